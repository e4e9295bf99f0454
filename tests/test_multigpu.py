"""Multi-GPU tests (need >= 2 CUDA devices; skipped otherwise): the fused
all-gather->GEMM and GEMM->reduce-scatter kernels against the NCCL + GEMM composition, and
the engine with tensor parallelism on GPUs against the single-GPU engine."""
import os
import socket
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args, errq):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        fn(rank, world, *args)
        torch.cuda.synchronize()
        dist.barrier()
    except Exception:
        errq.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_gpu_ranks(fn, world, *args, timeout=300):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            errs.append((-1, "rank timed out"))
    if errs:
        raise AssertionError("\n".join(f"[rank {r}]\n{tb}" for r, tb in errs))


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _fused_worker(rank, world, rows, h, n_out, iters):
    import torch.distributed as dist
    from dhellam_b200 import kernels as K
    from dhellam_b200.config import ModelConfig, ParallelConfig, TrainConfig
    from dhellam_b200.ops import comm as C
    from dhellam_b200.ops.fused_comm import FusedTP
    from dhellam_b200.ops.gemm import gemm_nn, gemm_nt
    from dhellam_b200.parallel import state as PS
    dev = torch.device("cuda", rank)
    ps = PS.initialize_model_parallel(ParallelConfig(tp=world))
    cfg = ModelConfig(hidden_size=h, seq_length=rows, num_attention_heads=h // 128, num_query_groups=h // 128)
    fused = FusedTP(ps, cfg, TrainConfig(micro_batch_size=1), dev, max_rows=rows, width=h)
    torch.manual_seed(100 + rank)
    side = torch.cuda.Stream()
    for it in range(iters):
        shard = (torch.randn(rows // world, h, device=dev)).to(torch.bfloat16)
        w = (torch.randn(n_out, h, device=dev) * 0.05).to(torch.bfloat16)
        # all-gather -> GEMM, forward form (B K-major) and dgrad form (B MN-major)
        full_ref, _ = C.gather_along_first_dim(shard, ps.tp_group)
        out, full = fused.ag_gemm(shard, w, "attn_c")
        torch.cuda.synchronize()
        assert torch.equal(full, full_ref), f"gathered operand differs (iter {it})"
        assert _rel(out, gemm_nt(full_ref, w)) < 1e-3
        wt = (torch.randn(h, n_out, device=dev) * 0.05).to(torch.bfloat16)
        out2, full2 = fused.ag_gemm(shard, wt, "mlp_l_bwd", transpose_w=True)
        assert _rel(out2, gemm_nn(full_ref, wt)) < 1e-3
        assert torch.equal(full2, full_ref)
        # the all-gather alone (push + counter wait), as used to re-gather for a weight gradient
        full3 = fused.all_gather(shard, "regather_mlp")
        torch.cuda.synchronize()
        assert torch.equal(full3, full_ref), f"stand-alone gather differs (iter {it})"
        # GEMM -> reduce-scatter, both forms
        a = torch.randn(rows, n_out, device=dev).to(torch.bfloat16)
        w2 = (torch.randn(h, n_out, device=dev) * 0.05).to(torch.bfloat16)
        ref, _ = C.reduce_scatter_along_first_dim(gemm_nt(a, w2), ps.tp_group)
        got = fused.gemm_rs(a, w2)
        assert _rel(got, ref) < 1e-2, _rel(got, ref)
        w3 = (torch.randn(n_out, h, device=dev) * 0.05).to(torch.bfloat16)
        ref3, _ = C.reduce_scatter_along_first_dim(gemm_nn(a, w3), ps.tp_group)
        got3 = fused.gemm_rs(a, w3, transpose_w=True)
        assert _rel(got3, ref3) < 1e-2, _rel(got3, ref3)
        # the reduce-scatter alone: a local GEMM into symmetric memory, then the in-switch
        # (or peer-load) reduction; with and without the multicast alias
        for mc in (fused.mc_ptr, 0):
            keep, fused.mc_ptr = fused.mc_ptr, mc
            part = fused.partial_buffer("head_bwd", rows, h)      # whole-buffer announcements: its own site
            gemm_nt(a, w2, out=part)
            got4 = fused.rs_reduce("head_bwd")
            fused.mc_ptr = keep
            assert _rel(got4, ref) < 1e-2, (_rel(got4, ref), mc)
        # tile-granular forms: the GEMM waits per 128-row block for the pushed rows inside the kernel (own shard
        # first), and the producing GEMM signals finished row blocks to the reduction kernel, which is launched
        # on another stream right after the GEMM's launch point
        fused.gather_start(shard, "attn_c", stream=side)
        view, sync = fused.gather_consume("attn_c")
        assert sync is not None
        out5 = gemm_nt(view, w, sync=sync)
        torch.cuda.synchronize()
        assert torch.equal(view, full_ref) and _rel(out5, gemm_nt(full_ref, w)) < 1e-3
        fused.gather_start(shard, "mlp_l_bwd", stream=side)
        view, sync = fused.gather_consume("mlp_l_bwd")
        out6 = gemm_nn(view, wt, sync=sync)
        assert _rel(out6, gemm_nn(full_ref, wt)) < 1e-3
        for mc in (fused.mc_ptr, 0):
            keep, fused.mc_ptr = fused.mc_ptr, mc
            part, sync = fused.partial_produce("mlp_l", rows, h)
            assert sync is not None
            launched = torch.cuda.Event()
            launched.record()
            gemm_nt(a, w2, out=part, sync=sync)
            side.wait_event(launched)
            with torch.cuda.stream(side):
                got7 = fused.rs_reduce("mlp_l")
            torch.cuda.current_stream().wait_stream(side)
            fused.mc_ptr = keep
            assert _rel(got7, ref) < 1e-2, (_rel(got7, ref), mc)
            part, sync = fused.partial_produce("mlp_c_bwd", rows, h)
            gemm_nn(a, w3, out=part, sync=sync)
            got8 = fused.rs_reduce("mlp_c_bwd")
            assert _rel(got8, ref3) < 1e-2, _rel(got8, ref3)
    torch.cuda.synchronize()
    st = K.read_status()
    assert st.code == 0, (st.code, st.where, st.extra)


def test_fused_ag_gemm_and_gemm_rs_match_nccl_composition():
    _need(2)
    world = 2 if torch.cuda.device_count() < 4 else 4
    run_gpu_ranks(_fused_worker, world, 2048, 1024, 768, 3)


def _engine_worker(rank, world, fused, out_path, policy="auto"):
    os.environ["DHELLAM_FUSED_POLICY"] = policy
    from dhellam_b200 import kernels as K
    from dhellam_b200.config import ModelConfig, ParallelConfig, TrainConfig
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.models.sharding import random_full_head, random_full_layer
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    cfg = ModelConfig(name="t-llama", num_layers=4, hidden_size=1024, ffn_hidden_size=2048, num_attention_heads=8,
                      num_query_groups=4, head_dim=128, vocab_size=4096, seq_length=512, rope_theta=500000.0)
    train = TrainConfig(micro_batch_size=2, global_batch_size=6, dtype="bf16", clip_grad=0.0, fused_comm=fused)
    tr = Trainer(cfg, ParallelConfig(tp=world), train, device=torch.device("cuda", rank))
    layers = [random_full_layer(cfg, i, 3) for i in range(cfg.num_layers)]
    head = random_full_head(cfg, 3)
    for i, w in enumerate(layers):
        tr.model.load_full_layer_weights(i, w)
    tr.model.load_full_head_weights(head)
    samples = [synthetic_tokens(cfg, 2, 40 + i) for i in range(3)]
    mbs = [make_microbatch(cfg, tr.ps, s, i, 40 + i, tr.device) for i, s in enumerate(samples)]
    tr.optimizer.zero_grad()
    losses = tr.engine.run_step(mbs)
    tr.optimizer.reduce_gradients()
    torch.cuda.synchronize()
    assert K.read_status().code == 0
    if rank == 0:
        torch.save({"losses": [float(l) for l in losses], "fused": bool(tr.env.fused_tp),
                    "g_ln": tr.model.dctb[0].ln_attn_weight_first.main_grad.cpu(),
                    "g_qkv": tr.model.dctb[0].column_attn_weight_first.main_grad.cpu()}, out_path)


def test_tp_engine_fused_matches_unfused(tmp_path):
    _need(2)
    b = str(tmp_path / "nccl.pt")
    run_gpu_ranks(_engine_worker, 2, False, b)
    rb = torch.load(b)
    assert not rb["fused"]
    # every collective inside its GEMM kernel / every collective as its own kernel on the
    # communication stream
    for policy in ("fused", "split"):
        a = str(tmp_path / f"{policy}.pt")
        run_gpu_ranks(_engine_worker, 2, True, a, policy)
        ra = torch.load(a)
        assert ra["fused"]
        for x, y in zip(ra["losses"], rb["losses"]):
            assert abs(x - y) / abs(y) < 1e-2, (policy, ra["losses"], rb["losses"])
        assert _rel(ra["g_ln"], rb["g_ln"]) < 5e-2, policy
        assert _rel(ra["g_qkv"], rb["g_qkv"]) < 5e-2, policy


def _cp_worker(rank, world, ring, out_path, tp=1):
    """Context parallelism on GPUs: ``ring`` = library point-to-point ring, else the peer-memory gather form."""
    os.environ["DHELLAM_CP_RING"] = "1" if ring else "0"
    from dhellam_b200 import kernels as K
    from dhellam_b200.config import ModelConfig, ParallelConfig, TrainConfig
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.models.sharding import random_full_head, random_full_layer
    from dhellam_b200.trainer import Trainer
    cfg = ModelConfig(name="t-llama", num_layers=2, hidden_size=1024, ffn_hidden_size=2048, num_attention_heads=8,
                      num_query_groups=4, head_dim=128, vocab_size=4096, seq_length=1024, rope_theta=500000.0)
    train = TrainConfig(micro_batch_size=2, global_batch_size=4, dtype="bf16", clip_grad=0.0)
    cp = world // tp
    tr = Trainer(cfg, ParallelConfig(cp=cp, tp=tp), train, device=torch.device("cuda", rank))
    assert (tr.env.fused_cp is not None) == (cp > 1 and not ring)
    for i in range(cfg.num_layers):
        tr.model.load_full_layer_weights(i, random_full_layer(cfg, i, 3))
    tr.model.load_full_head_weights(random_full_head(cfg, 3))
    samples = [synthetic_tokens(cfg, 2, 40 + i) for i in range(2)]
    mbs = [make_microbatch(cfg, tr.ps, s, i, 40 + i, tr.device) for i, s in enumerate(samples)]
    tr.optimizer.zero_grad()
    losses = tr.engine.run_step(mbs)
    tr.optimizer.reduce_gradients()
    torch.cuda.synchronize()
    assert K.read_status().code == 0
    if rank == 0:
        torch.save({"losses": [float(l) for l in losses],
                    "g_qkv": tr.model.dctb[0].column_attn_weight_first.main_grad.cpu(),
                    "g_ln": tr.model.dctb[0].ln_attn_weight_first.main_grad.cpu()}, out_path)


def test_context_parallel_gather_over_peer_memory_matches_ring_and_single_gpu(tmp_path):
    """cp = 2 on two GPUs: the peer-memory gather form (push K|V chunks, one causal call per query chunk, in-switch
    reduction of dK|dV) against the library ring and against one GPU without context parallelism."""
    _need(2)
    paths = {k: str(tmp_path / f"{k}.pt") for k in ("single", "ring", "gather")}
    run_gpu_ranks(_cp_worker, 1, True, paths["single"])
    run_gpu_ranks(_cp_worker, 2, True, paths["ring"])
    run_gpu_ranks(_cp_worker, 2, False, paths["gather"])
    ref = torch.load(paths["single"])
    for k in ("ring", "gather"):
        got = torch.load(paths[k])
        for x, y in zip(got["losses"], ref["losses"]):
            assert abs(x - y) / abs(y) < 1e-2, (k, got["losses"], ref["losses"])
        assert _rel(got["g_qkv"], ref["g_qkv"]) < 5e-2, (k, _rel(got["g_qkv"], ref["g_qkv"]))
        assert _rel(got["g_ln"], ref["g_ln"]) < 5e-2, k


def test_context_parallel_with_tensor_parallel_on_four_gpus(tmp_path):
    """tp = 2 x cp = 2 (the layout of the long-context configuration, scaled down) against one GPU."""
    _need(4)
    a, b = str(tmp_path / "single.pt"), str(tmp_path / "tp2cp2.pt")
    run_gpu_ranks(_cp_worker, 1, True, a)
    run_gpu_ranks(_cp_worker, 4, False, b, 2)
    ref, got = torch.load(a), torch.load(b)
    for x, y in zip(got["losses"], ref["losses"]):
        assert abs(x - y) / abs(y) < 1e-2, (got["losses"], ref["losses"])


def _moe_worker(rank, world, out_path):
    from dhellam_b200 import kernels as K
    from dhellam_b200.config import ModelConfig, ParallelConfig, TrainConfig
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.models.sharding import random_full_head, random_full_layer
    from dhellam_b200.trainer import Trainer
    cfg = ModelConfig(name="t-moe", num_layers=2, hidden_size=512, ffn_hidden_size=512, num_attention_heads=4,
                      num_query_groups=2, head_dim=128, vocab_size=2048, seq_length=256, num_experts=4, moe_top_k=2,
                      moe_aux_loss_coeff=0.0)
    train = TrainConfig(micro_batch_size=2, global_batch_size=2 * world, dtype="bf16", clip_grad=0.0)
    tr = Trainer(cfg, ParallelConfig(dp=world, ep=world), train, device=torch.device("cuda", rank))
    assert tr.env.moe_dev is not None and tr.env.moe_dev.ep == world
    for i in range(cfg.num_layers):
        tr.model.load_full_layer_weights(i, random_full_layer(cfg, i, 3))
    tr.model.load_full_head_weights(random_full_head(cfg, 3))
    # every data-parallel rank gets its own micro-batch; the single-GPU run sees both in turn
    samples = [synthetic_tokens(cfg, 2, 40 + r) for r in range(2)]
    if world == 1:
        mbs = [make_microbatch(cfg, tr.ps, s, i, 40 + i, tr.device) for i, s in enumerate(samples)]
    else:
        mbs = [make_microbatch(cfg, tr.ps, samples[rank], 0, 40 + rank, tr.device)]
    tr.optimizer.zero_grad()
    losses = tr.engine.run_step(mbs)
    torch.cuda.synchronize()
    assert K.read_status().code == 0
    torch.save({"losses": [float(l) for l in losses]}, out_path + f".{rank}")


def test_expert_parallel_device_exchange_matches_single_gpu(tmp_path):
    """ep = 2 over peer memory (device-side plan, push dispatch, grouped expert GEMMs, pull combine): each rank's
    micro-batch loss equals the loss of the same micro-batch on one GPU with all experts local."""
    _need(2)
    a, b = str(tmp_path / "one"), str(tmp_path / "two")
    run_gpu_ranks(_moe_worker, 1, a)
    run_gpu_ranks(_moe_worker, 2, b)
    ref = torch.load(a + ".0")["losses"]
    got = [torch.load(b + ".0")["losses"][0], torch.load(b + ".1")["losses"][0]]
    for x, y in zip(got, ref):
        assert abs(x - y) / abs(y) < 1e-2, (got, ref)


def _train_worker(rank, world, par, dist_opt, out_path):
    """Two optimizer steps of a small Llama under the given parallel layout; every rank sees the same global batch."""
    from dhellam_b200 import kernels as K
    from dhellam_b200.config import ModelConfig, ParallelConfig, TrainConfig
    from dhellam_b200.models.sharding import random_full_head, random_full_layer
    from dhellam_b200.trainer import Trainer
    cfg = ModelConfig(name="t-llama", num_layers=4, hidden_size=512, ffn_hidden_size=1024, num_attention_heads=4,
                      num_query_groups=2, head_dim=128, vocab_size=2048, seq_length=256, rope_theta=500000.0)
    train = TrainConfig(micro_batch_size=1, global_batch_size=4, dtype="bf16", lr=1e-3, weight_decay=0.0, clip_grad=1.0)
    tr = Trainer(cfg, ParallelConfig(**par), train, device=torch.device("cuda", rank), distributed_optimizer=dist_opt)
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    for i in range(cfg.num_layers):
        tr.model.load_full_layer_weights(i, random_full_layer(cfg, i, 3))       # a stage keeps only the layers it owns
    if tr.model.dchb is not None:
        tr.model.load_full_head_weights(random_full_head(cfg, 3))
    o = tr.optimizer
    o.master.copy_(tr.model.flat_param[o.lo:o.hi].float())
    tr.engine.time_pp = par.get("pp", 1) > 1
    losses = []
    dp, r = tr.ps.dp, tr.ps.dp_rank
    for step in range(2):
        # the same four samples per step whatever the layout; a data-parallel rank takes its share of them
        mine = [j for j in range(4) if j * dp // 4 == r]
        mbs = [make_microbatch(cfg, tr.ps, synthetic_tokens(cfg, 1, 900 + 10 * step + j), i, 900 + 10 * step + j, tr.device)
               for i, j in enumerate(mine)]
        l = tr.train_step(mbs)
        losses.append(float(l) if l is not None else None)
    torch.cuda.synchronize()
    assert K.read_status().code == 0
    if tr.engine.time_pp:
        assert tr.engine.pp_bubble_ms() > 0.0
    if losses[0] is not None and tr.ps.dp_rank == 0 and tr.ps.tp_rank == 0:
        torch.save({"losses": losses}, out_path)


@pytest.mark.parametrize("par,dist_opt", [(dict(pp=2), False), (dict(dp=2), True), (dict(dp=2), False)],
                         ids=["pp2", "dp2-distributed-optimizer", "dp2"])
def test_pipeline_and_data_parallel_training_on_gpus_match_one_gpu(tmp_path, par, dist_opt):
    """pp = 2 (folded 1F1B, per-strand overlapped exchange) and dp = 2 (bucketed gradient reduction under the
    backward pass; with the distributed optimizer a reduce-scatter into the optimizer shards) on two GPUs
    against the same two optimizer steps on one GPU."""
    _need(2)
    a, b = str(tmp_path / "one.pt"), str(tmp_path / "two.pt")
    run_gpu_ranks(_train_worker, 1, {}, False, a)
    run_gpu_ranks(_train_worker, 2, par, dist_opt, b)
    ref, got = torch.load(a)["losses"], torch.load(b)["losses"]
    for x, y in zip(got, ref):
        assert abs(x - y) / abs(y) < 2e-2, (got, ref)


def test_fused_collectives_at_world_8_with_headline_rows():
    """All eight GPUs of a box, 16384 rows x 8192 columns (the per-micro-batch activation of the headline run):
    one-kernel all-gather->GEMM and GEMM->reduce-scatter, the stand-alone push / row-block reduction with in-kernel
    waits and signals, with and without the NVSwitch multicast alias, against the NCCL + GEMM composition."""
    _need(8)
    run_gpu_ranks(_fused_worker, 8, 16384, 8192, 1024, 1, timeout=600)
