"""Training entry point (the role of ``pretrain_gpt.py`` under the reference's patch and of
its 1-click ``script/run.sh:149-160``):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 train.py \
        --num-layers 8 --hidden-size 8192 --ffn-hidden-size 28672 --num-attention-heads 64 \
        --group-query-attention --num-query-groups 8 --seq-length 4096 --vocab-size 128256 --swiglu \
        --tensor-model-parallel-size 8 --sequence-parallel --micro-batch-size 4 --global-batch-size 32 \
        --train-iters 10 --bf16 --dhellam --schedule-config config/best.json --log-throughput

Data is synthetic (uniform token ids of the configured shape).  ``--save`` / ``--load`` use
the Megatron-layout checkpoints of ``dhellam_b200.ckpt``; ``--metrics-jsonl`` writes one
JSON record per step.
"""
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def lr_at(args, it):
    """Linear warm-up then cosine decay, as the reference's run script configures Megatron."""
    import math
    warm = max(int(args.lr_warmup_fraction * args.lr_decay_iters), 1)
    if it < warm:
        return args.lr * (it + 1) / warm
    t = min((it - warm) / max(args.lr_decay_iters - warm, 1), 1.0)
    return args.min_lr + 0.5 * (args.lr - args.min_lr) * (1 + math.cos(math.pi * t))


def main(argv=None):
    import os
    if int(os.environ.get("WORLD_SIZE", "1")) == 1:   # library collectives are slow on growable segments
        os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    import torch
    import torch.distributed as dist
    from dhellam_b200.adaptor import initialize_dhellam_megatron
    from dhellam_b200.ckpt import load_checkpoint, save_checkpoint
    from dhellam_b200.common import print_rank0
    from dhellam_b200.data import TokenFileDataset, file_step_batches, synthetic_step_batches
    from dhellam_b200.runtime.metrics import MetricsLogger
    from dhellam_b200.trainer import Trainer

    args = initialize_dhellam_megatron(os.environ.get("MegaPath"), None, argv=argv)
    cfg, pcfg, train = args.model_config, args.parallel_config, args.train_config
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    tr = Trainer(cfg, pcfg, train, device=device, ps=args.parallel_state, distributed_optimizer=args.use_distributed_optimizer)
    start = 0
    if train.load:
        start = load_checkpoint(train.load, tr.model, tr.optimizer)
        print_rank0(f"resumed from {train.load} at iteration {start}")
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    ml = MetricsLogger(args.metrics_jsonl if args.rank == 0 else None, cfg, args.world_size, train.global_batch_size * cfg.seq_length,
                       measured_tflops=peaks.get("bf16_tflops_sustained"))
    print_rank0(f"model {cfg.total_params() / 1e9:.2f} B parameters, parallelism {pcfg.describe()}, "
                f"{train.num_microbatches(pcfg.dp)} micro-batches of {train.micro_batch_size} per step, "
                f"dual-strand {'on' if train.dhellam else 'off'}, fused comm {'on' if tr.env.fused_tp else 'off'}")
    dataset = None
    if args.data_path and not args.mock_data:
        # a flat token file (the payload of a Megatron .bin file); "<path>:<dtype>" selects the id type
        path, _, dt = args.data_path[-1].partition(":")
        dataset = TokenFileDataset(path, cfg.seq_length, dt or "int32", seed=train.seed)
        print_rank0(f"data: {path} ({len(dataset)} samples of {cfg.seq_length + 1} tokens)")
    tr.engine.time_pp = pcfg.pp > 1 and args.timing_log_level >= 2
    # Failure detection between steps: every rank beats on the rendezvous store and announces the
    # step it is about to launch; a rank that stopped is noticed on the host BEFORE the next launch.
    # After the step (the loop synchronises anyway) the device status word is read: a bounded wait
    # that gave up inside a kernel raises here, before the optimizer touched the master weights
    # (Trainer.check_status) and before any checkpoint is written.
    hb = gate = None
    if dist.is_initialized() and dist.get_world_size() > 1 and args.step_gate_timeout > 0:
        from dhellam_b200.runtime.watchdog import Heartbeat, StepGate
        hb = Heartbeat(interval=args.heartbeat_interval, timeout=args.heartbeat_timeout)
        gate = StepGate(timeout=args.step_gate_timeout, heartbeat=hb)
    tr.check_status = cuda
    inject = _parse_injection(os.environ.get("DHELLAM_INJECT_HOST_FAILURE"))
    try:
        _loop(args, tr, train, cfg, pcfg, dataset, device, cuda, start, ml, hb, gate, inject)
    finally:
        if hb is not None:
            hb.stop()
    if train.save:
        save_checkpoint(train.save, train.train_iters, tr.model, tr.optimizer)
    ml.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


def _parse_injection(spec):
    """``DHELLAM_INJECT_HOST_FAILURE=<rank>:<step>:<seconds>`` makes that rank stop beating and
    sleep on the host at that step, then exit with an error (a test hook; nothing on a GPU is
    faulted)."""
    if not spec:
        return None
    r, s, sec = spec.split(":")
    return int(r), int(s), float(sec)


def _loop(args, tr, train, cfg, pcfg, dataset, device, cuda, start, ml, hb, gate, inject):
    import torch
    import torch.distributed as dist
    from dhellam_b200.ckpt import save_checkpoint
    from dhellam_b200.common import print_rank0
    from dhellam_b200.data import file_step_batches, synthetic_step_batches
    for it in range(start, train.train_iters):
        if inject is not None and inject[0] == args.rank and inject[1] == it:
            if hb is not None:
                hb.pause()
            time.sleep(inject[2])
            raise RuntimeError(f"injected host failure on rank {args.rank} at step {it}")
        if gate is not None:
            gate.agree(it)                 # raises RankFailure: nothing of step `it` is launched, nothing is saved
        mbs = (file_step_batches(dataset, cfg, train, tr.ps, it, device) if dataset is not None
               else synthetic_step_batches(cfg, train, tr.ps, it, device))
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        loss = tr.train_step(mbs, lr_at(args, it))
        if cuda:
            torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        if dist.is_initialized():
            t = torch.tensor([ms], device=device if cuda else "cpu", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        lv = float(loss) if loss is not None else None
        extra = {"pp_bubble_ms": tr.engine.pp_bubble_ms()} if tr.engine.time_pp else None
        rec = ml.log(it + 1, ms, lv, float(tr.last_grad_norm) if tr.last_grad_norm is not None else None, extra)
        if (it + 1) % train.log_interval == 0:
            print_rank0(f" iteration {it + 1:6d}/{train.train_iters} | elapsed time per iteration (ms): {ms:.1f} | lm loss: "
                        f"{lv if lv is not None else float('nan'):.6E} | grad norm: {rec['grad_norm']} | throughput per GPU "
                        f"(TFLOP/s/GPU): {rec['model_tflops_per_gpu']:.1f} | tokens/s/GPU: {rec['tokens_per_s_per_gpu']:.0f}")
        if train.save and (it + 1) % train.save_interval == 0:
            save_checkpoint(train.save, it + 1, tr.model, tr.optimizer, {k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool, type(None)))})


if __name__ == "__main__":
    sys.exit(main())
