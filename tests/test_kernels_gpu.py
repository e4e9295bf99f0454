"""Numerics of every sm_100a kernel against the fp32 PyTorch reference of the same op
(the CPU path of the same ``ops`` function)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


@pytest.fixture(autouse=True)
def _seed_and_status():
    from dhellam_b200 import kernels as K
    torch.manual_seed(1234)
    yield
    torch.cuda.synchronize()
    st = K.read_status()
    assert st.code == 0, f"device status {st.code} at {st.where}"


@pytest.fixture(params=[False, True], ids=["atomic", "reproducible"])
def reduction_mode(request):
    """The kernels with cross-CTA reductions in both forms: order-dependent atomics (default) and the
    fixed-order forms of the reproducible mode."""
    from dhellam_b200 import kernels as K
    K.set_deterministic(request.param)
    yield request.param
    K.set_deterministic(False)


@pytest.fixture(params=[1, 2], ids=["single_cta", "cta_pair"])
def gemm_mode(request):
    from dhellam_b200.ops.gemm import set_gemm_mode
    set_gemm_mode(request.param)
    yield request.param
    set_gemm_mode(0)


@pytest.mark.parametrize("M,N,K_", [(128, 256, 64), (384, 1280, 1024), (200, 264, 136), (1024, 1024, 4096), (8, 4096, 256),
                                    (2048, 1536, 2048), (1100, 520, 328)])
def test_gemm_three_layouts(M, N, K_, gemm_mode):
    from dhellam_b200.ops.gemm import gemm_nn, gemm_nt, gemm_tn_acc
    x, w, dy = bf(M, K_), bf(N, K_), bf(M, N)
    assert rel(gemm_nt(x, w), x.float() @ w.float().t()) < 5e-3
    assert rel(gemm_nn(dy, w), dy.float() @ w.float()) < 5e-3
    g = torch.ones(N, K_, device=DEV)
    gemm_tn_acc(dy, x, g)
    assert rel(g, 1 + dy.float().t() @ x.float()) < 1e-4
    g2 = torch.full((N, K_), 7.0, device=DEV)
    gemm_tn_acc(dy, x, g2, accumulate=False)
    assert rel(g2, dy.float().t() @ x.float()) < 1e-4


@pytest.mark.parametrize("split", [2, 3, 4])
def test_gemm_weight_gradient_split_along_k_adds_atomically(split):
    """An accumulating GEMM may be cut into ``split`` work items per tile that each add their share
    into the fp32 output with the reducing bulk store; the result must not depend on the split."""
    from dhellam_b200.ops.gemm import gemm_tn_acc, set_gemm_mode, set_gemm_splitk
    set_gemm_mode(2)
    try:
        for M, N, K_ in ((4096, 520, 392), (1000, 256, 256), (8192, 1280, 512)):
            dy, x = bf(M, N), bf(M, K_)
            ref = 3.0 + dy.float().t() @ x.float()
            set_gemm_splitk(split)
            g = torch.full((N, K_), 3.0, device=DEV)
            gemm_tn_acc(dy, x, g)
            assert rel(g, ref) < 1e-4, (M, N, K_, rel(g, ref))
    finally:
        set_gemm_splitk(-1)
        set_gemm_mode(0)


@pytest.mark.parametrize("M,N,K_,kind", [(16384, 1280, 8192, "nt"), (16384, 8192, 1024, "nt"), (16384, 7168, 8192, "nn"),
                                         (16384, 16032, 2048, "nt"), (16384, 3584, 8192, "tn"), (16384, 1280, 8192, "tn")])
def test_gemm_headline_shapes_against_fp32(M, N, K_, kind):
    """The per-GPU shapes of the 8-way tensor-parallel headline run (16384 rows) against an fp32 product."""
    from dhellam_b200.ops.gemm import gemm_nn, gemm_nt, gemm_tn_acc
    if kind == "nt":
        x, w = bf(M, K_), bf(N, K_, scale=0.05)
        got, ref = gemm_nt(x, w), x.float() @ w.float().t()
        tol = 5e-3
    elif kind == "nn":
        dy, w = bf(M, N), bf(N, K_, scale=0.05)
        got, ref = gemm_nn(dy, w), dy.float() @ w.float()
        tol = 5e-3
    else:
        dy, x = bf(M, N, scale=0.1), bf(M, K_)
        got = torch.ones(N, K_, device=DEV)
        gemm_tn_acc(dy, x, got)
        ref = 1 + dy.float().t() @ x.float()
        tol = 1e-4
    assert rel(got, ref) < tol, rel(got, ref)


def test_gemm_sm_budget_and_strided_output(gemm_mode):
    from dhellam_b200.ops.gemm import gemm_nt
    x, w = bf(512, 512), bf(768, 512)
    big = torch.zeros(512, 1024, dtype=torch.bfloat16, device=DEV)
    out = gemm_nt(x, w, out=big[:, :768], sm_budget=16)
    assert rel(out, x.float() @ w.float().t()) < 5e-3
    assert float(big[:, 768:].abs().max()) == 0.0


@pytest.mark.parametrize("rows,h", [(64, 256), (300, 4096), (257, 8192), (33, 1024)])
def test_rmsnorm(rows, h, reduction_mode):
    from dhellam_b200.ops.norm import rmsnorm_bwd, rmsnorm_fwd
    x, w, dy, res = bf(rows, h), bf(h) * 0.1 + 1, bf(rows, h), bf(rows, h)
    y, rstd = rmsnorm_fwd(x, w, 1e-5)
    yr, rstdr = rmsnorm_fwd(x.cpu().float(), w.cpu().float(), 1e-5)
    assert rel(y, yr) < 5e-3 and rel(rstd, rstdr) < 1e-4
    mg = torch.zeros(h, device=DEV)
    dx, _ = rmsnorm_bwd(dy, x, w, rstd, weight_main_grad=mg, residual_grad=res)
    mgr = torch.zeros(h)
    dxr, _ = rmsnorm_bwd(dy.cpu().float(), x.cpu().float(), w.cpu().float(), rstdr, weight_main_grad=mgr, residual_grad=res.cpu().float())
    assert rel(dx, dxr) < 5e-3 and rel(mg, mgr) < 2e-3


@pytest.mark.parametrize("rows,h", [(64, 256), (129, 5120)])
def test_layernorm(rows, h, reduction_mode):
    from dhellam_b200.ops.norm import layernorm_bwd, layernorm_fwd
    x, w, b, dy = bf(rows, h) + 0.5, bf(h) * 0.1 + 1, bf(h) * 0.1, bf(rows, h)
    y, mu, rstd = layernorm_fwd(x, w, b, 1e-5)
    yr, mur, rstdr = layernorm_fwd(x.cpu().float(), w.cpu().float(), b.cpu().float(), 1e-5)
    assert rel(y, yr) < 5e-3 and rel(mu, mur) < 1e-3 and rel(rstd, rstdr) < 1e-3
    dx, dw, db = layernorm_bwd(dy, x, w, mu, rstd)
    dxr, dwr, dbr = layernorm_bwd(dy.cpu().float(), x.cpu().float(), w.cpu().float(), mur, rstdr)
    assert rel(dx, dxr) < 6e-3 and rel(dw, dwr) < 2e-3 and rel(db, dbr) < 2e-3


def test_swiglu_gelu():
    from dhellam_b200.ops.activation import gelu_bwd, gelu_fwd, swiglu_bwd, swiglu_fwd
    y, d = bf(300, 2 * 1032), bf(300, 1032)
    assert rel(swiglu_fwd(y), swiglu_fwd(y.cpu().float())) < 5e-3
    assert rel(swiglu_bwd(d, y), swiglu_bwd(d.cpu().float(), y.cpu().float())) < 5e-3
    x, dx = bf(77, 1024), bf(77, 1024)
    assert rel(gelu_fwd(x), gelu_fwd(x.cpu().float())) < 5e-3
    assert rel(gelu_bwd(dx, x), gelu_bwd(dx.cpu().float(), x.cpu().float())) < 5e-3


def test_bias_dropout_add_mask_matches_cpu_model():
    from dhellam_b200.ops.bda import bda_bwd, bda_fwd
    x, r, b = bf(130, 512), bf(130, 512), bf(512)
    for p in (0.0, 0.1):
        out = bda_fwd(x, r, b, p, seed=99)
        ref = bda_fwd(x.cpu().float(), r.cpu().float(), b.cpu().float(), p, seed=99)
        assert rel(out, ref) < 5e-3
    dx = bda_bwd(x, 0.1, seed=99)
    assert rel(dx, bda_bwd(x.cpu().float(), 0.1, seed=99)) < 5e-3


def test_rope_roundtrip_and_reference():
    from dhellam_b200.ops.rope import rope_apply_, rope_table
    T, nq, nkv, d = 96, 4, 2, 128
    qkv = bf(T, (nq + 2 * nkv) * d)
    pos = torch.randint(0, 64, (T,), dtype=torch.int32, device=DEV)
    cos, sin = rope_table(64, d, 500000.0, DEV)
    ref = rope_apply_(qkv.cpu().float().clone(), pos.cpu(), cos.cpu(), sin.cpu(), nq, nkv, d)
    orig = qkv.clone()
    out = rope_apply_(qkv, pos, cos, sin, nq, nkv, d)
    assert rel(out, ref) < 5e-3
    back = rope_apply_(out, pos, cos, sin, nq, nkv, d, inverse=True)
    assert rel(back, orig) < 1e-2


def test_embedding_and_cross_entropy(reduction_mode):
    from dhellam_b200.ops.embedding import embedding_bwd, embedding_fwd
    from dhellam_b200.ops.loss import ce_combine_stats, ce_local_stats, vocab_parallel_ce_bwd_
    T, h, Vl, v0 = 200, 256, 1000, 500
    tok = torch.randint(0, 2000, (T,), dtype=torch.int32, device=DEV)
    w = bf(Vl, h)
    assert rel(embedding_fwd(tok, w, v0), embedding_fwd(tok.cpu(), w.cpu().float(), v0)) < 1e-6
    d = bf(T, h)
    mg, mgr = torch.zeros(Vl, h, device=DEV), torch.zeros(Vl, h)
    embedding_bwd(d, tok, mg, v0)
    embedding_bwd(d.cpu().float(), tok.cpu(), mgr, v0)
    assert rel(mg, mgr) < 1e-5
    for dtype, Vc in ((torch.bfloat16, 1000), (torch.bfloat16, 1003), (torch.float32, 777)):
        buf = (torch.randn(T, 1008, device=DEV) * 3).to(dtype)
        logits = buf[:, :Vc]
        st = ce_local_stats(logits, tok, v0)
        str_ = ce_local_stats(logits.cpu().float(), tok.cpu(), v0)
        loss, lse = ce_combine_stats(st.unsqueeze(0))
        lossr, lser = ce_combine_stats(str_.unsqueeze(0))
        assert rel(lse, lser) < 1e-4 and rel(loss, lossr) < 1e-4
        gt = torch.rand(T, device=DEV)
        ref = vocab_parallel_ce_bwd_(logits.cpu().float().clone(), tok.cpu(), lser, gt.cpu(), v0)
        out = vocab_parallel_ce_bwd_(buf.clone()[:, :Vc], tok, lse, gt, v0)
        assert rel(out, ref) < 1e-2


def test_adam_and_sum_squares(reduction_mode):
    from dhellam_b200.optim.adam import adam_update, sum_squares
    n = 4096 * 3 + 4
    master = torch.randn(n, device=DEV)
    p = master.to(torch.bfloat16)
    m, v, g = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV), torch.randn(n, device=DEV)
    ref = [t.cpu().clone() for t in (p.float(), master, m, v, g)]
    for step in (1, 2):
        adam_update(p, master, m, v, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.5)
        adam_update(ref[0], ref[1], ref[2], ref[3], ref[4], 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 0.5)
    assert rel(master, ref[1]) < 1e-5 and rel(m, ref[2]) < 1e-5 and rel(v, ref[3]) < 1e-5 and rel(p, ref[1]) < 5e-3
    assert abs(float(sum_squares(g)) - float((g.double() ** 2).sum())) / float((g.double() ** 2).sum()) < 1e-4


def test_router_topk():
    from dhellam_b200.ops.moe import router_topk_fwd
    T, h, E, k = 333, 512, 8, 2
    x, w = bf(T, h), bf(E, h, scale=0.05)
    probs, topi, gates = router_topk_fwd(x, w, k)
    pr, ti, gr = router_topk_fwd(x.cpu().float(), w.cpu().float(), k)
    assert rel(probs, pr) < 1e-3
    same = (topi.cpu() == ti).all(dim=1)
    assert same.float().mean() > 0.99            # near-ties may order differently in bf16 vs fp32 accumulation
    assert rel(gates.cpu()[same], gr[same]) < 1e-3


@pytest.fixture(params=[0, 1], ids=["tile128", "pipelined64"])
def attn_bwd_mode(request):
    """Both dK/dV kernels: the default and the pipelined transposed-score form."""
    from dhellam_b200.ops.attention import set_attn_bwd_mode
    set_attn_bwd_mode(request.param)
    yield request.param
    set_attn_bwd_mode(0)


@pytest.mark.parametrize("Sq,Sk,B,Hq,Hk,causal", [(128, 128, 1, 1, 1, True), (256, 256, 2, 4, 2, True), (384, 384, 1, 2, 1, False),
                                                     (200, 200, 2, 2, 2, True), (128, 256, 1, 2, 1, False), (256, 128, 1, 2, 2, False)])
def test_attention_forward_backward(Sq, Sk, B, Hq, Hk, causal, attn_bwd_mode):
    from dhellam_b200.ops.attention import attn_bwd, attn_fwd
    d = 128
    # strided views into packed buffers, as the engine uses them
    qkv = bf(Sq, B, Hq + 2 * Hk, d)
    q = qkv[:, :, :Hq]
    if Sk == Sq:
        k, v = qkv[:, :, Hq:Hq + Hk], qkv[:, :, Hq + Hk:]
    else:
        kv = bf(Sk, B, 2 * Hk, d)
        k, v = kv[:, :, :Hk], kv[:, :, Hk:]
    scale = 1.0 / math.sqrt(d)
    o, lse = attn_fwd(q, k, v, causal, scale)
    qc, kc, vc = q.cpu().float(), k.cpu().float(), v.cpu().float()
    oref, lref = attn_fwd(qc, kc, vc, causal, scale)
    assert rel(o, oref) < 1e-2, rel(o, oref)
    assert rel(lse, lref) < 1e-3
    do = bf(Sq, B, Hq, d)
    dq, dk, dv = attn_bwd(do, q, k, v, o, lse, causal, scale)
    dqr, dkr, dvr = attn_bwd(do.cpu().float(), qc, kc, vc, oref, lref, causal, scale)
    assert rel(dq, dqr) < 2e-2, ("dq", rel(dq, dqr))
    assert rel(dk, dkr) < 2e-2, ("dk", rel(dk, dkr))
    assert rel(dv, dvr) < 2e-2, ("dv", rel(dv, dvr))


@pytest.mark.parametrize("Sq,Sk,B,Hq,Hk", [(4096, 4096, 1, 8, 1), (1024, 2048, 2, 4, 2), (2048, 2048, 4, 16, 2)])
def test_attention_large_shapes_against_fp32(Sq, Sk, B, Hq, Hk):
    """Causal attention at the sizes the training step uses, against plain fp32 PyTorch (explicit softmax and
    autograd on the GPU): 4096 positions with eight query heads on one KV head (the dK/dV kernel then splits the
    heads of that KV head over several CTAs), more keys than queries (mask aligned to the last key, the
    context-parallel case), and a batch that fills the GPU without a head split."""
    from dhellam_b200.ops.attention import attn_bwd, attn_fwd
    d = 128
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = bf(Sq, B, Hq, d), bf(Sk, B, Hk, d), bf(Sk, B, Hk, d), bf(Sq, B, Hq, d)
    o, lse = attn_fwd(q, k, v, True, scale)
    dq, dk, dv = attn_bwd(do, q, k, v, o, lse, True, scale)
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    g = Hq // Hk
    sc = torch.einsum("sbhd,tbhd->bhst", qf, kf.repeat_interleave(g, dim=2)) * scale
    i = torch.arange(Sq, device=DEV).unsqueeze(1)
    j = torch.arange(Sk, device=DEV).unsqueeze(0)
    sc = sc.masked_fill(j > i + (Sk - Sq), float("-inf"))
    ref_lse = torch.logsumexp(sc, dim=-1)
    oref = torch.einsum("bhst,tbhd->sbhd", torch.softmax(sc, dim=-1), vf.repeat_interleave(g, dim=2))
    oref.backward(do.float())
    assert rel(o, oref.detach()) < 1e-2 and rel(lse, ref_lse.detach()) < 1e-3
    assert rel(dq, qf.grad) < 2e-2, ("dq", rel(dq, qf.grad))
    assert rel(dk, kf.grad) < 2e-2, ("dk", rel(dk, kf.grad))
    assert rel(dv, vf.grad) < 2e-2, ("dv", rel(dv, vf.grad))


@pytest.mark.parametrize("budget", [1, 5, 24, 100])
def test_attention_sm_budget_gives_identical_results(budget):
    """With an SM budget the attention kernels run as consecutive launches of at most that many CTAs
    (tile columns split when one head alone has more tiles than the budget, else whole (head, batch)
    pairs per launch); every tile computes exactly what it computes without a budget."""
    from dhellam_b200.ops.attention import attn_bwd, attn_fwd
    Sq, B, Hq, Hk, d = 1024, 2, 4, 2, 128
    qkv = bf(Sq, B, Hq + 2 * Hk, d)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hk], qkv[:, :, Hq + Hk:]
    do = bf(Sq, B, Hq, d)
    scale = 1.0 / math.sqrt(d)
    o0, l0 = attn_fwd(q, k, v, True, scale)
    g0 = attn_bwd(do, q, k, v, o0, l0, True, scale)
    o1, l1 = attn_fwd(q, k, v, True, scale, sm_budget=budget)
    g1 = attn_bwd(do, q, k, v, o1, l1, True, scale, sm_budget=budget)
    torch.cuda.synchronize()
    assert torch.equal(o0, o1) and torch.equal(l0, l1)
    for a, b in zip(g0, g1):
        assert torch.equal(a, b)


def test_varlen_api_with_equal_lengths_uses_strided_views_of_the_packed_tensors():
    """``pymha_varlen_fwd / bwd`` on a packed batch of equal-length sequences (one launch over strided views)
    against the fixed-length entry points on contiguous [s, b, h, d] copies."""
    from dhellam_b200.ops.attention import attn_bwd, attn_fwd, pymha_varlen_bwd, pymha_varlen_fwd
    b, s, hq, hk, d = 3, 256, 4, 2, 128
    cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32, device=DEV)
    q, k, v, do = bf(b * s, hq, d), bf(b * s, hk, d), bf(b * s, hk, d), bf(b * s, hq, d)
    scale = 1.0 / math.sqrt(d)
    out, lse = pymha_varlen_fwd(q, k, v, cu, cu, s, s, 0.0, scale, True)
    dq, dk, dv = pymha_varlen_bwd(do, q, k, v, out, lse, cu, cu, s, s, 0.0, scale, True)
    sb = lambda t: t.view(b, s, t.shape[1], d).permute(1, 0, 2, 3).contiguous()
    o2, l2 = attn_fwd(sb(q), sb(k), sb(v), True, scale)
    g2 = attn_bwd(sb(do), sb(q), sb(k), sb(v), o2, l2, True, scale)
    assert torch.equal(sb(out), o2) and torch.equal(lse, l2)
    for a, r in zip((dq, dk, dv), g2):
        assert rel(sb(a), r) < 1e-3


def test_bounded_wait_reports_timeout_without_hanging():
    """A flag that nobody sets: the device-side wait gives up after its (short) budget and
    the host reads the status word; the context stays usable."""
    from dhellam_b200 import kernels as K
    from dhellam_b200.runtime.signals import probe_flag_wait
    st = probe_flag_wait(expect=1, budget_cycles=200000)
    assert st.code == 2 and st.extra == 1
    x = torch.ones(4, device=DEV)
    assert float(x.sum()) == 4.0
    assert K.read_status().code == 0


def test_communication_wait_entry_point_gives_up_after_its_budget():
    """The real wait in front of a consumer of gathered rows (``dh_wait_counters``) on counters that
    nothing raises, with a budget of about a millisecond: the kernel gives up, the status word says
    "flag timeout" at that site, and the context stays usable.  No peer is involved."""
    from ctypes import c_int, c_int64, c_uint, c_void_p
    from dhellam_b200 import kernels as K
    counters = torch.zeros(16, dtype=torch.int32, device=DEV)
    fn = K.proto("dh_wait_counters", [c_void_p, c_int, c_uint, c_int64, c_void_p])
    K.check(fn(counters.data_ptr(), 16, 3, 2_000_000, K.stream_ptr(None)), "dh_wait_counters")
    st = K.read_status(clear=True)
    assert st.code == 2 and st.where == 641 and st.extra == 3, (st.code, st.where, st.extra)
    counters.fill_(3)                          # the same wait succeeds at once when the counters are there
    K.check(fn(counters.data_ptr(), 16, 3, 2_000_000, K.stream_ptr(None)), "dh_wait_counters")
    assert K.read_status().code == 0
    assert float(torch.ones(4, device=DEV).sum()) == 4.0


def test_device_resident_moe_exchange_and_grouped_gemms():
    """Plan -> dispatch -> grouped expert GEMMs -> combine on one GPU (ep = 1) against plain PyTorch: the
    routing sizes never reach the host on the device path, the reference below sorts on the host."""
    from types import SimpleNamespace
    from dhellam_b200.ops.moe_native import DeviceMoE
    E, k, h, f, T = 4, 2, 512, 256, 300
    cfg = SimpleNamespace(num_experts=E, moe_top_k=k, hidden_size=h)
    ps = SimpleNamespace(ep=1, ep_rank=0, ep_group=None)
    dev = DeviceMoE(ps, cfg, None, torch.device(DEV), T)
    x = bf(T, h)
    logits = torch.randn(T, E, device=DEV)
    topi = logits.topk(k, dim=-1).indices.to(torch.int32).contiguous()
    gates = torch.softmax(torch.randn(T, k, device=DEV), -1).contiguous()
    plan = dev.plan(topi)
    slot, _ = dev.dispatch(plan, x, "xe", record=True)
    xe = dev.landed("xe", slot)
    torch.cuda.synchronize()
    offs, rows_e = plan.offs.cpu().tolist(), plan.rows_e.cpu().tolist()
    flat = topi.reshape(-1).cpu()
    assert int(plan.overflow) == 0 and all(o % 256 == 0 for o in offs)
    for e in range(E):
        idx = torch.nonzero(flat == e).squeeze(1)              # stable order of the copies of expert e
        assert rows_e[e] == idx.numel()
        got = xe[offs[e]:offs[e] + rows_e[e]].cpu()
        assert torch.equal(got, x.cpu()[idx // k]), e
        assert float(xe[offs[e] + rows_e[e]:offs[e + 1]].abs().max() if offs[e + 1] > offs[e] + rows_e[e] else 0.0) == 0.0
    w1 = bf(E, 2 * f, h, scale=0.05)
    w2 = bf(E, h, f, scale=0.05)
    z = dev.grouped_nt(xe, w1, plan)
    a = dev.swiglu_fwd(z, plan)
    y, yslot = dev.output_buffer("y")
    dev.grouped_nt(a, w2, plan, out=y)
    dev.publish("y", yslot)
    out, copies = dev.combine(plan, "y", yslot, gates=gates, keep_copies=True)
    torch.cuda.synchronize()
    # reference: per token, per choice
    xf = x.float()
    ref = torch.zeros(T, h, device=DEV)
    for j in range(k):
        for e in range(E):
            m = topi[:, j] == e
            if m.any():
                zz = (xf[m] @ w1[e].float().t()).to(torch.bfloat16).float()
                aa = (torch.nn.functional.silu(zz[:, :f]) * zz[:, f:]).to(torch.bfloat16).float()
                yy = (aa @ w2[e].float().t()).to(torch.bfloat16).float()
                ref[m] += gates[m, j:j + 1] * yy
    assert rel(out, ref) < 1e-2, rel(out, ref)
    # backward products on the same plan
    d_y = torch.zeros_like(y)
    for e in range(E):
        d_y[offs[e]:offs[e] + rows_e[e]] = bf(rows_e[e], h)
    d_a = dev.grouped_nn(d_y, w2, plan)
    g2 = torch.ones(E, h, f, device=DEV)
    dev.grouped_tn_acc(d_y, a, g2, plan)
    torch.cuda.synchronize()
    for e in range(E):
        lo, hi = offs[e], offs[e] + rows_e[e]
        assert rel(d_a[lo:hi], d_y[lo:hi].float() @ w2[e].float()) < 5e-3
        assert rel(g2[e], 1 + d_y[lo:hi].float().t() @ a[lo:hi].float()) < 1e-3
    # the pull without gates is the plain sum over a token's copies
    s2, sslot = dev.output_buffer("dxe")
    s2.copy_(y)
    dev.publish("dxe", sslot)
    summed, _ = dev.combine(plan, "dxe", sslot)
    assert rel(summed, copies.float().view(T, k, h).sum(1)) < 1e-2
