"""Names and contracts kept from the reference package, on CPU."""
import torch


def test_package_facade_exports_reference_names():
    import dhellam_b200 as d
    for n in ("gemm_fwd", "gemm_bwd", "gemm_fwd_event", "pylayernorm_fwd", "pylayernorm_bwd", "gather_along_first_dim",
              "reduce_scatter_along_first_dim", "pymha_varlen_fwd", "pymha_varlen_bwd", "_get_qkv_layout"):
        assert hasattr(d, n), n
    from dhellam_b200 import _Clib
    for n in ("add_tensors", "pygemm", "pygelu", "pybda", "pymha_varlen_fwd", "pymha_varlen_bwd"):
        assert hasattr(_Clib, n), n


def test_gemm_wrappers_match_matmul():
    from dhellam_b200 import gemm_bwd, gemm_fwd
    x, w = torch.randn(6, 8), torch.randn(5, 8)
    y, _ = gemm_fwd(None, x, w)
    assert torch.allclose(y, x @ w.t(), atol=1e-5)
    dy = torch.randn(6, 5)
    wg = torch.ones(5, 8)
    dx, wg2, _, _ = gemm_bwd(None, dy, w, x, None, wg, grad_accumulate=True)
    assert torch.allclose(dx, dy @ w, atol=1e-5)
    assert torch.allclose(wg2, 1 + dy.t() @ x, atol=1e-5)


def test_varlen_attention_matches_per_sequence_reference():
    from dhellam_b200 import pymha_varlen_bwd, pymha_varlen_fwd
    from dhellam_b200.ops.attention import attn_fwd
    torch.manual_seed(0)
    lens = [5, 9, 3]
    cu = torch.tensor([0, 5, 14, 17], dtype=torch.int32)
    q, k, v = torch.randn(17, 4, 16), torch.randn(17, 2, 16), torch.randn(17, 2, 16)
    out, lse = pymha_varlen_fwd(q, k, v, cu, cu, 9, 9, 0.0, 0.25, True)
    o1, _ = attn_fwd(q[5:14].unsqueeze(1), k[5:14].unsqueeze(1), v[5:14].unsqueeze(1), True, 0.25)
    assert torch.allclose(out[5:14], o1.squeeze(1), atol=1e-5)
    dq, dk, dv = pymha_varlen_bwd(torch.randn_like(out), q, k, v, out, lse, cu, cu, 9, 9, 0.0, 0.25, True)
    assert dq.shape == q.shape and dk.shape == k.shape and torch.isfinite(dv).all()


def test_varlen_attention_with_equal_lengths_runs_as_one_call_and_matches_the_per_sequence_path():
    """A packed batch of equal-length sequences (what the reference passes) takes the single-launch path; the
    result equals the per-sequence path, which unequal lengths force."""
    from dhellam_b200 import pymha_varlen_bwd, pymha_varlen_fwd
    from dhellam_b200.ops import attention as ATT
    torch.manual_seed(1)
    b, s, hq, hk, d = 3, 8, 4, 2, 16
    cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32)
    q, k, v = torch.randn(b * s, hq, d), torch.randn(b * s, hk, d), torch.randn(b * s, hk, d)
    dout = torch.randn(b * s, hq, d)
    calls = []
    real = ATT.attn_fwd
    ATT.attn_fwd = lambda *a, **kw: (calls.append(1), real(*a, **kw))[1]
    try:
        out, lse = pymha_varlen_fwd(q, k, v, cu, cu, s, s, 0.0, 0.25, True)
    finally:
        ATT.attn_fwd = real
    assert len(calls) == 1 and out.shape == q.shape and lse.shape == (b, hq, s)
    dq, dk, dv = pymha_varlen_bwd(dout, q, k, v, out, lse, cu, cu, s, s, 0.0, 0.25, True)
    for i in range(b):
        sl = slice(i * s, (i + 1) * s)
        c1 = torch.tensor([0, s], dtype=torch.int32)
        o_i, l_i = pymha_varlen_fwd(q[sl], k[sl], v[sl], c1, c1, s + 1, s + 1, 0.0, 0.25, True)     # max != length: loop path
        assert torch.allclose(out[sl], o_i, atol=1e-5) and torch.allclose(lse[i], l_i[0, :, :s], atol=1e-5)
        g = pymha_varlen_bwd(dout[sl], q[sl], k[sl], v[sl], o_i, l_i, c1, c1, s + 1, s + 1, 0.0, 0.25, True)
        assert torch.allclose(dq[sl], g[0], atol=1e-5) and torch.allclose(dk[sl], g[1], atol=1e-5) and torch.allclose(dv[sl], g[2], atol=1e-5)


def test_qkv_layout_probe():
    from dhellam_b200 import _get_qkv_layout
    s, b, h, d = 4, 2, 3, 8
    packed = torch.randn(s, b, 3, h, d)
    assert _get_qkv_layout(packed[:, :, 0], packed[:, :, 1], packed[:, :, 2]) == "sb3hd"
    packed2 = torch.randn(s, b, h, 3, d)
    assert _get_qkv_layout(packed2[..., 0, :], packed2[..., 1, :], packed2[..., 2, :]) == "sbh3d"
    q = torch.randn(s, b, h, d)
    kv = torch.randn(s, b, 2, h, d)
    assert _get_qkv_layout(q, kv[:, :, 0], kv[:, :, 1]) == "sbhd_sb2hd"
    assert _get_qkv_layout(q, torch.randn(s, b, h, d), torch.randn(s, b, h, d)) == "sbhd_sbhd_sbhd"


def test_adaptor_parses_megatron_flags_and_builds_configs():
    from dhellam_b200.adaptor import _add_dhellam_args, get_args, initialize_dhellam_megatron
    from dhellam_b200.parallel import state as PS
    PS.set_state(None)
    args = initialize_dhellam_megatron(None, None, argv=[
        "--num-layers", "4", "--hidden-size", "256", "--ffn-hidden-size", "688", "--num-attention-heads", "4",
        "--group-query-attention", "--num-query-groups", "2", "--seq-length", "128", "--vocab-size", "1024", "--swiglu",
        "--micro-batch-size", "2", "--global-batch-size", "8", "--tensor-model-parallel-size", "1", "--sequence-parallel",
        "--dhellam", "--schedule-config", "x.json", "--bf16", "--use-distributed-optimizer", "--disable-bias-linear"])
    assert args.dhellam and args.schedule_config == "x.json"
    assert get_args() is args
    cfg = args.model_config
    assert (cfg.num_layers, cfg.num_query_groups, cfg.activation, cfg.norm) == (4, 2, "swiglu", "rmsnorm")
    assert args.train_config.dtype == "bf16" and args.parallel_config.dp == 1
    PS.set_state(None)


def test_benchmark_harness_has_the_reference_entry_points():
    """benchmark, benchmark_ms, benchmark_ms_ops, benchmark_ms_ops_cp, benchmark_dhellam
    (dhellam/common/benchmark.py) exist and time plain callables on CPU."""
    import time

    import torch
    from dhellam_b200.common import benchmark, benchmark_dhellam, benchmark_ms_ops, benchmark_ms_ops_cp
    x = torch.randn(32, 32)
    assert benchmark(3, lambda a: a @ a, x) >= 0.0
    assert benchmark_ms_ops(3, None, None, [lambda: x @ x], [lambda: x + x], comm=lambda: x.sum()) >= 0.0
    assert benchmark_ms_ops_cp(3, None, None, [lambda: x @ x], [lambda: x + x], [lambda: x.sum(), lambda: x.mean()], wait_fwd=True) >= 0.0
    seq, par, sp = benchmark_dhellam(3, lambda: time.sleep(0.004), lambda: time.sleep(0.002))
    assert seq > par and sp > 1.2


def test_launch_templates_keep_the_reference_context_protocol():
    """``template_fwd_new`` returns ``[[inputs that require grad], outputs]`` and
    ``template_bwd_new`` differentiates that context (dhellam/common/template_launch.py:38-70)."""
    from dhellam_b200.common import template_bwd, template_bwd_new, template_fwd, template_fwd_new
    x = torch.randn(4, 3, requires_grad=True)
    w = torch.randn(3, 2, requires_grad=True)
    c = torch.randn(4, 2)                         # no grad: must not appear in the context
    ctx, ms = template_fwd_new(lambda a, b, k: a @ b + k, x, w, c)
    assert len(ctx[0]) == 2 and ctx[0][0] is x and ctx[0][1] is w and ms == 0
    g = torch.randn(4, 2)
    grads, _ = template_bwd_new(ctx, g)
    assert torch.allclose(grads[0], g @ w.t().detach(), atol=1e-6) and torch.allclose(grads[1], x.t().detach() @ g, atol=1e-6)
    ctx2, _ = template_fwd(lambda d: {"y": d["x"] * 2}, {"x": c})
    assert ctx2[0]["x"] is c and torch.equal(ctx2[1]["y"], c * 2)
    out, _ = template_bwd(lambda cx, go: go * 2, ctx2, g)
    assert torch.equal(out, g * 2)


def test_cross_entropy_wrappers_with_label_smoothing():
    """Dictionary protocol of the reference's loss op, with label smoothing, against a float64
    restatement of its formula taken over the whole vocabulary."""
    import torch.nn.functional as F
    from dhellam_b200.ops.loss import cross_entropy_bwd, cross_entropy_fwd
    torch.manual_seed(1)
    S, B, V, a = 5, 2, 32, 0.1
    logits = torch.randn(S, B, V)
    target = torch.randint(0, V, (S, B))
    ctx = cross_entropy_fwd({"vocab_parallel_logits": logits.clone(), "target": target}, label_smoothing=a)
    s = a * V / (V - 1)
    ref_in = logits.double().requires_grad_(True)
    logp = F.log_softmax(ref_in, -1)
    ref = (1 - s) * (-logp.gather(-1, target[..., None]).squeeze(-1)) - s * logp.mean(-1)
    assert torch.allclose(ctx["loss"].double(), ref, atol=1e-5)
    dout = torch.randn(S, B)
    (ref * dout.double()).sum().backward()
    g = cross_entropy_bwd(ctx, dout)
    assert torch.allclose(g.double(), ref_in.grad, atol=1e-5)
