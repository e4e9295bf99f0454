"""Strategy files, built-in schedules, the executor's launch order and the race checker."""
import json

import pytest

from dhellam_b200.config import preset
from dhellam_b200.models.transformer import build_layer_program
from dhellam_b200.sched.checker import Launch, RaceError, check_schedule, check_trace, launches_of
from dhellam_b200.sched.strategy import Block, Strategy, StrategyError, default_paired

# the reference's built-in paired schedule (dhellam/core/dstb.py:1043-1059), as a strategy file
REFERENCE_DEFAULT = {"DCBlocks": [
    [["ln_attn"], "None", "None"],
    ["None", ["bda_mlp_bwd"], ["allgather_attn"]],
    [["gemm_attn_c", "fl_attn"], "None", ["allgather_mlp_bwd"]],
    [["gemm_attn_l"], "None", "None"],
    ["None", ["gemm_dgrad_mlp_l", "gemm_wgrad_mlp_l"], ["reduce_scatter_attn"]],
    ["None", ["swiglu_bwd"], "None"],
    ["None", ["gemm_dgrad_mlp_c"], "None"],
    ["None", ["gemm_wgrad_mlp_c"], ["reduce_scatter_mlp_c_bwd"]],
    [["bda_attn", "ln_mlp"], "None", "None"],
    ["None", ["ln_mlp_bwd", "bda_attn_bwd"], ["allgather_mlp"]],
    [["gemm_mlp_c"], "None", ["allgather_attn_bwd"]],
    [["swiglu_mlp", "gemm_mlp_l"], "None", "None"],
    ["None", ["gemm_dgrad_attn_l", "gemm_wgrad_attn_l", "attn_bwd"], ["reduce_scatter_mlp"]],
    [["bda_mlp"], "None", "None"],
    ["None", ["gemm_dgrad_attn_c"], "None"],
    ["None", ["gemm_wgrad_attn_c"], ["reduce_scatter_attn_c_bwd"]],
    ["None", ["ln_attn_bwd"], "None"]]}


def _program(name="tiny-llama", cp=1):
    return build_layer_program(preset(name), cp=cp)


def test_reference_format_strategy_loads_validates_and_round_trips(tmp_path):
    prog = _program()
    s = Strategy.from_dict(REFERENCE_DEFAULT)
    s.validate(prog)
    p = tmp_path / "s.json"
    s.save(str(p))
    again = Strategy.load(str(p))
    assert again.to_dict() == s.to_dict()
    assert json.loads(p.read_text())["DCBlocks"][0] == [["ln_attn"], "None", "None"]
    check_schedule(prog, s)


def test_fused_search_names_are_split_and_budgets_parsed():
    prog = _program()
    d = json.loads(json.dumps(REFERENCE_DEFAULT))
    d["DCBlocks"][7] = ["None", ["gemm_wgrad_mlp_c_reduce_scatter_mlp_c_bwd"], "None"]
    d["DCBlocks"][2] = [["gemm_attn_c@96", "fl_attn"], "None", ["allgather_mlp_bwd"]]
    s = Strategy.from_dict(d)
    assert s.dcblocks[7].s2 == ["gemm_wgrad_mlp_c"] and s.dcblocks[7].s3 == ["reduce_scatter_mlp_c_bwd"]
    s.validate(prog)


def test_deferred_wgrad_marker_moves_the_op():
    prog = _program()
    d = json.loads(json.dumps(REFERENCE_DEFAULT))
    d["DCBlocks"][13] = [["bda_mlp"], ["gemm_wgrad_mlp_l_n"], "None"]
    s = Strategy.from_dict(d)
    s.validate(prog)
    names = [l.op for l in launches_of(prog, s.dcblocks)]
    assert names.index("gemm_wgrad_mlp_l") > names.index("bda_attn_bwd")
    check_schedule(prog, s)


def test_wgrad_handed_to_the_next_layer_run_executes_there_and_is_flushed_at_the_end():
    """``<op>_next`` hands a weight-gradient op to the next layer run, ``carried`` is where that
    run executes it; the last layer's hand-over runs when the engine flushes."""
    import torch
    from dhellam_b200.config import ParallelConfig, TrainConfig
    from dhellam_b200.data import make_microbatch, synthetic_tokens
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.trainer import Trainer
    cfg = preset("tiny-llama")
    d = json.loads(json.dumps(REFERENCE_DEFAULT))
    d["DCBlocks"][1] = ["None", ["bda_mlp_bwd", "carried"], ["allgather_attn"]]
    d["DCBlocks"][15] = ["None", ["gemm_wgrad_attn_c_next"], ["reduce_scatter_attn_c_bwd"]]
    strat = Strategy.from_dict(d)
    strat.validate(_program())
    check_schedule(_program(), strat)
    trace = []
    train = TrainConfig(micro_batch_size=1, global_batch_size=3, dtype="fp32")
    tr = Trainer(cfg, ParallelConfig(), train, device=torch.device("cpu"), ps=PS.initialize_model_parallel(ParallelConfig()),
                 strategy=strat, trace=trace)
    mbs = [make_microbatch(cfg, tr.ps, synthetic_tokens(cfg, 1, 3 + i), i, 3 + i, tr.device) for i in range(3)]
    tr.optimizer.zero_grad()
    tr.engine.run_step(mbs)
    wg = [i for i, t in enumerate(trace) if t[0] == "gemm_wgrad_attn_c"]
    # one weight gradient per (micro-batch, layer), none lost
    assert len(wg) == 3 * cfg.num_layers
    # in a paired run the op of layer L, micro-batch b shows up after the NEXT run's bda_mlp_bwd
    paired = [i for i in wg if i + 1 < len(trace) and trace[i - 1][0] == "bda_mlp_bwd" and trace[i - 1][2:] != trace[i][2:]]
    assert paired, "no weight gradient was executed inside the following layer run"
    # same gradients as the built-in schedule
    ref = Trainer(cfg, ParallelConfig(), train, device=torch.device("cpu"), ps=tr.ps, strategy=Strategy.from_dict(REFERENCE_DEFAULT))
    ref.model.flat_param.data.copy_(tr.model.flat_param.data)
    ref.optimizer.zero_grad()
    ref.engine.run_step(mbs)
    assert torch.allclose(ref.model.flat_grad, tr.model.flat_grad, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("bad", ["dup", "missing", "order", "lane"])
def test_invalid_strategies_are_rejected(bad):
    prog = _program()
    d = json.loads(json.dumps(REFERENCE_DEFAULT))
    if bad == "dup":
        d["DCBlocks"][3] = [["gemm_attn_l", "ln_attn"], "None", "None"]
    elif bad == "missing":
        d["DCBlocks"][5] = ["None", "None", "None"]
    elif bad == "order":
        d["DCBlocks"][2], d["DCBlocks"][3] = d["DCBlocks"][3], d["DCBlocks"][2]
    else:
        d["DCBlocks"][0] = ["None", ["ln_attn"], "None"]
    with pytest.raises(StrategyError):
        Strategy.from_dict(d).validate(prog)


@pytest.mark.parametrize("name,cp", [("tiny-llama", 1), ("tiny-llama", 2), ("tiny-llama", 4), ("tiny-gpt", 1), ("tiny-moe", 1)])
def test_builtin_schedules_are_valid_and_race_free(name, cp):
    prog = _program(name, cp)
    for streams in (1, 2):
        check_schedule(prog, Strategy(), compute_streams=streams)
    blocks = default_paired(prog)
    # no collective is launched in a block without compute of the other strand beside it, except at the ends
    if cp == 1:
        assert sum(1 for b in blocks if b.s3 and not (b.s1 or b.s2)) <= 1


def test_checker_catches_missing_wait_and_accepts_the_fix():
    racy = [Launch("ln", "S1"), Launch("allgather", "S3", waits=(), reads=("ln",))]
    with pytest.raises(RaceError):
        check_trace(racy)
    assert check_trace([Launch("ln", "S1"), Launch("allgather", "S3", waits=("ln",), reads=("ln",))])
    # transitive: gemm on S1 waits the collective, which waited ln
    ok = [Launch("ln", "S1"), Launch("ag", "S3", ("ln",), ("ln",)), Launch("other", "S2"),
          Launch("gemm", "S1", ("ag",), ("ag",)), Launch("wgrad", "S2", ("gemm",), ("ag", "gemm"))]
    assert check_trace(ok)
    bad = [Launch("ln", "S1"), Launch("ag", "S3", ("ln",), ("ln",)), Launch("wgrad", "S2", (), ("ag",))]
    with pytest.raises(RaceError):
        check_trace(bad)


def test_buffer_reuse_checker_accepts_builtin_and_rejects_single_slot():
    """Cross-rank write-after-read on the double-buffered symmetric slots: the built-in schedules
    are safe with two slots for one and two compute streams; with one slot the carried QKV weight
    gradient (which reads its re-gathered operand one layer run late) is caught."""
    from dhellam_b200.config import preset
    from dhellam_b200.models.transformer import FUSED_BUFFER_EFFECTS, build_layer_program
    from dhellam_b200.sched.checker import RaceError, check_buffer_reuse
    from dhellam_b200.sched.strategy import Strategy
    P = build_layer_program(preset("tiny-llama"))
    for cs in (1, 2):
        assert check_buffer_reuse(P, Strategy(), FUSED_BUFFER_EFFECTS, compute_streams=cs)
    with pytest.raises(RaceError) as ei:
        check_buffer_reuse(P, Strategy(), FUSED_BUFFER_EFFECTS, compute_streams=1, slots=1)
    assert "regather_attn" in str(ei.value) and "gemm_wgrad_attn_c" in str(ei.value)


def test_buffer_reuse_checker_replays_carried_ops_in_the_run_that_executes_them():
    from dhellam_b200.config import preset
    from dhellam_b200.models.transformer import FUSED_BUFFER_EFFECTS, build_layer_program
    from dhellam_b200.sched.checker import launches_of_runs
    from dhellam_b200.sched.strategy import Strategy
    P = build_layer_program(preset("tiny-llama"))
    strat = Strategy().completed(P)
    launches, notes = launches_of_runs(P, strat, ("pair", "pair"), 1, FUSED_BUFFER_EFFECTS)
    names = [l.op for l in launches]
    # the QKV weight gradient of run 0 executes inside run 1, after run 1 started and before run 1's own
    i = names.index("gemm_wgrad_attn_c#0")
    assert names.index("bda_mlp_bwd#1") < i < names.index("gemm_wgrad_attn_c#1")
    # and it waits on events of run 0's producers, not run 1's
    assert all(w.endswith("#0") for w in launches[i].waits)
