"""Strategy search: solver optimality, file formats, and the whole pipeline on CPU."""
import itertools
import json
import os
import random

import torch

from dhellam_b200.search import search as S
from dhellam_b200.search.op_table import get_candidate_operator_groups, has_collective, operator_list_prune


def _synthetic_table(fskel, bskel, seed):
    rnd = random.Random(seed)
    fg, bg = get_candidate_operator_groups(fskel, bskel)
    single = {}
    table = {}
    for f in fg:
        if f:
            single[("f", tuple(f))] = sum(rnd.uniform(0.1, 1.0) for _ in f)
            table[S._key(f, [])] = single[("f", tuple(f))]
    for b in bg:
        if b:
            single[("b", tuple(b))] = sum(rnd.uniform(0.1, 1.0) for _ in b)
            table[S._key([], b)] = single[("b", tuple(b))]
    for f in fg:
        for b in bg:
            if f and b and not (has_collective(f) and has_collective(b)):
                a, c = single[("f", tuple(f))], single[("b", tuple(b))]
                table[S._key(f, b)] = max(a, c) + rnd.uniform(0.0, 0.6) * min(a, c)
    return table


def test_solver_matches_brute_force_on_small_skeletons():
    fskel = [[24], [0], [16, 11, 17], [4], [13]]
    bskel = [[15], [3], [19, 23, 28], [9], [26]]
    for seed in range(4):
        table = _synthetic_table(fskel, bskel, seed)
        total, steps = S.solve(table, fskel, bskel)
        assert abs(total - S.brute_force(table, fskel, bskel)) < 1e-9
        # the steps cover both strands exactly once, in order
        assert [i for f, _ in steps for i in f] == [i for g in fskel for i in g]
        assert [i for _, b in steps for i in b] == [i for g in bskel for i in g]
        assert not any(S.illegal_pair(f, b) for f, b in steps)


def test_solver_on_reference_skeletons_produces_valid_strategy():
    from dhellam_b200.config import preset
    from dhellam_b200.models.transformer import build_layer_program
    (_, _, fskel), (_, _, bskel) = operator_list_prune(1)
    table = _synthetic_table(fskel, bskel, 11)
    total, steps = S.solve(table, fskel, bskel)
    program = build_layer_program(preset("tiny-llama"))
    strat = S.steps_to_strategy(steps, program)
    strat.validate(program)
    single = sum(table[S._key(g2, [])] for g in fskel for g2 in [g]) + sum(table[S._key([], g)] for g in bskel)
    assert total <= single + 1e-9


def test_profile_line_format_round_trip(tmp_path):
    p = tmp_path / "op_profile_num.txt"
    p.write_text("[[24, 0],[15]] speedup: 1.25 seq_time:2.0 para_time:1.6\n[[],[26]] speedup: 1.0 seq_time:0.5 para_time:0.5\nnoise\n")
    t = S.parse_op_file(str(p))
    assert t[S._key([24, 0], [15])] == 1.6 and t[S._key([], [26])] == 0.5 and len(t) == 2


def test_skeleton_from_program_matches_reference_for_llama():
    from dhellam_b200.config import preset
    from dhellam_b200.models.transformer import build_layer_program
    program = build_layer_program(preset("tiny-llama"))
    (_, _, f_ref), (_, _, b_ref) = operator_list_prune(1)
    (_, _, f), (_, _, b) = operator_list_prune(1, program)
    assert f == f_ref and b == b_ref


def test_search_pipeline_end_to_end_on_cpu(tmp_path):
    from dhellam_b200.parallel import state as PS
    from dhellam_b200.search.run import main
    from dhellam_b200.sched.strategy import Strategy
    PS.set_state(None)
    argv = ["--num-layers", "2", "--hidden-size", "64", "--ffn-hidden-size", "128", "--num-attention-heads", "4",
            "--group-query-attention", "--num-query-groups", "2", "--seq-length", "32", "--vocab-size", "128", "--swiglu",
            "--micro-batch-size", "1", "--global-batch-size", "2", "--search-dir", str(tmp_path), "--profile-repeat", "1"]
    assert main(argv) == 0
    best = tmp_path / "config" / "dhellam-cp1" / "best_result.json"
    assert best.exists()
    strat = Strategy.load(str(best))
    from dhellam_b200.config import preset
    from dhellam_b200.models.transformer import build_layer_program
    strat.validate(build_layer_program(preset("tiny-llama")))
    lines = (tmp_path / "op_profile_num.txt").read_text().strip().splitlines()
    assert len(lines) > 300
    PS.set_state(None)


def test_overlap_micro_benchmark_writes_both_tables_on_cpu(tmp_path):
    """The pairwise overlap benchmark (reference: micro_benchmark/overlap.py) runs on CPU tensors
    and writes speedup.csv and efficiency.csv into a directory it creates."""
    import csv

    from dhellam_b200.bench import overlap
    out = tmp_path / "new_dir"
    rc = overlap.main(["--rows", "64", "--hidden", "128", "--ffn", "256", "--heads", "2", "--kv-heads", "1", "--seq", "32",
                       "--repeat", "1", "--out-dir", str(out)])
    assert rc in (0, None)
    for name in ("speedup.csv", "efficiency.csv"):
        rows = list(csv.reader(open(out / name)))
        assert rows[0][0] == "fwd\\bwd" and len(rows) > 3 and len(rows[1]) == len(rows[0])
