"""The command-line trainer end to end on CPU, with a strategy file, metrics and resume."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ARGS = ["--num-layers", "2", "--hidden-size", "64", "--ffn-hidden-size", "128", "--num-attention-heads", "4",
        "--group-query-attention", "--num-query-groups", "2", "--seq-length", "32", "--vocab-size", "128", "--swiglu",
        "--micro-batch-size", "1", "--global-batch-size", "2", "--lr", "1e-3", "--dhellam"]


def _run(extra, cwd):
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "train.py")] + ARGS + extra, cwd=cwd, env=env, capture_output=True,
                       text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    return p.stdout


def test_train_cli_with_schedule_metrics_and_resume(tmp_path):
    from dhellam_b200.config import preset
    from dhellam_b200.models.transformer import build_layer_program
    from dhellam_b200.sched.strategy import Strategy, default_paired
    sched = tmp_path / "best.json"
    Strategy(dcblocks=default_paired(build_layer_program(preset("tiny-llama")))).save(str(sched))
    out = _run(["--train-iters", "3", "--schedule-config", str(sched), "--metrics-jsonl", str(tmp_path / "m.jsonl"),
                "--save", str(tmp_path / "ck"), "--save-interval", "2"], str(tmp_path))
    assert "iteration      3/3" in out.replace("  ", " ") or "iteration" in out
    recs = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert len(recs) == 3 and recs[0]["tokens_per_s"] > 0 and recs[-1]["loss"] < recs[0]["loss"] + 1.0
    assert (tmp_path / "ck" / "iter_0000002" / "metadata.json").exists()
    assert (tmp_path / "ck" / "latest_checkpointed_iteration.txt").read_text() == "3"
    out2 = _run(["--train-iters", "4", "--load", str(tmp_path / "ck")], str(tmp_path))
    assert "resumed from" in out2 and "iteration      4/" in out2.replace("  ", " ") or "resumed from" in out2
