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


def test_train_cli_reads_a_token_file_and_runs_fp16_style_loss_scaling(tmp_path):
    import numpy as np
    path = tmp_path / "tokens.bin"
    (np.arange(4000) % 128).astype(np.int32).tofile(str(path))
    out = _run(["--train-iters", "2", "--data-path", str(path), "--fp16", "--initial-loss-scale", "1024",
                "--metrics-jsonl", str(tmp_path / "m.jsonl")], str(tmp_path))
    assert "data:" in out and "tokens.bin" in out
    recs = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert len(recs) == 2 and all(r["loss"] == r["loss"] for r in recs)       # finite losses


def test_train_cli_two_ranks_tensor_and_sequence_parallel(tmp_path):
    """The launcher path of the one-click script on CPU ranks (gloo): torch.distributed.run + train.py."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29537", os.path.join(ROOT, "train.py")] + ARGS + [
               "--tensor-model-parallel-size", "2", "--sequence-parallel", "--train-iters", "2", "--timing-log-level", "2",
               "--metrics-jsonl", str(tmp_path / "m.jsonl")]
    p = subprocess.run(cmd, cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    recs = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert len(recs) == 2 and recs[0]["tokens_per_s"] > 0


def test_the_reference_launch_lines_parse_unchanged():
    """Every flag of the reference's one-click script (script/run.sh:55-160, both model types) is accepted by
    the Megatron-style parser, so a user of the reference can keep the launch line."""
    from dhellam_b200.adaptor.megatron import build_parser
    common = ["--num-layers", "8", "--hidden-size", "8192", "--num-attention-heads", "64", "--seq-length", "8192",
              "--max-position-embeddings", "8192", "--transformer-impl", "transformer_engine", "--vocab-size", "128256",
              "--global-batch-size", "16", "--micro-batch-size", "4", "--train-iters", "2", "--weight-decay", "0.1",
              "--adam-beta1", "0.9", "--adam-beta2", "0.95", "--init-method-std", "0.006", "--clip-grad", "1.0", "--lr", "6.0e-5",
              "--lr-decay-style", "cosine", "--min-lr", "6.0e-6", "--lr-warmup-fraction", ".001", "--lr-decay-iters", "430000",
              "--use-mcore-models", "--distributed-backend", "nccl", "--initial-loss-scale", "65536", "--disable-bias-linear",
              "--fp16", "--use-distributed-optimizer", "--use-flash-attn", "--tensor-model-parallel-size", "8",
              "--context-parallel-size", "1", "--pipeline-model-parallel-size", "1", "--distributed-timeout-minutes", "2",
              "--sequence-parallel", "--attention-mask-cuda-init", "--log-throughput", "--timing-log-level", "2",
              "--log-interval", "1", "--save-interval", "10000", "--eval-interval", "10000", "--eval-iters", "0",
              "--dhellam", "--schedule-config", "config/best.json"]
    llama = ["--data-cache-path", "d/cache", "--tokenizer-type", "Llama2Tokenizer", "--tokenizer-model", "d/tokenizer.model",
             "--data-path", "d/oscar_text_document", "--split", "949,50,1", "--ffn-hidden-size", "28672", "--swiglu",
             "--group-query-attention", "--num-query-groups", "8"]
    gpt = ["--data-path", "d/my-gpt2_text_document", "--vocab-file", "d/gpt2-vocab.json", "--merge-file", "d/gpt2-merges.txt",
           "--split", "949,50,1", "--tokenizer-type", "GPT2BPETokenizer"]
    parser = build_parser()
    a = parser.parse_args(common + llama)
    assert a.tensor_model_parallel_size == 8 and a.sequence_parallel and a.dhellam and a.schedule_config == "config/best.json"
    b = parser.parse_args(common + gpt)
    assert b.vocab_file == "d/gpt2-vocab.json" and b.merge_file == "d/gpt2-merges.txt"
