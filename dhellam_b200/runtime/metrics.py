"""Per-step metrics as JSON lines: loss, gradient norm, step time, tokens/s/GPU, model
TFLOP/s per GPU and MFU against the nominal and the measured bf16 peak.  The reference logs
through Megatron's training log (loss from its global dictionary, throughput from
``--log-throughput``; megatron.patch:786-812)."""
from __future__ import annotations

import json
import os
import time
from typing import Optional


class MetricsLogger:
    def __init__(self, path: Optional[str], cfg, n_gpus: int, tokens_per_step: int, nominal_tflops: float = 2250.0,
                 measured_tflops: Optional[float] = None):
        self.path, self.cfg, self.n_gpus, self.tokens = path, cfg, n_gpus, tokens_per_step
        self.nominal, self.measured = nominal_tflops, measured_tflops
        self.fp = open(path, "a") if path else None
        self.flops_per_token = cfg.flops_per_token()

    def log(self, iteration: int, step_ms: float, loss=None, grad_norm=None, extra: Optional[dict] = None) -> dict:
        tps = self.tokens / (step_ms / 1e3)
        tflops_gpu = tps * self.flops_per_token / self.n_gpus / 1e12
        rec = {"iteration": iteration, "time": time.time(), "step_ms": step_ms, "tokens_per_s": tps,
               "tokens_per_s_per_gpu": tps / self.n_gpus, "model_tflops_per_gpu": tflops_gpu,
               "mfu_nominal": tflops_gpu / self.nominal, "loss": loss, "grad_norm": grad_norm}
        if self.measured:
            rec["mfu_of_measured"] = tflops_gpu / self.measured
        if extra:
            rec.update(extra)
        if self.fp:
            self.fp.write(json.dumps(rec) + "\n")
            self.fp.flush()
        return rec

    def close(self):
        if self.fp:
            self.fp.close()
