"""Double-strand training engine.

One *tick* sweeps a pipeline stage's block pairs once: the forward strand of micro-batch
``a`` goes through one layer of every pair while the backward strand of micro-batch
``b = a - P`` goes through the partner layer, each pair executed by the dual-strand
``Executor``.  Stage ``p`` of ``P`` owns layer chunk ``p`` ("first") and chunk ``2P-1-p``
("second"); a *down* sweep runs first-chunk forward beside second-chunk backward and an
*up* sweep the opposite, so a micro-batch's forward visits stages ``0..P-1`` going down and
``P-1..0`` going up, with embedding and loss both on stage 0.

Capability parity: ``DSLLM.forward`` + autograd-driven second half + the patched Megatron
schedules of the reference (dhellam/core/dsllm.py:86-115, dhellam/core/dstb.py:1294-1364,
megatron.patch:131-195 for no-PP with N+1 rounds, megatron.patch:354-714 for 1F1B with
``num_microbatches += P``).  One explicit loop covers every pipeline size (P = 1 gives the
N+1-round schedule) and nothing is routed through autograd or a global dictionary.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig, TrainConfig
from ..models import head as H
from ..models.transformer import build_layer_program
from ..ops.rope import rope_table
from ..parallel import pp as PP
from ..sched.executor import Executor, StreamSet
from ..sched.ir import LayerRun
from ..sched.strategy import Strategy


@dataclass
class MicroBatch:
    """One micro-batch on this rank, rows in sequence-first order (row = s * batch + b)."""
    index: int
    tokens: torch.Tensor          # [T] integer ids
    labels: torch.Tensor          # [T]
    loss_mask: torch.Tensor       # [T]
    positions: torch.Tensor       # [T] int32 sequence position of each row (RoPE, causal order)
    batch: int
    seed: int = 0
    positions_local: Optional[torch.Tensor] = None   # [T/t] positions of this rank's sequence-parallel rows


class Env:
    """Everything the ops need besides tensors."""

    def __init__(self, cfg: ModelConfig, ps, train: TrainConfig, device, dtype, fused=None):
        self.cfg, self.ps, self.train = cfg, ps, train
        self.device, self.dtype = torch.device(device), dtype
        self.training = True
        self.fused = fused
        self.fused_tp = fused is not None and ps.tp > 1
        self.moe_dev = None           # DeviceMoE: device-resident expert exchange (set by the trainer on GPUs)
        self.fused_cp = None          # FusedCP: peer-memory key/value exchange of context parallelism (set by the trainer)
        self.cur_stream = None
        self.exposed = None           # ExposedTimer of the engine's executor (set by the engine)
        self.softmax_scale = 1.0 / math.sqrt(cfg.head_dim)
        self.rope_cos = self.rope_sin = None
        if cfg.position == "rope":
            c, s = rope_table(cfg.seq_length, cfg.head_dim, cfg.rope_theta)
            self.rope_cos, self.rope_sin = c.to(self.device), s.to(self.device)
        self.moe_aux = []             # auxiliary (load-balance) losses of the current step


def hand_over(obj, stream):
    """Marks every CUDA tensor inside ``obj`` (tensor, tuple, list or dict) as used on
    ``stream``.  Activations are allocated by the forward strand's stream and read, one round
    later, by the backward strand's stream; without this the caching allocator could recycle
    a block for the forward stream while the backward stream's kernels are still queued."""
    if stream is None or obj is None:
        return
    if isinstance(obj, torch.Tensor):
        if obj.is_cuda:
            obj.record_stream(stream)
    elif isinstance(obj, dict):
        for v in obj.values():
            hand_over(v, stream)
    elif isinstance(obj, (tuple, list)):
        for v in obj:
            hand_over(v, stream)


class DoubleStrandEngine:
    def __init__(self, model, env: Env, strategy: Optional[Strategy] = None, single_stream: bool = False,
                 profile: bool = False, trace=None, compute_streams: int = 2, sync_per_block: bool = False):
        self.model, self.env = model, env
        self.cfg, self.ps = env.cfg, env.ps
        self.program = build_layer_program(env.cfg, cp=env.ps.cp)
        self.streams = StreamSet(env.device if env.device.type == "cuda" else None, single_stream=single_stream,
                                 compute_streams=compute_streams)
        self.executor = Executor(self.program, strategy or Strategy(), self.streams, profile=profile, trace=trace,
                                 sync_per_block=sync_per_block)
        env.streams = self.streams
        env.exposed = self.executor.exposed      # shared with the head block and the in-kernel collectives
        self.acts: Dict[tuple, dict] = {}
        self.head_saved: Dict[int, dict] = {}
        self.fwd_done: Dict[int, object] = {}
        self.losses: List[torch.Tensor] = []
        self.grad_scale = 1.0
        self._carry = (None, None)
        self._inbox = {"next": [None, None], "prev": [None, None]}
        self.grad_reducer = None          # set by the trainer when data parallelism is on
        # "pp-bubble": time the communication stream spends in the pipeline exchanges of a step
        # (waiting for the neighbour stage included), measured with events on that stream instead
        # of the reference's extra 1-element exchange + device synchronisation (megatron.patch:82-96)
        self.time_pp = False
        self.loss_scale = 1.0             # factor on the loss gradient; the trainer copies the optimizer's value in
        self._pp_spans: List[tuple] = []

    # ------------------------------------------------------------------ helpers
    @property
    def P(self):
        return self.ps.pp

    def _layer_indices(self, j: int):
        c = len(self.model.blocks)
        first = self.ps.pp_rank * c + j
        return first, self.cfg.num_layers - 1 - first

    def _on(self, lane):
        return self.streams.ctx(self.streams.lane(lane))

    def _set_stream(self, lane):
        self.env.cur_stream = self.streams.lane(lane)

    def _rows_shape(self, mb_batch: int, seq_local: int):
        return (seq_local * mb_batch // self.ps.tp, self.cfg.hidden_size)

    # ------------------------------------------------------------------ one tick
    def tick(self, t: int, mbs: List[MicroBatch]):
        ps, P, N = self.ps, self.P, len(mbs)
        p = ps.pp_rank
        down, a, b, fa, fb = PP.tick_plan(t, p, P, N)
        st = self.streams
        x = g = None
        # ---- inputs
        if down:
            if p == 0:
                if fa:
                    self._set_stream("S1")
                    with self._on("S1"):
                        x = H.embed_fwd(self.env, self.model.head, mbs[a])
                if fb:
                    self._set_stream("S2")
                    if st.cuda and b in self.fwd_done:
                        st.s2.wait_event(self.fwd_done[b])
                    saved = self.head_saved.pop(b)
                    hand_over(saved, st.s2)
                    with self._on("S2"):
                        g = H.loss_bwd(self.env, self.model.head, mbs[b], saved, self.grad_scale)
            else:
                x, g = self._inbox["prev"]
        else:
            if p == P - 1:
                x, g = self._carry
                self._carry = (None, None)
            else:
                x, g = self._inbox["next"]
        self._inbox = {"next": [None, None], "prev": [None, None]}
        if st.cuda:
            evs, self._inbox_events = getattr(self, "_inbox_events", [None, None]), [None, None]
            if evs[0] is not None:
                st.s1.wait_event(evs[0])              # the forward strand waits for its activation only
            if evs[1] is not None:
                st.s2.wait_event(evs[1])              # the backward strand for its gradient only
        if fb and st.cuda and b in self.fwd_done:
            st.s2.wait_event(self.fwd_done[b])

        # ---- sweep over the block pairs
        blocks = self.model.blocks
        order = range(len(blocks)) if down else range(len(blocks) - 1, -1, -1)
        for j in order:
            first_idx, second_idx = self._layer_indices(j)
            first_params, second_params = blocks[j]
            f_params, f_idx = (first_params, first_idx) if down else (second_params, second_idx)
            b_params, b_idx = (second_params, second_idx) if down else (first_params, first_idx)
            frun = brun = None
            if fa:
                frun = LayerRun(f_params, self.acts.setdefault((a, f_idx), {}), mbs[a], self.env, {"x": x}, f_idx)
            if fb:
                saved_acts = self.acts.pop((b, b_idx))
                hand_over(saved_acts, st.s2)
                brun = LayerRun(b_params, saved_acts, mbs[b], self.env, {"dout": g}, b_idx)
            if self.env.fused is not None:
                self.env.fused.paired = frun is not None and brun is not None
            self.executor.run(frun, brun)
            if fa:
                x = frun.v["out"]
            if fb:
                g = brun.v["dx"]
                if b == N - 1 and self.grad_reducer is not None:
                    self.executor.flush_carry()       # a weight gradient handed to the next layer run belongs to this layer
                    self.grad_reducer.layer_final(b_idx, st.s2 if st.cuda else None)
        if fa and st.cuda:
            ev = torch.cuda.Event()
            ev.record(st.s1)
            self.fwd_done[a] = ev

        # ---- outputs
        send_next, send_prev = [None, None], [None, None]
        if down:
            if p == P - 1:
                self._carry = (x, g)
            else:
                send_next = [x if fa else None, g if fb else None]
        else:
            if p == 0:
                if fa:
                    self._set_stream("S1")
                    with self._on("S1"):
                        loss, saved = H.loss_fwd(self.env, self.model.head, mbs[a], x)
                    self.head_saved[a] = saved
                    self.losses.append(loss)
                    if st.cuda:
                        ev = torch.cuda.Event()
                        ev.record(st.s1)
                        self.fwd_done[a] = ev
                if fb:
                    self._set_stream("S2")
                    with self._on("S2"):
                        H.embed_bwd(self.env, self.model.head, mbs[b], g)
                    self.fwd_done.pop(b, None)
            else:
                send_prev = [x if fa else None, g if fb else None]
        if P > 1:
            self._exchange(t, mbs, send_next, send_prev)

    def _exchange(self, t, mbs, send_next, send_prev):
        """Sends this tick's outputs and receives the next tick's inputs."""
        ps, P, N = self.ps, self.P, len(mbs)
        p = ps.pp_rank
        recv_next, recv_prev = [False, False], [False, False]
        if t + 1 < PP.total_ticks(P, N):
            ndown, na, nb, nfa, nfb = PP.tick_plan(t + 1, p, P, N)
            if ndown and p > 0:
                recv_prev = [nfa, nfb]
            if (not ndown) and p < P - 1:
                recv_next = [nfa, nfb]
        st = self.streams
        mb0 = mbs[0]
        shape = (mb0.tokens.numel() // ps.tp, self.cfg.hidden_size)
        # One group per strand.  The forward strand's activation is ready when the last forward op of the sweep
        # has run, which in the paired schedule is well before the last backward op: its transfer overlaps the
        # rest of the backward strand.  The receiving side lets each strand of the next tick wait for its own
        # tensor only.
        last = {0: self.program.names("fwd")[-1], 1: self.program.names("bwd")[-1]}
        from_next, from_prev = [None, None], [None, None]
        events = [None, None]
        self._set_stream("S3")
        t0 = None
        if self.time_pp:
            if st.cuda:
                t0 = torch.cuda.Event(enable_timing=True)
                t0.record(st.s3)
            else:
                t0 = time.perf_counter()
        for slot in (0, 1):
            sending = [t for t in (send_next[slot], send_prev[slot]) if t is not None]
            if not sending and not (recv_next[slot] or recv_prev[slot]):
                continue
            if st.cuda:
                rec = self.executor._events.get(last[slot]) if sending else None
                if rec is not None:
                    st.s3.wait_event(rec[0])            # the op that produced this strand's tensor
                elif sending:
                    st.s3.wait_stream(st.s1 if slot == 0 else st.s2)
                for tns in sending:
                    if tns.is_cuda:
                        tns.record_stream(st.s3)
            with self._on("S3"):
                fn, fp = PP.exchange(ps, send_next, send_prev, recv_next, recv_prev, shape, self.env.dtype, self.env.device,
                                     slots=(slot,))
            from_next[slot], from_prev[slot] = fn[slot], fp[slot]
            if st.cuda:
                events[slot] = torch.cuda.Event()
                events[slot].record(st.s3)
        if t0 is not None:
            if st.cuda:
                t1 = torch.cuda.Event(enable_timing=True)
                t1.record(st.s3)
                self._pp_spans.append((t0, t1))
            else:
                self._pp_spans.append((t0, time.perf_counter()))
        self._inbox = {"next": from_next, "prev": from_prev}
        self._inbox_events = events

    def measure_exposed(self, on: bool):
        """Switches the exposed-communication measurement on or off (see ``ExposedTimer``)."""
        self.executor.exposed.enabled = bool(on) and self.streams.cuda
        self.executor.exposed.spans = []

    def exposed_ms(self) -> float:
        """Time, summed over the spans recorded since ``measure_exposed(True)``, that compute streams
        spent waiting for communication (synchronises)."""
        return self.executor.exposed.total_ms() if self.streams.cuda else 0.0

    def pp_bubble_ms(self) -> float:
        """Sum of the exchange spans recorded since the last call (synchronises on GPUs)."""
        spans, self._pp_spans = self._pp_spans, []
        if not spans:
            return 0.0
        if self.streams.cuda:
            torch.cuda.synchronize()
            return float(sum(a.elapsed_time(b) for a, b in spans))
        return float(sum(b - a for a, b in spans) * 1e3)

    # ------------------------------------------------------------------ whole step
    def run_step(self, mbs: List[MicroBatch]) -> List[torch.Tensor]:
        """Forward + backward of all micro-batches; gradients end up in ``main_grad``.
        Returns the per-micro-batch losses (first pipeline stage; empty elsewhere)."""
        N = len(mbs)
        self.losses = []
        self.env.moe_aux = []
        self.grad_scale = self.loss_scale / N
        self.env.grad_scale = self.grad_scale
        st = self.streams
        if self.grad_reducer is not None:
            self.grad_reducer.start_step()
        if st.cuda:
            st.fork_from(torch.cuda.current_stream())
        for t in range(PP.total_ticks(self.P, N)):
            self.tick(t, mbs)
        self.executor.flush_carry()
        if st.cuda:
            st.join_all_into(torch.cuda.current_stream())
        assert not self.acts, f"activations left over: {list(self.acts.keys())[:4]}"
        self.fwd_done.clear()
        return self.losses
