"""Search pipeline: profile -> solve -> execute, the role of the reference's
``search/search.sh:161-189``.

    torchrun --nproc-per-node 8 -m dhellam_b200.search.run --tensor-model-parallel-size 8 ...

takes the same Megatron-style flags as training and writes ``op_profile_num.txt``,
``config/dhellam-cp{c}/best_result.json`` and ``config/best.json`` (what
``--schedule-config`` then points at).
"""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist


def _extra(parser):
    g = parser.add_argument_group(title="search")
    g.add_argument("--search-dir", default=".")
    g.add_argument("--profile-repeat", type=int, default=5)
    g.add_argument("--profile-limit", type=int, default=None, help="measure at most this many two-sided pairs (smoke runs)")
    return parser


def main(argv=None):
    from ..adaptor.megatron import initialize_dhellam_megatron
    from ..common.common import print_rank0
    from .execute import run_execute
    from .harness import LayerHarness
    from .profiler import run_profiler
    from .search import run_search
    args = initialize_dhellam_megatron(None, _extra, argv=argv)
    ps, cfg, train = args.parallel_state, args.model_config, args.train_config
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    fused = None
    if train.fused_comm and device.type == "cuda" and ps.tp > 1:
        from ..ops.fused_comm import FusedTP
        fused = FusedTP(ps, cfg, train, device)
    h = LayerHarness(cfg, ps, train, device, fused=fused)
    os.makedirs(args.search_dir, exist_ok=True)
    prof = os.path.join(args.search_dir, "op_profile_num.txt")
    t0 = time.time()
    run_profiler(h, prof, repeat=args.profile_repeat, limit=args.profile_limit)
    if dist.is_initialized():
        dist.barrier()
    cfg_dir = os.path.join(args.search_dir, "config")
    if not dist.is_initialized() or dist.get_rank() == 0:
        total, path = run_search(prof, ps.cp, h.program, cfg_dir)
        print_rank0(f">>>> best paired schedule: {total:.3f} ms per block pair -> {path}")
    if dist.is_initialized():
        dist.barrier()
    best, sp = run_execute(h, os.path.join(cfg_dir, f"dhellam-cp{ps.cp}"), os.path.join(cfg_dir, "best.json"))
    print_rank0(f">>>> search finished in {time.time() - t0:.1f} s; best: {best} ({sp:.2f}% over sequential)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
