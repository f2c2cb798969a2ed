"""Exposed-communication table of the non-overlapped baseline.

    torchrun --nproc-per-node N -m fluidmoe_b200.tools.comm_ratio_table --model mixtral_8x7b

Runs the block stack with the scheduler off and library collectives (the ``fluidmoe-f`` arm), wraps
``dist.all_to_all_single``, ``dist.all_to_all``, ``dist.batch_isend_irecv`` and ``dist.all_reduce``
with timers, and prints per collective family: calls per iteration, milliseconds per iteration and
the share of the iteration (max over ranks).  With nothing overlapped, that share is the exposed
communication that the overlapped arms try to hide.  On CUDA the timers are CUDA events on the
calling stream; on CPU they are wall-clock (the gloo tests use that path).  The reference measures
the same table for its Megatron baseline by patching the same entry points
(tests/comm_ratio_table.py:52-98,128-257).
"""
from __future__ import annotations

import argparse
import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

_FAMILIES = {
    "all_to_all_single": "all_to_all",
    "all_to_all": "all_to_all",
    "batch_isend_irecv": "p2p",
    "all_reduce": "all_reduce",
}


class CommTimer:
    """Context manager that times every call of the patched ``torch.distributed`` entry points."""

    def __init__(self, device: torch.device):
        self.device = device
        self.cuda = device.type == "cuda"
        self._orig = {}
        self._events: List[Tuple[str, object, object]] = []
        self._wall: Dict[str, float] = defaultdict(float)
        self.calls: Dict[str, int] = defaultdict(int)

    def _wrap(self, name: str):
        orig = getattr(dist, name)
        fam = _FAMILIES[name]

        def timed(*a, **k):
            self.calls[fam] += 1
            if self.cuda:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                out = orig(*a, **k)      # asynchronous calls are charged up to their launch only
                e.record()
                self._events.append((fam, s, e))
                return out
            t0 = time.perf_counter()
            out = orig(*a, **k)
            self._wall[fam] += (time.perf_counter() - t0) * 1e3
            return out
        self._orig[name] = orig
        setattr(dist, name, timed)

    def __enter__(self):
        for name in _FAMILIES:
            if hasattr(dist, name):
                self._wrap(name)
        return self

    def __exit__(self, *exc):
        for name, fn in self._orig.items():
            setattr(dist, name, fn)
        self._orig.clear()

    def totals_ms(self) -> Dict[str, float]:
        out = defaultdict(float, self._wall)
        if self.cuda:
            torch.cuda.synchronize()
            for fam, s, e in self._events:
                out[fam] += s.elapsed_time(e)
        return dict(out)


def measure(step_fn, iters: int, device: torch.device):
    """Returns ``(iteration ms, {family: (calls per iteration, ms per iteration)})``."""
    with CommTimer(device) as timer:
        if device.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            step_fn()
        if device.type == "cuda":
            torch.cuda.synchronize()
        iter_ms = (time.perf_counter() - t0) * 1e3 / iters
        totals = timer.totals_ms()
        table = {fam: (timer.calls[fam] / iters, ms / iters) for fam, ms in totals.items()}
    return iter_ms, table


def format_table(iter_ms: float, table) -> str:
    lines = [f"{'collective':<14}{'calls/iter':>12}{'ms/iter':>12}{'share':>10}"]
    total = 0.0
    for fam in sorted(table):
        calls, ms = table[fam]
        total += ms
        lines.append(f"{fam:<14}{calls:>12.1f}{ms:>12.3f}{ms / iter_ms:>10.1%}")
    lines.append(f"{'all':<14}{'':>12}{total:>12.3f}{total / iter_ms:>10.1%}")
    lines.append(f"iteration {iter_ms:.3f} ms")
    return "\n".join(lines)


def main(argv=None):
    from ..parallel.scheduler import get_backward_scheduler
    from . import common
    from .experiment_configs import get_block_benchmark_defaults

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral_8x7b")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq-len", type=int, default=None, help="override the preset's sequence length")
    common.add_parallel_args(ap)
    args = ap.parse_args(argv)
    if common.handle_list_models(args):
        return
    bench = get_block_benchmark_defaults()
    over = {"num_layers": args.layers} if args.layers else {}
    if args.seq_len:
        over["seq_len"] = args.seq_len
    device, cfg, pc = common.setup(args.model, over, "a2a", args=args)
    model = common.build_model(cfg, bench, pc, device, "a2a")
    x = common.make_input(cfg, pc, device)
    get_backward_scheduler().disable()
    common.run_iters(model, x, args.warmup, pc)
    iter_ms, table = measure(lambda: common.run_iters(model, x, 1, pc), args.iters, device)
    if dist.is_initialized() and dist.get_world_size() > 1:       # max over ranks
        fams = sorted(_FAMILIES.values())
        vec = torch.tensor([iter_ms] + [table.get(f, (0, 0.0))[1] for f in dict.fromkeys(fams)],
                           dtype=torch.float64, device=device)
        dist.all_reduce(vec, op=dist.ReduceOp.MAX)
        iter_ms = vec[0].item()
        for i, f in enumerate(dict.fromkeys(fams)):
            if f in table:
                table[f] = (table[f][0], vec[1 + i].item())
    common.p0(format_table(iter_ms, table))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
