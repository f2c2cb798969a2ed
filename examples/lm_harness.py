"""What the three training examples share: data, a language-model wrapper around a stack of
blocks, gradient-norm and logging in one format, so that their logs can be compared line by line.

* ``batches``: synthetic token ids or fixed-length samples of a token file; every rank takes its
  contiguous block of the sequence (rank r trains on positions ``[r*s_local, (r+1)*s_local)``), the
  split the reference's example uses for its Megatron run (examples/pretrain_fluidmoe.py:97-117).
* ``BlockLM``: embedding -> any block stack (``[s, b, H] -> [s, b, H]``) -> LayerNorm -> head ->
  cross-entropy on shifted ids.  Used by the Megatron-Core and DeepSpeed arms; this framework's
  arm uses ``fluidmoe_b200.models.gpt.MoEGPT``, whose head and loss are its own kernels.
* ``log_line``: the Megatron log format the reference's comparison driver parses
  (examples/run_training.sh:246-290 reads ``lm loss``, ``grad norm`` and the iteration time).
"""
from __future__ import annotations

import os
import sys
from typing import Iterator, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def add_common_args(ap) -> None:
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=2048, help="positions per rank")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--log-interval", type=int, default=1)
    ap.add_argument("--data", default=os.environ.get("FLUIDMOE_DATASET_SOURCE", ""),
                    help="token file (.npy / .bin, see text_dataset.py); empty: uniform random ids")


def batches(args, rank: int, world: int, device) -> Iterator[torch.Tensor]:
    """Yields ``[seq + 1, batch]`` id tensors of this rank (one extra position for the labels)."""
    full_len = args.seq * world + 1
    data = None
    if args.data:
        from text_dataset import TokenFileDataset
        data = TokenFileDataset(args.data, full_len)
    gen = torch.Generator().manual_seed(args.seed)
    step = 0
    while True:
        if data is not None:
            full = torch.stack([data[(step * args.batch + j) % len(data)] for j in range(args.batch)], dim=1)
        else:
            full = torch.randint(0, args.vocab, (full_len, args.batch), generator=gen)
        yield full[rank * args.seq:(rank + 1) * args.seq + 1].to(device)
        step += 1


class BlockLM(torch.nn.Module):
    def __init__(self, blocks: torch.nn.Module, vocab: int, hidden: int, dtype, device, init_std: float = 0.02):
        super().__init__()
        self.embedding = torch.nn.Embedding(vocab, hidden, dtype=dtype, device=device)
        self.blocks = blocks
        self.final_norm = torch.nn.LayerNorm(hidden, dtype=dtype, device=device)
        self.head = torch.nn.Linear(hidden, vocab, bias=False, dtype=dtype, device=device)
        torch.nn.init.normal_(self.embedding.weight, std=init_std)
        torch.nn.init.normal_(self.head.weight, std=init_std)

    def forward(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        x = self.blocks(self.embedding(ids))
        x = x[0] if isinstance(x, tuple) else x
        logits = self.head(self.final_norm(x))
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.reshape(-1))


def grad_norm(params, expert_group=None) -> float:
    """Global L2 norm of the gradients: replicated parameters count once, expert-sharded ones
    (``param.allreduce is False``) are summed over the expert-parallel group."""
    dense = torch.zeros((), dtype=torch.float64)
    sharded = None
    for p in params:
        g = getattr(p, "main_grad", None)
        if g is None or not getattr(p, "_ar_buf_written", True):
            g = p.grad
        if g is None:
            continue
        sq = g.detach().double().pow(2).sum()
        if getattr(p, "allreduce", True) is False:
            sharded = sq if sharded is None else sharded + sq
        else:
            dense = dense.to(sq.device) + sq
    if sharded is not None:
        if dist.is_initialized() and dist.get_world_size(expert_group) > 1:
            dist.all_reduce(sharded, group=expert_group)
        dense = dense.to(sharded.device) + sharded
    return float(dense.sqrt().item())


def mean_over_ranks(value: torch.Tensor) -> float:
    v = value.detach().float().clone()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(v)
        v /= dist.get_world_size()
    return float(v.item())


def log_line(step: int, steps: int, ms: float, loss: float, gnorm: Optional[float], lr: float) -> str:
    line = (f" iteration {step:8d}/{steps:8d} | elapsed time per iteration (ms): {ms:.1f} | "
            f"learning rate: {lr:.6E} | lm loss: {loss:.6E} |")
    if gnorm is not None:
        line += f" grad norm: {gnorm:.3f} |"
    return line
