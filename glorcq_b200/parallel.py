"""Expert parallelism for the MoE block: which rank holds which expert, and the exchange.

The reference runs a block's experts on one device (inference/moe_block.py:381-436); sharding them
is this package's addition.  Expert ``e`` lives on rank ``e % world``.  Router and shared expert are
replicated, so every rank derives the same routing and numbers the (token, expert) entries alike;
each rank fills the down-projection rows of its own experts' entries in an ``(n_tokens*top_k, H)``
fp16 buffer and leaves the rest zero.  A sum all-reduce of that buffer then has exactly one non-zero
term per row, which makes it exact in fp16 whatever the reduction order: the combine that follows
sees the same bytes as a single device would, for every world size.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def owner(expert: int, world: int) -> int:
    return expert % world


def local_experts(num_experts: int, rank: int, world: int) -> List[int]:
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    return [e for e in range(num_experts) if owner(e, world) == rank]


def exchange_entries(entry_out: torch.Tensor, group: Optional["dist.ProcessGroup"] = None) -> torch.Tensor:
    """In-place sum over the ranks of the per-entry output buffer (enqueued on the current stream for
    NCCL groups).  Exact: each row is non-zero on one rank only."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(entry_out, op=dist.ReduceOp.SUM, group=group)
    return entry_out
