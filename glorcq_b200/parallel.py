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


class PeerExchange:
    """The exchange as this library's own kernel over peer-mapped memory (phase EXCHANGE of
    glq_moe_forward_ep) instead of an all-reduce.

    Every rank allocates the same buffer in symmetric memory: two halves of ``max_entries * H`` fp16
    (alternate steps use alternate halves) followed by one int32 flag word per rank; the rendezvous gives
    every rank the others' addresses, which are kept on the device as the pointer tables the kernel
    reads.  One instance serves every block of a model with the same hidden size (the blocks run one
    after another on one stream), so it is cached per (group, device, H).  NVLink multicast binding is
    not needed (plain peer stores) and is switched off for the allocation.
    """

    _cache: dict = {}

    wait_limit_seconds = 1.0      # longest wait of the exchange kernel for the other ranks' flags

    def __init__(self, group, device: torch.device, max_entries: int, H: int):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_entries, self.H = int(max_entries), int(H)
        self.half_elems = self.max_entries * self.H
        flag_bytes = (4 * self.world + 255) // 256 * 256
        with torch.cuda.device(device):
            self._buf = symm.empty(4 * self.half_elems + flag_bytes, dtype=torch.uint8, device=device)
            self._buf.zero_()
            self._hdl = symm.rendezvous(self._buf, group)
            torch.cuda.synchronize(device)
        dist.barrier(group)          # every rank's flags are zero before any peer writes them
        ptrs = [int(self._hdl.buffer_ptrs[r]) for r in range(self.world)]
        if ptrs[self.rank] != self._buf.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned a foreign address for the local buffer")
        self._bufs = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self._flags = torch.tensor([p + 4 * self.half_elems for p in ptrs], dtype=torch.int64, device=device)
        self._state = torch.zeros(2, dtype=torch.int32, device=device)      # step counter, error word
        self.peers = _lib.EpPeers(self._bufs.data_ptr(), self._flags.data_ptr(), self._state.data_ptr(),
                                  self._state.data_ptr() + 4, self.half_elems,
                                  int(float(os.environ.get("GLQ_EP_WAIT_SECONDS", self.wait_limit_seconds)) * 1e9))
        self.local_ptr = ptrs[self.rank]

    @classmethod
    def get(cls, group, device: torch.device, max_entries: int, H: int) -> "PeerExchange":
        key = (id(group), str(device), int(H))
        px = cls._cache.get(key)
        if px is None or px.max_entries < max_entries:
            px = cls(group, device, max(int(max_entries), 64), H)
            cls._cache[key] = px
        return px

    def error(self) -> int:
        """Step number of the first wait that ran out (0: none).  Synchronises."""
        return int(self._state[1].item())

    def raise_on_error(self):
        """To be called at the host's own synchronisation points (end of a generation, after a timed
        region): a wait that ran out means a rank did not publish its rows in time, and every result from
        that step on is incomplete."""
        step = self.error()
        if step:
            raise RuntimeError(f"expert-parallel exchange: the wait for the other ranks ran out at step {step} "
                               f"(limit {self.peers.wait_limit_ns / 1e9:g} s); results from that step on are incomplete")

    @classmethod
    def check_all(cls):
        for px in list(cls._cache.values()):
            px.raise_on_error()
