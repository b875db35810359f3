"""Expert-parallel host logic on CPU: two gloo ranks, each computing its own experts' rows with the
oracle, exchange them with glorcq_b200.parallel.exchange_entries; the summed buffer and the combine
must equal the single-rank oracle bit for bit."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from glorcq_b200 import parallel
from oracle import glorcq_oracle as O
from tests import cases


def test_partition_covers_every_expert_once():
    for E, world in ((60, 1), (60, 2), (60, 4), (60, 8), (8, 3)):
        seen = []
        for r in range(world):
            mine = parallel.local_experts(E, r, world)
            assert all(parallel.owner(e, world) == r for e in mine)
            seen += mine
        assert sorted(seen) == list(range(E))
    with pytest.raises(ValueError):
        parallel.local_experts(8, 2, 2)


def _entries(blk, x, rank, world):
    """(n*top_k, H) fp16 rows of this rank's experts, numbered by (expert, token) as the device plan
    numbers them; zero elsewhere.  Also returns the numbering and the routing."""
    ob = cases.to_oracle_moe(blk)
    logits, w, sel = O.route(ob, x)
    n, k = sel.shape
    order = sorted(range(n * k), key=lambda i: (int(sel.reshape(-1)[i]), i))
    entry_of = {i: pos for pos, i in enumerate(order)}
    buf = torch.zeros(n * k, blk["H"], dtype=torch.float16)
    xU = O._shared_xU(ob, x, range(ob.num_experts))
    for i in range(n * k):
        t, s = divmod(i, k)
        e = int(sel[t, s])
        if parallel.owner(e, world) != rank:
            continue
        ex = ob.experts[e]
        ag = xU["gate_proj"].get(ex.gate_proj.cluster_id)
        au = xU["up_proj"].get(ex.up_proj.cluster_id)
        y = O._expert_mlp(ex, x[t:t + 1], None if ag is None else ag[t:t + 1], None if au is None else au[t:t + 1])
        buf[entry_of[i]] = (y * w[t, s]).to(torch.float16).squeeze(0)
    return buf, entry_of, sel


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        blk = cases.make_moe(77, 128, 128, 8, 2, rank=16, experts_per_cluster=3)
        x = cases.make_x(78, 6, 128)
        mine, entry_of, sel = _entries(blk, x, rank, world)
        full, _, _ = _entries(blk, x, 0, 1)
        got = parallel.exchange_entries(mine.clone())
        ok_sum = torch.equal(got, full)
        # combine in expert order, as the block does above four tokens
        n, k = sel.shape
        out = torch.zeros(n, blk["H"], dtype=torch.float16)
        for t in range(n):
            for s in sorted(range(k), key=lambda s: int(sel[t, s])):
                out[t] += got[entry_of[t * k + s]]
        ref, _ = O.moe_forward(cases.to_oracle_moe(blk), x.reshape(1, 6, 128))
        q.put((rank, ok_sum, torch.equal(out, ref.reshape(6, 128)), int((mine != 0).any(1).sum())))
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_is_exact():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    rows = 0
    for rank, ok_sum, ok_out, nrows in res:
        assert ok_sum, f"rank {rank}: summed entry buffer differs from the single-rank buffer"
        assert ok_out, f"rank {rank}: combined output differs from the oracle block"
        rows += nrows
    assert rows == 12   # every entry was produced by exactly one rank


def test_peer_exchange_protocol_never_overwrites_rows_being_read():
    """The protocol of the peer-memory exchange (two buffer halves used by alternate steps, one flag word per
    rank holding the last published step, no second barrier), run as a model under random interleavings of
    the ranks: a rank's combine must always read the rows of its own step from every rank, i.e. no rank that
    is ahead may have overwritten them."""
    import random

    for world in (2, 3, 4):
        rng = random.Random(100 + world)
        for _ in range(60):
            steps = 6
            # buf[r][half][src] = step whose rows rank `src` last stored into that half of rank r's buffer
            buf = [[[0] * world for _ in range(2)] for _ in range(world)]
            flags = [[0] * world for _ in range(world)]     # flags[r][src]: last step src published to r
            pc = [("store", 1)] * world                      # per rank: (stage, step)
            done = 0
            while done < world:
                r = rng.randrange(world)
                stage, step = pc[r]
                if stage == "end":
                    continue
                if stage == "store":
                    for p in range(world):
                        buf[p][step & 1][r] = step
                    pc[r] = ("publish", step)
                elif stage == "publish":
                    for p in range(world):
                        flags[p][r] = step
                    pc[r] = ("wait", step)
                elif stage == "wait":
                    if all(f >= step for f in flags[r]):
                        pc[r] = ("combine", step)
                elif stage == "combine":
                    assert buf[r][step & 1] == [step] * world, (world, r, step, buf[r])
                    if step == steps:
                        pc[r] = ("end", step)
                        done += 1
                    else:
                        pc[r] = ("store", step + 1)
