"""MoE block parity: the device-side block (one C-ABI call) against the CPU oracle of the
reference's GraphCompatibleMoeBlock.forward, and against the golden vectors produced by the
reference itself.  Bars: routing decisions identical; router logits and routing weights within
rel-L2 1e-3; block output within rel-L2 2e-3 -- the block chains three fp16-rounded layers (gate/up,
SwiGLU, down) plus fp16 weighted sums, each of which is held to 1e-3 on its own in test_gpu_linear.py,
and the oracle rounds its dequantised weights to fp16 where the kernels keep (q - z) * s exact."""

import pytest
import torch

from oracle import glorcq_oracle as O
from tests import cases

pytestmark = pytest.mark.gpu
REL = 1e-3
REL_BLOCK = 2e-3


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from glorcq_b200 import _build
    _build.build()
    return torch.device("cuda:0")


def _run(blk, N, dev, seed):
    mb = cases.to_b200_moe(blk, dev)
    x = cases.make_x(seed, N, blk["H"]).reshape(1, N, blk["H"])
    y, logits = mb(x.to(dev))
    ref, ref_logits = O.moe_forward(cases.to_oracle_moe(blk), x)
    return mb, y.cpu(), logits.cpu(), ref, ref_logits


@pytest.mark.parametrize("N", [1, 2, 3, 4, 5, 8, 9, 20, 33])
@pytest.mark.parametrize("norm", [False, True])
def test_small_block(dev, N, norm):
    blk = cases.make_moe(300 + N, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3, norm_topk_prob=norm)
    mb, y, logits, ref, ref_logits = _run(blk, N, dev, 1300 + N)
    assert y.shape == ref.shape and logits.shape == ref_logits.shape
    assert cases.rel_l2(logits, ref_logits) <= REL
    # same experts chosen (ties aside, which the seeds avoid)
    _, w_ref, sel_ref = O.route(cases.to_oracle_moe(blk), cases.make_x(1300 + N, N, 256))
    assert torch.equal(mb.last_selected_experts.cpu().long(), sel_ref)
    assert cases.rel_l2(mb.last_routing_weights.cpu(), w_ref) <= REL
    assert cases.rel_l2(y, ref) <= REL_BLOCK


@pytest.mark.parametrize("N", [1, 8])
def test_no_shared_expert_and_top8(dev, N):
    blk = cases.make_moe(410 + N, 256, 128, 16, 8, I_shared=0, rank=16, experts_per_cluster=4, norm_topk_prob=True)
    mb, y, logits, ref, _ = _run(blk, N, dev, 1410 + N)
    assert cases.rel_l2(y, ref) <= REL_BLOCK


@pytest.mark.parametrize("N", [1, 7, 150])
def test_codebook_format_block(dev, N):
    blk = cases.make_moe(35, 256, 128, 6, 2, I_shared=256, rank=16, experts_per_cluster=2, fmt="turbo")
    for ex in blk["experts"] + [blk["shared_expert"]]:
        for p in ex.values():
            p["Pi"] = None
    mb, y, logits, ref, _ = _run(blk, N, dev, 1035)
    assert cases.rel_l2(y, ref) <= REL_BLOCK


@pytest.mark.parametrize("N", [1, 8, 32])
def test_qwen_moe_shape(dev, N):
    """Qwen1.5-MoE block shape: hidden 2048, 60 experts top-4, intermediate 1408, shared expert 5632,
    rank 64, U shared by clusters of 4 experts; 1, 8 and 32 tokens (32: the routing plan cuts an expert's
    entries into slots of at most 8 rows; 128 tokens: test_qwen_moe_shape_prefill)."""
    blk = cases.make_moe(2000 + N, 2048, 1408, 60, 4, I_shared=5632, rank=64, experts_per_cluster=4)
    mb, y, logits, ref, _ = _run(blk, N, dev, 3000 + N)
    assert cases.rel_l2(y, ref) <= REL_BLOCK


def test_against_golden(dev, golden):
    from tests.golden.make_golden import MOE_CASES
    for name, kw, N in MOE_CASES:
        blk = cases.make_moe(**kw)
        if blk["fmt"] == "turbo":
            for ex in blk["experts"] + [blk["shared_expert"]]:
                for p in ex.values():
                    p["Pi"] = None
        mb = cases.to_b200_moe(blk, dev)
        x = cases.make_x(kw["seed"] + 1000, N, kw["H"]).reshape(1, N, kw["H"])
        y, logits = mb(x.to(dev))
        g = golden["moe"][name]
        assert cases.rel_l2(logits.cpu(), g["router_logits"]) <= REL, name
        assert cases.rel_l2(y.cpu(), g["y"]) <= REL_BLOCK, name


def test_graph_capture_replay(dev):
    """The whole block is capturable: no host synchronisation, fixed launch shapes."""
    blk = cases.make_moe(77, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    mb = cases.to_b200_moe(blk, dev)
    xs = [cases.make_x(500 + i, 1, 256).reshape(1, 1, 256) for i in range(3)]
    static_x = xs[0].to(dev).clone()
    mb(static_x)                      # builds tables and workspaces outside the capture
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        mb(static_x)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_y, _ = mb(static_x)
    for x in xs:
        static_x.copy_(x.to(dev))
        graph.replay()
        ref, _ = O.moe_forward(cases.to_oracle_moe(blk), x)
        assert cases.rel_l2(static_y.cpu(), ref) <= REL_BLOCK


@pytest.mark.parametrize("N", [64, 200, 515])
def test_prefill_block_many_rows(dev, N):
    """Token counts that give experts more than 32 rows: the grouped tcgen05 path with device-side
    token lists, gather of the activation rows, SwiGLU and routing-weight epilogues."""
    blk = cases.make_moe(700 + N, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    mb, y, logits, ref, ref_logits = _run(blk, N, dev, 1700 + N)
    assert cases.rel_l2(y, ref) <= REL_BLOCK
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


def test_many_token_plan_matches_one_cta_plan(dev):
    """From 2048 entries (tokens x top-k) the routing plan runs as four launches over the SMs instead of one CTA.
    1100 tokens (2200 entries) against the oracle, and the first 1000 rows bit-equal to a call with 1000 tokens
    (2000 entries: the one-CTA plan) -- a token's output does not depend on the other tokens of the call."""
    blk = cases.make_moe(911, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    mb = cases.to_b200_moe(blk, dev)
    x = cases.make_x(912, 1100, 256).reshape(1, 1100, 256)
    y, logits = mb(x.to(dev))
    sel = mb.last_selected_experts.clone()
    ref, ref_logits = O.moe_forward(cases.to_oracle_moe(blk), x)
    assert cases.rel_l2(y.cpu().reshape(ref.shape), ref) <= REL_BLOCK
    y2, _ = mb(x[:, :1000].contiguous().to(dev))
    assert torch.equal(mb.last_selected_experts, sel[:1000])
    assert torch.equal(y2.reshape(1000, -1), y.reshape(1100, -1)[:1000])
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


def test_qwen_moe_shape_prefill(dev):
    blk = cases.make_moe(4242, 2048, 1408, 60, 4, I_shared=5632, rank=64, experts_per_cluster=4)
    mb, y, logits, ref, ref_logits = _run(blk, 128, dev, 4243)
    assert cases.rel_l2(y, ref) <= REL_BLOCK


def test_non_finite_hidden_state_keeps_indices_in_range(dev):
    """Overflowed activations give NaN router probabilities; routing must still pick k distinct experts
    (probabilities that are not numbers count as zero) so that no table index leaves its range."""
    blk = cases.make_moe(808, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    mb = cases.to_b200_moe(blk, dev)
    x = cases.make_x(809, 5, 256).reshape(1, 5, 256).to(dev)
    x[0, 1, :] = float("inf")
    x[0, 3, 7] = float("nan")
    y, _ = mb(x)
    torch.cuda.synchronize()
    sel = mb.last_selected_experts.cpu()
    assert int(sel.min()) >= 0 and int(sel.max()) < 8
    assert all(len(set(r.tolist())) == 2 for r in sel)
    assert torch.isfinite(y[0, [0, 2, 4]]).all()          # the other tokens are untouched
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


@pytest.mark.parametrize("N", [1, 5, 40])
def test_combine_with_residual_and_next_norm(dev, N):
    """The decoder's residual add and following RMS norm folded into the combine kernel give what the
    separate tensor ops give on the block output."""
    blk = cases.make_moe(840 + N, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    mb = cases.to_b200_moe(blk, dev)
    x = cases.make_x(1840 + N, N, 256).reshape(1, N, 256).to(dev)
    res = cases.make_x(2840 + N, N, 256).reshape(1, N, 256).to(dev)
    w = (1 + 0.1 * cases.make_x(3840, 1, 256).reshape(256)).to(dev)
    y, logits = mb(x)
    out, logits2, normed = mb(x, residual=res, next_norm=(w, 1e-6))
    assert torch.equal(logits, logits2)
    ref_out = res + y
    assert torch.equal(out, ref_out)
    ref_norm = torch.nn.functional.rms_norm(ref_out, (256,), w, 1e-6)
    assert cases.rel_l2(normed.cpu(), ref_norm.cpu()) <= 1e-3
    out3, _, normed3 = mb(x, next_norm=(None, 1e-3))
    assert torch.equal(out3, y)
    assert cases.rel_l2(normed3.cpu(), torch.nn.functional.rms_norm(y, (256,), None, 1e-3).cpu()) <= 1e-3


# ---- expert parallelism ---------------------------------------------------------------------------
@pytest.mark.parametrize("N,world", [(1, 2), (3, 2), (9, 2), (9, 4), (33, 3)])
def test_expert_parallel_emulated_on_one_gpu(dev, N, world):
    """Every rank's block (its own experts only) run in turn on one device; the exchange is emulated by
    summing the ranks' entry buffers.  The result must equal the single-device block bit for bit."""
    blk = cases.make_moe(900 + N, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    x = cases.make_x(1900 + N, N, 256).reshape(1, N, 256).to(dev)
    single, logits1 = cases.to_b200_moe(blk, dev)(x)
    bufs = {}
    outs = []
    for rank in list(range(world)) + [0]:        # second pass of rank 0 sees every other rank's rows
        mb = cases.to_b200_moe(blk, dev).set_expert_parallel(rank, world)
        second = rank == 0 and 0 in bufs

        def hook(entries, group, rank=rank, second=second):
            if second:
                for r, b in bufs.items():
                    if r != 0:
                        entries += b
            else:
                bufs[rank] = entries.clone()
            return entries
        mb._exchange = hook
        y, logits = mb(x)
        outs.append(y)
        assert torch.equal(logits, logits1)
    # each entry row is non-zero on exactly one rank
    nz = torch.stack([(b != 0).any(1) for b in bufs.values()]).sum(0)
    assert int(nz.max()) <= 1
    assert torch.equal(outs[-1], single)
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


class _OneDevicePeers:
    """The pointer tables of the peer-memory exchange for `world` ranks whose buffers all live on one device."""

    def __init__(self, world, entries, H, dev, flag_value):
        from glorcq_b200 import _lib
        self._lib, self.entries, self.half = _lib, entries, entries * H
        self.bufs = [torch.zeros(2 * self.half, dtype=torch.float16, device=dev) for _ in range(world)]
        self.flags = [torch.full((world,), flag_value, dtype=torch.int32, device=dev) for _ in range(world)]
        self.tb = torch.tensor([b.data_ptr() for b in self.bufs], dtype=torch.int64, device=dev)
        self.tf = torch.tensor([f.data_ptr() for f in self.flags], dtype=torch.int64, device=dev)

    def view(self, rank, limit_ns=0):
        import types
        state = torch.zeros(2, dtype=torch.int32, device=self.tb.device)
        return types.SimpleNamespace(
            peers=self._lib.EpPeers(self.tb.data_ptr(), self.tf.data_ptr(), state.data_ptr(), state.data_ptr() + 4,
                                    self.half, limit_ns),
            local_ptr=self.bufs[rank].data_ptr(), max_entries=self.entries, state=state, keep=self)


@pytest.mark.parametrize("N,world", [(1, 2), (5, 2), (8, 4), (16, 3)])
def test_peer_memory_exchange_emulated_on_one_gpu(dev, N, world):
    """Phase EXCHANGE with every rank's buffer on one device, the ranks run in turn.  The flag words start
    above the step number so that no rank waits for one that has not run yet; rank 0 runs once more at the
    end (again as step 1) and must then see every rank's rows: bit-identical to the single-device block."""
    blk = cases.make_moe(960 + N, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    x = cases.make_x(1960 + N, N, 256).reshape(1, N, 256).to(dev)
    single, _ = cases.to_b200_moe(blk, dev)(x)
    tables = _OneDevicePeers(world, N * 2, 256, dev, 1 << 20)
    y = None
    for rank in list(range(world)) + [0]:
        mb = cases.to_b200_moe(blk, dev).set_expert_parallel(rank, world)
        mb.peer_exchange_max_tokens = N
        mb._peers = tables.view(rank)
        y, _ = mb(x)
        assert mb._peers.state.tolist() == [1, 0]          # one step taken, no wait ran out
    assert torch.equal(y, single)
    # every rank's buffer holds the same rows in the half of step 1
    for b in tables.bufs[1:]:
        assert torch.equal(b, tables.bufs[0])
    assert not tables.bufs[0][:tables.half].any()           # the other half is untouched


def test_peer_memory_exchange_wait_runs_out(dev):
    """A flag that nothing sets: the exchange kernel gives up after the limit the caller configured (0.3 s
    here; one second by default), records the step in the error word and returns; the context stays usable.
    A second step runs out as well, and the error word keeps the FIRST step that did."""
    import time
    blk = cases.make_moe(970, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
    x = cases.make_x(1970, 2, 256).reshape(1, 2, 256).to(dev)
    tables = _OneDevicePeers(2, 4, 256, dev, 0)             # rank 1 never publishes
    mb = cases.to_b200_moe(blk, dev).set_expert_parallel(0, 2)
    mb.peer_exchange_max_tokens = 2
    mb._peers = tables.view(0, limit_ns=300_000_000)
    mb(x)                                                   # builds tables and workspaces (and is step 1)
    torch.cuda.synchronize()
    assert mb._peers.state.tolist() == [1, 1]               # step 1 taken; the wait of step 1 ran out
    t0 = time.time()
    y, _ = mb(x)
    torch.cuda.synchronize()
    assert 0.25 < time.time() - t0 < 3.0
    assert mb._peers.state.tolist() == [2, 1]               # step 2 ran out too; the first failure stays on record
    assert tables.flags[1].tolist() == [2, 0] and tables.flags[0].tolist() == [2, 0]
    single, _ = cases.to_b200_moe(blk, dev)(x)              # the device still works
    assert torch.isfinite(single.float()).all() and torch.isfinite(y.float()).all()


def _nccl_worker(rank, world, port, q):
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        d = torch.device("cuda", rank)
        blk = cases.make_moe(950, 256, 128, 8, 2, I_shared=256, rank=16, experts_per_cluster=3)
        res = []
        for N in (1, 9):
            x = cases.make_x(1950 + N, N, 256).reshape(1, N, 256).to(d)
            single, _ = cases.to_b200_moe(blk, d)(x)
            y, _ = cases.to_b200_moe(blk, d).set_expert_parallel(rank, world)(x)
            torch.cuda.synchronize()
            res.append(bool(torch.equal(y, single)))
            # the same through this library's exchange kernel over peer memory, several steps in a row
            mb = cases.to_b200_moe(blk, d).set_expert_parallel(rank, world)
            mb.peer_exchange_max_tokens = 16
            for _ in range(3):
                y, _ = mb(x)
            torch.cuda.synchronize()
            res.append(bool(torch.equal(y, single)) and mb._peers.error() == 0)
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_nccl(dev, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=170) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, oks in res:
        assert all(oks), f"rank {rank}: expert-parallel output differs from the single-device block"


# ---- fused-experts adapter --------------------------------------------------------------------------
def _b200_experts(blk, dev):
    import torch.nn.functional as F
    from glorcq_b200.quantized_linear import GLoRCQExperts
    ge = GLoRCQExperts(blk["E"], blk["H"], blk["I"], F.silu)
    shared_u = {}
    for e, ex in enumerate(blk["experts"]):
        ge.gate_experts[e] = cases.to_b200_linear(ex["gate_proj"], dev, shared_u)
        ge.up_experts[e] = cases.to_b200_linear(ex["up_proj"], dev, shared_u)
        ge.down_experts[e] = cases.to_b200_linear(ex["down_proj"], dev, shared_u)
    return ge


def test_experts_adapter_against_golden_and_oracle(dev, golden):
    g = golden["experts"]["experts_10"]
    blk = cases.make_moe(**g["args"])
    ge = _b200_experts(blk, dev)
    x = cases.make_x(g["x_seed"], g["T"], g["args"]["H"])
    y = ge(x.to(dev), g["idx"].to(dev), g["w"].to(dev)).cpu()
    assert y.shape == g["y"].shape and y.dtype == torch.float16
    assert cases.rel_l2(y, g["y"]) <= REL_BLOCK
    ob = cases.to_oracle_moe(blk)
    assert cases.rel_l2(y, O.experts_forward(ob.experts, x, g["idx"], g["w"])) <= REL_BLOCK


@pytest.mark.parametrize("T", [1, 3, 50])
def test_experts_adapter_token_counts_and_dropped_slots(dev, T):
    kw = dict(seed=61, H=256, I=128, E=6, top_k=2, I_shared=0, rank=16, experts_per_cluster=2)
    blk = cases.make_moe(**kw)
    ge = _b200_experts(blk, dev)
    x = cases.make_x(62 + T, T, 256)
    gen = torch.Generator().manual_seed(63 + T)
    idx = torch.stack([torch.randperm(6, generator=gen)[:2] for _ in range(T)])
    w = torch.rand(T, 2, generator=gen).to(torch.float16)
    ref = O.experts_forward(cases.to_oracle_moe(blk).experts, x, idx, w)
    assert cases.rel_l2(ge(x.to(dev), idx.to(dev), w.to(dev)).cpu(), ref) <= REL_BLOCK
    # index == num_experts marks a dropped slot: it contributes nothing
    idx2 = idx.clone()
    idx2[0, 1] = 6
    w2 = w.clone()
    w2[0, 1] = 0
    idx_ref = idx2.clone()
    idx_ref[0, 1] = idx2[0, 0] ^ 1          # any other expert, weight zero
    ref2 = O.experts_forward(cases.to_oracle_moe(blk).experts, x, idx_ref, w2)
    assert cases.rel_l2(ge(x.to(dev), idx2.to(dev), w2.to(dev)).cpu(), ref2) <= REL_BLOCK


# ---- other model families' block shapes ---------------------------------------------------------------
@pytest.mark.parametrize("N", [1, 5, 40])
def test_many_experts_top8_renormalised(dev, N):
    """Qwen3-MoE style routing: 128 experts, top-8, renormalised weights, no shared expert."""
    blk = cases.make_moe(520 + N, 256, 128, 128, 8, I_shared=0, rank=16, experts_per_cluster=8, norm_topk_prob=True)
    mb, y, logits, ref, ref_logits = _run(blk, N, dev, 1520 + N)
    assert cases.rel_l2(y, ref) <= REL_BLOCK
    assert cases.rel_l2(logits.float(), ref_logits.float()) <= REL


@pytest.mark.parametrize("N", [1, 16])
def test_two_of_eight_experts_renormalised(dev, N):
    """Mixtral style routing: 8 experts, top-2 always renormalised, no shared expert, wide intermediate."""
    blk = cases.make_moe(530 + N, 256, 896, 8, 2, I_shared=0, rank=16, experts_per_cluster=2, norm_topk_prob=True)
    mb, y, logits, ref, ref_logits = _run(blk, N, dev, 1530 + N)
    assert cases.rel_l2(y, ref) <= REL_BLOCK


@pytest.mark.timeout(900)
@pytest.mark.parametrize("N", [1, 16])
def test_mixtral_8x7b_block_shape(dev, N):
    """Mixtral-8x7B block at its own dimensions: hidden 4096, 8 experts top-2 (always renormalised),
    intermediate 14336, no shared expert, 2-bit g128 codes with a rank-64 correction; batch 1 and 16."""
    blk = cases.make_moe(5400 + N, 4096, 14336, 8, 2, I_shared=0, rank=64, experts_per_cluster=2, norm_topk_prob=True)
    mb, y, logits, ref, ref_logits = _run(blk, N, dev, 6400 + N)
    assert cases.rel_l2(logits.float(), ref_logits.float()) <= REL
    assert cases.rel_l2(y, ref) <= REL_BLOCK
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


@pytest.mark.timeout(900)
def test_qwen3_30b_a3b_block_shape(dev):
    """Qwen3-30B-A3B block at its own dimensions: hidden 2048, 128 experts top-8 (renormalised),
    intermediate 768, no shared expert, rank 64 with U shared by clusters; 64 tokens (one decode step of
    64 concurrent streams)."""
    blk = cases.make_moe(5500, 2048, 768, 128, 8, I_shared=0, rank=64, n_clusters=16, norm_topk_prob=True)
    mb, y, logits, ref, ref_logits = _run(blk, 64, dev, 6500)
    assert cases.rel_l2(logits.float(), ref_logits.float()) <= REL
    assert cases.rel_l2(y, ref) <= REL_BLOCK
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None
