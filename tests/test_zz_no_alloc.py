"""The allocation-free entry point, glq_turbo_dequant_matmul_static, against the existing
glq_turbo_dequant_matmul, both called through the C ABI.

Some hosts may not allocate device memory while they serve: all of it was handed to one arena at
start-up, and a cudaMalloc in the request path would synchronise the device.  For them the library
keeps the scratch of its split-k reduction in a fixed array of its own.  That array is shared by
every call and remembers the previous one, so the check runs the call twice in a row: the second
call must not be disturbed by what the first one left behind.  This file sorts last on purpose, so a
run that stops at the first failure has already run every other test."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
REL = 1e-3   # the tolerance of the other kernel tests (fp16 output, fp32 accumulation)


def _rel_l2(a, b):
    a, b = a.double().reshape(-1), b.double().reshape(-1)
    return float((a - b).norm() / (b.norm() + 1e-30))


def _operands(B, N, K, dev, seed):
    g = torch.Generator().manual_seed(seed)
    packed = torch.randint(0, 256, (N, K // 4), generator=g, dtype=torch.int32).to(torch.uint8)
    norms = torch.randn(N, generator=g).abs() + 0.1
    centroids = torch.randn(4, generator=g)
    x = torch.randn(B, K, generator=g).half()
    return [t.to(dev) for t in (x, packed, norms, centroids)], (x, packed, norms, centroids)


@pytest.mark.parametrize("B,N,K,splits", [(1, 1408, 2048, True), (4, 2048, 1408, True), (1, 96, 256, False)])
def test_static_scratch_variant_matches(B, N, K, splits):
    """Against the existing entry point AND against the CPU oracle of the reference's kernel, twice in a
    row.  The first two shapes plan a k split over CTAs, the only case that touches the fixed array; the
    third plans none and must work without it."""
    assert torch.cuda.is_available()
    from glorcq_b200 import _build, _lib
    from oracle import glorcq_oracle as O
    _build.build()
    L = _lib.lib()
    dev = torch.device("cuda:0")
    (x, packed, norms, centroids), host = _operands(B, N, K, dev, B * 7 + N + K)
    st = torch.cuda.current_stream().cuda_stream
    needed = L.glq_static_scratch_needed(B, N, K)
    assert (needed > 0) == splits and needed <= L.glq_static_scratch_bytes()

    ref = torch.empty(B, N, dtype=torch.float16, device=dev)
    _lib.check(L.glq_turbo_dequant_matmul(x.data_ptr(), packed.data_ptr(), norms.data_ptr(), centroids.data_ptr(),
                                          ref.data_ptr(), B, N, K, st), "turbo_dequant_matmul")
    outs = []
    for _ in range(2):                       # twice in a row: the array keeps the last call's contents
        y = torch.full((B, N), float("nan"), dtype=torch.float16, device=dev)
        _lib.check(L.glq_turbo_dequant_matmul_static(x.data_ptr(), packed.data_ptr(), norms.data_ptr(),
                                                     centroids.data_ptr(), y.data_ptr(), B, N, K, st),
                   "turbo_dequant_matmul_static")
        torch.cuda.synchronize()
        outs.append(y)
    oracle = O.turbo_matmul(*host)
    for y in outs:
        assert torch.isfinite(y.float()).all()
        assert _rel_l2(y, ref) <= REL
        assert _rel_l2(y.cpu(), oracle) <= REL
    assert torch.equal(outs[0], outs[1])     # deterministic, and unaffected by the leftovers of the first call


def test_static_scratch_reused_in_stream_order():
    """Different shapes enqueued back to back on one non-default stream, with no synchronisation in
    between: stream order alone must make the shared array safe to reuse (each call clears its counters on
    the stream before its launch)."""
    from glorcq_b200 import _build, _lib
    _build.build()
    L = _lib.lib()
    dev = torch.device("cuda:0")
    shapes = [(4, 2048, 1408), (1, 1408, 2048), (4, 2048, 1408), (2, 5632, 2048), (1, 96, 256)]
    ops = [_operands(B, N, K, dev, 100 + i)[0] for i, (B, N, K) in enumerate(shapes)]
    refs, outs = [], []
    main = torch.cuda.current_stream().cuda_stream
    for (B, N, K), (x, packed, norms, centroids) in zip(shapes, ops):
        r = torch.empty(B, N, dtype=torch.float16, device=dev)
        _lib.check(L.glq_turbo_dequant_matmul(x.data_ptr(), packed.data_ptr(), norms.data_ptr(), centroids.data_ptr(),
                                              r.data_ptr(), B, N, K, main), "turbo_dequant_matmul")
        refs.append(r)
        outs.append(torch.full((B, N), float("nan"), dtype=torch.float16, device=dev))
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            for (B, N, K), (x, packed, norms, centroids), y in zip(shapes, ops, outs):
                _lib.check(L.glq_turbo_dequant_matmul_static(x.data_ptr(), packed.data_ptr(), norms.data_ptr(),
                                                             centroids.data_ptr(), y.data_ptr(), B, N, K,
                                                             side.cuda_stream), "turbo_dequant_matmul_static")
    side.synchronize()
    for y, r in zip(outs, refs):
        assert _rel_l2(y, r) <= REL


def test_static_scratch_limit_is_enforced():
    from glorcq_b200 import _build, _lib
    _build.build()
    L = _lib.lib()
    assert L.glq_static_scratch_bytes() == 4 << 20
    dev = torch.device("cuda:0")
    # 128 rows of a 5632 x 2048 matrix: the split would need 5.8 MB of partial sums, more than the array has
    B, N, K = 128, 5632, 2048
    packed = torch.zeros(N, K // 4, dtype=torch.uint8, device=dev)
    norms = torch.ones(N, device=dev)
    centroids = torch.ones(4, device=dev)
    x = torch.zeros(B, K, dtype=torch.float16, device=dev)
    y = torch.zeros(B, N, dtype=torch.float16, device=dev)
    rc = L.glq_turbo_dequant_matmul_static(x.data_ptr(), packed.data_ptr(), norms.data_ptr(), centroids.data_ptr(),
                                           y.data_ptr(), B, N, K, torch.cuda.current_stream().cuda_stream)
    assert rc == -5, rc
    assert b"fixed array" in L.glq_status_string(rc)
    torch.cuda.synchronize()
