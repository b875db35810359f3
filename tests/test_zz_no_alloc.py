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


@pytest.mark.parametrize("B,N,K", [(1, 1408, 2048), (4, 2048, 1408), (1, 96, 256)])
def test_static_scratch_variant_matches(B, N, K):
    assert torch.cuda.is_available()
    from glorcq_b200 import _build, _lib
    _build.build()
    L = _lib.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(B * 7 + N + K)
    packed = torch.randint(0, 256, (N, K // 4), generator=g, dtype=torch.int32).to(torch.uint8).to(dev)
    norms = (torch.randn(N, generator=g).abs() + 0.1).to(dev)
    centroids = torch.randn(4, generator=g).to(dev)
    x = torch.randn(B, K, generator=g).half().to(dev)
    st = torch.cuda.current_stream().cuda_stream

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
    for y in outs:
        assert torch.isfinite(y.float()).all()
        assert _rel_l2(y, ref) <= REL
    assert torch.equal(outs[0], outs[1])     # deterministic, and unaffected by the leftovers of the first call


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
