"""The three drop-in entry points against the reference's OWN CUDA kernels, when those have been built for this
GPU (oracle/build_ref.py compiles the reference's two extension sources, unchanged, for sm_100 into
oracle/_ref/; without that folder these tests are skipped and the CPU oracle remains the only checker).
Bars between the two GPU implementations (both accumulate in fp32): rel-L2 <= 1e-3, and no element further apart
than two fp16 roundings at the largest output magnitude (the reference's own kernel tests use the absolute bound
max|err| < 0.01 on outputs of order one, inference/kernels/test_kernels.py:105; these cases reach tens)."""

import pytest
import torch

from oracle import build_ref
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from glorcq_b200 import _build
    _build.build()
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ref_turbo():
    m = build_ref.load_module("ref_turbo_matmul_cuda")
    if m is None:
        pytest.skip("the reference's kernels have not been built (python oracle/build_ref.py)")
    return m


@pytest.fixture(scope="module")
def ref_gptq():
    m = build_ref.load_module("ref_gptq_matmul_cuda")
    if m is None:
        pytest.skip("the reference's kernels have not been built (python oracle/build_ref.py)")
    return m


def _close_fp16(ours, ref):
    bound = max(0.01, 2.0 * float(ref.float().abs().max()) * 2.0 ** -10)
    assert float((ours.float() - ref.float()).abs().max()) <= bound
    assert cases.rel_l2(ours.cpu(), ref.cpu()) <= 1e-3


@pytest.mark.parametrize("B,N,K", [(1, 1408, 2048), (4, 2048, 1408), (16, 512, 2048), (5, 5632, 2048), (0, 64, 64)])
def test_turbo_matmul_against_reference_kernel(dev, ref_turbo, B, N, K):
    import glorcq_b200.kernels as GK
    d = cases.make_linear(600 + N + B, N, K, fmt="turbo", with_lora=False)
    x = cases.make_x(601 + B, B, K).to(dev)
    ops = [d["packed_indices"].to(dev), d["norms"].to(dev), d["centroids"].to(dev)]
    ours = GK.turbo_dequant_matmul(x, *ops)
    ref = ref_turbo.turbo_dequant_matmul(x, *ops)
    torch.cuda.synchronize()
    assert ours.shape == ref.shape and ours.dtype == ref.dtype == torch.float16
    if B:
        _close_fp16(ours, ref)


@pytest.mark.parametrize("E,n_out,K", [(3, 16, 128), (60, 2048, 1408)])
def test_turbo_grouped_gemv_against_reference_kernel(dev, ref_turbo, E, n_out, K):
    import glorcq_b200.kernels as GK
    d = cases.make_linear(610 + E, E * n_out, K, fmt="turbo", with_lora=False)
    x = cases.make_x(611 + E, E, K).to(dev)
    ops = [d["packed_indices"].to(dev), d["norms"].to(dev), d["centroids"].to(dev)]
    ours = GK.turbo_dequant_grouped_gemv(x, *ops, n_out)
    ref = ref_turbo.turbo_dequant_grouped_gemv(x, *ops, n_out)
    torch.cuda.synchronize()
    _close_fp16(ours, ref)


@pytest.mark.parametrize("B,N,K,sym,lora", [(1, 1408, 2048, False, False), (8, 2048, 1408, False, True), (3, 100, 392, True, False)])
def test_gptq_matmul_against_reference_kernel(dev, ref_gptq, B, N, K, sym, lora):
    import glorcq_b200.kernels as GK
    d = cases.make_linear(620 + N, N, K, fmt="gptq", with_lora=False, int_zeros=False, sym=sym, signed_codes=True)
    x = cases.make_x(621, B, K, torch.float32).to(dev)
    lo = (cases.make_x(622, B, N, torch.float32) * 0.1).to(dev) if lora else torch.empty(0, device=dev)
    args = [x, d["qweight_int"].to(torch.int8).to(dev), d["scales"].to(dev), d["zeros"].to(dev), 128, sym, lo]
    ours = GK.gptq_dequant_matmul(*args)
    ref = ref_gptq.gptq_dequant_matmul(*args)
    torch.cuda.synchronize()
    assert ours.shape == ref.shape and ours.dtype == ref.dtype == torch.float32
    assert float((ours - ref).abs().max()) < 0.01
    assert cases.rel_l2(ours.cpu(), ref.cpu()) <= 1e-4
