"""Parity of the CUDA kernels with the CPU oracle, through the C ABI (ctypes) and the Python
classes that mirror the reference.  Bars: dequantised tiles bit-exact; layer outputs
rel-L2 <= 1e-3 (fp16 storage, fp32 accumulation); the reference's own kernel-test bound
max|err| < 0.01 (inference/kernels/test_kernels.py:105) on its data distributions."""

import pytest
import torch

from oracle import glorcq_oracle as O
from tests import cases

pytestmark = pytest.mark.gpu
REL = 1e-3


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from glorcq_b200 import _build
    _build.build()
    return torch.device("cuda:0")


# ---- tiles ---------------------------------------------------------------------------------
@pytest.mark.parametrize("N,K,bits,gs,int_zeros", [
    (1408, 2048, 2, 128, True), (2048, 1408, 2, 128, True), (40, 200, 2, 128, True), (17, 128, 2, 128, False),
    (64, 256, 4, 128, True), (2048, 2048, 4, 128, True), (33, 192, 4, 64, False), (48, 512, 2, 256, True)])
def test_gptq_tiles_bit_exact(dev, N, K, bits, gs, int_zeros):
    from glorcq_b200.tiled import TiledWeight
    d = cases.make_linear(101 + N + K, N, K, fmt="gptq", bits=bits, groupsize=gs, int_zeros=int_zeros, with_lora=False)
    tw = TiledWeight.from_gptq(d["qweight_int"].to(dev), d["scales"].to(dev), d["zeros"].to(dev), bits, gs)
    W = tw.dequantize().cpu()
    ref = O.gptq_tile_fp16(d["qweight_int"], d["scales"], d["zeros"], gs)
    assert torch.equal(W, ref)


@pytest.mark.parametrize("N,K", [(1408, 2048), (72, 256), (19, 132), (64, 64)])
def test_turbo_tiles_bit_exact(dev, N, K):
    from glorcq_b200.tiled import TiledWeight
    d = cases.make_linear(202 + N, N, K, fmt="turbo", with_lora=False)
    tw = TiledWeight.from_turbo(d["packed_indices"].to(dev), d["norms"].to(dev), d["centroids"].to(dev))
    W = tw.dequantize().cpu()
    assert torch.equal(W, O.turbo_tile(d["packed_indices"], d["norms"], d["centroids"], K))


# ---- GLoRCQLinear.forward ------------------------------------------------------------------
LIN = [
    # N, K, rank, fmt, bits, groupsize, sym
    (1408, 2048, 64, "gptq", 2, 128, False),     # expert gate/up projection
    (2048, 1408, 64, "gptq", 2, 128, False),     # expert down projection, 11 groups
    (5632, 2048, 64, "gptq", 2, 128, False),     # shared expert
    (2048, 5632, 64, "gptq", 2, 128, True),
    (2048, 2048, 128, "gptq", 4, 128, False),    # attention projection, 4-bit
    (100, 392, 16, "gptq", 2, 128, False),       # ragged rows, K not a multiple of 128
    (24, 128, 0, "gptq", 2, 128, False),
    (1408, 2048, 64, "turbo", 2, 0, False),
    (2048, 1408, 64, "turbo", 2, 0, False),
    (52, 192, 16, "turbo", 2, 0, False),
]


@pytest.mark.parametrize("B", [1, 2, 5, 8, 13, 16, 33, 70])
@pytest.mark.parametrize("N,K,rank,fmt,bits,gs,sym", LIN)
def test_linear_forward(dev, N, K, rank, fmt, bits, gs, sym, B):
    if B > 16 and N * K > 3_000_000:
        pytest.skip("large batch only on the smaller shapes")
    d = cases.make_linear(7 * N + K + B, N, K, rank=max(rank, 16), fmt=fmt, bits=bits, groupsize=gs or 128, sym=sym,
                          with_lora=rank > 0)
    lin = cases.to_b200_linear(d, dev)
    x = cases.make_x(N + K + 31 * B, B, K)
    y = lin(x.to(dev)).cpu()
    ref = O.linear_forward(cases.to_oracle_linear(d), x, x_rot_half=True)
    assert y.dtype == torch.float16 and y.shape == ref.shape
    assert cases.rel_l2(y, ref) <= REL
    if rank > 0:
        a = (x @ d["U"])
        y2 = lin(x.to(dev), precomputed_xU=a.to(dev)).cpu()
        assert cases.rel_l2(y2, ref) <= REL


def _hostile_rows(B, K, seed):
    """Activation rows that attack the block fixed-point staging of the integer decode path (each 128-channel
    block of a row is scaled by a power of two taken from its largest magnitude): one element 2^10 times the
    rest of its block, a block of fp16 subnormals, a block of zeros, elements at +-60000 beside ordinary
    values, a row of tiny values, and blocks whose sign pattern makes the plain sum cancel."""
    x = cases.make_x(seed, B, K).float()
    nb = K // 128
    for b in range(B):
        x[b, (b % nb) * 128 + 5] *= 1024.0                               # outlier 2^10 x its block
        blk = (b + 1) % nb
        x[b, blk * 128:(blk + 1) * 128] = x[b, blk * 128:(blk + 1) * 128] * 3e-7    # fp16 subnormals
        blk = (b + 2) % nb
        x[b, blk * 128:(blk + 1) * 128] = 0.0
        blk = (b + 3) % nb
        x[b, blk * 128 + 17] = 60000.0
        x[b, blk * 128 + 90] = -60000.0
        blk = (b + 4) % nb
        half = x[b, blk * 128:blk * 128 + 64].clone()
        x[b, blk * 128 + 64:(blk + 1) * 128] = -half                       # sum of the block cancels exactly
    if B > 1:
        x[B - 1] *= 1e-3
    return x.to(torch.float16)


@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("N,K,bits", [(1408, 2048, 2), (2048, 1408, 2), (2048, 2048, 4)])
def test_integer_path_hostile_activations(dev, N, K, bits, B):
    """Up to 8 rows of affine codes run on the integer path, which rounds every 128-channel block of x to
    16-bit fixed point relative to the block maximum (exact within 2^-13 of it, absolute error <= 2^-16 of it
    below); the reference multiplies the exact fp16 values.  Outliers, subnormals and near-overflow values
    must still land within the layer bar, rel-L2 <= 1e-3, per row as well as over all rows."""
    d = cases.make_linear(77 * B + N + bits, N, K, rank=64, bits=bits)
    lin = cases.to_b200_linear(d, dev)
    x = _hostile_rows(B, K, 4000 + B + N)
    y = lin(x.to(dev)).cpu()
    ref = O.linear_forward(cases.to_oracle_linear(d), x)
    assert torch.isfinite(ref.float()).all() and torch.isfinite(y.float()).all()
    assert cases.rel_l2(y, ref) <= REL
    for b in range(B):
        assert cases.rel_l2(y[b], ref[b]) <= REL, f"row {b}"


@pytest.mark.parametrize("N,K,rank,B,int_zeros", [(1408, 2048, 64, 128, True), (2048, 1408, 64, 300, True),
                                                   (100, 392, 16, 200, True), (256, 256, 16, 64, False),
                                                   (24, 128, 0, 40, True), (5632, 2048, 64, 96, True)])
def test_many_rows_tensor_core_path(dev, N, K, rank, B, int_zeros):
    """More than 32 rows of 2-bit affine codes go to the tcgen05 kernel: ragged feature and channel
    counts, token counts that do not fill a tile, non-integer zero points."""
    d = cases.make_linear(11 * N + K + B, N, K, rank=max(rank, 16), with_lora=rank > 0, int_zeros=int_zeros)
    lin = cases.to_b200_linear(d, dev)
    x = cases.make_x(N + 3 * K + B, B, K)
    y = lin(x.to(dev)).cpu()
    ref = O.linear_forward(cases.to_oracle_linear(d), x)
    assert cases.rel_l2(y, ref) <= REL
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


@pytest.mark.parametrize("N,K,rank,B,int_zeros", [(5632, 2048, 64, 1300, True), (2816, 1024, 16, 2100, False)])
def test_many_rows_more_items_than_sms(dev, N, K, rank, B, int_zeros):
    """Prefill-sized calls whose (token tile, feature tile) items outnumber the SMs: every CTA of the persistent
    tcgen05 kernel takes several items, so the rings run across item boundaries, the accumulator is handed back
    and forth and the results of one item are written while the next one is multiplied.  Last token tile ragged."""
    d = cases.make_linear(5 * N + K + B, N, K, rank=rank, int_zeros=int_zeros)
    lin = cases.to_b200_linear(d, dev)
    x = cases.make_x(N + 7 * K + B, B, K)
    y = lin(x.to(dev)).cpu()
    ref = O.linear_forward(cases.to_oracle_linear(d), x)
    assert cases.rel_l2(y, ref) <= REL
    for b in (0, 255, 256, 1023, 1024, B - 1):
        assert cases.rel_l2(y[b], ref[b]) <= REL, f"row {b}"
    y2 = lin(x.to(dev)).cpu()
    assert torch.equal(y, y2), "two calls in a row differ"
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("B", [1, 40])
def test_mixtral_expert_projection_shapes(dev, N, K, B):
    """The largest projections of the benchmark configurations (expert up / down of a Mixtral-8x7B-shaped
    layer): long reductions (112 k blocks) and many row tiles."""
    d = cases.make_linear(3 * N + K + B, N, K, rank=64)
    lin = cases.to_b200_linear(d, dev)
    x = cases.make_x(N + K + B, B, K)
    y = lin(x.to(dev)).cpu()
    ref = O.linear_forward(cases.to_oracle_linear(d), x)
    assert cases.rel_l2(y, ref) <= REL
    from glorcq_b200 import tiled
    assert tiled.debug_error() is None


def test_linear_batch_dims_and_empty(dev):
    d = cases.make_linear(5, 96, 256, rank=16)
    lin = cases.to_b200_linear(d, dev)
    x = cases.make_x(6, 6, 256).reshape(2, 3, 256)
    y = lin(x.to(dev))
    assert y.shape == (2, 3, 96)
    ref = O.linear_forward(cases.to_oracle_linear(d), x)
    assert cases.rel_l2(y.cpu(), ref) <= REL
    y0 = lin(torch.empty(0, 256, dtype=torch.float16, device=dev))
    assert y0.shape == (0, 96)
    torch.cuda.synchronize()


def test_linear_turbo_with_rotation(dev):
    d = cases.make_linear(21, 72, 256, rank=16, fmt="turbo")
    g = torch.Generator().manual_seed(5021)
    q, _ = torch.linalg.qr(torch.randn(256, 256, generator=g))
    d["Pi"] = q.to(torch.float16)
    lin = cases.to_b200_linear(d, dev)
    x = cases.make_x(1021, 4, 256)
    ref = O.linear_forward(cases.to_oracle_linear(d), x, x_rot_half=True)
    assert cases.rel_l2(lin(x.to(dev)).cpu(), ref) <= REL
    xr = (x.float() @ d["Pi"].float().T).half()
    assert cases.rel_l2(lin(x.to(dev), precomputed_x_rot=xr.to(dev)).cpu(), ref) <= REL


@pytest.mark.parametrize("B", [1, 3, 8, 13])
@pytest.mark.parametrize("N,K,rank", [(1408, 2048, 64), (2048, 1408, 64), (52, 192, 16)])
@pytest.mark.parametrize("residue", [0.0, 2e-7])
def test_linear_turbo_symmetric_codebook(dev, N, K, rank, B, residue):
    """A codebook (-a, -b, b, a), the shape a Lloyd-Max fit of a symmetric density gives (exactly, or up to the
    residue of the fit's last iteration): up to 8 rows take the integer path with two integer products per
    block; the sorted random codebooks of the other cases take its three-product form."""
    d = cases.make_linear(900 + N + B, N, K, rank=rank, fmt="turbo")
    c = torch.tensor([-1.51, -0.4528, 0.4528, 1.51], dtype=torch.float64) / K ** 0.5
    c[3] += residue * c[3]
    d["centroids"] = c.float()
    lin = cases.to_b200_linear(d, dev)
    x = cases.make_x(901 + B, B, K)
    ref = O.linear_forward(cases.to_oracle_linear(d), x, x_rot_half=True)
    assert cases.rel_l2(lin(x.to(dev)).cpu(), ref) <= REL


def test_shared_u_is_tiled_once(dev):
    from glorcq_b200 import tiled
    blk = cases.make_moe(77, 256, 128, 4, 2, rank=16, experts_per_cluster=2)
    shared = {}
    lins = [cases.to_b200_linear(ex["gate_proj"], dev, shared) for ex in blk["experts"]]
    assert lins[0]._ut is lins[1]._ut and lins[2]._ut is lins[3]._ut and lins[0]._ut is not lins[2]._ut
    assert lins[0].U.data_ptr() == lins[1].U.data_ptr()


def test_against_golden(dev, golden):
    from tests.golden.make_golden import LINEAR_CASES
    for name, kw, B in LINEAR_CASES:
        d = cases.make_linear(**kw)
        if d["fmt"] == "turbo":
            gen = torch.Generator().manual_seed(kw["seed"] + 5000)
            q, _ = torch.linalg.qr(torch.randn(kw["K"], kw["K"], generator=gen))
            d["Pi"] = q.to(torch.float16)
        lin = cases.to_b200_linear(d, dev)
        x = cases.make_x(kw["seed"] + 1000, B, kw["K"])
        y = lin(x.to(dev)).cpu()
        assert cases.rel_l2(y, golden["linear"][name]["y"]) <= REL, name


# ---- drop-ins for the reference's native modules ---------------------------------------------
@pytest.mark.parametrize("B,N,K", [(1, 1408, 2048), (4, 2048, 1408), (5, 1408, 2048), (16, 4096, 4096),
                                   (32, 512, 14336), (1, 64, 64), (3, 30, 36), (1, 2048, 5632), (8, 5632, 2048)])
def test_turbo_dropin(dev, B, N, K):
    import glorcq_b200.kernels as GK
    g = torch.Generator().manual_seed(B * 1000 + N + K)
    packed = torch.randint(0, 256, (N, K // 4), generator=g, dtype=torch.int32).to(torch.uint8)
    norms = torch.randn(N, generator=g).abs() + 0.1
    centroids = torch.randn(4, generator=g)
    x = torch.randn(B, K, generator=g).half()
    y = GK.turbo_dequant_matmul_fused(None, packed.to(dev), norms.to(dev), None, centroids.to(dev), 2, K,
                                      precomputed_x_rot=x.to(dev))
    ref = O.turbo_matmul(x, packed, norms, centroids)
    assert y.dtype == torch.float16 and tuple(y.shape) == (B, N)
    assert cases.rel_l2(y.cpu(), ref) <= REL


def test_turbo_dropin_empty_batch(dev):
    import glorcq_b200.kernels as GK
    packed = torch.zeros(8, 16, dtype=torch.uint8, device=dev)
    y = GK.turbo_dequant_matmul(torch.empty(0, 64, dtype=torch.float16, device=dev), packed,
                                torch.ones(8, device=dev), torch.ones(4, device=dev))
    assert tuple(y.shape) == (0, 8)
    torch.cuda.synchronize()      # the context stays healthy
    with pytest.raises(RuntimeError):
        GK.turbo_dequant_matmul(torch.empty(1, 64, dtype=torch.float32, device=dev), packed,
                                torch.ones(8, device=dev), torch.ones(4, device=dev))


@pytest.mark.parametrize("E,n_out,K", [(3, 16, 128), (60, 2048, 1408), (5, 100, 256)])
def test_turbo_grouped_dropin(dev, E, n_out, K):
    import glorcq_b200.kernels as GK
    d = cases.make_linear(43 + E, E * n_out, K, fmt="turbo", with_lora=False)
    x = cases.make_x(44 + E, E, K)
    y = GK.turbo_dequant_grouped_gemv_fused(x.to(dev), d["packed_indices"].to(dev), d["norms"].to(dev),
                                            d["centroids"].to(dev), n_out)
    ref = O.turbo_grouped_gemv(x, d["packed_indices"], d["norms"], d["centroids"], n_out)
    assert tuple(y.shape) == (E * n_out,)
    assert cases.rel_l2(y.cpu(), ref) <= REL


@pytest.mark.parametrize("B,N,K,sym,lora", [(1, 1408, 2048, False, False), (4, 2048, 1408, False, True),
                                            (5, 100, 392, True, False), (9, 64, 256, False, True),
                                            (0, 16, 128, False, False)])
def test_gptq_i8_dropin(dev, B, N, K, sym, lora):
    import glorcq_b200.kernels as GK
    d = cases.make_linear(900 + N, N, K, fmt="gptq", with_lora=False, int_zeros=False, sym=sym, signed_codes=True)
    x = cases.make_x(901, B, K, torch.float32)
    lo = cases.make_x(902, B, N, torch.float32) * 0.1 if lora else torch.empty(0)
    q8 = d["qweight_int"].to(torch.int8)
    y = GK.gptq_dequant_matmul(x.to(dev), q8.to(dev), d["scales"].to(dev), d["zeros"].to(dev), 128, sym, lo.to(dev))
    assert y.dtype == torch.float32 and tuple(y.shape) == (B, N)
    if B:
        ref = O.gptq_matmul(x, d["qweight_int"], d["scales"], d["zeros"], 128, sym, lo if lora else None)
        assert cases.rel_l2(y.cpu(), ref) <= 1e-5
        assert float((y.cpu() - ref).abs().max()) < 0.01
        yh = GK.gptq_dequant_matmul_fused(x.half().to(dev), d["qweight_int"].to(dev), d["scales"].to(dev),
                                          d["zeros"].to(dev), 128, sym)
        assert yh.dtype == torch.float16


# ---- routes around the packed formats ----------------------------------------------------------------
def test_dense_weight_route_dtype_and_reference_op_names(dev):
    """Pre-dequantised weights (a checkpoint's ``weight_quant`` records and the legacy load_turbo_predequant)
    run dense through the fp16 kernels with the low-rank term; a bf16 / fp32 input gets its own dtype back;
    the reference's custom-op names ``torch.ops.glorcq.*`` bind to this package's kernels."""
    from glorcq_b200.quantized_linear import GLoRCQLinear
    import glorcq_b200.kernels as GK
    g = torch.Generator().manual_seed(77)
    N, K, r = 96, 256, 16
    W = (torch.randn(N, K, generator=g) * 0.05).half()
    U = (torch.randn(K, r, generator=g) * 0.01).half()
    SV = (torch.randn(N, r, generator=g) * 0.01).half()
    x = cases.make_x(78, 5, K)
    ref = (x.float() @ W.float().T + (x.float() @ U.float()) @ SV.float().T)
    lin = GLoRCQLinear(K, N)
    lin.load_dense(W, device=dev)
    lin.load_sv(U.to(dev), SV, device=dev)
    y = lin(x.to(dev))
    assert y.dtype == torch.float16 and cases.rel_l2(y.cpu(), ref) <= REL
    for dt in (torch.bfloat16, torch.float32):
        assert lin(x.to(dev).to(dt)).dtype == dt
    d = cases.make_linear(79, N, K, rank=r)
    assert cases.to_b200_linear(d, dev)(x.to(dev).float()).dtype == torch.float32

    class _Quantizer:                      # stands in for the third-party quantizer object
        def dequantize(self, q):
            assert q.bits == 2 and q.indices.shape == (N, K // 4)
            return W.to(q.indices.device)
    lin2 = GLoRCQLinear(K, N)
    lin2.load_turbo_predequant({"packed_indices": torch.zeros(N, K // 4, dtype=torch.uint8), "norms": torch.ones(N),
                                "bits": 2, "dim": K}, _Quantizer(), device=dev)
    assert lin2.quant_type == "turbo" and cases.rel_l2(lin2(x.to(dev)).cpu(), x.float() @ W.float().T) <= REL

    t = cases.make_linear(80, 72, 256, fmt="turbo", with_lora=False)
    y1 = torch.ops.glorcq.turbo_dequant_matmul(x.to(dev), t["packed_indices"].to(dev), t["norms"].to(dev), t["centroids"].to(dev))
    assert cases.rel_l2(y1.cpu(), O.turbo_matmul(x, t["packed_indices"], t["norms"], t["centroids"])) <= REL
    q = cases.make_linear(81, 64, 256, fmt="gptq", with_lora=False, signed_codes=True)
    q32 = q["qweight_int"].to(dev)
    y2 = torch.ops.glorcq.gptq_dequant_matmul(x.float().to(dev), q32.to(torch.int8), q["scales"].to(dev), q["zeros"].to(dev), 128,
                                              False, torch.empty(0, device=dev))
    assert cases.rel_l2(y2.cpu(), O.gptq_matmul(x.float(), q["qweight_int"], q["scales"], q["zeros"], 128, False, None)) <= 1e-5
    # the int8 copy of int32 codes is made once per tensor, and again after the tensor changed
    a8 = GK._int8_codes(q32)
    assert GK._int8_codes(q32) is a8
    q32 += 0
    assert GK._int8_codes(q32) is not a8
