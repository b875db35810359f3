"""The CPU oracle against vectors produced by the unmodified reference
(tests/golden/make_golden.py).  Integer results and weight tiles must be bit-exact; matmul
outputs are compared with a tolerance of a few fp16 ulps because a different host may sum in a
different order than the host that wrote the vectors."""

import hashlib

import pytest
import torch

from oracle import glorcq_oracle as O
from tests import cases
from tests.golden.make_golden import linear_digest, moe_digest, digest, LINEAR_CASES, MOE_CASES


def close16(a, b, tol=2e-3):
    """max |a-b| <= tol * max|b|  (fp16 outputs: one ulp is 9.8e-4 relative)."""
    a, b = a.float(), b.float()
    return float((a - b).abs().max()) <= tol * float(b.abs().max() + 1e-12)


def test_unpack_and_turbo_fallback(golden):
    g = golden["kernel"]["turbo_unpack"]
    d = cases.make_linear(**g["args"])
    assert linear_digest(d) == g["digest"], "seeded inputs drifted from the ones the golden file was made with"
    assert torch.equal(O.unpack_codes_2bit(d["packed_indices"], 192).to(torch.uint8), g["codes_u8"])
    assert torch.equal(O.unpack_codes(d["packed_indices"], 2, 192).to(torch.uint8), g["codes_u8"])
    x = cases.make_x(g["x_seed"], g["B"], 192)
    y = O.turbo_matmul(x.float(), d["packed_indices"], d["norms"], d["centroids"])
    assert cases.rel_l2(y, g["y_fallback"]) < 1e-6
    assert cases.rel_l2(y, g["y_fused"]) < 1e-6


def test_turbo_grouped(golden):
    g = golden["kernel"]["turbo_grouped"]
    d = cases.make_linear(**g["args"])
    assert linear_digest(d) == g["digest"]
    x = cases.make_x(g["x_seed"], g["E"], 128)
    y = O.turbo_grouped_gemv(x, d["packed_indices"], d["norms"], d["centroids"], g["n_out"])
    assert y.dtype == torch.float16 and y.shape == g["y"].shape
    assert close16(y, g["y"])


@pytest.mark.parametrize("name", ["gptq_i8_asym", "gptq_i8_sym"])
def test_gptq_fallback(golden, name):
    g = golden["kernel"][name]
    d = cases.make_linear(**g["args"])
    assert linear_digest(d) == g["digest"]
    K, N = g["args"]["K"], g["args"]["N"]
    x = cases.make_x(g["x_seed"], g["B"], K, torch.float32)
    lora = cases.make_x(g["lora_seed"], g["B"], N, torch.float32) * 0.1
    y = O.gptq_matmul(x, d["qweight_int"], d["scales"], d["zeros"], 128, d["sym"])
    assert cases.rel_l2(y, g["y"]) < 1e-6
    yl = O.gptq_matmul(x, d["qweight_int"], d["scales"], d["zeros"], 128, d["sym"], lora)
    assert cases.rel_l2(yl, g["y_lora"]) < 1e-6
    assert close16(y.half(), g["y_fused_half"])


@pytest.mark.parametrize("name,kw,B", LINEAR_CASES, ids=[c[0] for c in LINEAR_CASES])
def test_linear_forward(golden, name, kw, B):
    g = golden["linear"][name]
    d = cases.make_linear(**kw)
    if d["fmt"] == "turbo":
        gen = torch.Generator().manual_seed(kw["seed"] + 5000)
        q, _ = torch.linalg.qr(torch.randn(kw["K"], kw["K"], generator=gen))
        d["Pi"] = q.to(torch.float16)
    assert linear_digest(d) == g["digest"]
    p = cases.to_oracle_linear(d)
    x = cases.make_x(kw["seed"] + 1000, B, kw["K"])
    if d["fmt"] == "gptq":
        W = O.gptq_tile_fp16(d["qweight_int"], d["scales"], d["zeros"], d["groupsize"], d["sym"])
        assert torch.equal(W[:8, :256], g["tile_fp16_head"])          # bit-exact tile
        assert digest(W) == g["tile_digest"]
        if d["zeros"].float().frac().abs().max() == 0:
            # integer zero points: the fp32 formula rounds to the same fp16 bits
            W32 = O.gptq_tile_fp32(d["qweight_int"], d["scales"], d["zeros"], d["groupsize"], d["sym"])
            assert torch.equal(W32.half(), W)
    y = O.linear_forward(p, x)
    assert y.dtype == g["y"].dtype and y.shape == g["y"].shape
    assert close16(y, g["y"])
    if "SV" in d:
        y2 = O.linear_forward(p, x, precomputed_xU=x @ d["U"])
        assert close16(y2, g["y_pre_xU"])


@pytest.mark.parametrize("name,kw,N", MOE_CASES, ids=[c[0] for c in MOE_CASES])
def test_moe_forward(golden, name, kw, N):
    g = golden["moe"][name]
    blk = cases.make_moe(**kw)
    assert moe_digest(blk) == g["digest"]
    ob = cases.to_oracle_moe(blk)
    x = cases.make_x(kw["seed"] + 1000, N, kw["H"]).reshape(1, N, kw["H"])
    y, logits = O.moe_forward(ob, x)
    assert y.shape == g["y"].shape and y.dtype == g["y"].dtype
    assert close16(logits, g["router_logits"])
    assert close16(y, g["y"], tol=4e-3)
    assert cases.rel_l2(y, g["y"]) < 1e-3


def test_experts_adapter(golden):
    g = golden["experts"]["experts_10"]
    blk = cases.make_moe(**g["args"])
    assert moe_digest(blk) == g["digest"]
    ob = cases.to_oracle_moe(blk)
    x = cases.make_x(g["x_seed"], g["T"], g["args"]["H"])
    y = O.experts_forward(ob.experts, x, g["idx"], g["w"])
    assert close16(y, g["y"], tol=4e-3)
    assert cases.rel_l2(y, g["y"]) < 1e-3
