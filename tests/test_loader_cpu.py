"""On-disk format decoders, the low-rank assignment rules and the Hadamard helpers, on CPU: the oracle
and the package's host logic against vectors produced by the reference's own functions
(tests/golden/make_golden.py)."""

import pytest
import torch

from glorcq_b200 import model_builder as MB
from glorcq_b200 import synthetic
from glorcq_b200.hadamard_rotation import generate_rht_signs
from oracle import glorcq_oracle as O
from tests.golden.make_golden import LOADER_CFG, LOADER_FORMATS, LOADER_MODULES, RHT_SIGN_CASES


def test_int4_and_intN_decoders(golden):
    g = golden["loader"]["unpack_int4"]
    assert torch.equal(O.unpack_int4(g["packed"], g["rows"]), g["out"])
    assert torch.equal(MB._unpack_int4(g["packed"], g["rows"]), g["out"])
    assert torch.equal(MB._unpack_int4(MB._pack_int4(g["out"]), g["rows"]), g["out"])       # writer <-> reader
    d = golden["loader"]["dequant_intN"]
    for fn in (O.dequant_intN, MB._dequant_intN):
        assert torch.equal(fn(d["q"], d["scale"], 8), d["out8"])
        assert torch.equal(fn(d["q"].clamp(-7, 7), d["scale"], 4), d["out4"])


@pytest.mark.parametrize("fmt", LOADER_FORMATS)
def test_low_rank_factors_as_the_reference_loads_them(golden, fmt):
    md, cr, _ = synthetic.make_checkpoint(LOADER_CFG, seed=62, rank=8, attn_rank=8, n_clusters=2, u_format=fmt,
                                          sv_format=fmt)
    layers = O.checkpoint_layers(md, cr)
    cc = cr["config"]
    uc = MB.SharedUCache(cr["shared_matrices"], cc["uv_bits"], device="cpu", u_bits=cc["u_bits"])
    for name in LOADER_MODULES:
        ref = golden["loader"][fmt][name]
        ql = layers[0][name]
        if ref["U"] is None:                       # the shared expert gets no low-rank term
            assert ql.U is None and ql.SV is None and "shared_expert" in name
            continue
        assert torch.equal(ql.U, ref["U"]) and torch.equal(ql.SV, ref["SV"])
        assert tuple(ql.cluster_id) == tuple(ref["cluster_id"])
        assert torch.equal(uc.get(*ref["cluster_id"])[0], ref["U"])


def test_module_keys_and_assignment_lookup():
    assert MB.module_key("self_attn.q_proj") == ("q_proj", -1)
    assert MB.module_key("mlp.experts.17.up_proj") == ("up_proj", 17)
    assert MB.module_key("mlp.shared_expert.down_proj") == ("down_proj", -2)
    assert MB.module_key("block_sparse_moe.experts.3.w1") == ("gate_proj", 3)
    assert MB.module_key("block_sparse_moe.experts.3.w2") == ("down_proj", 3)
    assert MB.module_key("block_sparse_moe.experts.3.w3") == ("up_proj", 3)
    assert MB.module_key("mlp.gate") == (None, -1)
    look = MB.assignment_lookup({"up_proj": [{"layer": 0, "expert": 2, "group_id": 5}, {"layer": 1, "expert": 2, "group_id": 7}]})
    assert look[("up_proj", 1, 2)] == (7, "up_proj", 1)


def test_checkpoint_write_read_round_trip(tmp_path):
    md, cr, dense = synthetic.write_checkpoint(str(tmp_path), LOADER_CFG, seed=3, rank=8, attn_rank=8, n_clusters=2)
    mc, layers, cross, hf = MB.read_checkpoint(str(tmp_path))
    assert hf == LOADER_CFG and mc == md["model_config"]
    assert torch.equal(layers[0]["mlp.experts.1.up_proj"]["qweight_int"], md["layers"][0]["mlp.experts.1.up_proj"]["qweight_int"])
    assert cross["assignments"] == cr["assignments"]
    assert MB.lora_bits(mc, cross["config"]) == (8, 4, 4)
    with pytest.raises(FileNotFoundError):
        MB.read_checkpoint(str(tmp_path / "missing"))


def test_global_u_pool_shapes():
    md, cr, _ = synthetic.make_checkpoint(LOADER_CFG, seed=4, rank=8, attn_rank=8, n_clusters=3, u_format="fp16")
    uc = MB.SharedUCache(cr["shared_matrices"], 8, device="cpu")
    pools, ids = MB._build_global_u_pool(uc)
    assert pools["gate"].shape == (64, 3 * 8) and pools["down"].shape == (32, 3 * 8)
    assert ids["up"][("up_proj", 2)] == 2


@pytest.mark.parametrize("d,seed", RHT_SIGN_CASES)
def test_rht_signs_match_the_reference(golden, d, seed):
    ref = golden["rht_signs"][f"{d}_{seed}"].float()
    assert torch.equal(O.generate_rht_signs(d, seed), ref)
    assert torch.equal(generate_rht_signs(d, seed=seed, device="cpu"), ref)


def test_rht_oracle_properties():
    from scipy.linalg import hadamard
    x = torch.randn(3, 64, generator=torch.Generator().manual_seed(5))
    s = O.generate_rht_signs(64, 1)
    y = O.rht_forward(x, s)
    ref = (x * s).double() @ torch.tensor(hadamard(64), dtype=torch.float64).T / 8.0
    assert torch.allclose(y.double(), ref, atol=1e-6)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)                 # norm preserving
    back = O.rht_forward(y, torch.ones(64)) * s                                       # D (1/sqrt d) H y
    assert torch.allclose(back, x, atol=1e-5)
    # a dimension that is not a power of two: zero-padded to the next one, first d outputs, scale 1/sqrt(d)
    x2 = torch.randn(2, 48, generator=torch.Generator().manual_seed(6))
    s2 = O.generate_rht_signs(48, 2)
    ref2 = (torch.nn.functional.pad((x2 * s2).double(), (0, 16)) @ torch.tensor(hadamard(64), dtype=torch.float64).T)[:, :48] / 48 ** 0.5
    assert torch.allclose(O.rht_forward(x2, s2).double(), ref2, atol=1e-6)
