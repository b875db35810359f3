"""Generate the golden vectors that pin the CPU oracle to the reference.

Run where the unmodified reference tree is mounted (it cannot travel with the repository):

    python tests/golden/make_golden.py --ref <checkout of the reference>

It imports the reference's own modules (``inference.kernels`` falls back to its pure-PyTorch
functions when its CUDA extensions are absent; ``inference.quantized_linear.GLoRCQLinear``;
``inference.moe_block.GraphCompatibleMoeBlock``), feeds them the seeded inputs of
``tests/cases.py`` and writes ``tests/golden/golden.pt``: for every case the generator arguments,
a SHA-256 of the input bytes (so a drifting random generator is detected, not silently accepted)
and the reference's outputs.  Nothing here is imported by the shipped package.

Two workarounds keep the reference unmodified:
* ``GraphCompatibleMoeBlock._build_cluster_map`` lost its ``def`` line; its body now runs inside
  ``set_global_pool`` (inference/moe_block.py:85-115), so ``set_global_pool({}, {})`` is called once.
* the block expects a transformers-4.45-shaped sparse block; a stand-in with the same attribute
  names is built here, as inference/test_cluster_parallel.py:65-88 does.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests import cases  # noqa: E402


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().cpu().numpy().tobytes())
    return h.hexdigest()


def linear_digest(d) -> str:
    keys = ["qweight_int", "scales", "zeros", "packed_indices", "norms", "centroids", "U", "SV"]
    return digest(*[d[k] for k in keys if k in d])


def moe_digest(blk) -> str:
    ts = [blk["gate_weight"]]
    for ex in blk["experts"]:
        for p in ("gate_proj", "up_proj", "down_proj"):
            d = ex[p]
            ts += [d[k] for k in ("qweight_int", "scales", "zeros", "packed_indices", "norms", "U", "SV") if k in d]
    if blk.get("shared_expert"):
        for p in ("gate_proj", "up_proj", "down_proj"):
            d = blk["shared_expert"][p]
            ts += [d[k] for k in ("qweight_int", "scales", "zeros", "packed_indices", "norms", "U", "SV") if k in d]
        ts.append(blk["shared_gate_weight"])
    return digest(*ts)


class FakeRotationCache:
    """Stands in for model_builder.RotationCache (inference/model_builder.py:86-137), whose real
    constructor needs the absent third-party turboquant package: it hands out a given Pi and codebook."""

    def __init__(self, Pi, centroids):
        self._pi, self._c = Pi, centroids

    def register(self, dim, bits, seed=42):
        pass

    def get_pi(self, dim, bits, seed=42):
        return self._pi

    def get_centroids(self, dim, bits, seed=42):
        return self._c


def ref_linear(RefLinear, d):
    lin = RefLinear(d["K"], d["N"])
    if d["fmt"] == "gptq":
        lin.load_gptq({"qweight_int": d["qweight_int"], "scales": d["scales"], "zeros": d["zeros"],
                       "bits": d["bits"], "groupsize": d["groupsize"], "sym": d["sym"]}, device="cpu")
    else:
        Pi = d.get("Pi")
        if Pi is None:
            Pi = torch.eye(d["K"], dtype=torch.float16)
        lin.load_turbo({"packed_indices": d["packed_indices"], "norms": d["norms"], "bits": 2,
                        "dim": d["K"], "seed": 42}, FakeRotationCache(Pi, d["centroids"]), device="cpu")
    if "SV" in d:
        lin.load_sv(d["U"], d["SV"], device="cpu")
        lin.cluster_id = d.get("cluster_id")
    return lin


class RefExpert(nn.Module):
    def __init__(self, RefLinear, ex):
        super().__init__()
        self.gate_proj = ref_linear(RefLinear, ex["gate_proj"])
        self.up_proj = ref_linear(RefLinear, ex["up_proj"])
        self.down_proj = ref_linear(RefLinear, ex["down_proj"])
        self.act_fn = F.silu

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class RefHFBlock:
    def __init__(self, RefLinear, blk):
        self.num_experts = blk["E"]
        self.top_k = blk["top_k"]
        self.norm_topk_prob = blk["norm_topk_prob"]
        self.gate = nn.Linear(blk["H"], blk["E"], bias=False).half()
        self.gate.weight.data.copy_(blk["gate_weight"])
        self.experts = nn.ModuleList([RefExpert(RefLinear, ex) for ex in blk["experts"]])
        self.shared_expert = RefExpert(RefLinear, blk["shared_expert"])
        self.shared_expert_gate = nn.Linear(blk["H"], 1, bias=False).half()
        self.shared_expert_gate.weight.data.copy_(blk["shared_gate_weight"])


LINEAR_CASES = [
    # name, kwargs of cases.make_linear, batch
    ("gptq2_asym", dict(seed=11, N=96, K=256, rank=16, fmt="gptq", bits=2), 3),
    ("gptq2_sym", dict(seed=12, N=80, K=384, rank=16, fmt="gptq", bits=2, sym=True), 1),
    ("gptq4_asym", dict(seed=13, N=64, K=256, rank=32, fmt="gptq", bits=4), 5),
    ("gptq2_fraczero", dict(seed=14, N=48, K=256, rank=16, fmt="gptq", bits=2, int_zeros=False), 2),
    ("gptq2_nolora", dict(seed=15, N=40, K=128, rank=0, fmt="gptq", bits=2, with_lora=False), 1),
    ("gptq2_c1", dict(seed=1234, N=1408, K=2048, rank=64, fmt="gptq", bits=2), 1),
    ("turbo_small", dict(seed=21, N=72, K=256, rank=16, fmt="turbo"), 4),
    ("turbo_nolora", dict(seed=22, N=64, K=64, rank=0, fmt="turbo", with_lora=False), 1),
]

MOE_CASES = [
    ("moe_decode_1", dict(seed=31, H=256, I=128, E=8, top_k=2, I_shared=256, rank=16, experts_per_cluster=3), 1),
    ("moe_decode_1_norm", dict(seed=32, H=256, I=128, E=8, top_k=2, I_shared=256, rank=16, experts_per_cluster=3,
                               norm_topk_prob=True), 1),
    ("moe_sparse_9", dict(seed=33, H=256, I=128, E=8, top_k=2, I_shared=256, rank=16, experts_per_cluster=3), 9),
    ("moe_sparse_20_norm", dict(seed=34, H=256, I=256, E=12, top_k=4, I_shared=384, rank=16, experts_per_cluster=4,
                                norm_topk_prob=True), 20),
    ("moe_turbo_7", dict(seed=35, H=256, I=128, E=6, top_k=2, I_shared=256, rank=16, experts_per_cluster=2,
                         fmt="turbo"), 7),
    # the Qwen1.5-MoE block at its own dimensions, 8 tokens
    ("moe_qwen15_shape_8", dict(seed=36, H=2048, I=1408, E=60, top_k=4, I_shared=5632, rank=64, experts_per_cluster=4), 8),
]


RHT_SIGN_CASES = [(2048, 42), (1408, 42), (768, 7), (64, 0)]
LOADER_CFG = dict(hidden_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, vocab_size=32,
                  num_experts=2, num_experts_per_tok=1, moe_intermediate_size=32, shared_expert_intermediate_size=32)
LOADER_FORMATS = ("int4", "fp16", "int8")
LOADER_MODULES = ("self_attn.q_proj", "mlp.experts.1.down_proj", "mlp.experts.0.gate_proj", "mlp.shared_expert.up_proj")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("GLORCQ_REFERENCE"), required=os.environ.get("GLORCQ_REFERENCE") is None,
                    help="checkout of the unmodified reference (or set GLORCQ_REFERENCE)")
    ap.add_argument("--out", default=os.path.join(HERE, "golden.pt"))
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    torch.set_num_threads(1)   # fixed reduction order for the stored outputs

    import inference.kernels as RK                                  # noqa: E402
    from inference.quantized_linear import GLoRCQLinear, GLoRCQExperts  # noqa: E402
    from inference.moe_block import GraphCompatibleMoeBlock          # noqa: E402
    assert not RK.is_cuda_available() and not RK.is_gptq_cuda_available()

    gold = {"torch": torch.__version__, "linear": {}, "kernel": {}, "moe": {}, "experts": {}}

    # ---- kernel-level fallbacks (inference/kernels/__init__.py) ----
    d = cases.make_linear(41, 52, 192, fmt="turbo", with_lora=False)
    x = cases.make_x(42, 3, 192)
    gold["kernel"]["turbo_unpack"] = {
        "args": dict(seed=41, N=52, K=192, fmt="turbo", with_lora=False), "digest": linear_digest(d),
        "codes_u8": RK._unpack_indices_2bit(d["packed_indices"], 192).to(torch.uint8),
        "y_fallback": RK._pytorch_fallback(x.float(), d["packed_indices"], d["norms"], d["centroids"], 192),
        "y_fused": RK.turbo_dequant_matmul_fused(x, d["packed_indices"], d["norms"], None, d["centroids"], 2, 192,
                                                 precomputed_x_rot=x.float()),
        "x_seed": 42, "B": 3,
    }
    E, n_out = 3, 16
    dg = cases.make_linear(43, E * n_out, 128, fmt="turbo", with_lora=False)
    xg = cases.make_x(44, E, 128)
    gold["kernel"]["turbo_grouped"] = {
        "args": dict(seed=43, N=E * n_out, K=128, fmt="turbo", with_lora=False), "digest": linear_digest(dg),
        "y": RK.turbo_dequant_grouped_gemv_fused(xg, dg["packed_indices"], dg["norms"], dg["centroids"], n_out),
        "x_seed": 44, "E": E, "n_out": n_out,
    }
    for nm, kw in [("gptq_i8_asym", dict(seed=45, N=40, K=320, fmt="gptq", with_lora=False, int_zeros=False,
                                         signed_codes=True)),
                   ("gptq_i8_sym", dict(seed=46, N=24, K=256, fmt="gptq", with_lora=False, sym=True,
                                        signed_codes=True))]:
        d = cases.make_linear(**kw)
        x = cases.make_x(47, 2, kw["K"], torch.float32)
        lora = cases.make_x(48, 2, kw["N"], torch.float32) * 0.1
        q8 = d["qweight_int"].to(torch.int8)
        y = RK._gptq_pytorch_fallback(x, q8, d["scales"], d["zeros"], 128, d["sym"])
        gold["kernel"][nm] = {"args": kw, "digest": linear_digest(d), "y": y, "y_lora": y + lora,
                              "y_fused_half": RK.gptq_dequant_matmul_fused(x, d["qweight_int"], d["scales"],
                                                                            d["zeros"], 128, d["sym"]),
                              "x_seed": 47, "lora_seed": 48, "B": 2}

    # ---- GLoRCQLinear.forward (inference/quantized_linear.py:286-355) ----
    for name, kw, B in LINEAR_CASES:
        d = cases.make_linear(**kw)
        if d["fmt"] == "turbo":
            g = torch.Generator().manual_seed(kw["seed"] + 5000)
            q, _ = torch.linalg.qr(torch.randn(kw["K"], kw["K"], generator=g))
            d["Pi"] = q.to(torch.float16)
        lin = ref_linear(GLoRCQLinear, d)
        x = cases.make_x(kw["seed"] + 1000, B, kw["K"])
        entry = {"args": kw, "B": B, "digest": linear_digest(d), "y": lin(x)}
        if d["fmt"] == "gptq":
            entry["tile_fp16_head"] = lin._dequant_gptq()[:8, :256].clone()
            entry["tile_digest"] = digest(lin._dequant_gptq())
        if "SV" in d:
            a = (x @ d["U"])
            entry["y_pre_xU"] = lin(x, precomputed_xU=a)
        gold["linear"][name] = entry

    # ---- GraphCompatibleMoeBlock.forward, graph_mode off (inference/moe_block.py:381-436) ----
    for name, kw, N in MOE_CASES:
        blk = cases.make_moe(**kw)
        if blk["fmt"] == "turbo":
            for ex in blk["experts"] + [blk["shared_expert"]]:
                for p in ex.values():
                    p["Pi"] = None
        rb = GraphCompatibleMoeBlock(RefHFBlock(GLoRCQLinear, blk))
        rb.set_global_pool({}, {})          # builds the cluster map (see module docstring)
        x = cases.make_x(kw["seed"] + 1000, N, kw["H"]).reshape(1, N, kw["H"])
        with torch.no_grad():
            y, logits = rb(x)
        gold["moe"][name] = {"args": kw, "N": N, "digest": moe_digest(blk), "y": y, "router_logits": logits}

    # ---- GLoRCQExperts.forward (inference/quantized_linear.py:395-428) ----
    kw = dict(seed=51, H=256, I=128, E=6, top_k=2, I_shared=128, rank=16, experts_per_cluster=2)
    blk = cases.make_moe(**kw)
    ge = GLoRCQExperts(blk["E"], blk["H"], blk["I"], F.silu)
    for e, ex in enumerate(blk["experts"]):
        ge.gate_experts[e] = ref_linear(GLoRCQLinear, ex["gate_proj"])
        ge.up_experts[e] = ref_linear(GLoRCQLinear, ex["up_proj"])
        ge.down_experts[e] = ref_linear(GLoRCQLinear, ex["down_proj"])
    T = 10
    x = cases.make_x(52, T, kw["H"])
    g = torch.Generator().manual_seed(53)
    idx = torch.stack([torch.randperm(kw["E"], generator=g)[:2] for _ in range(T)])
    w = torch.rand(T, 2, generator=g).to(torch.float16)
    with torch.no_grad():
        y = ge(x, idx, w)
    gold["experts"]["experts_10"] = {"args": kw, "T": T, "digest": moe_digest(blk), "idx": idx, "w": w, "y": y,
                                      "x_seed": 52}

    # ---- Hadamard sign vectors (hadamard_rotation.py:33-47) ----
    import hadamard_rotation as RH                                   # noqa: E402
    gold["rht_signs"] = {f"{d}_{seed}": RH.generate_rht_signs(d, seed=seed, device="cpu").to(torch.int8)
                         for d, seed in RHT_SIGN_CASES}

    # ---- loader: integer decoders, SharedUCache, _load_lora_for_module (inference/model_builder.py) ----
    from inference import model_builder as RMB                       # noqa: E402
    from glorcq_b200 import synthetic                                # noqa: E402
    gold["loader"] = {}
    g = torch.Generator().manual_seed(61)
    packed = torch.randint(0, 256, (5, 6), generator=g, dtype=torch.int32).to(torch.uint8)
    gold["loader"]["unpack_int4"] = {"packed": packed, "rows": 9, "out": RMB._unpack_int4(packed, 9)}
    q = torch.randint(-127, 128, (7, 4), generator=g, dtype=torch.int32).to(torch.int8)
    sc = torch.rand(4, generator=g).half()
    gold["loader"]["dequant_intN"] = {"q": q, "scale": sc, "out8": RMB._dequant_intN(q, sc, 8),
                                      "out4": RMB._dequant_intN(q.clamp(-7, 7), sc, 4)}
    for fmt in LOADER_FORMATS:
        md, cr, _ = synthetic.make_checkpoint(LOADER_CFG, seed=62, rank=8, attn_rank=8, n_clusters=2, u_format=fmt,
                                              sv_format=fmt)
        cc = cr["config"]
        uc = RMB.SharedUCache(cr["shared_matrices"], cc["uv_bits"], device="cpu", u_bits=cc["u_bits"])
        lookup = {}
        for wtype, recs in cr["assignments"].items():
            for li, rec in enumerate(recs):
                lookup[(wtype, rec["layer"], rec["expert"])] = (rec["group_id"], wtype, li)
        mods = {}
        for name in LOADER_MODULES:
            D = md["layers"][0][name]
            N, K = D["qweight_int"].shape
            ql = GLoRCQLinear(K, N)
            ql.load_gptq(D, device="cpu")
            RMB._load_lora_for_module(ql, 0, name, lookup, uc, cr["per_expert_V"], cc["uv_bits"], "cpu",
                                      sv_bits=cc["sv_bits"])
            mods[name] = {"U": ql.U, "SV": ql.SV, "cluster_id": getattr(ql, "cluster_id", None)}
        gold["loader"][fmt] = mods

    torch.save(gold, args.out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
