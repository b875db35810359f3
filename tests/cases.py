"""Seeded synthetic inputs for the hot path, in a neutral dict-of-tensors form.

The same dicts feed the CPU oracle, the CUDA path and (in tests/golden/make_golden.py only) the
reference's own modules, so all three see identical bits.  Value distributions follow the
benchmark configurations: 2-bit codes uniform in {0..3}, per-group fp16 scale |N(0, 0.02)| and
integer fp16 zero point uniform in {0..3}, low-rank factors N(0, 0.01) fp16, activations N(0, 1).
"""

from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def make_linear(seed, N, K, rank=64, fmt="gptq", bits=2, groupsize=128, sym=False,
                int_zeros=True, with_lora=True, signed_codes=False):
    """One quantized linear layer.  fmt 'gptq': codes (N,K) int32 + scales/zeros (N,G) fp16.
    fmt 'turbo': packed (N,K/4) uint8 + norms (N,) fp32 + centroids (4,) fp32 (sorted)."""
    g = _gen(seed)
    d = {"fmt": fmt, "N": N, "K": K, "rank": rank if with_lora else 0}
    if fmt == "gptq":
        G = (K + groupsize - 1) // groupsize
        if signed_codes:      # the reference's own kernel tests draw codes in [-2, 2]
            q = torch.randint(-2, 3, (N, K), generator=g, dtype=torch.int32)
        else:
            q = torch.randint(0, 2 ** bits, (N, K), generator=g, dtype=torch.int32)
        scales = (torch.randn(N, G, generator=g) * 0.02).abs().to(torch.float16)
        if sym:
            zeros = torch.zeros(N, G, dtype=torch.float16)
        elif int_zeros:
            zeros = torch.randint(0, 2 ** bits, (N, G), generator=g).to(torch.float16)
        else:
            zeros = (torch.randn(N, G, generator=g) * 0.5).to(torch.float16)
        d.update(qweight_int=q, scales=scales, zeros=zeros, bits=bits, groupsize=groupsize, sym=sym)
    elif fmt == "turbo":
        assert K % 4 == 0
        packed = torch.randint(0, 256, (N, K // 4), generator=g, dtype=torch.int32).to(torch.uint8)
        norms = torch.randn(N, generator=g).abs() + 0.1
        centroids = torch.sort(torch.randn(4, generator=g))[0] * 0.05
        d.update(packed_indices=packed, norms=norms.float(), centroids=centroids.float(), bits=2)
    else:
        raise ValueError(fmt)
    if with_lora:
        d["U"] = (torch.randn(K, rank, generator=g) * 0.01).to(torch.float16)
        d["SV"] = (torch.randn(N, rank, generator=g) * 0.01).to(torch.float16)
    return d


def make_x(seed, B, K, dtype=torch.float16):
    return torch.randn(B, K, generator=_gen(seed)).to(dtype)


def make_moe(seed, H, I, E, top_k, I_shared=0, rank=64, experts_per_cluster=4, fmt="gptq",
             bits=2, groupsize=128, norm_topk_prob=False, n_clusters=None, router_std=0.02):
    """A Qwen2-MoE shaped block.  U is shared by clusters: expert e of projection p belongs to
    cluster (p, e // experts_per_cluster), or to a seeded random one of `n_clusters` if given."""
    g = _gen(seed)
    blk = {"H": H, "I": I, "E": E, "top_k": top_k, "I_shared": I_shared, "rank": rank,
           "norm_topk_prob": norm_topk_prob, "fmt": fmt}
    blk["gate_weight"] = (torch.randn(E, H, generator=g) * router_std).to(torch.float16)
    if n_clusters is None:
        nclu = (E + experts_per_cluster - 1) // experts_per_cluster
        assign = {p: [e // experts_per_cluster for e in range(E)] for p in ("gate_proj", "up_proj", "down_proj")}
    else:
        nclu = n_clusters
        assign = {p: torch.randint(0, nclu, (E,), generator=g).tolist() for p in ("gate_proj", "up_proj", "down_proj")}
    dims = {"gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
    sharedU = {}
    for p, (n, k) in dims.items():
        for c in range(nclu):
            sharedU[(p, c)] = (torch.randn(k, rank, generator=g) * 0.01).to(torch.float16)
    experts = []
    for e in range(E):
        ex = {}
        for pi, (p, (n, k)) in enumerate(dims.items()):
            lin = make_linear(seed * 100003 + e * 7 + pi + 1, n, k, rank, fmt, bits, groupsize)
            cid = (p, assign[p][e])
            lin["U"] = sharedU[cid]
            lin["cluster_id"] = cid
            ex[p] = lin
        experts.append(ex)
    blk["experts"] = experts
    blk["sharedU"] = sharedU
    if I_shared:
        sdims = {"gate_proj": (I_shared, H), "up_proj": (I_shared, H), "down_proj": (H, I_shared)}
        blk["shared_expert"] = {p: make_linear(seed * 100003 + 900001 + pi, n, k, rank, fmt, bits, groupsize)
                                for pi, (p, (n, k)) in enumerate(sdims.items())}
        blk["shared_gate_weight"] = (torch.randn(1, H, generator=g) * 0.02).to(torch.float16)
    return blk


# --------------------------------------------------------------------------------------
# Conversions to the oracle's structures
# --------------------------------------------------------------------------------------
def to_oracle_linear(d):
    from oracle import glorcq_oracle as O
    kw = dict(in_features=d["K"], out_features=d["N"], quant_type=d["fmt"],
              U=d.get("U"), SV=d.get("SV"), cluster_id=d.get("cluster_id"))
    if d["fmt"] == "gptq":
        kw.update(qweight_int=d["qweight_int"], scales=d["scales"], zeros=d["zeros"],
                  gptq_bits=d["bits"], gptq_groupsize=d["groupsize"], gptq_sym=d["sym"])
    else:
        kw.update(packed_indices=d["packed_indices"], norms=d["norms"], centroids=d["centroids"],
                  Pi=d.get("Pi"))
        if d.get("rht_seed") is not None:     # rotation_type "hadamard": signs from the layer's seed
            kw.update(rht_signs=O.generate_rht_signs(d["K"], d["rht_seed"]))
    return O.QuantLinear(**kw)


def to_oracle_moe(blk):
    from oracle import glorcq_oracle as O
    experts = [O.Expert(*(to_oracle_linear(ex[p]) for p in ("gate_proj", "up_proj", "down_proj")))
               for ex in blk["experts"]]
    shared = None
    if blk.get("shared_expert") is not None:
        shared = O.Expert(*(to_oracle_linear(blk["shared_expert"][p]) for p in ("gate_proj", "up_proj", "down_proj")))
    return O.MoeBlock(num_experts=blk["E"], top_k=blk["top_k"], norm_topk_prob=blk["norm_topk_prob"],
                      gate_weight=blk["gate_weight"], experts=experts, shared_expert=shared,
                      shared_gate_weight=blk.get("shared_gate_weight"))


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().reshape(-1)
    b = b.double().reshape(-1)
    return float((a - b).norm() / (b.norm() + 1e-30))


# --------------------------------------------------------------------------------------
# Conversions to the CUDA package's modules (need a GPU)
# --------------------------------------------------------------------------------------
class FixedRotationCache:
    """Hands a given rotation and codebook to GLoRCQLinear.load_turbo (the reference builds them
    with a third-party package that is not part of this repository)."""

    def __init__(self, Pi, centroids):
        self._pi, self._c = Pi, centroids

    def register(self, dim, bits, seed=42):
        pass

    def get_pi(self, dim, bits, seed=42):
        return self._pi

    def get_centroids(self, dim, bits, seed=42):
        return self._c


def to_b200_linear(d, device="cuda", shared_u=None):
    """Build glorcq_b200's GLoRCQLinear from a case dict.  shared_u: dict id(U cpu tensor) -> device
    tensor, so that layers of one cluster share one device U."""
    from glorcq_b200.quantized_linear import GLoRCQLinear
    lin = GLoRCQLinear(d["K"], d["N"])
    if d["fmt"] == "gptq":
        lin.load_gptq({"qweight_int": d["qweight_int"], "scales": d["scales"], "zeros": d["zeros"],
                       "bits": d["bits"], "groupsize": d["groupsize"], "sym": d["sym"]}, device=device)
    else:
        Pi = d.get("Pi")
        if Pi is None:
            Pi = torch.eye(d["K"], dtype=torch.float16)
        lin.load_turbo({"packed_indices": d["packed_indices"], "norms": d["norms"], "bits": 2,
                        "dim": d["K"], "seed": 42},
                       FixedRotationCache(Pi.to(device), d["centroids"].to(device)), device=device)
        if d.get("rht_seed") is not None:
            from glorcq_b200.hadamard_rotation import generate_rht_signs
            lin._rht_signs = generate_rht_signs(d["K"], seed=d["rht_seed"], device=device)
    if "SV" in d:
        U = d["U"]
        if shared_u is not None:
            if id(U) not in shared_u:
                shared_u[id(U)] = U.to(device)
            U = shared_u[id(U)]
        else:
            U = U.to(device)
        lin.load_sv(U, d["SV"], device=device)
        lin.cluster_id = d.get("cluster_id")
    return lin


class _B200Expert(torch.nn.Module):
    def __init__(self, ex, device, shared_u):
        super().__init__()
        self.gate_proj = to_b200_linear(ex["gate_proj"], device, shared_u)
        self.up_proj = to_b200_linear(ex["up_proj"], device, shared_u)
        self.down_proj = to_b200_linear(ex["down_proj"], device, shared_u)
        self.act_fn = torch.nn.functional.silu


class _HFBlock:
    """Stand-in with the attribute names of a transformers-4.45 Qwen2MoeSparseMoeBlock."""


def to_b200_moe(blk, device="cuda"):
    """glorcq_b200's GraphCompatibleMoeBlock from a case dict."""
    from glorcq_b200.moe_block import GraphCompatibleMoeBlock
    shared_u = {}
    hf = _HFBlock()
    hf.num_experts, hf.top_k, hf.norm_topk_prob = blk["E"], blk["top_k"], blk["norm_topk_prob"]
    hf.gate = torch.nn.Linear(blk["H"], blk["E"], bias=False).half().to(device)
    hf.gate.weight.data.copy_(blk["gate_weight"])
    hf.experts = torch.nn.ModuleList([_B200Expert(ex, device, shared_u) for ex in blk["experts"]])
    if blk.get("shared_expert") is not None:
        hf.shared_expert = _B200Expert(blk["shared_expert"], device, shared_u)
        hf.shared_expert_gate = torch.nn.Linear(blk["H"], 1, bias=False).half().to(device)
        hf.shared_expert_gate.weight.data.copy_(blk["shared_gate_weight"])
    else:
        hf.shared_expert, hf.shared_expert_gate = None, None
    return GraphCompatibleMoeBlock(hf)
