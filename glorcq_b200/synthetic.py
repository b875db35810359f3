"""Seeded synthetic Qwen2-MoE-shaped blocks built directly on the device (benchmarks, smoke test).

Value distributions follow the benchmark configurations: 2-bit codes uniform in {0..3}, fp16 scale
|N(0, 0.02)| and integer zero point in {0..3} per group of 128 input channels, low-rank factors
N(0, 0.01) with U shared by clusters of experts, router weights N(0, 0.02)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .moe_block import GraphCompatibleMoeBlock
from .quantized_linear import GLoRCQLinear


def _linear(gen, N, K, rank, U, device, bits=2, groupsize=128):
    G = (K + groupsize - 1) // groupsize
    lin = GLoRCQLinear(K, N)
    lin.load_gptq({
        "qweight_int": torch.randint(0, 2 ** bits, (N, K), generator=gen, device=device, dtype=torch.int32),
        "scales": (torch.randn(N, G, generator=gen, device=device) * 0.02).abs().half(),
        "zeros": torch.randint(0, 2 ** bits, (N, G), generator=gen, device=device).half(),
        "bits": bits, "groupsize": groupsize, "sym": False}, device=device, check_range=False)
    if rank > 0:
        lin.load_sv(U, (torch.randn(N, rank, generator=gen, device=device) * 0.01).half(), device=device)
    return lin


class _Expert(nn.Module):
    def __init__(self, gen, H, I, rank, Ug, Uu, Ud, device):
        super().__init__()
        self.gate_proj = _linear(gen, I, H, rank, Ug, device)
        self.up_proj = _linear(gen, I, H, rank, Uu, device)
        self.down_proj = _linear(gen, H, I, rank, Ud, device)
        self.act_fn = F.silu


class _SparseBlock:
    pass


def make_moe_block(seed, device, H=2048, I=1408, E=60, top_k=4, I_shared=5632, rank=64, experts_per_cluster=4,
                   norm_topk_prob=False, release_linear_tiles=True, pools=None, n_clusters=None,
                   ep_rank=0, ep_world=1, ep_group=None):
    """One MoE block of the Qwen1.5-MoE shape.  `pools` (dict) lets several blocks share the cluster U
    factors across layers, as the cross-layer clustering of the reference does.  With ep_world > 1
    only the experts of rank ep_rank are materialised; every tensor is drawn from its own seeded
    generator, so all ranks see the same router, shared expert and (for the experts they hold) weights."""
    def generator(index):
        g = torch.Generator(device=device)
        g.manual_seed(seed * 100003 + index)
        return g
    gen = generator(0)
    pools = {} if pools is None else pools
    kinds = {"gate": 1, "up": 2, "down": 3, "sgate": 4, "sup": 5, "sdown": 6}

    def U(kind, c, K):
        key = (kind, c)
        if key not in pools:
            g = torch.Generator(device=device)
            g.manual_seed(7919 * kinds[kind] + int(c))        # the pool is shared by blocks: not seeded per block
            pools[key] = (torch.randn(K, rank, generator=g, device=device) * 0.01).half()
        return pools[key]

    if n_clusters:   # cross-layer clusters assigned at random per (expert, projection)
        assign = torch.randint(0, n_clusters, (3, E), generator=gen, device=device).tolist()
    else:
        assign = [[e // experts_per_cluster for e in range(E)]] * 3

    hf = _SparseBlock()
    hf.num_experts, hf.top_k, hf.norm_topk_prob = E, top_k, norm_topk_prob
    hf.gate = nn.Linear(H, E, bias=False).half().to(device)
    hf.gate.weight.data.copy_((torch.randn(E, H, generator=gen, device=device) * 0.02).half())
    hf.experts = [
        _Expert(generator(1 + e), H, I, rank, U("gate", assign[0][e], H), U("up", assign[1][e], H),
                U("down", assign[2][e], I), device) if e % ep_world == ep_rank else None for e in range(E)]
    if I_shared:
        hf.shared_expert = _Expert(generator(100001), H, I_shared, rank, U("sgate", seed, H), U("sup", seed, H),
                                   U("sdown", seed, I_shared), device)
        hf.shared_expert_gate = nn.Linear(H, 1, bias=False).half().to(device)
        hf.shared_expert_gate.weight.data.copy_((torch.randn(1, H, generator=gen, device=device) * 0.02).half())
    else:
        hf.shared_expert, hf.shared_expert_gate = None, None
    blk = GraphCompatibleMoeBlock(hf)
    if ep_world > 1:
        blk.set_expert_parallel(ep_rank, ep_world, ep_group)
    blk.prepare(device, release_linear_tiles=release_linear_tiles)
    return blk


def block_bytes_per_token(H=2048, I=1408, top_k=4, I_shared=5632, rank=64, E=60, groupsize=128, bits=2):
    """Algorithmic bytes one decode token moves through a block: routed experts and the shared expert
    (codes, scales and zeros, SV, U once per projection), the router, activations in and out."""
    def lin(N, K):
        return N * K * bits // 8 + 2 * N * ((K + groupsize - 1) // groupsize) * 2 + K * rank * 2 + N * rank * 2 + K * 2 + N * 2
    routed = top_k * (2 * lin(I, H) + lin(H, I))
    shared = (2 * lin(I_shared, H) + lin(H, I_shared)) if I_shared else 0
    router = (E + (1 if I_shared else 0)) * H * 2
    return routed + shared + router


# ---- synthetic checkpoints in the reference's on-disk format ---------------------------------------
def make_checkpoint(hf_config: dict, seed=0, qbit=2, attn_bits=4, rank=64, attn_rank=None, groupsize=128,
                    n_clusters=8, u_format="int4", sv_format="int4", uv_bits=8):
    """Seeded random model in the format ``load_glorcq_model`` reads (CPU tensors):
    returns (model_data, cross_layer_info, dense) = the contents of glorcq_model.pt,
    cross_layer_info.pt and dense_weights.pt.  Codes uniform, scales |N(0, 0.02)|, integer zero points,
    low-rank factors N(0, 0.01) quantised to `u_format` / `sv_format` ("fp16", "int4", "int8"), cluster
    of every (layer, expert, projection) drawn at random from `n_clusters`; attention projections carry
    `attn_bits` codes and their own clusters (expert index -1); the shared expert has no low-rank term,
    as in the reference's loader."""
    from .model_builder import _pack_int4
    g = torch.Generator()
    g.manual_seed(seed)
    c = hf_config
    H, L = c["hidden_size"], c["num_hidden_layers"]
    nh, nkv = c["num_attention_heads"], c.get("num_key_value_heads") or c["num_attention_heads"]
    hd = c.get("head_dim") or H // nh
    E = c.get("num_experts", c.get("num_local_experts", 0))
    mixtral = "num_local_experts" in c
    I = c.get("moe_intermediate_size", c.get("intermediate_size"))
    Ish = c.get("shared_expert_intermediate_size", 0)
    mp = "block_sparse_moe" if mixtral else "mlp"
    names = ("w1", "w3", "w2") if mixtral else ("gate_proj", "up_proj", "down_proj")
    attn_rank = attn_rank or rank

    def codes(N, K, bits):
        G = (K + groupsize - 1) // groupsize
        return {"qweight_int": torch.randint(0, 2 ** bits, (N, K), generator=g, dtype=torch.int32),
                "scales": (torch.randn(N, G, generator=g) * 0.02).abs().half(),
                "zeros": torch.randint(0, 2 ** bits, (N, G), generator=g).half(),
                "bits": bits, "groupsize": groupsize, "sym": False}

    def quant(M, fmt, prefix):
        """(rows, r) fp32 factor -> stored form with a per-column scale."""
        if fmt == "fp16":
            return {f"{prefix}_fp16": M.half()}
        bits = 4 if fmt == "int4" else uv_bits
        maxval = 2 ** (bits - 1) - 1
        scale = M.abs().amax(0).clamp_min(1e-8)
        q = torch.round(M / scale * maxval).clamp(-maxval, maxval).to(torch.int8)
        if fmt == "int4":
            return {f"{prefix}_int4_packed": _pack_int4(q), f"{prefix}_scale": scale.half(),
                    f"{prefix}_orig_rows": torch.tensor(M.shape[0])}
        return {f"{prefix}_int8": q, f"{prefix}_scale": scale.half()}

    layers, dense = {}, {}
    assignments = {w: [] for w in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")}
    per_v = {w: [] for w in assignments}
    shapes = {"q_proj": (nh * hd, H), "k_proj": (nkv * hd, H), "v_proj": (nkv * hd, H), "o_proj": (H, nh * hd),
              "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
    wt_of = dict(zip(names, ("gate_proj", "up_proj", "down_proj")))

    def add(layer, expert, wtype, r):
        gid = int(torch.randint(0, n_clusters, (1,), generator=g))
        assignments[wtype].append({"layer": layer, "expert": expert, "group_id": gid})
        per_v[wtype].append(quant(torch.randn(shapes[wtype][0], r, generator=g) * 0.01, sv_format, "SV"))

    for l in range(L):
        mods = {}
        for w in ("q_proj", "k_proj", "v_proj", "o_proj"):
            mods[f"self_attn.{w}"] = codes(*shapes[w], attn_bits)
            add(l, -1, w, attn_rank)
        if E:
            for e in range(E):
                for nm in names:
                    mods[f"{mp}.experts.{e}.{nm}"] = codes(*shapes[wt_of[nm]], qbit)
                    add(l, e, wt_of[nm], rank)
            if Ish:
                mods[f"{mp}.shared_expert.gate_proj"] = codes(Ish, H, qbit)
                mods[f"{mp}.shared_expert.up_proj"] = codes(Ish, H, qbit)
                mods[f"{mp}.shared_expert.down_proj"] = codes(H, Ish, qbit)
                dense[f"model.layers.{l}.{mp}.shared_expert_gate.weight"] = (torch.randn(1, H, generator=g) * 0.02).half()
            dense[f"model.layers.{l}.{mp}.gate.weight"] = (torch.randn(E, H, generator=g) * 0.02).half()
        else:
            for nm in ("gate_proj", "up_proj", "down_proj"):
                mods[f"mlp.{nm}"] = codes(*shapes[nm], qbit)
                add(l, -1, nm, rank)
        layers[l] = mods
        dense[f"model.layers.{l}.input_layernorm.weight"] = torch.ones(H).half()
        dense[f"model.layers.{l}.post_attention_layernorm.weight"] = torch.ones(H).half()
    shared = {}
    for w, (N, K) in shapes.items():
        r = attn_rank if w.endswith(("q_proj", "k_proj", "v_proj", "o_proj")) else rank
        shared[w] = {gid: quant(torch.randn(K, r, generator=g) * 0.01, u_format, "U") for gid in range(n_clusters)}
    dense["model.embed_tokens.weight"] = (torch.randn(c["vocab_size"], H, generator=g) * 0.02).half()
    dense["lm_head.weight"] = (torch.randn(c["vocab_size"], H, generator=g) * 0.02).half()
    dense["model.norm.weight"] = torch.ones(H).half()
    model_data = {"model_config": {"model_path": "synthetic", "qbit": qbit, "rank": rank, "groupsize": groupsize,
                                   "n_iter": 0, "use_turboquant": False, "act_alpha": 0.0, "uv_bits": uv_bits,
                                   "rotation_type": "qr"},
                  "layers": layers}
    cross = {"config": {"uv_bits": uv_bits, "u_bits": 4 if u_format == "int4" else uv_bits,
                        "sv_bits": 4 if sv_format == "int4" else uv_bits},
             "assignments": assignments, "shared_matrices": shared, "per_expert_V": per_v}
    return model_data, cross, dense


def write_checkpoint(path, hf_config: dict, **kw):
    """make_checkpoint written as config.json, glorcq_model.pt, cross_layer_info.pt and dense_weights.pt."""
    import json
    import os
    os.makedirs(path, exist_ok=True)
    model_data, cross, dense = make_checkpoint(hf_config, **kw)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf_config, f)
    torch.save(model_data, os.path.join(path, "glorcq_model.pt"))
    torch.save(cross, os.path.join(path, "cross_layer_info.pt"))
    torch.save(dense, os.path.join(path, "dense_weights.pt"))
    return model_data, cross, dense


def make_decoder(hf_config: dict, device, seed=0, qbit=2, attn_bits=4, rank=64, attn_rank=64, groupsize=128,
                 n_clusters=128, ep_rank=0, ep_world=1, ep_group=None, peer_exchange_max_tokens=0):
    """A whole random decoder of the given shape built directly on the device (no files: the int32 code
    tensors of the on-disk format would be 4 bytes per weight).  Same distributions and cluster rule as
    make_checkpoint: every (layer, expert, projection) draws its U cluster from `n_clusters`; attention
    projections are `attn_bits` codes with their own clusters; the shared expert has no low-rank term.
    Every module draws from its own seeded generator, so with ep_world > 1 (expert e of every layer on rank
    e % ep_world, the others not materialised) all ranks hold identical replicated tensors and identical
    copies of the experts they share with an unsharded build."""
    from .decoder import GLoRCQDecoder
    c = hf_config
    H, L = c["hidden_size"], c["num_hidden_layers"]
    nh, nkv = c["num_attention_heads"], c.get("num_key_value_heads") or c["num_attention_heads"]
    hd = c.get("head_dim") or H // nh
    E = c.get("num_experts", c.get("num_local_experts", 0))
    mixtral = "num_local_experts" in c
    I = c.get("moe_intermediate_size", c.get("intermediate_size"))
    Ish = c.get("shared_expert_intermediate_size", 0)
    mp = "block_sparse_moe" if mixtral else "mlp"
    names = ("w1", "w3", "w2") if mixtral else ("gate_proj", "up_proj", "down_proj")
    wt_of = dict(zip(names, ("gate_proj", "up_proj", "down_proj")))
    shapes = {"q_proj": (nh * hd, H), "k_proj": (nkv * hd, H), "v_proj": (nkv * hd, H), "o_proj": (H, nh * hd),
              "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
    wtypes = list(shapes)
    pools = {}

    def generator(*key):
        g = torch.Generator(device=device)
        g.manual_seed((seed * 1000003 + sum((i + 1) * 7919 ** (n + 1) * int(k) for n, (i, k) in enumerate(enumerate(key))))
                      % (2 ** 62))
        return g

    def U(wtype, r, gen):
        gid = int(torch.randint(0, n_clusters, (1,), generator=gen, device=device))
        if (wtype, gid) not in pools:     # the pool is shared by every layer: seeded by the cluster alone
            pools[(wtype, gid)] = (torch.randn(shapes[wtype][1], r, generator=generator(9, wtypes.index(wtype), gid),
                                               device=device) * 0.01).half()
        return pools[(wtype, gid)]

    layers, dense = {}, {}
    for l in range(L):
        mods = {}
        for wi, w in enumerate(("q_proj", "k_proj", "v_proj", "o_proj")):
            gen = generator(1, l, wi)
            mods[f"self_attn.{w}"] = _linear(gen, *shapes[w], attn_rank, U(w, attn_rank, gen), device, bits=attn_bits,
                                             groupsize=groupsize)
        if E:
            for e in range(E):
                if e % ep_world != ep_rank:
                    continue
                for ni, nm in enumerate(names):
                    w = wt_of[nm]
                    gen = generator(2, l, e, ni)
                    mods[f"{mp}.experts.{e}.{nm}"] = _linear(gen, *shapes[w], rank, U(w, rank, gen), device, bits=qbit,
                                                             groupsize=groupsize)
            gen = generator(3, l)
            if Ish:
                mods[f"{mp}.shared_expert.gate_proj"] = _linear(gen, Ish, H, 0, None, device, bits=qbit, groupsize=groupsize)
                mods[f"{mp}.shared_expert.up_proj"] = _linear(gen, Ish, H, 0, None, device, bits=qbit, groupsize=groupsize)
                mods[f"{mp}.shared_expert.down_proj"] = _linear(gen, H, Ish, 0, None, device, bits=qbit, groupsize=groupsize)
                dense[f"model.layers.{l}.{mp}.shared_expert_gate.weight"] = (torch.randn(1, H, generator=gen, device=device) * 0.02).half()
            dense[f"model.layers.{l}.{mp}.gate.weight"] = (torch.randn(E, H, generator=gen, device=device) * 0.02).half()
        else:
            for ni, nm in enumerate(("gate_proj", "up_proj", "down_proj")):
                gen = generator(4, l, ni)
                mods[f"mlp.{nm}"] = _linear(gen, *shapes[nm], rank, U(nm, rank, gen), device, bits=qbit, groupsize=groupsize)
        layers[l] = mods
        dense[f"model.layers.{l}.input_layernorm.weight"] = torch.ones(H, device=device).half()
        dense[f"model.layers.{l}.post_attention_layernorm.weight"] = torch.ones(H, device=device).half()
    gen = generator(5)
    dense["model.embed_tokens.weight"] = (torch.randn(c["vocab_size"], H, generator=gen, device=device) * 0.02).half()
    dense["lm_head.weight"] = (torch.randn(c["vocab_size"], H, generator=gen, device=device) * 0.02).half()
    dense["model.norm.weight"] = torch.ones(H, device=device).half()
    return GLoRCQDecoder(hf_config, layers, dense=dense, device=device, ep_rank=ep_rank, ep_world=ep_world,
                         ep_group=ep_group, peer_exchange_max_tokens=peer_exchange_max_tokens)


QWEN15_MOE_A27B = dict(hidden_size=2048, num_hidden_layers=24, num_attention_heads=16, num_key_value_heads=16,
                       vocab_size=151936, num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408,
                       shared_expert_intermediate_size=5632, norm_topk_prob=False, rms_norm_eps=1e-6,
                       rope_theta=1000000.0, max_position_embeddings=8192)

MIXTRAL_8X7B = dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                    vocab_size=32000, num_local_experts=8, num_experts_per_tok=2, intermediate_size=14336,
                    rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=8192)
QWEN3_30B_A3B = dict(hidden_size=2048, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                     vocab_size=151936, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                     norm_topk_prob=True, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=8192)
