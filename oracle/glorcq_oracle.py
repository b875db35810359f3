"""CPU restatement of the GLoRCQ real-quant inference hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the CUDA path is compared against.  Nothing that ships
(``glorcq_b200``) imports it; only the tests, the smoke check and the CPU-baseline leg of
the benchmark do.  It restates, in plain torch-on-CPU tensor arithmetic, what the reference
computes when neither of its CUDA extensions is present:

* 2-bit codebook ("turbo") weights       -- inference/kernels/__init__.py:113-146,
                                            inference/quantized_linear.py:72-146
* integer-code + scale/zero ("gptq")      -- inference/quantized_linear.py:271-284 (fp16 tile),
                                            inference/kernels/__init__.py:149-178 (fp32 tile)
* quantized linear + low-rank correction  -- inference/quantized_linear.py:286-355
* grouped GEMV over experts               -- inference/kernels/__init__.py:242-278
* the MoE block (router, shared U, decode and sparse dispatch, shared expert)
                                          -- inference/moe_block.py:381-478, 592-602, 704-740
* the fused-experts adapter               -- inference/quantized_linear.py:395-428

Parity is pinned: ``tests/golden/make_golden.py`` imports the reference itself (unmodified)
and stores its inputs and outputs; ``tests/test_oracle_golden.py`` checks this module
against those vectors.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# Code unpacking and weight tiles
# --------------------------------------------------------------------------------------
def unpack_codes_2bit(packed: torch.Tensor, K: int) -> torch.Tensor:
    """(N, K/4) uint8 -> (N, K) int64.  Code j of a byte sits in bits [2j, 2j+1]
    (inference/kernels/__init__.py:113-118)."""
    p = packed.to(torch.int64)
    cols = [(p >> s) & 3 for s in (0, 2, 4, 6)]
    codes = torch.stack(cols, dim=-1).reshape(packed.shape[0], -1)
    return codes[:, :K]


def unpack_codes(packed: torch.Tensor, bits: int, K: int) -> torch.Tensor:
    """General unpack (inference/quantized_linear.py:115-146): 1, 2 or (3..4 -> 4) bits per code,
    low bits first; more than 4 bits means one code per byte."""
    if bits == 1:
        per, width = 8, 1
    elif bits == 2:
        per, width = 4, 2
    elif bits <= 4:
        per, width = 2, 4
    else:
        return packed.to(torch.int64)
    p = packed.to(torch.int64)
    cols = [(p >> (i * width)) & ((1 << width) - 1) for i in range(per)]
    codes = torch.stack(cols, dim=-1).reshape(*packed.shape[:-1], -1)
    return codes[..., :K]


def turbo_tile(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor, K: int) -> torch.Tensor:
    """fp32 weight tile W[n,k] = centroids[idx[n,k]] * norms[n] (inference/kernels/__init__.py:142-143)."""
    idx = unpack_codes_2bit(packed, K)
    return centroids.float()[idx] * norms.float()[:, None]


def gptq_tile_fp16(q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, groupsize: int,
                   sym: bool = False) -> torch.Tensor:
    """fp16 weight tile, every step in fp16 as the reference layer does
    (inference/quantized_linear.py:271-284): fp16((fp16(q) - z) * s)."""
    N, K = q.shape
    W = torch.zeros(N, K, dtype=torch.float16)
    for g in range(scales.shape[1]):
        a, b = g * groupsize, min((g + 1) * groupsize, K)
        qs = q[:, a:b].to(torch.float16)
        if sym:
            W[:, a:b] = qs * scales[:, g:g + 1]
        else:
            W[:, a:b] = (qs - zeros[:, g:g + 1]) * scales[:, g:g + 1]
    return W


def gptq_tile_fp32(q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, groupsize: int,
                   sym: bool = False) -> torch.Tensor:
    """fp32 weight tile (q - z) * s with q, z, s widened first (inference/kernels/__init__.py:168-176)."""
    N, K = q.shape
    G = scales.shape[1]
    gidx = torch.arange(K) // groupsize
    gidx = gidx.clamp(max=G - 1)
    s = scales.float()[:, gidx]
    if sym:
        return q.float() * s
    return (q.float() - zeros.float()[:, gidx]) * s


# --------------------------------------------------------------------------------------
# Kernel-level functions (what the two native modules compute)
# --------------------------------------------------------------------------------------
def turbo_matmul(x_rot: torch.Tensor, packed: torch.Tensor, norms: torch.Tensor,
                 centroids: torch.Tensor) -> torch.Tensor:
    """y = x_rot @ W.T in fp32, W from :func:`turbo_tile` (inference/kernels/__init__.py:121-146).
    Returns fp32 (B, N); the native kernel rounds this to fp16 when it stores."""
    K = x_rot.shape[1]
    return x_rot.float() @ turbo_tile(packed, norms, centroids, K).T


def turbo_grouped_gemv(x_grouped: torch.Tensor, packed_cat: torch.Tensor, norms_cat: torch.Tensor,
                       centroids: torch.Tensor, n_out: int) -> torch.Tensor:
    """E independent GEMVs, expert e uses x_grouped[e] and rows [e*n_out, (e+1)*n_out);
    each result rounded to fp16 (inference/kernels/__init__.py:268-278).  Returns (E*n_out,) fp16."""
    E = x_grouped.shape[0]
    outs = []
    for e in range(E):
        rows = slice(e * n_out, (e + 1) * n_out)
        y = turbo_matmul(x_grouped[e:e + 1], packed_cat[rows], norms_cat[rows], centroids)
        outs.append(y.to(torch.float16).reshape(-1))
    if not outs:
        return torch.empty(0, dtype=torch.float16)
    return torch.cat(outs)


def gptq_matmul(x: torch.Tensor, q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                groupsize: int, sym: bool = False, lora_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 y = x @ ((q - z) * s).T (+ lora_out) (inference/kernels/__init__.py:149-178, 338-344)."""
    y = x.float() @ gptq_tile_fp32(q, scales, zeros, groupsize, sym).T
    if lora_out is not None and lora_out.numel() > 0:
        y = y + lora_out.float()
    return y


# --------------------------------------------------------------------------------------
# Randomized Hadamard rotation (hadamard_rotation.py:33-65)
# --------------------------------------------------------------------------------------
def generate_rht_signs(d: int, seed: int = 42) -> torch.Tensor:
    """(d,) float32 of +-1 from a CPU generator seeded with `seed` (hadamard_rotation.py:33-47)."""
    rng = torch.Generator(device="cpu")
    rng.manual_seed(seed)
    return (torch.randint(0, 2, (d,), generator=rng) * 2 - 1).float()


def sylvester_hadamard(n: int) -> torch.Tensor:
    """H_n for n a power of two, by the Sylvester construction: H_1 = [1], H_2n = [[H, H], [H, -H]]."""
    assert n > 0 and n & (n - 1) == 0
    H = torch.ones(1, 1, dtype=torch.float64)
    while H.shape[0] < n:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return H


def rht_forward(x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """y = (1/sqrt(d)) H diag(signs) x over the last dimension (hadamard_rotation.py:50-65).

    The reference delegates H to the third-party fast-hadamard-transform 1.1.0, which is absent here
    (parity unpinned for it).  Restated from its published behaviour: the Walsh-Hadamard transform in
    natural (Sylvester) order; a dimension that is not a power of two is zero-padded to the next one
    and the result is cut back to d, while the scale stays 1/sqrt(d) as the caller passes it.
    """
    d = x.shape[-1]
    n = 1 << max(0, (d - 1).bit_length())
    xs = (x.double() * signs.double())
    if n != d:
        xs = torch.nn.functional.pad(xs, (0, n - d))
    y = xs @ sylvester_hadamard(n).T
    return (y[..., :d] * (1.0 / d ** 0.5)).to(x.dtype)


# --------------------------------------------------------------------------------------
# Quantized linear layer
# --------------------------------------------------------------------------------------
@dataclass
class QuantLinear:
    """Tensors of one quantized linear layer, named as the reference layer names them
    (inference/quantized_linear.py:162-193)."""
    in_features: int
    out_features: int
    quant_type: str                              # "gptq" | "turbo"
    # gptq
    qweight_int: Optional[torch.Tensor] = None   # (N, K) int32
    scales: Optional[torch.Tensor] = None        # (N, G) fp16
    zeros: Optional[torch.Tensor] = None         # (N, G) fp16
    gptq_bits: int = 2
    gptq_groupsize: int = 128
    gptq_sym: bool = False
    # turbo
    packed_indices: Optional[torch.Tensor] = None  # (N, K/4) uint8
    norms: Optional[torch.Tensor] = None           # (N,) fp32
    centroids: Optional[torch.Tensor] = None       # (4,) fp32
    Pi: Optional[torch.Tensor] = None              # (K, K) fp16 rotation, or None = identity
    rht_signs: Optional[torch.Tensor] = None       # (K,) +-1: randomized Hadamard rotation instead of Pi
    # low-rank correction
    U: Optional[torch.Tensor] = None               # (K, r) fp16, shared by a cluster
    SV: Optional[torch.Tensor] = None              # (N, r) fp16, per layer
    cluster_id: Optional[Tuple] = None
    bias: Optional[torch.Tensor] = None


def linear_forward(p: QuantLinear, x: torch.Tensor, precomputed_xU: Optional[torch.Tensor] = None,
                   x_rot_half: bool = False) -> torch.Tensor:
    """GLoRCQLinear.forward on the route without native kernels
    (inference/quantized_linear.py:286-355).

    gptq : W = fp16 tile, y = x @ W.T in the activation dtype.
    turbo: x_rot = x.float() @ Pi.float().T, fp32 product with the fp32 tile, result cast to
           fp16 (inference/quantized_linear.py:97-112).  ``x_rot_half=True`` rounds x_rot to fp16
           first, which is what the route with the native kernel does
           (inference/kernels/__init__.py:212).
    then y += (precomputed_xU or x @ U) @ SV.T, then bias.
    """
    shape = x.shape
    x2 = x.reshape(-1, p.in_features)
    if p.quant_type == "gptq":
        W = gptq_tile_fp16(p.qweight_int, p.scales, p.zeros, p.gptq_groupsize, p.gptq_sym)
        y = x2 @ W.to(x2.dtype).T
    elif p.quant_type == "turbo":
        if p.rht_signs is not None:          # inference/moe_block.py:349-351, 523-525
            xr = rht_forward(x2.float(), p.rht_signs).to(torch.float16).float()
        else:
            xr = x2.float() if p.Pi is None else x2.float() @ p.Pi.float().T
        if x_rot_half:
            xr = xr.to(torch.float16).float()
        y = turbo_matmul(xr, p.packed_indices, p.norms, p.centroids).to(torch.float16)
    else:
        raise RuntimeError(f"Unknown quant_type: {p.quant_type}")
    if p.SV is not None:
        a = precomputed_xU if precomputed_xU is not None else x2 @ p.U
        y = y + a @ p.SV.T
    if p.bias is not None:
        y = y + p.bias
    if len(shape) > 2:
        y = y.reshape(*shape[:-1], p.out_features)
    return y


# --------------------------------------------------------------------------------------
# MoE block
# --------------------------------------------------------------------------------------
@dataclass
class Expert:
    gate_proj: QuantLinear
    up_proj: QuantLinear
    down_proj: QuantLinear


@dataclass
class MoeBlock:
    """Sub-modules of a Qwen2-MoE style sparse block (inference/moe_block.py:45-55)."""
    num_experts: int
    top_k: int
    norm_topk_prob: bool
    gate_weight: torch.Tensor                      # (E, H) router
    experts: List[Expert] = field(default_factory=list)
    shared_expert: Optional[Expert] = None         # None = no shared expert (Mixtral / Qwen3 style)
    shared_gate_weight: Optional[torch.Tensor] = None  # (1, H)
    graph_threshold: int = 4                       # inference/moe_block.py:60


def route(blk: MoeBlock, x: torch.Tensor):
    """Router (inference/moe_block.py:386-392): logits in the activation dtype, softmax in fp32,
    top-k, optional renormalisation, weights cast back to the activation dtype."""
    logits = x @ blk.gate_weight.T
    w = F.softmax(logits, dim=1, dtype=torch.float)
    w, sel = torch.topk(w, blk.top_k, dim=-1)
    if blk.norm_topk_prob:
        w = w / w.sum(dim=-1, keepdim=True)
    return logits, w.to(x.dtype), sel


def _expert_mlp(e: Expert, x: torch.Tensor, xU_gate=None, xU_up=None) -> torch.Tensor:
    """SwiGLU expert (inference/moe_block.py:367-379): down(silu(gate(x)) * up(x))."""
    g = linear_forward(e.gate_proj, x, precomputed_xU=xU_gate)
    u = linear_forward(e.up_proj, x, precomputed_xU=xU_up)
    return linear_forward(e.down_proj, F.silu(g) * u)


def _shared_xU(blk: MoeBlock, x: torch.Tensor, experts: Sequence[int]) -> Dict[str, Dict]:
    """x @ U once per distinct cluster among `experts`, for gate and up only
    (inference/moe_block.py:272-322)."""
    cache: Dict[str, Dict] = {"gate_proj": {}, "up_proj": {}}
    for name in ("gate_proj", "up_proj"):
        # the first expert seen in index order donates the U of its cluster
        owners = {}
        for ei in range(blk.num_experts):
            lin = getattr(blk.experts[ei], name)
            if lin.cluster_id is not None and lin.cluster_id not in owners:
                owners[lin.cluster_id] = lin.U
        for ei in experts:
            cid = getattr(blk.experts[ei], name).cluster_id
            if cid is not None and cid not in cache[name] and owners.get(cid) is not None:
                cache[name][cid] = x @ owners[cid]
    return cache


def moe_forward(blk: MoeBlock, hidden: torch.Tensor):
    """GraphCompatibleMoeBlock.forward with graph_mode off (inference/moe_block.py:381-436).

    Tokens <= graph_threshold take the per-token decode loop (inference/moe_block.py:438-478:
    weighted sum in top-k slot order; each token uses its own row of the shared x @ U -- the
    reference hands the whole (N, r) matrix to a one-token call, which only works for N == 1); otherwise the sparse loop over all experts
    (inference/moe_block.py:704-740: index_add in expert order).  The shared expert, gated by a
    sigmoid, is added last.  Returns (out (B,S,H), router_logits (B*S,E)).
    """
    Bsz, S, H = hidden.shape
    x = hidden.reshape(-1, H)
    logits, w, sel = route(blk, x)
    N = x.shape[0]
    out = torch.zeros(N, H, dtype=x.dtype)

    if N <= blk.graph_threshold:
        xU = _shared_xU(blk, x, sel.reshape(-1).tolist())
        for t in range(N):
            xt = x[t:t + 1]
            ids = sel[t].tolist()
            hs = []
            for ei in ids:
                e = blk.experts[ei]
                ag = xU["gate_proj"].get(e.gate_proj.cluster_id)
                au = xU["up_proj"].get(e.up_proj.cluster_id)
                g = linear_forward(e.gate_proj, xt, precomputed_xU=None if ag is None else ag[t:t + 1])
                u = linear_forward(e.up_proj, xt, precomputed_xU=None if au is None else au[t:t + 1])
                hs.append(F.silu(g) * u)
            for k, ei in enumerate(ids):
                d = linear_forward(blk.experts[ei].down_proj, hs[k])
                out[t] += w[t, k] * d.squeeze(0)
    else:
        xU = _shared_xU(blk, x, range(blk.num_experts))
        mask = F.one_hot(sel, num_classes=blk.num_experts).permute(2, 1, 0)
        for ei in range(blk.num_experts):
            slot, tok = torch.where(mask[ei])
            if tok.numel() == 0:
                continue
            e = blk.experts[ei]
            xs = x[tok]
            ag = xU["gate_proj"].get(e.gate_proj.cluster_id)
            au = xU["up_proj"].get(e.up_proj.cluster_id)
            y = _expert_mlp(e, xs, None if ag is None else ag[tok], None if au is None else au[tok])
            y = y * w[tok, slot, None]
            out.index_add_(0, tok, y.to(x.dtype))

    if blk.shared_expert is not None:
        sh = _expert_mlp(blk.shared_expert, x)
        if blk.shared_gate_weight is not None:
            sh = torch.sigmoid(x @ blk.shared_gate_weight.T) * sh
        out = out + sh
    return out.reshape(Bsz, S, H), logits


def experts_forward(experts: List[Expert], hidden: torch.Tensor, top_k_index: torch.Tensor,
                    top_k_weights: torch.Tensor) -> torch.Tensor:
    """Fused-experts adapter (inference/quantized_linear.py:395-428): for each expert that is hit,
    gather its tokens, run the SwiGLU MLP, scale by the routing weight, index_add in expert order."""
    E = len(experts)
    out = torch.zeros_like(hidden)
    mask = F.one_hot(top_k_index, num_classes=E).permute(2, 1, 0)
    for ei in range(E):
        slot, tok = torch.where(mask[ei])
        if tok.numel() == 0:
            continue
        y = _expert_mlp(experts[ei], hidden[tok])
        y = y * top_k_weights[tok, slot, None]
        out.index_add_(0, tok, y.to(out.dtype))
    return out


# --------------------------------------------------------------------------------------
# On-disk format -> layers (inference/model_builder.py:27-80, 335-450, 465-544)
# --------------------------------------------------------------------------------------
def dequant_intN(q: torch.Tensor, scale: torch.Tensor, nbits: int) -> torch.Tensor:
    """q / (2^(nbits-1) - 1) * scale in fp32, per-column scale (inference/model_builder.py:69-72)."""
    return q.float() / (2 ** (nbits - 1) - 1) * scale.float()


def unpack_int4(packed: torch.Tensor, orig_rows: int) -> torch.Tensor:
    """Two rows per byte: low nibble = even row, high nibble = odd row, stored value = q + 7
    (inference/model_builder.py:75-80)."""
    lo = (packed & 0xF).to(torch.int8) - 7
    hi = ((packed >> 4) & 0xF).to(torch.int8) - 7
    return torch.stack([lo, hi], dim=1).reshape(-1, packed.shape[1])[:orig_rows]


def _decode_factor(d: dict, prefix: str, bits: int) -> torch.Tensor:
    if f"{prefix}_fp16" in d:
        return d[f"{prefix}_fp16"].half()
    if f"{prefix}_int4_packed" in d:
        rows = int(d[f"{prefix}_orig_rows"].item())
        return dequant_intN(unpack_int4(d[f"{prefix}_int4_packed"], rows), d[f"{prefix}_scale"], 4).half()
    return dequant_intN(d[f"{prefix}_int8"], d[f"{prefix}_scale"], bits).half()


def checkpoint_layers(model_data: dict, cross: dict) -> Dict[int, Dict[str, QuantLinear]]:
    """{layer: {module name: QuantLinear}} as the loader builds them: U from the cluster the
    (projection type, layer, expert) record assigns (expert -1 for attention / dense projections, the
    shared expert gets no low-rank term), SV from per_expert_V at the record's list position; Mixtral's
    w1/w2/w3 are gate/down/up (inference/model_builder.py:345-351, 473-544)."""
    mc, cc = model_data["model_config"], cross["config"]
    uv_bits = cc.get("uv_bits", mc.get("uv_bits", 8))
    u_bits, sv_bits = cc.get("u_bits", uv_bits), cc.get("sv_bits", uv_bits)
    lookup = {}
    for wtype, recs in cross["assignments"].items():
        for li, rec in enumerate(recs):
            lookup[(wtype, rec["layer"], rec["expert"])] = (rec["group_id"], li)
    U_cache = {}
    out = {}
    for l, mods in model_data["layers"].items():
        out[l] = {}
        for name, D in mods.items():
            N, K = D["qweight_int"].shape
            ql = QuantLinear(in_features=K, out_features=N, quant_type="gptq", qweight_int=D["qweight_int"],
                             scales=D["scales"], zeros=D["zeros"], gptq_bits=D["bits"],
                             gptq_groupsize=D["groupsize"], gptq_sym=D.get("sym", False))
            parts = name.split(".")
            if "shared_expert" in name:
                expert = -2
            elif "experts" in parts:
                expert = int(parts[parts.index("experts") + 1])
            else:
                expert = -1
            wt = {"w1": "gate_proj", "w2": "down_proj", "w3": "up_proj"}.get(parts[-1], parts[-1])
            if expert != -2 and (wt, l, expert) in lookup:
                gid, li = lookup[(wt, l, expert)]
                if (wt, gid) not in U_cache:
                    U_cache[(wt, gid)] = _decode_factor(cross["shared_matrices"][wt][gid], "U", u_bits)
                v = cross["per_expert_V"][wt][li]
                ql.U = U_cache[(wt, gid)]
                if "V_int8" in v:   # old format: S kept with the cluster, fused here (quantized_linear.py:249-259)
                    V = dequant_intN(v["V_int8"], v["V_scale"], uv_bits).half()
                    ql.SV = (V * cross["shared_matrices"][wt][gid]["S"].half().unsqueeze(0)).half()
                else:
                    ql.SV = _decode_factor(v, "SV", sv_bits)
                ql.cluster_id = (wt, gid)
            out[l][name] = ql
    return out


# --------------------------------------------------------------------------------------
# Decoder around the layers: what the transformers Qwen2-MoE / Mixtral / Qwen3-MoE models compute
# (the reference borrows them, inference/model_builder.py:234-243), restated with plain tensor ops
# --------------------------------------------------------------------------------------
def _rms_norm(x, w, eps):
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return (w.float() * v).to(x.dtype)


def decoder_forward(cfg: dict, layers: Dict[int, Dict[str, QuantLinear]], dense: Dict[str, torch.Tensor],
                    input_ids: torch.Tensor) -> torch.Tensor:
    """Logits (B, T, V) of a full causal forward without a cache, fp16 activations: embedding, per
    layer RMSNorm -> attention (rotary embedding, grouped-query, softmax in fp32) -> residual -> RMSNorm
    -> MoE block (moe_forward) or dense SwiGLU MLP -> residual, final RMSNorm, lm_head."""
    H, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or H // nh
    eps, theta = cfg.get("rms_norm_eps", 1e-6), cfg.get("rope_theta", 10000.0)
    mixtral = "num_local_experts" in cfg
    E = cfg.get("num_experts", cfg.get("num_local_experts", 0))
    mp = "block_sparse_moe" if mixtral else "mlp"
    gn, un, dn = ("w1", "w3", "w2") if mixtral else ("gate_proj", "up_proj", "down_proj")
    B, T = input_ids.shape
    x = dense["model.embed_tokens.weight"][input_ids]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    fr = torch.outer(torch.arange(T, dtype=torch.float32), inv)
    emb = torch.cat([fr, fr], -1)
    cos, sin = emb.cos().half()[None, None], emb.sin().half()[None, None]

    def rot(v):
        h = v.shape[-1] // 2
        return torch.cat([-v[..., h:], v[..., :h]], -1)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for l in range(cfg["num_hidden_layers"]):
        m = layers[l]
        pre = f"model.layers.{l}"
        h = _rms_norm(x, dense[f"{pre}.input_layernorm.weight"], eps)
        q = linear_forward(m["self_attn.q_proj"], h).view(B, T, nh, hd)
        k = linear_forward(m["self_attn.k_proj"], h).view(B, T, nkv, hd)
        v = linear_forward(m["self_attn.v_proj"], h).view(B, T, nkv, hd)
        if f"{pre}.self_attn.q_norm.weight" in dense:
            q = _rms_norm(q, dense[f"{pre}.self_attn.q_norm.weight"], eps)
            k = _rms_norm(k, dense[f"{pre}.self_attn.k_norm.weight"], eps)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        q = q * cos + rot(q) * sin
        k = k * cos + rot(k) * sin
        k = k.repeat_interleave(nh // nkv, dim=1)
        v = v.repeat_interleave(nh // nkv, dim=1)
        s = (q.float() @ k.float().transpose(-1, -2)) / hd ** 0.5
        s = s.masked_fill(~causal, float("-inf"))
        p = torch.softmax(s, dim=-1).to(x.dtype)
        a = (p @ v).transpose(1, 2).reshape(B, T, nh * hd)
        x = x + linear_forward(m["self_attn.o_proj"], a)
        h = _rms_norm(x, dense[f"{pre}.post_attention_layernorm.weight"], eps)
        if f"{mp}.experts.0.{gn}" in m:
            experts = [Expert(m[f"{mp}.experts.{e}.{gn}"], m[f"{mp}.experts.{e}.{un}"], m[f"{mp}.experts.{e}.{dn}"])
                       for e in range(E)]
            shared = None
            if f"{mp}.shared_expert.gate_proj" in m:
                shared = Expert(m[f"{mp}.shared_expert.gate_proj"], m[f"{mp}.shared_expert.up_proj"],
                                m[f"{mp}.shared_expert.down_proj"])
            blk = MoeBlock(num_experts=E, top_k=cfg["num_experts_per_tok"],
                           norm_topk_prob=True if mixtral else cfg.get("norm_topk_prob", False),
                           gate_weight=dense[f"{pre}.{mp}.gate.weight"], experts=experts, shared_expert=shared,
                           shared_gate_weight=dense.get(f"{pre}.{mp}.shared_expert_gate.weight"))
            y, _ = moe_forward(blk, h)
        else:
            g = linear_forward(m["mlp.gate_proj"], h)
            u = linear_forward(m["mlp.up_proj"], h)
            y = linear_forward(m["mlp.down_proj"], F.silu(g) * u)
        x = x + y
    x = _rms_norm(x, dense["model.norm.weight"], eps)
    return x @ dense.get("lm_head.weight", dense["model.embed_tokens.weight"]).T
