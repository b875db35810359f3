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
