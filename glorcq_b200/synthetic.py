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
