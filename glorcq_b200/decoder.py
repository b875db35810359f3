"""A decoder assembled from the quantized layers: the host model the reference borrows from
transformers (inference/model_builder.py:234-243 instantiates ``AutoModelForCausalLM`` and swaps its
linear layers; inference/graph_wrapper.py:84-127 calls it with ``input_ids, cache_position,
past_key_values, use_cache, return_dict``).  It is written here so that the path does not depend on
the transformers version: RMSNorm, rotary embedding, grouped-query attention over a static key/value
cache, and per layer either a ``GraphCompatibleMoeBlock`` or a dense SwiGLU MLP, all built from
``GLoRCQLinear`` modules.  Covers the Qwen2-MoE (shared expert, optional top-k renormalisation),
Mixtral (w1/w3/w2 naming, top-2 renormalised, no shared expert) and Qwen3-MoE (per-head q/k norms, no
shared expert) layouts.

The quantized projections and the MoE block run on this package's kernels, and so does the attention
of a decode step (``glq_attn_decode``: q/k norms, rotary embedding, cache write and attention over the
live positions in one launch) and the fp16 ``lm_head`` product of up to 64 rows (``glq_lm_head``: a streaming
kernel over the row-major vocabulary matrix with the greedy arg-max folded in).  A prompt written at positions
0..T-1 runs its norms, rotary embedding and cache write in ``glq_rope_prefill`` and its causal attention in
``glq_attn_prefill`` (head sizes 64 and 128; prompts of 2048 tokens and more, where the library's kernel is
measurably faster, and prompts appended to a filled cache go through ``scaled_dot_product_attention``).  The first
layer norm, the embedding lookup and the logits of a whole prompt are plain library calls.
"""

from __future__ import annotations

from types import SimpleNamespace
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

import os

from . import _lib, tiled
from .moe_block import GraphCompatibleMoeBlock
from .quantized_linear import GLoRCQLinear

# Prompts of at least this many tokens hand their causal attention to the library call instead of
# glq_attn_prefill (GLQ_PROMPT_ATTN_LIBRARY_FROM; 0 = always the library, a huge value = never).  Measured on the
# 24-layer model, whole prompt pass with this kernel / with the library: 512 tokens 15.5 / 15.5 ms, 1024: 19.0 / 18.7,
# 2048: 28.0 / 26.6, 4096: 48.4 / 43.6.
_PROMPT_ATTN_LIBRARY_FROM = int(os.environ.get("GLQ_PROMPT_ATTN_LIBRARY_FROM", "2048"))


class StaticKVCache:
    """Fixed-size key/value cache, one (B, kv_heads, max_len, head_dim) pair per layer: the role of
    transformers' StaticCache in inference/graph_wrapper.py:41-47 (``reset`` included)."""

    def __init__(self, config, max_batch_size, max_cache_len, device, dtype=torch.float16):
        c = config
        self.max_batch_size, self.max_cache_len = max_batch_size, max_cache_len
        shape = (c.num_hidden_layers, max_batch_size, c.num_key_value_heads, max_cache_len, c.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)

    def reset(self):
        self.k.zero_()
        self.v.zero_()

    def update(self, layer, k_new, v_new, cache_position):
        """Write (B, kv_heads, T, D) at positions cache_position (T,) and return the layer's full buffers."""
        b = k_new.shape[0]
        self.k[layer, :b].index_copy_(2, cache_position, k_new)
        self.v[layer, :b].index_copy_(2, cache_position, v_new)
        return self.k[layer, :b], self.v[layer, :b]


def _rope_tables(head_dim, max_len, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(max_len, device=device, dtype=torch.float32), inv)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().half(), emb.sin().half()


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def _add_rmsnorm(x, delta, weight, eps):
    """(x + delta, rms_norm(x + delta) * weight) in one launch for fp16 rows of up to 8192 columns."""
    H = x.shape[-1]
    if not (x.is_cuda and x.dtype == torch.float16 and delta.dtype == torch.float16 and H % 8 == 0 and H <= 8192):
        y = x + delta
        return y, F.rms_norm(y, (H,), weight, eps)
    x, delta = x.contiguous(), delta.contiguous()
    x_out, h_out = torch.empty_like(x), torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().glq_add_rmsnorm(x.data_ptr(), delta.data_ptr(), weight.data_ptr(), float(eps),
                                              x.numel() // H, H, x_out.data_ptr(), h_out.data_ptr(),
                                              tiled._stream_ptr(x.device)), "add_rmsnorm")
    return x_out, h_out


class _Attention(nn.Module):
    def __init__(self, cfg, layer_idx, mods: Dict[str, GLoRCQLinear], dense, prefix, device):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.q_proj, self.k_proj = mods["self_attn.q_proj"], mods["self_attn.k_proj"]
        self.v_proj, self.o_proj = mods["self_attn.v_proj"], mods["self_attn.o_proj"]
        for nm, lin in (("q_proj", self.q_proj), ("k_proj", self.k_proj), ("v_proj", self.v_proj)):
            b = dense.get(f"{prefix}.self_attn.{nm}.bias")
            if b is not None:
                lin.set_bias(b.to(device))
        self.q_norm = dense.get(f"{prefix}.self_attn.q_norm.weight")
        self.k_norm = dense.get(f"{prefix}.self_attn.k_norm.weight")
        if self.q_norm is not None:
            self.q_norm, self.k_norm = self.q_norm.to(device).half(), self.k_norm.to(device).half()
        # q, k and v of one shape (no grouped-query sharing): one grouped launch pair for the decode step
        self._qkv = None
        tl = [getattr(m, "_tiled", None) for m in (self.q_proj, self.k_proj, self.v_proj)]
        uts = [getattr(m, "_ut", None) for m in (self.q_proj, self.k_proj, self.v_proj)]
        if all(t is not None for t in tl) and len({(t.fmt, t.N, t.K, t.group_size, t.rank) for t in tl}) == 1 and \
                (all(u is not None for u in uts) or all(u is None for u in uts)):
            self._qkv = tiled.GroupedLinear(tl, uts if uts[0] is not None else None)
        # grouped-query attention: k and v still share a shape -- one launch pair for the two
        self._kv = None
        if self._qkv is None and all(t is not None for t in tl[1:]) and \
                len({(t.fmt, t.N, t.K, t.group_size, t.rank) for t in tl[1:]}) == 1 and \
                (all(u is not None for u in uts[1:]) or all(u is None for u in uts[1:])):
            self._kv = tiled.GroupedLinear(tl[1:], uts[1:] if uts[1] is not None else None)

    def forward(self, x, cache_position, cache: StaticKVCache, cos, sin, kv_len=None):
        c = self.cfg
        B, T, _ = x.shape
        if T == 1 and cache_position.numel() == 1 and c.head_dim in (32, 64, 128, 256):
            # decode step: norms, rotary embedding, cache write and attention over the live positions in
            # one launch; the position stays on the device (graph replay)
            if self._qkv is not None:
                q, k, v = self._qkv.forward(x.view(B, -1).contiguous())
            elif self._kv is not None:
                q = self.q_proj(x).view(B, -1)
                k, v = self._kv.forward(x.view(B, -1).contiguous())
            else:
                q, k, v = self.q_proj(x).view(B, -1), self.k_proj(x).view(B, -1), self.v_proj(x).view(B, -1)
            y = torch.empty_like(q)
            kc, vc = cache.k[self.layer_idx], cache.v[self.layer_idx]
            with torch.cuda.device(x.device):
                L = _lib.lib()
                ws, ctr = tiled.workspace(x.device, L.glq_attn_decode_workspace_bytes(
                    B, c.num_attention_heads, c.head_dim, cache.max_cache_len), B * c.num_attention_heads)
                _lib.check(L.glq_attn_decode(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(), cache_position.data_ptr(),
                    kc.data_ptr(), vc.data_ptr(), y.data_ptr(), B, c.num_attention_heads, c.num_key_value_heads,
                    c.head_dim, cache.max_cache_len, None if self.q_norm is None else self.q_norm.data_ptr(),
                    None if self.k_norm is None else self.k_norm.data_ptr(), float(c.rms_norm_eps),
                    ws.data_ptr(), ws.numel(), ctr.data_ptr(), ctr.numel(), tiled._stream_ptr(x.device)), "attn_decode")
            return self.o_proj(y.view(B, 1, -1))
        if self._qkv is not None and x.is_cuda:
            # q, k and v of one shape: one grouped launch pair for the whole prompt too
            q, k, v = self._qkv.forward(x.reshape(B * T, -1).contiguous())
            q = q.view(B, T, c.num_attention_heads, c.head_dim)
            k = k.view(B, T, c.num_key_value_heads, c.head_dim)
            v = v.view(B, T, c.num_key_value_heads, c.head_dim)
        elif self._kv is not None and x.is_cuda:
            q = self.q_proj(x).view(B, T, c.num_attention_heads, c.head_dim)
            k, v = self._kv.forward(x.reshape(B * T, -1).contiguous())
            k = k.view(B, T, c.num_key_value_heads, c.head_dim)
            v = v.view(B, T, c.num_key_value_heads, c.head_dim)
        else:
            q = self.q_proj(x).view(B, T, c.num_attention_heads, c.head_dim)
            k = self.k_proj(x).view(B, T, c.num_key_value_heads, c.head_dim)
            v = self.v_proj(x).view(B, T, c.num_key_value_heads, c.head_dim)
        if x.is_cuda and q.dtype == torch.float16 and c.head_dim in (32, 64, 128, 256) and cache_position.numel() == T:
            # norms, rotary embedding and the cache write of the whole prompt in one launch
            q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
            kc, vc = cache.k[self.layer_idx], cache.v[self.layer_idx]
            with torch.cuda.device(x.device):
                _lib.check(_lib.lib().glq_rope_prefill(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                    cache_position.to(torch.int64).contiguous().data_ptr(), kc.data_ptr(), vc.data_ptr(), B, T,
                    c.num_attention_heads, c.num_key_value_heads, c.head_dim, cache.max_cache_len,
                    None if self.q_norm is None else self.q_norm.data_ptr(),
                    None if self.k_norm is None else self.k_norm.data_ptr(), float(c.rms_norm_eps),
                    tiled._stream_ptr(x.device)), "rope_prefill")
            if kv_len is not None and kv_len == T and c.head_dim in (64, 128) and T < _PROMPT_ATTN_LIBRARY_FROM:
                # a prompt written at positions 0..T-1: causal attention over the new keys, in the projections' layout
                y = torch.empty_like(q)
                with torch.cuda.device(x.device):
                    _lib.check(_lib.lib().glq_attn_prefill(
                        q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), B, T, c.num_attention_heads,
                        c.num_key_value_heads, c.head_dim, tiled._stream_ptr(x.device)), "attn_prefill")
                return self.o_proj(y.view(B, T, c.num_attention_heads * c.head_dim))
            q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
            k_all, v_all = kc[:B], vc[:B]
            return self._prompt_attention(q, k, v, k_all, v_all, cache, cache_position, kv_len, B, T)
        if self.q_norm is not None:
            q = F.rms_norm(q, (c.head_dim,), self.q_norm, c.rms_norm_eps)
            k = F.rms_norm(k, (c.head_dim,), self.k_norm, c.rms_norm_eps)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        cs, sn = cos[cache_position][None, None], sin[cache_position][None, None]
        q = q * cs + _rotate_half(q) * sn
        k = k * cs + _rotate_half(k) * sn
        k_all, v_all = cache.update(self.layer_idx, k, v, cache_position)
        return self._prompt_attention(q, k, v, k_all, v_all, cache, cache_position, kv_len, B, T)

    def _prompt_attention(self, q, k, v, k_all, v_all, cache, cache_position, kv_len, B, T):
        c = self.cfg
        gqa = c.num_key_value_heads != c.num_attention_heads
        if kv_len is not None and kv_len == T:
            # a prompt written at positions 0..T-1: causal attention over the new keys only
            y = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=gqa)
        else:
            # position mask over the live part of the static cache: key j is visible to query t when j <= position(t)
            n_live = cache.max_cache_len if kv_len is None else kv_len
            mask = torch.arange(n_live, device=q.device)[None, :] <= cache_position[:, None]
            y = F.scaled_dot_product_attention(q, k_all[:, :, :n_live], v_all[:, :, :n_live], attn_mask=mask[None, None],
                                               enable_gqa=gqa)
        return self.o_proj(y.transpose(1, 2).reshape(B, T, c.num_attention_heads * c.head_dim))


class _DenseMLP(nn.Module):
    def __init__(self, gate, up, down):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate, up, down
        self.act_fn = F.silu

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class _Expert(nn.Module):
    def __init__(self, gate, up, down):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate, up, down
        self.act_fn = F.silu


def _config(hf: dict):
    c = SimpleNamespace(**hf)
    c.num_key_value_heads = hf.get("num_key_value_heads") or hf["num_attention_heads"]
    c.head_dim = hf.get("head_dim") or hf["hidden_size"] // hf["num_attention_heads"]
    c.rms_norm_eps = hf.get("rms_norm_eps", 1e-6)
    c.rope_theta = hf.get("rope_theta", 10000.0)
    c.num_experts = hf.get("num_experts", hf.get("num_local_experts", 0))
    c.num_experts_per_tok = hf.get("num_experts_per_tok", 0)
    mixtral = "num_local_experts" in hf
    c.norm_topk_prob = True if mixtral else hf.get("norm_topk_prob", False)
    c.moe_prefix = "block_sparse_moe" if mixtral else "mlp"
    c.expert_names = ("w1", "w3", "w2") if mixtral else ("gate_proj", "up_proj", "down_proj")
    c.max_position_embeddings = hf.get("max_position_embeddings", 4096)
    return c


class GLoRCQDecoder(nn.Module):
    """``layers``: {layer_idx: {module_name: GLoRCQLinear}} from ``model_builder.build_layers``.
    ``dense``: fp16 tensors under their state-dict names (model.embed_tokens.weight,
    model.layers.N.input_layernorm.weight, model.layers.N.post_attention_layernorm.weight,
    model.layers.N.mlp.gate.weight, model.layers.N.mlp.shared_expert_gate.weight, model.norm.weight,
    lm_head.weight, attention biases and q/k norms); what is missing is zero, as the reference's loader
    leaves every parameter it does not replace (inference/model_builder.py:314-330, 431-447)."""

    def __init__(self, hf_config: dict, layers, dense: Optional[dict] = None, device="cuda:0", ep_rank=0, ep_world=1,
                 ep_group=None, peer_exchange_max_tokens=0):
        """With ``ep_world`` > 1 the routed experts of every block are sharded (expert e on rank e % ep_world;
        ``layers`` then only needs this rank's experts); everything else is replicated, and the ranks exchange the
        experts' outputs once per block (glorcq_b200.parallel)."""
        super().__init__()
        c = self.config = _config(hf_config)
        dense = dense or {}
        dev = torch.device(device)
        H = c.hidden_size

        def dense_param(name, shape):
            t = dense.get(name)
            if t is None:
                t = torch.zeros(shape, dtype=torch.float16)
            return nn.Parameter(t.to(dev).half(), requires_grad=False)

        self.embed_tokens = dense_param("model.embed_tokens.weight", (c.vocab_size, H))
        self.norm = dense_param("model.norm.weight", (H,))
        lm = dense.get("lm_head.weight")
        self.lm_head = self.embed_tokens if lm is None else nn.Parameter(lm.to(dev).half(), requires_grad=False)
        self.ln1, self.ln2 = nn.ParameterList(), nn.ParameterList()
        self.attn, self.mlp = nn.ModuleList(), nn.ModuleList()
        for l in range(c.num_hidden_layers):
            mods = layers[l]
            pre = f"model.layers.{l}"
            self.ln1.append(dense_param(f"{pre}.input_layernorm.weight", (H,)))
            self.ln2.append(dense_param(f"{pre}.post_attention_layernorm.weight", (H,)))
            self.attn.append(_Attention(c, l, mods, dense, pre, dev))
            mp, (gn, un, dn) = c.moe_prefix, c.expert_names
            if any(k.startswith(f"{mp}.experts.") for k in mods):     # (with expert parallelism: this rank's experts only)
                blk = SimpleNamespace()
                blk.num_experts, blk.top_k, blk.norm_topk_prob = c.num_experts, c.num_experts_per_tok, c.norm_topk_prob
                blk.gate = nn.Linear(H, c.num_experts, bias=False, device=dev, dtype=torch.float16)
                blk.gate.weight.data.copy_(dense_param(f"{pre}.{mp}.gate.weight", (c.num_experts, H)))
                blk.experts = [_Expert(mods[f"{mp}.experts.{e}.{gn}"], mods[f"{mp}.experts.{e}.{un}"],
                                       mods[f"{mp}.experts.{e}.{dn}"]) if e % ep_world == ep_rank else None
                               for e in range(c.num_experts)]
                if ep_world == 1:
                    blk.experts = nn.ModuleList(blk.experts)
                if f"{mp}.shared_expert.gate_proj" in mods:
                    blk.shared_expert = _Expert(mods[f"{mp}.shared_expert.gate_proj"], mods[f"{mp}.shared_expert.up_proj"],
                                                mods[f"{mp}.shared_expert.down_proj"])
                    blk.shared_expert_gate = nn.Linear(H, 1, bias=False, device=dev, dtype=torch.float16)
                    blk.shared_expert_gate.weight.data.copy_(dense_param(f"{pre}.{mp}.shared_expert_gate.weight", (1, H)))
                else:
                    blk.shared_expert, blk.shared_expert_gate = None, None
                moe = GraphCompatibleMoeBlock(blk)
                if ep_world > 1:
                    moe.set_expert_parallel(ep_rank, ep_world, ep_group)
                    moe.peer_exchange_max_tokens = peer_exchange_max_tokens
                moe.prepare(dev, release_linear_tiles=True)
                self.mlp.append(moe)
            else:
                self.mlp.append(_DenseMLP(mods["mlp.gate_proj"], mods["mlp.up_proj"], mods["mlp.down_proj"]))
        self._rope = None
        self._own_cache = None
        self._lm_ws = {}
        self.last_argmax = None     # (B * kept positions,) int64 greedy tokens of the last forward, when the kernel ran

    def _tables(self, need, device):
        if self._rope is None or self._rope[0].shape[0] < need:
            n = max(need, self.config.max_position_embeddings)
            self._rope = _rope_tables(self.config.head_dim, n, self.config.rope_theta, device)
        return self._rope

    def _lm_head(self, x):
        """(rows, H) fp16 -> (rows, V) logits; up to 64 rows go through this package's streaming kernel (8 rows
        per pass of the weights) with the greedy arg-max of every row folded in (kept in ``last_argmax``),
        longer inputs (the logits of a whole prompt) through a dense library product."""
        rows, H = x.shape
        V = self.lm_head.shape[0]
        if not (x.is_cuda and 0 < rows <= 64 and H % 32 == 0 and H <= 8192 and self.lm_head.is_contiguous()):
            self.last_argmax = None
            return x @ self.lm_head.t()
        x = x.contiguous()
        logits = torch.empty(rows, V, dtype=torch.float16, device=x.device)
        best = torch.empty(rows, dtype=torch.int64, device=x.device)
        L = _lib.lib()
        with torch.cuda.device(x.device):
            key = ("lm_head", x.device.index, tiled._stream_ptr(x.device))
            if key not in self._lm_ws:
                self._lm_ws[key] = (torch.empty(L.glq_lm_head_workspace_bytes() + 16, dtype=torch.uint8, device=x.device),
                                    torch.zeros(1, dtype=torch.int32, device=x.device))
            ws, ctr = self._lm_ws[key]
            for r0 in range(0, rows, 8):
                nb = min(8, rows - r0)
                _lib.check(L.glq_lm_head(x[r0:].data_ptr(), x.stride(0), self.lm_head.data_ptr(), nb, V, H,
                                         logits[r0:].data_ptr(), V, best[r0:].data_ptr(),
                                         (ws.data_ptr() + 15) // 16 * 16, ws.numel() - 16, ctr.data_ptr(),
                                         tiled._stream_ptr(x.device)), "lm_head")
        self.last_argmax = best
        return logits

    def forward(self, input_ids=None, cache_position=None, past_key_values=None, use_cache=True, return_dict=False,
                logits_to_keep=0, **_unused):
        """``logits_to_keep`` = k > 0 computes the logits of the last k positions only (the greedy loop needs
        one); 0 keeps them all, as the transformers models do by default."""
        c = self.config
        B, T = input_ids.shape
        if past_key_values is None:
            if self._own_cache is None or self._own_cache.max_batch_size < B:
                self._own_cache = StaticKVCache(c, B, c.max_position_embeddings, input_ids.device)
            past_key_values = self._own_cache
        if cache_position is None:
            cache_position = torch.arange(T, device=input_ids.device)
        cos, sin = self._tables(past_key_values.max_cache_len, input_ids.device)
        x = F.embedding(input_ids, self.embed_tokens)
        L = c.num_hidden_layers
        h = F.rms_norm(x, (c.hidden_size,), self.ln1[0], c.rms_norm_eps) if L > 0 else x
        # a prompt (T > 1, eager only): its first position is read back once, so that attention sees the live
        # part of the static cache instead of all of it
        kv_len = (int(cache_position[0]) + T) if T > 1 else None
        for l in range(L):
            x, h = _add_rmsnorm(x, self.attn[l](h, cache_position, past_key_values, cos, sin, kv_len), self.ln2[l],
                                c.rms_norm_eps)
            nxt = self.ln1[l + 1] if l + 1 < L else self.norm          # the norm that follows this layer
            mlp = self.mlp[l]
            if isinstance(mlp, GraphCompatibleMoeBlock) and c.hidden_size <= 8192:
                # residual add and the following norm run inside the block's combine kernel
                x, _, h = mlp(h, residual=x, next_norm=(nxt, c.rms_norm_eps))
            else:
                m = mlp(h)
                x = x + (m[0] if isinstance(m, tuple) else m)
                h = F.rms_norm(x, (c.hidden_size,), nxt, c.rms_norm_eps)
        x = h if L > 0 else F.rms_norm(x, (c.hidden_size,), self.norm, c.rms_norm_eps)
        if logits_to_keep and logits_to_keep < T:
            x = x[:, T - logits_to_keep:]
        keep = x.shape[1]
        logits = self._lm_head(x.reshape(B * keep, c.hidden_size)).view(B, keep, -1)
        return (logits, past_key_values)

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=100, do_sample=False):
        """Greedy generation without a graph (the comparison leg of run_speed_benchmark)."""
        B, T = input_ids.shape
        cache = StaticKVCache(self.config, B, T + max_new_tokens, input_ids.device)
        logits = self(input_ids=input_ids, cache_position=torch.arange(T, device=input_ids.device), past_key_values=cache)[0]
        out = input_ids
        for i in range(max_new_tokens):
            nxt = torch.argmax(logits[:, -1, :], dim=-1, keepdim=True)
            out = torch.cat([out, nxt], dim=1)
            if i + 1 < max_new_tokens:
                pos = torch.full((1,), T + i, device=input_ids.device, dtype=torch.long)
                logits = self(input_ids=nxt, cache_position=pos, past_key_values=cache)[0]
        return out
