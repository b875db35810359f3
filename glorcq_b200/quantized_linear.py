"""Quantized linear layer and fused-experts adapter on the sm_100a kernels.

Same class names, attributes, loaders and forward signature as the reference's
``inference.quantized_linear`` (inference/quantized_linear.py:152-428):

    y = dequant(W_q) x + (x U) SV^T + bias

The loaders additionally re-tile the weights for the kernels (glorcq_b200.tiled); forward runs
one fused launch for the quantized matmul with the low-rank epilogue (plus a small launch for
a = x U when it is not handed in).  Nothing falls back to PyTorch arithmetic.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from . import tiled
from .kernels import gptq_dequant_matmul_fused, is_cuda_available, is_gptq_cuda_available
from .tiled import TiledWeight

_HAS_FUSED_KERNEL = is_cuda_available()
_HAS_GPTQ_FUSED_KERNEL = is_gptq_cuda_available()


def _tileable(bits, groupsize):
    kb = {2: 128, 4: 64}.get(bits)
    return kb is not None and groupsize is not None and groupsize > 0 and groupsize % kb == 0


class GLoRCQLinear(nn.Module):
    """Drop-in for the reference layer (inference/quantized_linear.py:152-362)."""

    def __init__(self, in_features, out_features, bias=False):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.quant_type = None       # "gptq" or "turbo"

        # integer-code format
        self.qweight_int = None      # (out_d, in_d) int32; dropped after tiling unless keep_raw
        self.scales = None           # (out_d, n_groups) fp16
        self.zeros = None            # (out_d, n_groups) fp16
        self.gptq_bits = None
        self.gptq_groupsize = None
        self.gptq_sym = False

        # codebook format
        self.packed_indices = None   # (out_d, in_d/4) uint8
        self.norms = None            # (out_d,) fp32
        self.turbo_bits = None
        self.turbo_dim = None
        self.turbo_seed = 42
        self._rotation_cache = None
        self._rht_signs = None
        self._turbo_dequant_W = None

        # low-rank correction
        self.U = None                # (in_d, rank) fp16, shared by a cluster
        self.SV = None               # (out_d, rank) fp16
        self.cluster_id = None

        self.bias_param = None       # (out_d,) fp16

        # device layout of the kernels
        self._tiled = None           # TiledWeight
        self._dense = None           # TiledWeight of pre-dequantised fp16 weights (load_dense)
        self._sv_dense = None        # TiledWeight of SV for the dense route
        self._ut = None              # TiledWeight of U^T (shared through tiled.tiled_ut)

    # ---- loaders (inference/quantized_linear.py:195-269) ---------------------------------
    def load_gptq(self, packed_data, device="cuda", keep_raw=False, check_range=True):
        """Integer codes + per-group scale/zero.  2- and 4-bit codes with a group size that is a
        multiple of 128 (64 for 4-bit) are re-tiled for the fused kernel; anything else keeps the
        (N,K) codes and runs through the int8 drop-in kernel."""
        self.quant_type = "gptq"
        q = packed_data["qweight_int"].to(device)
        self.scales = packed_data["scales"].to(device).to(torch.float16)
        self.zeros = packed_data["zeros"].to(device).to(torch.float16)
        self.gptq_bits = packed_data["bits"]
        self.gptq_groupsize = packed_data["groupsize"]
        self.gptq_sym = packed_data.get("sym", False)
        in_range = True
        if check_range and _tileable(self.gptq_bits, self.gptq_groupsize):
            in_range = bool(((q >= 0) & (q < 2 ** self.gptq_bits)).all())   # load time only
        if _tileable(self.gptq_bits, self.gptq_groupsize) and in_range:
            self._tiled = TiledWeight.from_gptq(q, self.scales, self.zeros, self.gptq_bits,
                                                self.gptq_groupsize, self.gptq_sym)
            self.qweight_int = q if keep_raw else None
        else:
            self._tiled = None
            self.qweight_int = q
        self._sync_tiled()

    def load_turbo(self, compressed_data, rotation_cache, device="cuda"):
        """2-bit codebook indices for runtime dequant; the codes stay packed on the device."""
        self.quant_type = "turbo"
        self.turbo_bits = compressed_data["bits"]
        self.turbo_dim = compressed_data["dim"]
        self.turbo_seed = compressed_data.get("seed", 42)
        if self.turbo_bits != 2:
            raise RuntimeError(f"codebook kernels cover bits == 2, got {self.turbo_bits}")
        self.packed_indices = compressed_data["packed_indices"].to(device)
        self.norms = compressed_data["norms"].float().to(device)
        self._rotation_cache = rotation_cache
        rotation_cache.register(self.turbo_dim, self.turbo_bits, self.turbo_seed)
        centroids = rotation_cache.get_centroids(self.turbo_dim, self.turbo_bits, self.turbo_seed)
        self._tiled = TiledWeight.from_turbo(self.packed_indices, self.norms, centroids.to(device))
        self._sync_tiled()

    def load_dense(self, weight, device="cuda", quant_type="dense"):
        """Pre-dequantised fp16 weights (``weight_quant`` records of a checkpoint,
        inference/model_builder.py:386-415): kept dense, run through the dense fp16 kernels."""
        self.quant_type = quant_type
        W = weight.to(device=device, dtype=torch.float16).contiguous()
        self._turbo_dequant_W = W
        self._dense = TiledWeight.from_dense(W)
        self._tiled = None
        self._sync_tiled()

    def load_turbo_predequant(self, compressed_data, turbo_quantizer, device="cuda"):
        """Legacy route of the reference (inference/quantized_linear.py:229-247): the codebook weights are
        dequantised once by the quantizer that produced them (a third-party object with a
        ``dequantize(MSEQuantized(indices, norms, bits))`` method) and cached as dense fp16; forward is then
        x . W^T on the unrotated input."""
        from collections import namedtuple
        self.turbo_bits = compressed_data["bits"]
        self.turbo_dim = compressed_data["dim"]
        MSEQuantized = namedtuple("MSEQuantized", ["indices", "norms", "bits"])
        q = MSEQuantized(indices=compressed_data["packed_indices"].to(device), norms=compressed_data["norms"].to(device),
                         bits=compressed_data["bits"])
        self.load_dense(turbo_quantizer.dequantize(q), device=device, quant_type="turbo")

    def load_lora(self, U, S, V, device="cuda"):
        """Old format: pre-fuse S into V (inference/quantized_linear.py:249-259)."""
        if U is not None:
            self.U = U.half().to(device)
            self.SV = (V * S.unsqueeze(0)).half().to(device)
            self._sync_tiled()

    def load_sv(self, U, SV, device="cuda"):
        """New format: SV already fused.  Pass the cluster's shared U tensor itself (not a copy) so
        that every layer of the cluster uses one tiled U^T."""
        if U is not None:
            dev = torch.device(device)
            same = U.dtype == torch.float16 and U.is_cuda and (dev.type == "cuda") and \
                (dev.index is None or dev.index == U.device.index)
            self.U = U if same else U.half().to(device)
            self.SV = SV.half().to(device).contiguous()
            self._sync_tiled()

    def set_bias(self, bias):
        self.bias_param = None if bias is None else bias.half()
        self._sync_tiled()

    def _sync_tiled(self):
        if self._tiled is None:
            if self._dense is not None:
                ok = self.U is not None and self.SV is not None
                self._ut = tiled.tiled_ut(self.U) if ok else None
                self._sv_dense = TiledWeight.from_dense(self.SV.contiguous()) if ok else None
            return
        if self.SV is not None:
            self._tiled.put_sv(0, self.SV)
        else:
            self._tiled.clear_sv()
        self._tiled.set_bias(self.bias_param)
        self._ut = tiled.tiled_ut(self.U) if (self.U is not None and self.SV is not None) else None

    # ---- checks -------------------------------------------------------------------------------
    def _dequant_gptq(self):
        """fp16 weight tile fp16((q - z) * s) read back from the tiled codes
        (inference/quantized_linear.py:271-284)."""
        if self._tiled is None:
            raise RuntimeError("weights are not in the tiled layout")
        return self._tiled.dequantize()

    # ---- forward (inference/quantized_linear.py:286-355) ------------------------------------
    def _rotate(self, x):
        if self._rht_signs is not None:
            from .hadamard_rotation import rht_forward_half
            return rht_forward_half(x, self._rht_signs)
        Pi = self._rotation_cache.get_pi(self.turbo_dim, self.turbo_bits, self.turbo_seed)
        return (x.float() @ Pi.float().T).half()

    def _forward_dense(self, x, a):
        y = tiled.dense_matmul(self._dense, x)
        if self.SV is not None:
            if a is None:
                a = tiled.dense_matmul(self._ut, x)
            y = y + tiled.dense_matmul(self._sv_dense, a.contiguous())
        if self.bias_param is not None:
            y = y + self.bias_param
        return y

    def forward(self, x, precomputed_xU=None, precomputed_x_rot=None):
        orig_shape = x.shape
        in_dtype = x.dtype
        if x.dim() != 2:
            x = x.reshape(-1, self.in_features)
        if x.dtype != torch.float16:
            x = x.half()
        x = x.contiguous()
        a = None
        if precomputed_xU is not None and self.SV is not None:
            a = precomputed_xU.reshape(-1, self.SV.shape[1]).to(torch.float16)

        if self._tiled is None and self._dense is not None:
            y = self._forward_dense(x, a)
        elif self.quant_type == "gptq":
            if self._tiled is not None:
                y = tiled.linear_forward(self._tiled, x, ut=self._ut, a=a)
            else:
                y = gptq_dequant_matmul_fused(x, self.qweight_int, self.scales, self.zeros,
                                              self.gptq_groupsize, self.gptq_sym, lora_USV=None)
                if self.SV is not None:
                    if a is None:
                        a = tiled.dense_matmul(tiled.tiled_ut(self.U), x)
                    y = y + a @ self.SV.T
                if self.bias_param is not None:
                    y = y + self.bias_param
        elif self.quant_type == "turbo":
            if self._tiled is None:
                raise RuntimeError("TurboQuant weights not loaded")
            if precomputed_x_rot is not None:
                x_rot = precomputed_x_rot.reshape(-1, self.in_features)
                if x_rot.dtype != torch.float16:
                    x_rot = x_rot.half()
                x_rot = x_rot.contiguous()
            else:
                x_rot = self._rotate(x)
            if self.SV is not None and a is None:
                a = tiled.dense_matmul(self._ut, x)          # the low-rank term sees the unrotated x
            y = tiled.linear_forward(self._tiled, x_rot, ut=None, a=a)
        else:
            raise RuntimeError(f"Unknown quant_type: {self.quant_type}")

        if len(orig_shape) != 2:
            y = y.reshape(*orig_shape[:-1], self.out_features)
        # the kernels compute in fp16; other floating-point inputs get their own dtype back
        return y if in_dtype == torch.float16 or not in_dtype.is_floating_point else y.to(in_dtype)

    def extra_repr(self):
        s = f"in_features={self.in_features}, out_features={self.out_features}, quant_type={self.quant_type}"
        if self.U is not None:
            s += f", lora_rank={self.U.shape[1]}"
        return s


# ---------------------------------------------------------------------------------------------
# GLoRCQExperts: fused-experts adapter (inference/quantized_linear.py:368-428)
# ---------------------------------------------------------------------------------------------
class GLoRCQExperts(nn.Module):
    """Drop-in for the transformers-5.x style ``XxxExperts`` modules: three per-expert lists of
    ``GLoRCQLinear`` (gate, up, down) and ``forward(hidden_states (T,H), top_k_index (T,k), top_k_weights
    (T,k)) -> (T,H)``.

    The reference loops over the experts that were hit on the host (one-hot mask, ``nonzero``, three
    linears per expert, ``index_add_``).  Here the routing tensors go to the device-side block path
    (per-expert token lists, grouped gate|up + SwiGLU and down kernels, sum in expert order) in one call;
    nothing is read back and the call can be captured into a graph.  ``act_fn`` must be SiLU.
    """

    def __init__(self, num_experts, hidden_dim, intermediate_dim, act_fn):
        super().__init__()
        self.num_experts = num_experts
        self.hidden_dim = hidden_dim
        self.intermediate_dim = intermediate_dim
        self.gate_experts = nn.ModuleList([GLoRCQLinear(hidden_dim, intermediate_dim) for _ in range(num_experts)])
        self.up_experts = nn.ModuleList([GLoRCQLinear(hidden_dim, intermediate_dim) for _ in range(num_experts)])
        self.down_experts = nn.ModuleList([GLoRCQLinear(intermediate_dim, hidden_dim) for _ in range(num_experts)])
        self.act_fn = act_fn
        self._block = None

    def _routed(self, top_k):
        if self._block is None or self._block.top_k != top_k:
            import torch.nn.functional as F
            from types import SimpleNamespace
            from .moe_block import GraphCompatibleMoeBlock
            if self.act_fn not in (F.silu,) and not isinstance(self.act_fn, nn.SiLU):
                raise RuntimeError("the fused expert kernels implement SiLU gating only")
            shim = SimpleNamespace(num_experts=self.num_experts, top_k=top_k, norm_topk_prob=False, gate=None,
                                   experts=[SimpleNamespace(gate_proj=g, up_proj=u, down_proj=d) for g, u, d in
                                            zip(self.gate_experts, self.up_experts, self.down_experts)],
                                   shared_expert=None, shared_expert_gate=None)
            blk = GraphCompatibleMoeBlock(shim)
            blk._graph_threshold = 0          # always the expert-order sum of index_add_
            self._block = blk
        return self._block

    def forward(self, hidden_states, top_k_index, top_k_weights):
        if not hidden_states.is_cuda:
            raise RuntimeError("GLoRCQExperts runs on a CUDA device only (no CPU path)")
        T, H = hidden_states.shape
        blk = self._routed(top_k_index.shape[1])
        out, _ = blk(hidden_states.reshape(1, T, H), top_k_index=top_k_index, top_k_weights=top_k_weights)
        return out.reshape(T, H).to(hidden_states.dtype)
