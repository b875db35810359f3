"""Reader of the reference's on-disk format and builder of the quantized layers.

Mirror of the loader in inference/model_builder.py (lines 27-66 SharedUCache, 69-80 the integer
decoders, 86-137 RotationCache, 143-183 the U pool, 335-450 layer replacement, 465-544 low-rank
loading, 203-312 load_glorcq_model).  The format is unchanged:

``glorcq_model.pt``      {"model_config": {...}, "layers": {layer_idx: {module_name: D}}} with D one of
    {qweight_int (N,K) int32, scales (N,G) fp16, zeros (N,G) fp16, bits, groupsize, sym}          (integer codes)
    {packed_indices (N,K/4) uint8, norms (N,), bits, dim, seed[, rotation_type]}                 (codebook)
``cross_layer_info.pt``  {"config", "assignments": {wtype: [{layer, expert, group_id}]},
    "shared_matrices": {wtype: {gid: {U_fp16} | {U_int4_packed, U_scale, U_orig_rows} | {U_int8, U_scale} [, S]}},
    "per_expert_V": {wtype: [{SV_int4_packed, SV_scale, SV_orig_rows} | {SV_fp16} | {SV_int8, SV_scale}
                             | {V_int8, V_scale}]}}

Where the reference instantiates a transformers model and swaps its ``nn.Linear`` modules, this reader
is independent of the transformers version: ``build_layers`` returns the ``GLoRCQLinear`` modules keyed
by (layer index, module name), and ``load_glorcq_model`` assembles them into this package's decoder
(``glorcq_b200.decoder``) from the checkpoint's ``config.json``.
"""

from __future__ import annotations

import json
import logging
import os
import sys
from typing import Dict, Optional, Tuple

import torch

from .quantized_linear import GLoRCQLinear

logger = logging.getLogger(__name__)

WTYPES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "w1", "w2", "w3")
_MIXTRAL = {"w1": "gate_proj", "w2": "down_proj", "w3": "up_proj"}


# ---- integer decoders (inference/model_builder.py:69-80) -----------------------------------------
def _dequant_intN(q, scale, nbits):
    """intN codes held in int8 -> float32 with a per-column scale: q / (2^(nbits-1) - 1) * scale."""
    maxval = 2 ** (nbits - 1) - 1
    return q.float() / maxval * scale.float()


def _unpack_int4(packed, orig_rows):
    """((rows+1)//2, cols) uint8 -> (orig_rows, cols) int8 in [-7, 7]; even rows in the low nibble, odd
    rows in the high nibble, each stored as q + 7."""
    lo = (packed & 0xF).to(torch.int8) - 7
    hi = ((packed >> 4) & 0xF).to(torch.int8) - 7
    return torch.stack([lo, hi], dim=1).reshape(-1, packed.shape[1])[:orig_rows]


def _pack_int4(q):
    """Inverse of _unpack_int4 (the writer's side, cross_layer_share.py:622-648): (rows, cols) int8 in
    [-7, 7] -> ((rows+1)//2, cols) uint8."""
    rows = q.shape[0]
    if rows % 2:
        q = torch.cat([q, torch.zeros(1, q.shape[1], dtype=q.dtype, device=q.device)], 0)
    u = (q + 7).to(torch.uint8)
    return (u[0::2] | (u[1::2] << 4)).contiguous()


# ---- shared U factors (inference/model_builder.py:27-66) ------------------------------------------
class SharedUCache:
    """All cluster-shared U matrices, decoded to fp16 on the device once.  ``get(wtype, gid)`` returns
    (U (in, r) fp16, S or None); every layer of a cluster receives the same tensor object, so the
    tiled U^T is built once per cluster (glorcq_b200.tiled.tiled_ut)."""

    def __init__(self, shared_matrices, uv_bits, device="cuda", u_bits=None):
        self._cache = {}
        _u_bits = u_bits if u_bits is not None else uv_bits
        for wtype, groups in shared_matrices.items():
            for gid, data in groups.items():
                if "U_fp16" in data:
                    U = data["U_fp16"].half().to(device)
                elif "U_int4_packed" in data:
                    rows = int(data["U_orig_rows"].item())
                    U = _dequant_intN(_unpack_int4(data["U_int4_packed"].to(device), rows), data["U_scale"].to(device), 4).half()
                else:
                    U = _dequant_intN(data["U_int8"].to(device), data["U_scale"].to(device), _u_bits).half()
                S = data["S"].half().to(device) if "S" in data else None
                self._cache[(wtype, gid)] = (U.contiguous(), S)

    def get(self, wtype, group_id):
        return self._cache.get((wtype, group_id), (None, None))

    def preload_for_layer(self, layer_idx, active_experts=None):
        pass

    def evict(self, wtype=None, group_id=None):
        pass


# ---- rotations of the codebook format (inference/model_builder.py:86-137) ---------------------------
class RotationCache:
    """Rotation matrix Pi (dim, dim) fp16 and codebook centroids (2^bits,) fp32 per (dim, bits, seed).

    The reference derives both from the third-party ``turboquant`` package (expected under
    ``thirdpart/turboquant``).  ``register`` does the same when that package can be imported; hosts that
    have the tensors already hand them over with ``put``.
    """

    def __init__(self, device="cuda", turboquant_path: Optional[str] = None):
        self._device = device
        self._pi, self._centroids = {}, {}
        self._tq_path = turboquant_path

    def put(self, dim, bits, seed, Pi, centroids):
        self._pi[(dim, bits, seed)] = Pi.to(self._device).half()
        self._centroids[(dim, bits, seed)] = centroids.to(self._device).float()

    def register(self, dim, bits, seed=42):
        key = (dim, bits, seed)
        if key in self._pi:
            return
        if self._tq_path and self._tq_path not in sys.path:
            sys.path.insert(0, self._tq_path)
        try:
            from turboquant.quantizer import TurboQuantMSE
        except ImportError as e:
            raise RuntimeError(
                f"rotation ({dim}, {bits}, {seed}) is not registered and the turboquant package that derives it "
                "is not importable; call RotationCache.put(dim, bits, seed, Pi, centroids) or pass "
                "turboquant_path") from e
        tq = TurboQuantMSE(dim=dim, bits=bits, device=self._device, dtype=torch.float32, seed=seed)
        self._pi[key] = tq.Pi.half()
        self._centroids[key] = tq.centroids

    def get_pi(self, dim, bits, seed=42):
        return self._pi[(dim, bits, seed)]

    def get_centroids(self, dim, bits, seed=42):
        return self._centroids[(dim, bits, seed)]


# ---- module names (utils/moe_utils.py:9-36) ---------------------------------------------------------
def is_shared_expert(name: str) -> bool:
    return "shared_expert" in name


def is_regular_expert(name: str) -> bool:
    return (".experts." in name or name.startswith("experts.")) and not is_shared_expert(name)


def extract_expert_index(name: str) -> Optional[int]:
    parts = name.split(".")
    return int(parts[parts.index("experts") + 1]) if "experts" in parts else None


def module_key(module_name: str) -> Tuple[Optional[str], int]:
    """(projection type, expert index) as the loader derives them (inference/model_builder.py:473-497):
    expert index -1 for attention and dense projections, -2 for the shared expert (which gets no low-rank
    term), the routed expert's number otherwise; Mixtral's w1/w2/w3 map to gate/down/up."""
    if is_regular_expert(module_name):
        idx = extract_expert_index(module_name)
        expert = idx if idx is not None else -3
    elif is_shared_expert(module_name):
        expert = -2
    else:
        expert = -1
    wtype = None
    for wt in WTYPES:
        if module_name == wt or module_name.endswith("." + wt):
            wtype = _MIXTRAL.get(wt, wt)
            break
    return wtype, expert


def assignment_lookup(assignments) -> Dict[Tuple[str, int, int], Tuple[int, str, int]]:
    """(wtype, layer, expert) -> (group id, wtype, index into per_expert_V[wtype])."""
    out = {}
    for wtype, records in assignments.items():
        for li, rec in enumerate(records):
            out[(wtype, rec["layer"], rec["expert"])] = (rec["group_id"], wtype, li)
    return out


def _load_lora_for_module(ql, layer_idx, module_name, lookup, u_cache, per_expert_V, uv_bits, device, sv_bits=None):
    """Attach (U, SV) to one layer (inference/model_builder.py:465-544): new formats carry the fused SV
    (int4-packed, fp16 or intN), the old one V and the cluster's S."""
    wtype, expert = module_key(module_name)
    if wtype is None or expert == -2:
        return
    key = (wtype, layer_idx, expert)
    if key not in lookup:
        return
    group_id, wtype_key, local_idx = lookup[key]
    U, S_shared = u_cache.get(wtype_key, group_id)
    if U is None:
        return
    v_list = per_expert_V.get(wtype_key)
    if v_list is None or v_list[local_idx] is None:
        return
    v = v_list[local_idx]
    if "SV_int4_packed" in v:
        rows = int(v["SV_orig_rows"].item())
        SV = _dequant_intN(_unpack_int4(v["SV_int4_packed"].to(device), rows), v["SV_scale"].to(device), 4).half()
        ql.load_sv(U, SV, device=device)
    elif "SV_fp16" in v:
        ql.load_sv(U, v["SV_fp16"].to(device).half(), device=device)
    elif "SV_int8" in v:
        bits = sv_bits if sv_bits is not None else uv_bits
        ql.load_sv(U, _dequant_intN(v["SV_int8"].to(device), v["SV_scale"].to(device), bits).half(), device=device)
    else:
        V = _dequant_intN(v["V_int8"].to(device), v["V_scale"].to(device), uv_bits).half()
        ql.load_lora(U, S_shared, V, device=device)
    ql.cluster_id = (wtype_key, group_id)


# ---- checkpoint -> layers ------------------------------------------------------------------------------
def read_checkpoint(model_path):
    """(model_config, layers_data, cross_layer_info, hf_config) of a real-quant checkpoint directory."""
    gp = os.path.join(model_path, "glorcq_model.pt")
    cp = os.path.join(model_path, "cross_layer_info.pt")
    if not os.path.exists(gp):
        raise FileNotFoundError(f"glorcq_model.pt not found in {model_path}. This model was likely saved in "
                                "fake-quant mode. Use standard HF loading instead.")
    model_data = torch.load(gp, map_location="cpu", weights_only=False)
    cross = torch.load(cp, map_location="cpu", weights_only=False)
    hf = {}
    cj = os.path.join(model_path, "config.json")
    if os.path.exists(cj):
        with open(cj) as f:
            hf = json.load(f)
    return model_data["model_config"], model_data["layers"], cross, hf


def lora_bits(model_config, cl_config):
    uv_bits = cl_config.get("uv_bits", model_config.get("uv_bits", 8))
    return uv_bits, cl_config.get("u_bits", uv_bits), cl_config.get("sv_bits", uv_bits)


def build_layers(model_config, layers_data, cross_layer_info, device="cuda", rotation_cache=None, u_cache=None,
                 biases=None):
    """{layer_idx: {module_name: GLoRCQLinear}} for every quantized module of the checkpoint
    (the body of _replace_linear_layers, inference/model_builder.py:335-450, without the host model).
    `biases` may map (layer_idx, module_name) to a bias tensor.  Returns (layers, u_cache)."""
    uv_bits, u_bits, sv_bits = lora_bits(model_config, cross_layer_info["config"])
    if u_cache is None:
        u_cache = SharedUCache(cross_layer_info["shared_matrices"], uv_bits, device=device, u_bits=u_bits)
    if rotation_cache is None and model_config.get("use_turboquant", False):
        rotation_cache = RotationCache(device=device)
    lookup = assignment_lookup(cross_layer_info["assignments"])
    per_expert_V = cross_layer_info["per_expert_V"]
    out = {}
    for layer_idx, layer_data in layers_data.items():
        mods = {}
        for module_name, packed in layer_data.items():
            if "qweight_int" in packed:
                out_f, in_f = packed["qweight_int"].shape
                ql = GLoRCQLinear(in_f, out_f)
                ql.load_gptq(packed, device=device)
            elif "packed_indices" in packed:
                out_f, in_f = packed["packed_indices"].shape[0], packed["dim"]
                ql = GLoRCQLinear(in_f, out_f)
                if rotation_cache is None:
                    raise RuntimeError("codebook-format layers need a RotationCache")
                ql.load_turbo(packed, rotation_cache, device=device)
            elif "weight_quant" in packed:
                # pre-dequantised weights: kept dense (inference/model_builder.py:386-415 loads them the same way)
                out_f, in_f = packed["weight_quant"].shape
                ql = GLoRCQLinear(in_f, out_f)
                ql.load_dense(packed["weight_quant"], device=device, quant_type=packed.get("quant_method", "dense"))
            else:
                # unknown record: the reference leaves the original (zero-initialised) layer in place
                logger.warning("layer %s module %s: unknown record %s, skipped", layer_idx, module_name, sorted(packed))
                continue
            _load_lora_for_module(ql, layer_idx, module_name, lookup, u_cache, per_expert_V, uv_bits, device,
                                  sv_bits=sv_bits)
            if biases and (layer_idx, module_name) in biases:
                ql.set_bias(biases[(layer_idx, module_name)].to(device))
            mods[module_name] = ql
        out[layer_idx] = mods
    if model_config.get("rotation_type", "qr") == "hadamard":          # inference/model_builder.py:277-286
        from .hadamard_rotation import generate_rht_signs
        for mods in out.values():
            for m in mods.values():
                if m.quant_type == "turbo":
                    m._rht_signs = generate_rht_signs(m.turbo_dim, seed=m.turbo_seed, device=device)
    return out, u_cache


def _build_global_u_pool(u_cache):
    """Pools of the unique cluster U matrices per projection type and the (wtype, gid) -> column index
    maps (inference/model_builder.py:143-172).  This package keeps one tiled U^T per distinct tensor
    instead (tiled.tiled_ut), so the pools are informational."""
    by_type = {"gate_proj": [], "up_proj": [], "down_proj": []}
    for (wtype, gid), (U, _S) in u_cache._cache.items():
        if wtype in by_type:
            by_type[wtype].append((gid, U))
    pools, id_maps = {}, {}
    for wtype, items in by_type.items():
        if not items:
            continue
        items.sort(key=lambda it: it[0])
        key = wtype.split("_")[0]
        pools[key] = torch.cat([u for _, u in items], dim=1)
        id_maps[key] = {(wtype, gid): i for i, (gid, _) in enumerate(items)}
    return pools, id_maps


def load_glorcq_model(model_path, device="cuda:0", rotation_cache=None):
    """Load a real-quant checkpoint directory (config.json, glorcq_model.pt, cross_layer_info.pt) into
    this package's decoder; same call as the reference's loader (inference/model_builder.py:203)."""
    from .decoder import GLoRCQDecoder
    model_config, layers_data, cross, hf = read_checkpoint(model_path)
    if not hf:
        raise FileNotFoundError(f"config.json not found in {model_path}")
    layers, u_cache = build_layers(model_config, layers_data, cross, device=device, rotation_cache=rotation_cache)
    extra = None
    ep = os.path.join(model_path, "dense_weights.pt")     # embeddings, norms, lm_head, router weights (fp16)
    if os.path.exists(ep):
        extra = torch.load(ep, map_location="cpu", weights_only=False)
    model = GLoRCQDecoder(hf, layers, dense=extra, device=device)
    model.seqlen = 4096
    model.u_cache = u_cache
    return model
