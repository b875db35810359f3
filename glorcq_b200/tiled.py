"""Weights in the tiled device layout of the sm_100a kernels, and the calls that consume them.

`TiledWeight` owns the re-tiled tensors of one matrix (built once at load time by the
glq_pack_* entry points) and hands out the glq_weight_t descriptor the C ABI takes.  The shared
input-side factor U of a cluster is tiled once (as U^T, dense fp16) and cached by storage, so
every layer of the cluster points at the same device memory -- the "global U pool" the reference's
loader builds (inference/model_builder.py:143-173) but its compute path never reads.
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import FMT_F16, FMT_Q2, FMT_Q4, FMT_T2, Weight


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _need_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (glorcq_b200 has no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


class TiledWeight:
    """One weight matrix (N, K) in the tiled layout."""

    def __init__(self, fmt: int, N: int, K: int, group_size: int = 0):
        self.fmt, self.N, self.K, self.group_size = fmt, N, K, group_size
        self.codes = self.sz = self.norms = self.centroids = self.sv = self.bias = None
        self.rank = 0
        self._desc = None

    # ---- constructors -------------------------------------------------------------------
    @classmethod
    def from_gptq(cls, qweight_int, scales, zeros, bits, groupsize, sym=False):
        """(N,K) int32 codes in [0, 2^bits) + (N,G) fp16 scales/zeros -> Q2 / Q4 tiles."""
        _need_cuda(qweight_int, "qweight_int")
        _need_cuda(scales, "scales")
        if bits not in (2, 4):
            raise RuntimeError(f"tiled layout covers 2- and 4-bit codes, got bits={bits}")
        N, K = qweight_int.shape
        kb = 128 if bits == 2 else 64
        if groupsize <= 0 or groupsize % kb != 0:
            raise RuntimeError(f"group size {groupsize} must be a positive multiple of {kb} for {bits}-bit codes")
        G = scales.shape[1]
        if G != (K + groupsize - 1) // groupsize:
            raise RuntimeError("scales shape does not match K / groupsize")
        L = _lib.lib()
        fmt = FMT_Q2 if bits == 2 else FMT_Q4
        self = cls(fmt, N, K, groupsize)
        dev = qweight_int.device
        q32 = qweight_int if qweight_int.dtype == torch.int32 else qweight_int.to(torch.int32)
        self.codes = torch.empty(L.glq_tiled_codes_bytes(fmt, N, K), dtype=torch.uint8, device=dev)
        self.sz = torch.empty(L.glq_tiled_sz_bytes(N, G), dtype=torch.uint8, device=dev)
        st = _stream_ptr(dev)
        with torch.cuda.device(dev):
            _lib.check(L.glq_pack_codes_i32(q32.data_ptr(), bits, N, K, self.codes.data_ptr(), st), "pack_codes_i32")
            z = None if (sym or zeros is None) else zeros.to(torch.float16).contiguous()
            s = scales.to(torch.float16).contiguous()
            _lib.check(L.glq_pack_sz(s.data_ptr(), _ptr(z), N, G, self.sz.data_ptr(), st), "pack_sz")
        return self

    @classmethod
    def from_turbo(cls, packed_indices, norms, centroids):
        """(N,K/4) uint8 2-bit indices + (N,) norms + (4,) codebook -> T2 tiles."""
        _need_cuda(packed_indices, "packed_indices")
        N, K4 = packed_indices.shape
        K = K4 * 4
        L = _lib.lib()
        self = cls(FMT_T2, N, K)
        dev = packed_indices.device
        self.codes = torch.empty(L.glq_tiled_codes_bytes(FMT_T2, N, K), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(L.glq_pack_codes_u8(packed_indices.data_ptr(), N, K, self.codes.data_ptr(), _stream_ptr(dev)),
                       "pack_codes_u8")
        self.norms = norms.to(device=dev, dtype=torch.float32).contiguous()
        self.centroids = centroids.to(device=dev, dtype=torch.float32).contiguous()
        return self

    @classmethod
    def from_dense(cls, W: torch.Tensor, transposed: bool = False):
        """fp16 matrix -> F16 tiles.  transposed=True tiles W^T, i.e. W is (K, N) as U is."""
        if not W.is_cuda:
            raise RuntimeError("W must be a CUDA tensor")
        W = W.to(torch.float16)
        if transposed:
            K, N = W.shape
            sn, sk = W.stride(1), W.stride(0)
        else:
            N, K = W.shape
            sn, sk = W.stride(0), W.stride(1)
        L = _lib.lib()
        self = cls(FMT_F16, N, K)
        self.codes = torch.empty(L.glq_tiled_codes_bytes(FMT_F16, N, K), dtype=torch.uint8, device=W.device)
        with torch.cuda.device(W.device):
            _lib.check(L.glq_pack_f16(W.data_ptr(), sn, sk, N, K, self.codes.data_ptr(), _stream_ptr(W.device)),
                       "pack_f16")
        self._keep = W
        return self

    # ---- low-rank / bias attachments ------------------------------------------------------
    def set_sv(self, SV: Optional[torch.Tensor]):
        if SV is None:
            self.sv, self.rank = None, 0
        else:
            if SV.shape[0] != self.N or SV.shape[1] % 16 != 0:
                raise RuntimeError("SV must be (N, rank) with rank a multiple of 16")
            self.sv = SV.to(torch.float16).contiguous()
            self.rank = SV.shape[1]
        self._desc = None

    def set_bias(self, bias: Optional[torch.Tensor]):
        self.bias = None if bias is None else bias.to(torch.float16).contiguous()
        self._desc = None

    @property
    def desc(self) -> Weight:
        if self._desc is None:
            self._desc = Weight(_ptr(self.codes), _ptr(self.sz), _ptr(self.norms), _ptr(self.centroids),
                                _ptr(self.sv), _ptr(self.bias), self.N, self.K, self.rank, 0)
        return self._desc

    def desc_bytes(self) -> bytes:
        return bytes(self.desc)

    @property
    def device(self):
        return self.codes.device

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.codes, self.sz, self.norms, self.sv, self.bias)
                   if t is not None)

    # ---- checks ------------------------------------------------------------------------------
    def dequantize(self) -> torch.Tensor:
        """Dequantised (N,K) weights from the tiles: fp16 for Q2/Q4, fp32 for T2."""
        L = _lib.lib()
        dt = torch.float32 if self.fmt == FMT_T2 else torch.float16
        out = torch.empty(self.N, self.K, dtype=dt, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(L.glq_dequant_tiled(self.fmt, C.byref(self.desc), self.group_size, out.data_ptr(),
                                           _stream_ptr(self.device)), "dequant_tiled")
        return out


# ---- shared U pool ---------------------------------------------------------------------------
_UT_POOL: Dict[Tuple[int, int, int, int], TiledWeight] = {}


def tiled_ut(U: torch.Tensor) -> TiledWeight:
    """U^T of a shared (K, r) factor in the dense tiled layout, one copy per distinct storage."""
    key = (U.device.index or 0, U.data_ptr(), U.shape[0], U.shape[1])
    tw = _UT_POOL.get(key)
    if tw is None:
        tw = TiledWeight.from_dense(U, transposed=True)
        _UT_POOL[key] = tw
    return tw


def clear_pool():
    _UT_POOL.clear()


# ---- workspaces ------------------------------------------------------------------------------
_WS: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]] = {}


def workspace(device, nbytes: int, ncounters: int = 0):
    """(scratch, counters) for the current stream of `device`.  The scratch holds split-k partial
    sums and small intermediates and needs no initialisation.  The counters are arrival counters:
    they must be zero before a call and every kernel leaves them zero, so they are cleared only
    when the array is (re)allocated."""
    key = (torch.device(device).index or 0, _stream_ptr(device))
    ws, ctr = _WS.get(key, (None, None))
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    if ctr is None or ctr.numel() < ncounters:
        ctr = torch.zeros(max(ncounters, 1 << 16), dtype=torch.int32, device=device)
    _WS[key] = (ws, ctr)
    return ws, ctr


# ---- calls -----------------------------------------------------------------------------------
def linear_forward(w: TiledWeight, x: torch.Tensor, ut: Optional[TiledWeight] = None,
                   a: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = Q(x) + a . SV^T + bias on (B, K) fp16 rows; a = x . U is taken from `a`, or computed
    from `ut`, or absent."""
    if x.dtype != torch.float16:
        raise RuntimeError("x must be fp16")
    _need_cuda(x, "x")
    B = x.shape[0]
    y = torch.empty(B, w.N, dtype=torch.float16, device=x.device)
    if B == 0 or w.N == 0:
        return y
    L = _lib.lib()
    if a is not None:
        if a.dtype != torch.float16 or a.shape != (B, w.rank):
            raise RuntimeError("precomputed x@U must be fp16 of shape (B, rank)")
        a = a.contiguous()
    with torch.cuda.device(x.device):
        nbytes = L.glq_linear_workspace_bytes(w.fmt, w.group_size, C.byref(w.desc), B)
        nctr = L.glq_linear_counters(w.fmt, w.group_size, C.byref(w.desc), B)
        ws, ctr = workspace(x.device, nbytes, nctr)
        _lib.check(L.glq_linear_forward(w.fmt, w.group_size, C.byref(w.desc), None if ut is None else _ptr(ut.codes),
                                        x.data_ptr(), x.stride(0), _ptr(a), y.data_ptr(), w.N, B,
                                        ws.data_ptr(), ws.numel(), ctr.data_ptr(), ctr.numel(),
                                        _stream_ptr(x.device)), "linear_forward")
    return y


def dense_matmul(w: TiledWeight, x: torch.Tensor) -> torch.Tensor:
    """y = x . W^T for a dense tiled weight (used for a = x . U with W = U^T)."""
    return linear_forward(w, x)
