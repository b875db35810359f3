"""Weights in the tiled device layout of the sm_100a kernels, and the calls that consume them.

`TiledWeight` owns the re-tiled tensors of one matrix -- or of a fused gate|up pair -- built once at
load time by the glq_pack_* entry points, and hands out the glq_weight_t descriptor the C ABI takes.
The shared input-side factor U of a cluster is tiled once (as U^T, dense fp16) and cached by
storage, so every layer of the cluster points at the same device memory: the "global U pool" the
reference's loader builds (inference/model_builder.py:143-173) but its compute path never reads.
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
    """One weight matrix (N, K) -- or two of the same shape fused tile by tile (count == 2: slot 0
    is the gate projection, slot 1 the up projection) -- in the tiled layout."""

    def __init__(self, fmt: int, N: int, K: int, group_size: int = 0, count: int = 1, device=None):
        self.fmt, self.N, self.K, self.group_size, self.count = fmt, N, K, group_size, count
        self.codes = self.norms = self.centroids = self.sv = self.bias = None
        self.rank = 0
        self._desc = None
        self._device = device
        L = _lib.lib()
        if fmt == FMT_F16:
            nbytes = L.glq_tiled_f16_bytes(N, K)
        else:
            nbytes = L.glq_tiled_bytes(fmt, N, K, count)
        # zero-filled: padding tiles and padding columns are never written by the pack kernels
        self.codes = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        if fmt == FMT_T2:
            self.norms = torch.zeros(L.glq_rows_f32_count(N, count), dtype=torch.float32, device=device)

    # ---- filling one slot -----------------------------------------------------------------
    def put_gptq(self, slot, qweight_int, scales, zeros, bits, sym=False):
        _need_cuda(qweight_int, "qweight_int")
        _need_cuda(scales, "scales")
        N, K = qweight_int.shape
        if (N, K) != (self.N, self.K):
            raise RuntimeError("shape mismatch between fused matrices")
        G = scales.shape[1]
        if G != (K + self.group_size - 1) // self.group_size:
            raise RuntimeError("scales shape does not match K / groupsize")
        q32 = qweight_int if qweight_int.dtype == torch.int32 else qweight_int.to(torch.int32)
        s = scales.to(torch.float16).contiguous()
        z = None if (sym or zeros is None) else zeros.to(torch.float16).contiguous()
        with torch.cuda.device(self.codes.device):
            _lib.check(_lib.lib().glq_pack_gptq(q32.data_ptr(), s.data_ptr(), _ptr(z), bits, N, K, self.group_size,
                                                self.codes.data_ptr(), slot, self.count,
                                                _stream_ptr(self.codes.device)), "pack_gptq")

    def put_turbo(self, slot, packed_indices, norms, centroids):
        _need_cuda(packed_indices, "packed_indices")
        N, K4 = packed_indices.shape
        if (N, K4 * 4) != (self.N, self.K):
            raise RuntimeError("shape mismatch between fused matrices")
        dev = self.codes.device
        nrm = norms.to(device=dev, dtype=torch.float32).contiguous()
        cen = centroids.to(device=dev, dtype=torch.float32).contiguous()
        if self.centroids is not None and not torch.equal(self.centroids, cen):
            raise RuntimeError("fused codebook weights must share one codebook")
        self.centroids = cen
        L = _lib.lib()
        with torch.cuda.device(dev):
            _lib.check(L.glq_pack_turbo(packed_indices.data_ptr(), N, self.K, self.codes.data_ptr(), slot, self.count,
                                        _stream_ptr(dev)), "pack_turbo")
            _lib.check(L.glq_pack_rows_f32(nrm.data_ptr(), N, self.norms.data_ptr(), slot, self.count,
                                           _stream_ptr(dev)), "pack_rows_f32")

    def put_sv(self, slot, SV: Optional[torch.Tensor]):
        """Attach the (N, rank) output-side factor of the matrix in `slot` (packed layout)."""
        self._desc = None
        if SV is None:
            return
        if SV.shape[0] != self.N or SV.shape[1] % 16 != 0:
            raise RuntimeError("SV must be (N, rank) with rank a multiple of 16")
        rank = SV.shape[1]
        L = _lib.lib()
        dev = self.codes.device
        if self.sv is None or self.rank != rank:
            self.sv = torch.zeros(L.glq_sv_bytes(self.N, rank, self.count), dtype=torch.uint8, device=dev)
            self.rank = rank
        src = SV.to(device=dev, dtype=torch.float16).contiguous()
        with torch.cuda.device(dev):
            _lib.check(L.glq_pack_sv(src.data_ptr(), self.N, rank, self.sv.data_ptr(), slot, self.count,
                                     _stream_ptr(dev)), "pack_sv")

    def clear_sv(self):
        self.sv, self.rank, self._desc = None, 0, None

    def set_bias(self, bias: Optional[torch.Tensor]):
        if bias is not None and self.count != 1:
            raise RuntimeError("bias is only supported on plain (un-fused) weights")
        self.bias = None if bias is None else bias.to(device=self.codes.device, dtype=torch.float16).contiguous()
        self._desc = None

    # ---- constructors -------------------------------------------------------------------
    @staticmethod
    def _gptq_fmt(bits, groupsize):
        if bits not in (2, 4):
            raise RuntimeError(f"tiled layout covers 2- and 4-bit codes, got bits={bits}")
        kb = 128 if bits == 2 else 64
        if groupsize <= 0 or groupsize % kb != 0:
            raise RuntimeError(f"group size {groupsize} must be a positive multiple of {kb} for {bits}-bit codes")
        return FMT_Q2 if bits == 2 else FMT_Q4

    @classmethod
    def from_gptq(cls, qweight_int, scales, zeros, bits, groupsize, sym=False):
        """(N,K) int32 codes in [0, 2^bits) + (N,G) fp16 scales/zeros -> Q2 / Q4 tiles."""
        fmt = cls._gptq_fmt(bits, groupsize)
        N, K = qweight_int.shape
        self = cls(fmt, N, K, groupsize, 1, qweight_int.device)
        self.put_gptq(0, qweight_int, scales, zeros, bits, sym)
        return self

    @classmethod
    def from_turbo(cls, packed_indices, norms, centroids):
        """(N,K/4) uint8 2-bit indices + (N,) norms + (4,) codebook -> T2 tiles."""
        N, K4 = packed_indices.shape
        self = cls(FMT_T2, N, K4 * 4, 0, 1, packed_indices.device)
        self.put_turbo(0, packed_indices, norms, centroids)
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
        self = cls(FMT_F16, N, K, 0, 1, W.device)
        with torch.cuda.device(W.device):
            _lib.check(_lib.lib().glq_pack_f16(W.data_ptr(), sn, sk, N, K, self.codes.data_ptr(),
                                               _stream_ptr(W.device)), "pack_f16")
        return self

    # ---- descriptor ---------------------------------------------------------------------------
    @property
    def desc(self) -> Weight:
        if self._desc is None:
            self._desc = Weight(_ptr(self.codes), None, _ptr(self.norms), _ptr(self.centroids),
                                _ptr(self.sv), _ptr(self.bias), self.N, self.K, self.rank, 0)
        return self._desc

    def desc_bytes(self) -> bytes:
        return bytes(self.desc)

    @property
    def device(self):
        return self.codes.device

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.codes, self.norms, self.sv, self.bias)
                   if t is not None)

    # ---- checks ------------------------------------------------------------------------------
    def dequantize(self, slot: int = 0) -> torch.Tensor:
        """Dequantised (N,K) weights of the matrix in `slot`: fp16 for Q2/Q4, fp32 for T2."""
        L = _lib.lib()
        dt = torch.float32 if self.fmt == FMT_T2 else torch.float16
        out = torch.empty(self.N, self.K, dtype=dt, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(L.glq_dequant_tiled(self.fmt, self.codes.data_ptr(), _ptr(self.norms), _ptr(self.centroids),
                                           self.N, self.K, slot, self.count, out.data_ptr(),
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
        tw._keep = U           # the key is the storage address: keep it alive
        _UT_POOL[key] = tw
    return tw


_UT_RM_POOL: Dict[Tuple[int, int, int, int], torch.Tensor] = {}


def rowmajor_ut(U: torch.Tensor) -> torch.Tensor:
    """U^T of a shared (K, r) factor as a plain row-major (r, K) fp16 tensor, one copy per distinct storage:
    the operand of the persistent decode kernel's dense row tasks (one warp per row of U^T)."""
    key = (U.device.index or 0, U.data_ptr(), U.shape[0], U.shape[1])
    t = _UT_RM_POOL.get(key)
    if t is None:
        t = U.to(torch.float16).t().contiguous()
        t._keep = U
        _UT_RM_POOL[key] = t
    return t


def clear_pool():
    _UT_POOL.clear()
    _UT_RM_POOL.clear()


# ---- workspaces ------------------------------------------------------------------------------
_WS: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]] = {}


def workspace(device, nbytes: int, ncounters: int = 0):
    """(scratch, counters) for the current stream of `device`.  The scratch holds split-k partial
    sums and small intermediates and needs no initialisation.  The counters are arrival counters:
    they must be zero before a call and every kernel leaves them zero, so they are cleared only
    when the array is (re)allocated."""
    key = (torch.device(device).index or 0, _stream_ptr(device))
    ws, ctr = _WS.get(key, (None, None))
    if (ws is None or ctr is None) and torch.cuda.is_current_stream_capturing():
        # no allocation (and no zero fill) inside a capture: the workspace of the warm-up calls on this device serves
        # the captured calls too (they run in stream order after them)
        for (dev_idx, _), (ows, octr) in _WS.items():
            if dev_idx == key[0] and ows.numel() >= nbytes and octr.numel() >= ncounters:
                ws, ctr = ows, octr
                break
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    if ctr is None or ctr.numel() < ncounters:
        ctr = torch.zeros(max(ncounters, 1 << 16), dtype=torch.int32, device=device)
    _WS[key] = (ws, ctr)
    return ws, ctr


def debug_error(clear: bool = True):
    """First bounds violation / timed-out wait recorded by a kernel, or None."""
    out = (C.c_ulonglong * 4)()
    _lib.check(_lib.lib().glq_debug_error(out, int(clear)), "debug_error")
    vals = [int(v) for v in out]
    return None if vals[0] == 0 else vals


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


class GroupedLinear:
    """Several quantized layers of one shape applied to the same activation rows in two launches (x.U of
    all of them, then the quantized products with the low-rank term), through ``glq_grouped_matmul``:
    e.g. the q, k and v projections of an attention layer.  ``forward(x (B,K))`` returns (P, B, N)."""

    def __init__(self, weights, uts):
        w0 = weights[0]
        for w in weights:
            if (w.fmt, w.N, w.K, w.group_size, w.rank) != (w0.fmt, w0.N, w0.K, w0.group_size, w0.rank):
                raise RuntimeError("grouped layers must share format, shape, group size and rank")
        self.weights, self.uts = list(weights), list(uts) if uts else None
        dev = w0.device
        self._table = torch.frombuffer(bytearray(b"".join(w.desc_bytes() for w in weights)), dtype=torch.uint8).to(dev)
        self._ut_table = None
        if self.uts:
            descs = [_lib.Weight(u.codes.data_ptr(), None, None, None, None, None, u.N, u.K, 0, 0) for u in self.uts]
            self._ut_table = torch.frombuffer(bytearray(b"".join(bytes(d) for d in descs)), dtype=torch.uint8).to(dev)
        self._rows = {}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w0, P = self.weights[0], len(self.weights)
        B = x.shape[0]
        dev = x.device
        L = _lib.lib()
        if B not in self._rows:     # every problem reads the same B activation rows
            self._rows[B] = torch.arange(B, dtype=torch.int32, device=dev).repeat(P)
        rows = self._rows[B]
        y = torch.empty(P, B, w0.N, dtype=torch.float16, device=dev)
        st = _stream_ptr(dev)

        def call(fmt, gs, table, N, K, rank, out, a):
            m = _lib.MMArgs()
            if a is not None:
                m.flags = 1      # GLQ_MM_A_FROM_PREVIOUS_LAUNCH: x.U was launched directly before
            m.fmt, m.group_size, m.epilogue, m.n_problems, m.max_rows, m.rows_stride = fmt, gs, 0, P, B, B
            m.N, m.K, m.rank, m.total_rows = N, K, rank, P * B
            m.w_table = table.data_ptr()
            m.entry_row = rows.data_ptr()
            m.x, m.ldx = x.data_ptr(), x.stride(0)
            if a is not None:
                m.a0, m.lda = a.data_ptr(), a.shape[-1]
            m.y, m.ldy = out.data_ptr(), N
            nbytes, nctr = L.glq_mm_workspace_bytes(C.byref(m)), L.glq_mm_counters(C.byref(m))
            ws, ctr = workspace(dev, nbytes, nctr)
            m.workspace, m.workspace_bytes = ws.data_ptr(), ws.numel()
            m.counters, m.n_counters = ctr.data_ptr(), ctr.numel()
            _lib.check(L.glq_grouped_matmul(C.byref(m), st), "grouped_matmul")

        with torch.cuda.device(dev):
            a = None
            if self._ut_table is not None and w0.rank > 0:
                a = torch.empty(P, B, w0.rank, dtype=torch.float16, device=dev)
                call(_lib.FMT_F16, 0, self._ut_table, w0.rank, w0.K, 0, a, None)
            call(w0.fmt, w0.group_size, self._table, w0.N, w0.K, w0.rank if a is not None else 0, y, a)
        return y
