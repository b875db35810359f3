"""Python boundary of the fused dequant + matmul kernels.

Same function names, arguments and return types as the reference's ``inference.kernels``
(inference/kernels/__init__.py:39-57, 184-346), backed by the C ABI of libglorcq_b200 instead of the
two pybind11 modules.  Differences, on purpose:

* there is no PyTorch fallback: a failed call raises RuntimeError (the reference logs and retries
  in PyTorch, inference/kernels/__init__.py:224-232);
* bits other than 2 for the codebook format raise instead of falling back.
"""

from __future__ import annotations

import logging

import torch

from .. import _lib

logger = logging.getLogger(__name__)

_empty_tensor_cache: dict = {}


def _empty_lora(device):
    key = (str(device), torch.float32)
    if key not in _empty_tensor_cache:
        _empty_tensor_cache[key] = torch.empty(0, dtype=torch.float32, device=device)
    return _empty_tensor_cache[key]


_int8_cache: dict = {}


def _int8_codes(qweight_int):
    """int8 copy of an (N, K) code tensor, made once per tensor (the reference converts on every call,
    inference/kernels/__init__.py:305-309).  The cache holds a weak reference to the source: an entry dies with it,
    and a tensor whose storage or version changed is converted again."""
    import weakref
    if qweight_int.dtype == torch.int8:
        return qweight_int
    key = id(qweight_int)
    hit = _int8_cache.get(key)
    if hit is not None:
        ref, ptr, ver, q8 = hit
        if ref() is qweight_int and ptr == qweight_int.data_ptr() and ver == qweight_int._version:
            return q8
    q8 = qweight_int.to(torch.int8)
    _int8_cache[key] = (weakref.ref(qweight_int, lambda _r, k=key: _int8_cache.pop(k, None)), qweight_int.data_ptr(),
                        qweight_int._version, q8)
    return q8


def _available() -> bool:
    try:
        _lib.lib()
    except (RuntimeError, OSError):
        return False
    return torch.cuda.is_available()


def is_cuda_available():
    """True when the codebook-format kernels can run (library built, CUDA device present)."""
    return _available()


def is_gptq_cuda_available():
    """True when the integer-code kernels can run."""
    return _available()


_HAS_GROUPED_GEMV = True


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _check_cuda(t, name, dtype):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}")


# ---------------------------------------------------------------------------------------------
# native-level functions (same signatures as the reference's pybind11 modules)
# ---------------------------------------------------------------------------------------------
def turbo_dequant_matmul(x_rot, packed_indices, norms, centroids):
    """(B,K) fp16 x (N,K/4) uint8 -> (B,N) fp16 (inference/kernels/turbo_matmul.cu:255-318)."""
    _check_cuda(x_rot, "x_rot", torch.float16)
    _check_cuda(packed_indices, "packed_indices", torch.uint8)
    _check_cuda(norms, "norms", torch.float32)
    _check_cuda(centroids, "centroids", torch.float32)
    if centroids.numel() != 4:
        raise RuntimeError("centroids must have 4 elements")
    B, K = x_rot.shape
    N = packed_indices.shape[0]
    if K % 4 != 0:
        raise RuntimeError("K must be divisible by 4 for 2-bit packing")
    if packed_indices.shape[1] != K // 4:
        raise RuntimeError("packed_indices shape mismatch: expected (N, K/4)")
    if norms.shape[0] != N:
        raise RuntimeError("norms shape mismatch")
    y = torch.empty(B, N, dtype=torch.float16, device=x_rot.device)
    if B == 0 or N == 0:
        return y
    with torch.cuda.device(x_rot.device):
        _lib.check(_lib.lib().glq_turbo_dequant_matmul(x_rot.data_ptr(), packed_indices.data_ptr(), norms.data_ptr(),
                                                       centroids.data_ptr(), y.data_ptr(), B, N, K, _stream(x_rot)),
                   "turbo_dequant_matmul")
    return y


def turbo_dequant_grouped_gemv(x_grouped, packed_cat, norms_cat, centroids, N_out):
    """E GEMVs with their own inputs -> (E*N_out,) fp16 (inference/kernels/turbo_matmul.cu:417-464)."""
    _check_cuda(x_grouped, "x_grouped", torch.float16)
    _check_cuda(packed_cat, "packed_cat", torch.uint8)
    _check_cuda(norms_cat, "norms_cat", torch.float32)
    _check_cuda(centroids, "centroids", torch.float32)
    E, K = x_grouped.shape
    if packed_cat.shape[0] != E * N_out:
        raise RuntimeError("packed_cat first dim must be E * N_out")
    if K % 4 != 0 or packed_cat.shape[1] != K // 4:
        raise RuntimeError("packed_cat col dim must be K/4")
    if norms_cat.shape[0] != E * N_out:
        raise RuntimeError("norms_cat size mismatch")
    y = torch.empty(E * N_out, dtype=torch.float16, device=x_grouped.device)
    if E == 0 or N_out == 0:
        return y
    with torch.cuda.device(x_grouped.device):
        _lib.check(_lib.lib().glq_turbo_dequant_grouped_gemv(x_grouped.data_ptr(), packed_cat.data_ptr(),
                                                             norms_cat.data_ptr(), centroids.data_ptr(), y.data_ptr(),
                                                             E, N_out, K, _stream(x_grouped)),
                   "turbo_dequant_grouped_gemv")
    return y


def gptq_dequant_matmul(x, qweight_i8, scales, zeros, groupsize, sym, lora_out):
    """(B,K) fp32 x (N,K) int8 -> (B,N) fp32 (inference/kernels/gptq_matmul.cu:223-315);
    a zero-element lora_out means no low-rank term."""
    _check_cuda(x, "x", torch.float32)
    _check_cuda(qweight_i8, "qweight_i8", torch.int8)
    _check_cuda(scales, "scales", torch.float16)
    _check_cuda(zeros, "zeros", torch.float16)
    B, K = x.shape
    N = qweight_i8.shape[0]
    G = scales.shape[1]
    if qweight_i8.shape[1] != K:
        raise RuntimeError("qweight_i8 shape mismatch: expected (N, K)")
    if scales.shape[0] != N or zeros.shape[0] != N or zeros.shape[1] != G:
        raise RuntimeError("scales / zeros shape mismatch")
    lora_ptr = None
    if lora_out is not None and lora_out.numel() > 0:
        _check_cuda(lora_out, "lora_out", torch.float32)
        if tuple(lora_out.shape) != (B, N):
            raise RuntimeError("lora_out shape mismatch")
        lora_ptr = lora_out.data_ptr()
    y = torch.empty(B, N, dtype=torch.float32, device=x.device)
    if B == 0 or N == 0:
        return y
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().glq_gptq_dequant_matmul(x.data_ptr(), qweight_i8.data_ptr(), scales.data_ptr(),
                                                      zeros.data_ptr(), lora_ptr, y.data_ptr(), B, N, K,
                                                      int(groupsize), G, int(bool(sym)), _stream(x)),
                   "gptq_dequant_matmul")
    return y


# ---------------------------------------------------------------------------------------------
# torch.library custom ops, so that a tracing compiler sees opaque calls with known output shapes
# (inference/kernels/__init__.py:68-107)
# ---------------------------------------------------------------------------------------------
try:
    @torch.library.custom_op("glorcq_b200::turbo_dequant_matmul", mutates_args=())
    def _turbo_dequant_matmul_op(x_rot: torch.Tensor, packed_indices: torch.Tensor, norms: torch.Tensor,
                                 centroids: torch.Tensor) -> torch.Tensor:
        return turbo_dequant_matmul(x_rot, packed_indices, norms, centroids)

    @_turbo_dequant_matmul_op.register_fake
    def _turbo_fake(x_rot, packed_indices, norms, centroids):
        return torch.empty(x_rot.shape[0], packed_indices.shape[0], dtype=torch.float16, device=x_rot.device)

    @torch.library.custom_op("glorcq_b200::gptq_dequant_matmul", mutates_args=())
    def _gptq_dequant_matmul_op(x: torch.Tensor, qweight_i8: torch.Tensor, scales: torch.Tensor,
                                zeros: torch.Tensor, groupsize: int, sym: bool,
                                lora_out: torch.Tensor) -> torch.Tensor:
        return gptq_dequant_matmul(x, qweight_i8, scales, zeros, groupsize, sym, lora_out)

    @_gptq_dequant_matmul_op.register_fake
    def _gptq_fake(x, qweight_i8, scales, zeros, groupsize, sym, lora_out):
        return torch.empty(x.shape[0], qweight_i8.shape[0], dtype=torch.float32, device=x.device)
except Exception as e:  # pragma: no cover - registration is optional
    logger.debug("custom op registration skipped: %s", e)
    _turbo_dequant_matmul_op = turbo_dequant_matmul
    _gptq_dequant_matmul_op = gptq_dequant_matmul

# The reference registers its ops as ``glorcq::turbo_dequant_matmul`` / ``glorcq::gptq_dequant_matmul``
# (inference/kernels/__init__.py:69, 88); code that calls ``torch.ops.glorcq.*`` binds to this package the same
# way, unless the reference package itself has been imported in this process and owns the names.
try:
    @torch.library.custom_op("glorcq::turbo_dequant_matmul", mutates_args=())
    def _ref_name_turbo(x_rot: torch.Tensor, packed_indices: torch.Tensor, norms: torch.Tensor,
                        centroids: torch.Tensor) -> torch.Tensor:
        return turbo_dequant_matmul(x_rot, packed_indices, norms, centroids)

    @_ref_name_turbo.register_fake
    def _ref_name_turbo_fake(x_rot, packed_indices, norms, centroids):
        return torch.empty(x_rot.shape[0], packed_indices.shape[0], dtype=torch.float16, device=x_rot.device)

    @torch.library.custom_op("glorcq::gptq_dequant_matmul", mutates_args=())
    def _ref_name_gptq(x: torch.Tensor, qweight_i8: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                       groupsize: int, sym: bool, lora_out: torch.Tensor) -> torch.Tensor:
        return gptq_dequant_matmul(x, qweight_i8, scales, zeros, groupsize, sym, lora_out)

    @_ref_name_gptq.register_fake
    def _ref_name_gptq_fake(x, qweight_i8, scales, zeros, groupsize, sym, lora_out):
        return torch.empty(x.shape[0], qweight_i8.shape[0], dtype=torch.float32, device=x.device)
except Exception as e:  # pragma: no cover - the names are taken when the reference package is loaded too
    logger.debug("glorcq:: op names not registered: %s", e)


# ---------------------------------------------------------------------------------------------
# Public API: codebook format
# ---------------------------------------------------------------------------------------------
def turbo_dequant_matmul_fused(x, packed_indices, norms, Pi, centroids, bits, dim, lora_USV=None,
                               precomputed_x_rot=None):
    """Rotate (or take the pre-rotated input), run the fused 2-bit dequant + matmul, optionally add
    the Python-level low-rank term ((x@U)*S)@V^T.  Returns (B,N) fp16
    (inference/kernels/__init__.py:184-239)."""
    if bits != 2:
        raise RuntimeError(f"codebook kernels cover bits == 2, got {bits}")
    if precomputed_x_rot is not None:
        x_rot = precomputed_x_rot
    else:
        x_rot = (x.float() @ Pi.float().T).half()
    if x_rot.dtype != torch.float16:
        x_rot = x_rot.half()
    y = _turbo_dequant_matmul_op(x_rot.contiguous(), packed_indices.contiguous(), norms.contiguous(),
                                 centroids.contiguous())
    if lora_USV is not None:
        U, S, V = lora_USV
        y = y + ((x @ U) * S @ V.T)
    return y


def turbo_dequant_grouped_gemv_fused(x_grouped, packed_cat, norms_cat, centroids, N_out):
    """E experts with their own inputs in one launch (inference/kernels/__init__.py:242-278)."""
    return turbo_dequant_grouped_gemv(x_grouped.contiguous(), packed_cat.contiguous(), norms_cat.contiguous(),
                                      centroids.contiguous(), N_out)


# ---------------------------------------------------------------------------------------------
# Public API: integer-code format
# ---------------------------------------------------------------------------------------------
def gptq_dequant_matmul_fused(x, qweight_int, scales, zeros, groupsize, sym=False, lora_USV=None):
    """int32 -> int8 codes if needed, optional Python-level low-rank term, fused dequant + matmul.
    Returns (B,N) fp16 (inference/kernels/__init__.py:284-346)."""
    qweight_i8 = _int8_codes(qweight_int)
    lora_out = _empty_lora(x.device)
    if lora_USV is not None:
        U, S, V = lora_USV
        lora_out = ((x @ U) * S @ V.T).float()
    y = _gptq_dequant_matmul_op(x.float().contiguous(), qweight_i8.contiguous(), scales.contiguous(),
                                zeros.contiguous(), groupsize, sym, lora_out.contiguous())
    return y.half()
