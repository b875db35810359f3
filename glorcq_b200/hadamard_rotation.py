"""Randomized Hadamard rotation on the GPU: mirror of the reference's ``hadamard_rotation`` module
(hadamard_rotation.py:28-83), which wraps the third-party fast-hadamard-transform.

    y = (1/sqrt(d)) * H * diag(signs) * x

H is the Walsh-Hadamard matrix in natural (Sylvester) order of the next power of two >= d; x is
zero-padded to it and the first d outputs are kept.  The transform runs in ``glq_rht_forward`` (one CTA
per row, fp32 butterflies in shared memory); there is no CPU path.
"""

from __future__ import annotations

import torch

from . import _lib, tiled


def is_hadamard_available() -> bool:
    """True when the native library is built (the reference asks whether its third-party kernel is installed)."""
    try:
        _lib.lib()
        return True
    except RuntimeError:
        return False


def generate_rht_signs(d, seed=42, device="cuda"):
    """(d,) float32 of +-1, drawn exactly as the reference draws them: a CPU generator seeded with
    `seed`, ``randint(0, 2, (d,)) * 2 - 1`` (hadamard_rotation.py:33-47)."""
    rng = torch.Generator(device="cpu")
    rng.manual_seed(seed)
    signs = torch.randint(0, 2, (d,), generator=rng) * 2 - 1
    return signs.float().to(device)


def _transform(x: torch.Tensor, signs: torch.Tensor, out_dtype) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("rht_forward runs on a CUDA device only (no CPU path)")
    if x.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("rht_forward takes fp16 or fp32 activations")
    d = x.shape[-1]
    if signs.shape != (d,):
        raise RuntimeError(f"signs must have shape ({d},)")
    signs = signs.to(device=x.device, dtype=torch.float32).contiguous()
    x2 = x.reshape(-1, d).contiguous()
    y = torch.empty(x2.shape, dtype=out_dtype, device=x.device)
    if x2.shape[0] > 0:
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().glq_rht_forward(x2.data_ptr(), int(x2.dtype == torch.float32), d, signs.data_ptr(),
                                                  x2.shape[0], d, 1.0 / d ** 0.5, y.data_ptr(),
                                                  int(out_dtype == torch.float32), d, tiled._stream_ptr(x.device)),
                       "rht_forward")
    return y.reshape(x.shape)


def rht_forward(x, signs):
    """y = (1/sqrt(d)) H diag(signs) x over the last dimension; same dtype out as in (hadamard_rotation.py:50-65)."""
    return _transform(x, signs, x.dtype)


def rht_forward_half(x, signs):
    """The form the MoE block uses: ``rht_forward(x.float(), signs).half()`` in one launch
    (inference/moe_block.py:349-351)."""
    return _transform(x, signs, torch.float16)


def rht_backward(y, signs):
    """x = diag(signs) (1/sqrt(d)) H y (hadamard_rotation.py:68-83); exact inverse for power-of-two d."""
    ones = torch.ones_like(signs)
    return _transform(y, ones, y.dtype) * signs.to(device=y.device, dtype=y.dtype)
