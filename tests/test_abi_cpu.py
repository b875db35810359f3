"""CPU checks of the C ABI: the library builds, loads, and exports every symbol the header declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def libpath():
    from glorcq_b200 import _build
    return _build.build()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "glorcq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(glq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(libpath):
    L = ctypes.CDLL(libpath)
    syms = header_symbols()
    assert len(syms) >= 15
    missing = [s for s in syms if not hasattr(L, s)]
    assert not missing, f"declared in include/glorcq_b200.h but not exported: {missing}"


def test_binding_covers_header(libpath):
    from glorcq_b200 import _lib
    assert set(header_symbols()) <= set(_lib.exported_symbols())


def test_status_strings_and_sizes(libpath):
    from glorcq_b200 import _lib
    L = _lib.lib()
    assert L.glq_version() >= 100
    for st in (0, -1, -2, -3, -4, -5):
        assert len(L.glq_status_string(st)) > 0
    # C1 expert projection 1408 x 2048, 2-bit: 44 tile pairs x 16 blocks x 2 tiles x (512 B codes + 64 B scales)
    assert L.glq_tiled_bytes(_lib.FMT_Q2, 1408, 2048, 1) == 44 * 16 * 2 * 576
    # the same fused with a second matrix of that shape (gate | up): twice the pairs
    assert L.glq_tiled_bytes(_lib.FMT_Q2, 1408, 2048, 2) == 88 * 16 * 2 * 576
    assert L.glq_tiled_bytes(_lib.FMT_Q4, 2048, 2048, 1) == 64 * 32 * 2 * 576
    assert L.glq_tiled_bytes(_lib.FMT_T2, 1408, 2048, 1) == 1408 * 2048 // 4
    assert L.glq_tiled_f16_bytes(64, 2048) == 64 * 2048 * 2
    assert L.glq_sv_bytes(1408, 64, 1) == 44 * 4096 == 1408 * 64 * 2
    # ragged shapes are padded to whole tile pairs and k blocks
    assert L.glq_tiled_bytes(_lib.FMT_T2, 17, 130, 1) == 1 * 2 * 2 * 512
    assert L.glq_rows_f32_count(17, 1) == 32


def test_host_side_argument_checks(libpath):
    """Errors decided on the host, before any launch: no GPU needed."""
    from glorcq_b200 import _lib
    L = _lib.lib()
    assert L.glq_turbo_dequant_matmul(None, None, None, None, None, 1, 8, 64, None) == -1
    assert L.glq_turbo_dequant_matmul(None, None, None, None, None, 0, 8, 64, None) == 0      # B == 0: no-op
    assert L.glq_turbo_dequant_matmul(None, None, None, None, None, -1, 8, 64, None) == -1
    assert L.glq_gptq_dequant_matmul(None, None, None, None, None, None, 0, 8, 64, 128, 1, 0, None) == 0
    assert L.glq_pack_gptq(None, None, None, 2, 16, 128, 128, None, 0, 1, None) == -1
    assert L.glq_grouped_matmul(None, None) == -1
    # expert-parallel phases: the peer-memory exchange needs its pointer tables, the other phases must not get them
    import ctypes as C
    d = _lib.MoeDesc()
    d.top_k, d.H, d.E = 2, 64, 4
    dummy = C.create_string_buffer(64)
    ptr = C.cast(dummy, C.c_void_p).value

    def ep_call(ep):
        return L.glq_moe_forward_ep(C.byref(d), ptr, 1, ptr, None, None, None, None, 0, None, 0, None, None, None, None,
                                    C.byref(ep))
    ep = _lib.MoeEp(0, 2, _lib.MOE_PHASE_EXCHANGE, 0, ptr, None, None)
    assert ep_call(ep) == -1                                   # no peers
    peers = _lib.EpPeers(ptr, ptr, ptr, ptr, 0)
    ep.peers = C.pointer(peers)
    assert ep_call(ep) == -1                                   # buffers too small for the step (half_elems 0)
    ep.phase = _lib.MOE_PHASE_EXPERTS
    assert ep_call(ep) == -1                                   # the staging buffer is not exchanged
    assert ep_call(_lib.MoeEp(2, 2, _lib.MOE_PHASE_EXPERTS, 0, ptr, None, None)) == -1   # rank outside the world
    assert ep_call(_lib.MoeEp(0, 2, _lib.MOE_PHASE_ALL, 0, ptr, None, None)) == -1      # world > 1 needs phases


def test_no_fallback_without_gpu():
    """Without a CUDA device the product path must fail loudly, not compute on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from tests import cases
    d = cases.make_linear(1, 32, 128, rank=16)
    with pytest.raises((RuntimeError, AssertionError)):
        cases.to_b200_linear(d, device="cpu")
