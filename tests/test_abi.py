"""The C-ABI boundary without a GPU: the library loads, exports every symbol the
header declares, refuses to open without a B200 (no CPU fallback), and its
host-side integer unpack equals the oracle's restatement of kernels.extract."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT
from jitllm_b200 import _lib, synth
from jitllm_b200.device import unpack_host


def _declared():
    text = open(os.path.join(ROOT, "include", "jitllm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jl_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_name_the_same_symbols():
    assert _declared() == sorted(_lib.SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in _declared():
        assert hasattr(lib, name), name
    assert lib.jl_abi_version() == 2
    assert b"sm_100a" in lib.jl_version()


def test_struct_sizes_match_the_header_layout():
    # natural C layout of the structs in include/jitllm_b200.h
    assert C.sizeof(_lib.Opts) == 56
    assert C.sizeof(_lib.Choice) == 44
    assert C.sizeof(_lib.Stats) == 72
    assert C.sizeof(_lib.MoeDesc) == 136


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="a GPU is present")
def test_open_fails_loudly_without_a_gpu():
    from jitllm_b200 import Device, DeviceError
    with pytest.raises(DeviceError):
        Device(0)


@pytest.mark.parametrize("t", [_lib.Q4_K, _lib.Q8_0, _lib.MXFP4, _lib.Q4_0, _lib.Q5_0, _lib.Q5_1, _lib.Q5_K, _lib.Q6_K])
def test_host_unpack_equals_the_oracle(orc, t):
    rng = synth.rng_for(100 + t)
    w = synth.matrix(rng, t, 5, 768 if _lib.BLOCK[t][0] == 32 else 1024)
    nb = w.size // _lib.BLOCK[t][1]
    got = unpack_host(t, w, nb)
    want = orc.unpack(t, w, nb)
    for g, x in zip(got, want):
        assert np.array_equal(g, x)


def test_host_unpack_on_reference_goldens(orc, golden):
    for name, t in [("q4_k_tiny", 12), ("q8_0_gemma", 8), ("mxfp4", 39), ("q4_0_gemma", 2), ("q5_k_tiny", 13), ("q6_k_tiny", 14)]:
        blocks = golden[name + "_blocks"]
        nb = blocks.size // _lib.BLOCK[t][1]
        for g, x in zip(unpack_host(t, blocks, nb), orc.unpack(t, blocks, nb)):
            assert np.array_equal(g, x)


def test_unpack_rejects_unknown_types():
    lib = _lib.load()
    b = np.zeros(64, np.uint8)
    o = np.zeros(64, np.uint8)
    assert lib.jl_unpack(3, b.ctypes.data, 1, o.ctypes.data, o.ctypes.data, o.ctypes.data, o.ctypes.data,
                         o.ctypes.data) == _lib.ENOTSUP


def test_aux_entry_points_refuse_misaligned_pointers_on_the_host():
    """The decode-step neighbour kernels use 16-byte accesses; a misaligned pointer is refused before any launch
    (so this needs no GPU)."""
    from jitllm_b200 import _lib
    L = _lib.load()
    good, bad = 0x10000, 0x10004
    assert L.jl_aux_add_rmsnorm(bad, None, None, 1e-5, good, None, 1, 256, None) == -1
    assert L.jl_aux_add_rmsnorm(good, bad, None, 1e-5, good, None, 1, 256, None) == -1
    assert L.jl_aux_add_rmsnorm(good, None, None, 1e-5, None, None, 1, 256, None) == -1      # neither out nor operand
    assert L.jl_aux_add_rmsnorm(good, None, None, 1e-5, good, None, 1, 250, None) == -1      # h % 4
    assert L.jl_aux_add_rmsnorm_gemm(bad, None, None, 1e-5, good, good, 1, 256, None) == -1
    assert L.jl_aux_add_rmsnorm_gemm(good, None, None, 1e-5, bad, good, 1, 256, None) == -1
    assert L.jl_aux_add_rmsnorm_gemm(good, None, None, 1e-5, None, good, 1, 256, None) == -1   # no operand to write
    assert L.jl_aux_add_rmsnorm_gemm(good, None, None, 1e-5, good, good, 1, 384, None) == -1   # whole super-blocks only
    assert L.jl_gemm_operand(None, None, 1, None, None) == -1
    assert L.jl_matmul_dev_prepared(None, good, 0, None, 1, None) == -1
    assert L.jl_aux_silu_mul(good, None, bad, 1, 256, None) == -1
    assert L.jl_aux_attn_decode(good, None, good, bad, good, good, good, 1, 4, 1, 128, 64, None) == -1
    assert L.jl_aux_attn_decode(good, None, good, good, good, good, good, 1, 4, 1, 64, 64, None) == -1   # head_dim != 128
    assert L.jl_aux_attn_scratch_bytes(1, 4, 3, 64) == 0                                       # hq % hkv
