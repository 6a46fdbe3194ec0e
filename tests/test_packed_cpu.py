"""Container-packed planes (nn.Packed{QS, D, SC, Row, Stride}) on the CPU: the library's plane -> block
re-interleave is the exact inverse of the reference's packer, restated in the oracle from
jit/gpu/kernels/pack.go:27-239 (payload words [sub-block][word][row], the d plane's shared words, the 96-bit
scale stream). The reference commits no packed golden (its TestPackAgainstRealWeights needs model files), so the
packer restatement is pinned by construction: its planes are checked field by field against the integer view."""
import numpy as np
import pytest

from jitllm_b200 import _lib, synth
from jitllm_b200.device import packed_desc, packed_to_blocks

TYPES = [_lib.Q4_K, _lib.Q8_0, _lib.MXFP4]


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("nrows,k", [(1, 256), (5, 512), (7, 1024), (64, 2048), (33, 256)])
def test_planes_to_blocks_is_the_inverse_of_the_packer(orc, t, nrows, k):
    rng = synth.rng_for(0xC0 + t + nrows + k)
    w = synth.matrix(rng, t, nrows, k)
    qs, d, sc = orc.pack_weights(t, w, nrows, k)
    got = packed_to_blocks(t, packed_desc(qs, d, sc), nrows, k)
    assert np.array_equal(got, w.reshape(-1))


@pytest.mark.parametrize("t", TYPES)
def test_an_expert_inside_a_bank_is_addressed_by_row_and_stride(orc, t):
    """Rows are interleaved through the whole buffer: expert e of a bank is Row = e * rows in a Stride-row buffer
    (engine/nn/device.go:68-73), and rows of different experts share d words on the narrow formats."""
    rng = synth.rng_for(0xC9 + t)
    E, rows, k = 3, 6, 512                      # 18 rows: not a multiple of four, so MXFP4's last d word is shared unevenly
    ws = [synth.matrix(rng, t, rows, k) for _ in range(E)]
    planes = None
    for e, w in enumerate(ws):
        planes = orc.pack_weights(t, w, rows, k, row0=e * rows, stride=E * rows, into=planes)
    qs, d, sc = planes
    for e, w in enumerate(ws):
        got = packed_to_blocks(t, packed_desc(qs, d, sc, row=e * rows, stride=E * rows), rows, k)
        assert np.array_equal(got, w.reshape(-1)), e


def test_packer_restatement_places_every_field_where_the_reference_says(orc):
    """Q4_K, spot-checked against the layout's definition: payload word (si*4 + w)*nrows + r holds elements
    4w..4w+3 (low nibbles) and 16+4w.. (high nibbles) of sub-block si; d word sup*nrows + r = d | dmin << 16; the
    scale of sub-block s is the 6-bit field at bit 12 s of the row's 96-bit stream, its minimum at 12 s + 6."""
    rng = synth.rng_for(0xCC)
    nrows, k = 9, 512
    w = synth.q4k_matrix(rng, nrows, k)
    qs, d, sc = orc.pack_weights(_lib.Q4_K, w, nrows, k)
    q, db, dmb, scv, mv = orc.unpack(_lib.Q4_K, w, nrows * k // 256)
    q = q.reshape(nrows, k // 32, 32)
    for r in (0, 4, 8):
        for si in (0, 7, 15):
            for wd in range(4):
                word = int(qs[(si * 4 + wd) * nrows + r])
                for b in range(4):
                    byte = (word >> (8 * b)) & 0xFF
                    assert byte & 15 == q[r, si, 4 * wd + b] and byte >> 4 == q[r, si, 16 + 4 * wd + b]
            sup, s = si // 8, si % 8
            rec = r * (k // 32) + si
            assert int(d[sup * nrows + r]) == int(db[rec]) | int(dmb[rec]) << 16
            stream = sum(int(sc[(sup * 3 + i) * nrows + r]) << (32 * i) for i in range(3))
            assert (stream >> (12 * s)) & 63 == scv[rec] and (stream >> (12 * s + 6)) & 63 == mv[rec]


def test_bad_planes_are_refused():
    qs, d = np.zeros(16, np.uint32), np.zeros(4, np.uint32)
    lib = _lib.load()
    out = np.zeros(4096, np.uint8)
    import ctypes as C
    p = packed_desc(qs, d, None)
    assert lib.jl_packed_to_blocks(_lib.Q4_K, C.byref(p), 4, 256, out.ctypes.data, out.nbytes) == _lib.EINVAL   # planes too short, no sc
    assert lib.jl_packed_to_blocks(_lib.Q6_K, C.byref(p), 4, 256, out.ctypes.data, out.nbytes) == _lib.DECLINED
