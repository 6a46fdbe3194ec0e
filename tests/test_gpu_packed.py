"""Packed-plane weights on a B200: MatVecPacked / MatMulPacked give the raw-block entry points' results bit for bit,
and the device copy made from the planes unpacks to the integer view of the blocks they were packed from."""
import numpy as np
import pytest

from conftest import parity_err
from jitllm_b200 import MXFP4, Q4_K, Q8_0, Device, synth
from jitllm_b200.device import packed_desc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t", [Q4_K, Q8_0, MXFP4])
@pytest.mark.parametrize("nrows,k", [(37, 512), (4096, 4096)])
def test_packed_matvec_equals_raw_matvec_bit_for_bit(orc, t, nrows, k):
    rng = synth.rng_for(0xD0 + t + nrows)
    w = synth.matrix(rng, t, nrows, k)
    x = synth.activations(rng, 1, k)[0]
    qs, d, sc = orc.pack_weights(t, w, nrows, k)
    p = packed_desc(qs, d, sc)
    with Device(0) as dev:
        raw = np.full(nrows, np.nan, np.float32)
        assert dev.MatVec(raw, t, w, x, nrows, k), dev.Err()
        got = np.full(nrows, np.nan, np.float32)
        assert dev.MatVecPacked(got, t, p, x, nrows, k), dev.Err()
        assert np.array_equal(got.view(np.uint32), raw.view(np.uint32))
        assert parity_err(got, orc.matmul_f64(t, w, x, nrows, k, 1)[0]) <= 2e-3
        n_up = dev.Stats().uploads
        assert dev.MatVecPacked(got, t, p, x, nrows, k) and dev.Stats().uploads == n_up      # resident: no second upload
        dev.Forget(qs)
        assert dev.MatVecPacked(got, t, p, x, nrows, k) and dev.Stats().uploads == n_up + 1  # forgotten: uploaded again
        # batched
        xs = synth.activations(rng, 5, k)
        a, b = np.empty((5, nrows), np.float32), np.empty((5, nrows), np.float32)
        assert dev.MatMul(a, t, w, xs, nrows, k, 5) and dev.MatMulPacked(b, t, p, xs, nrows, k, 5)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("t", [Q4_K, Q8_0, MXFP4])
def test_device_copy_made_from_planes_unpacks_bit_exact(orc, t):
    from jitllm_b200._lib import BLOCK
    rng = synth.rng_for(0xD7 + t)
    E, rows, k = 2, 24, 1024 if t == Q4_K else 640
    ws = [synth.matrix(rng, t, rows, k) for _ in range(E)]
    planes = None
    for e, w in enumerate(ws):
        planes = orc.pack_weights(t, w, rows, k, row0=e * rows, stride=E * rows, into=planes)
    with Device(0) as dev:
        for e, w in enumerate(ws):
            h = dev.UploadPacked(t, packed_desc(*planes, row=e * rows, stride=E * rows), rows, k)
            for g, want in zip(h.unpack(), orc.unpack(t, w, w.size // BLOCK[t][1])):
                assert np.array_equal(g, want)
            h.free()
