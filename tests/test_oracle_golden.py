"""The CPU oracle against the reference's committed golden vectors and its own
construction-level known answers. CPU only."""
import numpy as np
import pytest

from conftest import nmse
from jitllm_b200 import synth

CASES = [("q4_k_tiny", 12), ("q8_0_gemma", 8), ("q8_0_minilm", 8), ("q8_0_stories", 8), ("mxfp4", 39),
         ("q4_0_gemma", 2), ("q4_0_stories", 2), ("q5_k_tiny", 13), ("q6_k_tiny", 14)]


@pytest.mark.parametrize("name,t", CASES)
def test_decoders_match_reference_goldens_bit_for_bit(orc, golden, name, t):
    # convert/gguf/gguf_test.go:247-314 and format/quant/mxfp4_test.go:18-66 assert the same bytes.
    blocks, bits = golden[name + "_blocks"], golden[name + "_bits"]
    assert blocks.size % orc.block_bytes(t) == 0
    assert bits.size == blocks.size // orc.block_bytes(t) * orc.block_elems(t)
    got = orc.dequant32(t, blocks, bits.size).view(np.uint32)
    assert np.array_equal(got, bits)
    assert np.count_nonzero(bits & 0x7FFFFFFF) >= bits.size // 2, "degenerate golden"
    # format/quant/dequant32_test.go:12-58: the f64 destination holds the same value.
    got64 = orc.dequant64(t, blocks, bits.size)
    want = bits.view(np.float32).astype(np.float64)
    fin = np.isfinite(want)
    assert np.array_equal(got64[fin], want[fin])


def test_half_codec_round_trips_every_pattern(orc):
    # format/quant/dequant.go:478-517: EncodeHalf is the exact inverse of DecodeHalf.
    ref = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float64)
    for u in range(65536):
        v = orc.half_decode(u)
        if np.isnan(ref[u]):
            assert np.isnan(v)
            continue
        assert v == ref[u]
        assert orc.half_encode(np.float32(v)) == u


def test_half_encode_rounds_to_nearest_even(orc):
    xs = np.random.default_rng(1).standard_normal(20000).astype(np.float32) * np.float32(300.0)
    want = xs.astype(np.float16).view(np.uint16)
    got = np.array([orc.half_encode(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("t", [12, 8, 39])
def test_unpack_reassembles_to_the_decoder(orc, t):
    # value = scale*q - bias (jit/gpu/kernels/matvec.go:73-85) over extract's integers equals Dequant32.
    rng = synth.rng_for(0xB200 + t)
    k = 512
    w = synth.matrix(rng, t, 6, k)
    nb = 6 * k // orc.block_elems(t)
    q, d, dmin, sc, m = orc.unpack(t, w, nb)
    ref = orc.dequant32(t, w, 6 * k)
    q = q.reshape(-1, 32).astype(np.float32)
    if t == 12:
        df = d.view(np.float16).astype(np.float32)
        mf = dmin.view(np.float16).astype(np.float32)
        val = (df * sc.astype(np.float32))[:, None] * q - (mf * m.astype(np.float32))[:, None]
        assert q.min() >= 0 and q.max() <= 15 and sc.max() <= 63 and m.max() <= 63
    elif t == 8:
        val = d.view(np.float16).astype(np.float32)[:, None] * q
    else:
        table = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], np.float32)
        scale = ((d.astype(np.uint32) & 0xFF) << 23).view(np.float32)  # stored byte e-1 -> 2^(e-128)
        val = table[q.astype(np.int64)] * scale[:, None]
    assert np.array_equal(val.reshape(-1).view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("t", [2, 6, 7, 13, 14])
def test_unpack_reassembles_to_the_decoder_more_formats(orc, t):
    """The integer view of Q4_0, Q5_0, Q5_1, Q5_K and Q6_K (extract, jit/gpu/kernels/pack.go:252-386) put back
    together as value = scale * q - bias equals Dequant32 bit for bit. The reference commits no golden for Q5_0 /
    Q5_1; for those this identity against the decoder restated from dequant.go:103-146 is the pin."""
    rng = synth.rng_for(0xB300 + t)
    k = 512
    w = synth.matrix(rng, t, 6, k)
    nb = 6 * k // orc.block_elems(t)
    q, d, dmin, sc, m = orc.unpack(t, w, nb)
    ref = orc.dequant32(t, w, 6 * k)
    sub = 16 if t == 14 else 32
    q = q.reshape(-1, sub).astype(np.float32)
    df = d.view(np.float16).astype(np.float32)
    if t == 2:
        val = df[:, None] * (q - 8)
    elif t == 6:
        val = df[:, None] * (q - 16)
    elif t == 7:   # dmin carries m with its sign flipped: value = d q - (-m)
        mf = (dmin ^ 0x8000).view(np.float16).astype(np.float64)
        val = (df.astype(np.float64)[:, None] * q.astype(np.float64) + mf[:, None]).astype(np.float32)
    elif t == 13:
        mf = dmin.view(np.float16).astype(np.float32)
        val = (df * sc.astype(np.float32))[:, None] * q - (mf * m.astype(np.float32))[:, None]
        assert q.max() <= 31 and sc.max() <= 63
    else:
        val = (df * (sc.astype(np.float32) - 128))[:, None] * (q - 32)
        assert q.min() >= 0 and q.max() <= 63
    assert np.array_equal(val.reshape(-1).view(np.uint32), ref.view(np.uint32))


def test_synth_encoders_are_inverse_of_the_decoder(orc):
    rng = synth.rng_for(7)
    n = 40
    sc = rng.integers(0, 64, (n, 8), dtype=np.uint8)
    m = rng.integers(0, 64, (n, 8), dtype=np.uint8)
    codes = rng.integers(0, 16, (n, 256), dtype=np.uint8)
    d = np.resize(synth.planted_f16_scales(), n)
    dmin = np.resize(synth.planted_f16_scales()[::-1], n)
    blk = synth.q4k_from_parts(d, dmin, sc, m, codes)
    q, db, dmb, s2, m2 = orc.unpack(12, blk, n)
    assert np.array_equal(q.reshape(n, 256), codes.astype(np.int8))
    assert np.array_equal(s2.reshape(n, 8), sc) and np.array_equal(m2.reshape(n, 8), m)
    assert np.array_equal(db.reshape(n, 8)[:, 0], d) and np.array_equal(dmb.reshape(n, 8)[:, 0], dmin)


def test_float_oracle_matches_f64_twin(orc):
    rng = synth.rng_for(11)
    for t in (12, 8, 39):
        w = synth.matrix(rng, t, 33, 1024)
        x = synth.activations(rng, 1, 1024)[0]
        a = orc.matvec(t, w, x, 33, 1024)
        b = orc.matmul_f64(t, w, x, 33, 1024, 1)[0]
        c = orc.matmul_f64_blas(t, w, x, 33, 1024, 1)[0]
        assert nmse(a, b) < 1e-13
        assert nmse(c, b) < 1e-25


def test_quantizer_known_answers(orc):
    # internal/oracle/quantize.go:80-119: d = amax/127, round half away from zero, pair = -sum*biasC/8.
    x = np.zeros(64, np.float32)
    x[0], x[1], x[2], x[3] = 127.0, -63.5, 0.5, -0.5
    x[32:] = 0
    q, pairs = orc.quantize_q8_window(x, 1.0, 32)
    assert pairs[0] == np.float32(1.0)
    assert list(q[:4]) == [127, -64, 1, -1]
    assert pairs[1] == np.float32(-(127 - 64 + 1 - 1) / 8)
    assert pairs[2] == 0 and pairs[3] == 0 and not q[32:].any()
    # a 256 window shares one scale across its 8 blocks
    y = synth.activations(synth.rng_for(3), 1, 512)[0]
    _, p256 = orc.quantize_q8_window(y, 128.0, 256)
    assert len(set(p256[0:16:2].tolist())) == 1 and len(set(p256[16:32:2].tolist())) == 1
    assert p256[0] == np.float32(np.abs(y[:256]).max() / np.float32(127))


@pytest.mark.parametrize("t", [12, 8, 39])
def test_int8_twin_arms_agree_and_sit_where_the_reference_says(orc, t):
    # jit/cpu/matvec_test.go:135: re-orderings of the same quantity agree to NMSE <= 1e-10;
    # :142-184: int8 activations cost ~1e-5 NMSE against the exact dot (logged, not gated, there).
    rng = synth.rng_for(21 + t)
    nrows, k, ntok = 48, 2048, 3
    w = synth.matrix(rng, t, nrows, k)
    x = synth.activations(rng, ntok, k)
    scalar = orc.matmul_int8(t, w, x, nrows, k, ntok, window=32, nthreads=2, simd=0)
    ref = orc.matmul_f64(t, w, x, nrows, k, ntok)
    if orc.simd_level() >= 1:
        simd = orc.matmul_int8(t, w, x, nrows, k, ntok, window=32, nthreads=3, simd=1)
        assert nmse(simd, scalar) < 1e-10
    assert nmse(scalar, ref) < 2e-4
    assert nmse(scalar, ref) > 1e-9, "int8 activations cannot be this exact: the twin is not quantizing"


def test_int8_twin_evaluates_its_own_quantity_exactly(orc):
    # jit/cpu/matvec_test.go:117-130: sum_b d_a[b] * sum_i w[32b+i] * q[32b+i] in f64.
    rng = synth.rng_for(5)
    nrows, k = 16, 1024
    for t in (12, 8):
        w = synth.matrix(rng, t, nrows, k)
        x = synth.activations(rng, 1, k)[0]
        q, pairs = orc.quantize_q8_window(x, orc.bias_c(t), 32)
        xq = (q.astype(np.float64).reshape(-1, 32) * pairs[0::2].astype(np.float64)[:, None]).reshape(-1)
        wd = orc.dequant64(t, w, nrows * k).reshape(nrows, k)
        want = wd @ xq
        got = orc.matmul_int8(t, w, x, nrows, k, 1, window=32, simd=0)[0]
        assert nmse(got, want) < 1e-10


def test_router_known_answers(orc):
    # internal/oracle/moe.go:197-359.
    s = np.array([0.1, 0.4, 0.4, 0.05, 0.05], np.float32)
    sel, ordv, wt, owt, sm = orc.moe_router(s, 2, norm=True)
    assert list(sel) == [1, 2], "ties go to the lowest index"
    assert list(ordv) == [1, 2]
    assert sm == np.float32(np.float32(0.4) + np.float32(0.4)) + np.float32(1e-20)
    assert wt[0] == np.float32(0.4) / np.float32(sm)
    s = np.array([0.3, np.nan, 0.2, 0.5], np.float32)
    sel, ordv, wt, owt, sm = orc.moe_router(s, 3, norm=False)
    assert list(sel) == [3, 0, 2] and list(ordv) == [0, 2, 3], "a NaN is never eligible; ord ascends"
    assert list(wt) == [np.float32(0.5), np.float32(0.3), np.float32(0.2)]
    assert list(owt) == [np.float32(0.3), np.float32(0.2), np.float32(0.5)]
    # the divisor is summed in selection order (moe.go:267-291), not ascending id
    s = np.array([1e-8, 1.0, 3e-8, 0.5], np.float32)
    sel, _, _, _, sm = orc.moe_router(s, 4, norm=True)
    want = np.float32(0)
    for e in sel:
        want = np.float32(want + s[e])
    assert sm == np.float32(want + np.float32(1e-20))
    # bias moves the selection, never the weights
    sel, _, wt, _, _ = orc.moe_router(np.array([0.5, 0.4, 0.1], np.float32), 1, norm=False,
                                      bias=np.array([0, 0.2, 0], np.float32))
    assert list(sel) == [1] and wt[0] == np.float32(0.4)
    # all-underflowed selection stays finite (the +1e-20 floor)
    _, _, wt, _, _ = orc.moe_router(np.zeros(4, np.float32), 2, norm=True)
    assert np.isfinite(wt).all()


def test_activations(orc):
    assert orc.silu(0.0) == 0.0
    assert abs(orc.silu(2.0) - 2.0 / (1 + np.exp(-2.0))) < 1e-15
    # gate clamped at 7 from above, up to [-7, 7], (up + 1) multiplies (oracle.go:131-137)
    assert orc.swiglu_oai(9.0, 9.0) == orc.swiglu_oai(7.0, 7.0)
    assert orc.swiglu_oai(-9.0, -9.0) == orc.swiglu_oai(-9.0, -7.0)
    assert abs(orc.swiglu_oai(1.0, 2.0) - 1.0 / (1 + np.exp(-1.702)) * 3.0) < 1e-15


def test_moe_layer_matches_a_numpy_restatement_and_sums_ascending(orc):
    rng = synth.rng_for(31)
    E, topk, hidden, ffn, ntok = 6, 2, 64, 96, 5
    gate = synth.mxfp4_matrix(rng, E * ffn, hidden)
    up = synth.mxfp4_matrix(rng, E * ffn, hidden)
    down = synth.mxfp4_matrix(rng, E * hidden, ffn)
    h = synth.activations(rng, ntok, hidden)
    logits = synth.activations(rng, ntok, E)
    sel = np.zeros((ntok, topk), np.int32)
    wt = np.zeros((ntok, topk), np.float32)
    for i in range(ntok):
        s, _, w, _, _ = orc.moe_router(orc.softmax(logits[i]), topk)
        sel[i], wt[i] = s, w
    got = orc.moe_layer(h, 39, gate, up, down, sel, wt, E, hidden, ffn, act_kind=0, nthreads=2)
    G = orc.dequant64(39, gate, E * ffn * hidden).reshape(E, ffn, hidden)
    U = orc.dequant64(39, up, E * ffn * hidden).reshape(E, ffn, hidden)
    D = orc.dequant64(39, down, E * hidden * ffn).reshape(E, hidden, ffn)
    want = np.zeros((ntok, hidden), np.float32)
    for i in range(ntok):
        for e in sorted(sel[i]):
            j = list(sel[i]).index(e)
            g = (G[e] @ h[i].astype(np.float64)).astype(np.float32).astype(np.float64)
            u = (U[e] @ h[i].astype(np.float64)).astype(np.float32).astype(np.float64)
            a = (g / (1 + np.exp(-g)) * u).astype(np.float32)
            y = (D[e] @ a.astype(np.float64)).astype(np.float32)
            want[i] = (want[i] + wt[i, j] * y).astype(np.float32)
    assert nmse(got, want) < 1e-12


def test_router_floors_the_divisor(orc):
    """Mirror of the reference's TestMoERouterFloorsTheDivisor (engine/nn/moev3_test.go:341): an all-zero selection
    gives finite, exactly-zero weights (divisor = sum + 1e-20), and an ordinary one still renormalises to 1."""
    n_exp, k = 8, 4
    dead = np.zeros(n_exp, np.float32)
    sel, _, wt, _, sm = orc.moe_router(dead, k)
    assert len(wt) == k and np.isfinite(wt).all() and not wt.any()
    assert sorted(sel.tolist()) == [0, 1, 2, 3]                # ties go to the lowest ids
    rng = np.random.default_rng(7)
    ordinary = (1.0 / (1.0 + np.exp(-rng.standard_normal(n_exp)))).astype(np.float32)
    _, _, wt, _, _ = orc.moe_router(ordinary, k)
    assert abs(float(np.sum(wt, dtype=np.float32)) - 1.0) <= 1e-6
