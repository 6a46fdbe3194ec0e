"""Decode-operator parity on a B200, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

from conftest import nmse, parity_err
from jitllm_b200 import DECLINED, K_MMA, K_SIMT, MXFP4, Q4_K, Q8_0, Device, synth
from jitllm_b200._lib import FORM_FUSED, FORM_L1, FORM_SPLIT, FORM_WIDE

pytestmark = pytest.mark.gpu

BAR = 2e-3  # max_i |got-ref| / max(|ref_i|, rms(ref)), f32 accumulate


def _check(dev, orc, t, nrows, k, seed, x=None):
    rng = synth.rng_for(seed)
    w = synth.matrix(rng, t, nrows, k)
    if x is None:
        x = synth.activations(rng, 1, k)[0]
    out = np.full(nrows, np.nan, np.float32)  # poisoned: every row must be written
    assert dev.MatVec(out, t, w, x, nrows, k), dev.Err()
    ref = orc.matmul_f64(t, w, x, nrows, k, 1)[0]
    assert np.isfinite(out).all()
    err = parity_err(out, ref)
    assert err <= BAR, (err, nmse(out, ref))
    dev.Forget(w)
    return out, ref, w, x


@pytest.mark.parametrize("t", [Q4_K, Q8_0, MXFP4])
@pytest.mark.parametrize("nrows,k", [(16, 256), (1, 256), (37, 512), (256, 2048), (4096, 4096)])
def test_matvec_check_kernel_matches_oracle(orc, t, nrows, k):
    with Device(0, pin_kernel=K_SIMT) as d:
        out, ref, _, _ = _check(d, orc, t, nrows, k, 0xB200 + nrows + k + t)
        assert nmse(out, ref) < 1e-10


@pytest.mark.parametrize("t", [2, 6, 7, 13, 14])
@pytest.mark.parametrize("nrows,k,ntok", [(16, 256, 1), (1, 256, 1), (37, 512, 3), (256, 2048, 1), (4096, 4096, 1), (128256 // 64, 4096, 2)])
def test_more_formats_on_the_row_kernel_match_dequant32(orc, t, nrows, k, ntok):
    """Q4_0, Q5_0, Q5_1, Q5_K, Q6_K (what real Q4_K_M files carry beside Q4_K: Q6_K in the head and in half of the
    v / down projections) stay as raw blocks on the device and run on the one-warp-per-row kernel, every weight formed
    exactly as quant.Dequant32 forms it: f32 accumulation is the only difference from the f64 oracle."""
    rng = synth.rng_for(0xB400 + t + nrows + k)
    w = synth.matrix(rng, t, nrows, k)
    x = synth.activations(rng, ntok, k)
    with Device(0) as d:
        ch = d.Select(t, nrows, k, ntok)
        assert ch is not None and ch.kernel == K_SIMT
        out = np.full((ntok, nrows), np.nan, np.float32)
        assert d.MatMul(out, t, w, x, nrows, k, ntok), d.Err()
        ref = orc.matmul_f64(t, w, x, nrows, k, ntok)
        assert np.isfinite(out).all()
        assert parity_err(out, ref) <= BAR
        assert nmse(out, ref) < 1e-10


@pytest.mark.parametrize("warps", [4, 8, 16])
@pytest.mark.parametrize("nrows,k", [(16, 256), (16, 512), (5, 256), (100, 1024), (4096, 4096), (1024, 4096),
                                      (4096, 14336), (14336, 4096)])
def test_q4k_tensor_core_decode_matches_oracle(orc, warps, nrows, k):
    with Device(0, pin_kernel=K_MMA, pin_warps=warps) as d:
        ch = d.Select(Q4_K, nrows, k, 1)
        assert ch is not None and ch.kernel == K_MMA
        out, ref, _, _ = _check(d, orc, Q4_K, nrows, k, 0xB200 + nrows * 3 + k + warps)
        # far inside the reference's own bar for its f16 tensor-core GEMM (NMSE <= 1e-5,
        # jit/gpu/backend/mmavolta_test.go:278); the f32 check kernel above meets 1e-10
        assert nmse(out, ref) < 1e-8


def test_q4k_decode_equals_oracle_matvec_config0(dev, orc):
    """The headline workload verbatim: 4096x4096 Q4_K, x ~ N(0,1) f32, one seed."""
    rng = synth.rng_for(0xB200)
    w = synth.q4k_matrix(rng, 4096, 4096)
    x = synth.activations(rng, 1, 4096)[0]
    out = np.full(4096, np.nan, np.float32)
    assert dev.MatVec(out, Q4_K, w, x, 4096, 4096), dev.Err()
    ref32 = orc.matvec(Q4_K, w, x, 4096, 4096)          # oracle.MatVec, compensated f32
    ref64 = orc.matmul_f64(Q4_K, w, x, 4096, 4096, 1)[0]
    assert parity_err(out, ref64) <= BAR
    assert parity_err(out, ref32) <= BAR
    assert nmse(out, ref64) < 1e-8
    # same bits twice: the cross-warp reduction has a fixed order
    out2 = np.empty_like(out)
    assert dev.MatVec(out2, Q4_K, w, x, 4096, 4096)
    assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))
    # the reference's int8-activation CPU path sits ~1e-5 NMSE away (reported, not gated there)
    twin = orc.matmul_int8(Q4_K, w, x, 4096, 4096, 1, window=256)[0]
    assert nmse(twin, ref64) < 2e-4
    dev.Forget(w)


@pytest.mark.parametrize("dist", ["uniform", "student_t", "one_huge", "tiny", "huge", "zeros"])
def test_q4k_decode_input_distributions(dev, orc, dist):
    # jit/cpu/matvec_test.go:56-115 runs four activation distributions; the scaled hi/lo split
    # must also survive ranges f16 alone cannot hold.
    rng = synth.rng_for(77)
    k = 2048
    if dist == "uniform":
        x = rng.uniform(-1, 1, k)
    elif dist == "student_t":
        x = rng.standard_t(3, k)
    elif dist == "one_huge":
        x = rng.standard_normal(k); x[::32] *= 1000.0
    elif dist == "tiny":
        x = rng.standard_normal(k) * 1e-9
    elif dist == "huge":
        x = rng.standard_normal(k) * 1e9
    else:
        x = np.zeros(k)
    out, ref, _, _ = _check(dev, orc, Q4_K, 64, k, 78, x=x.astype(np.float32))
    if dist == "zeros":
        assert not out.any()


def test_planted_scales(dev, orc):
    # quant.PlantScales (format/quant/types.go:158-216): subnormal and extreme f16 super-scales.
    rng = synth.rng_for(9)
    n, k = 32, 1024
    nb = n * k // 256
    scales = synth.planted_f16_scales()
    blk = synth.q4k_from_parts(np.resize(scales, nb), np.resize(scales[::-1], nb),
                               rng.integers(0, 64, (nb, 8)), rng.integers(0, 64, (nb, 8)),
                               rng.integers(0, 16, (nb, 256))).reshape(n, -1)
    x = synth.activations(rng, 1, k)[0]
    for pin in (K_SIMT, K_MMA):
        with Device(0, pin_kernel=pin) as d:
            out = np.full(n, np.nan, np.float32)
            assert d.MatVec(out, Q4_K, blk, x, n, k), d.Err()
            ref = orc.matmul_f64(Q4_K, blk, x, n, k, 1)[0]
            assert parity_err(out, ref) <= BAR


def test_small_batch_matmul_matches_oracle(dev, orc):
    rng = synth.rng_for(55)
    for t, nrows, k, ntok in [(Q4_K, 128, 1024, 3), (Q8_0, 96, 512, 5), (MXFP4, 64, 320 * 2, 2)]:
        w = synth.matrix(rng, t, nrows, k)
        x = synth.activations(rng, ntok, k)
        out = np.full((ntok, nrows), np.nan, np.float32)
        assert dev.MatMul(out, t, w, x, nrows, k, ntok), dev.Err()
        ref = orc.matmul_f64(t, w, x, nrows, k, ntok)
        assert parity_err(out, ref) <= BAR
        dev.Forget(w)


@pytest.mark.parametrize("t", [Q4_K, Q8_0, MXFP4, 2, 6, 7, 13, 14])
def test_resident_copy_unpacks_bit_exact(dev, orc, t):
    # the repack at upload is a permutation: codes, scales and raw d bits survive it exactly
    from jitllm_b200._lib import BLOCK
    rng = synth.rng_for(200 + t)
    nrows, k = 24, 1024 if BLOCK[t][0] == 256 else 640
    w = synth.matrix(rng, t, nrows, k)
    h = dev.Upload(t, w, nrows, k)
    got = h.unpack()
    want = orc.unpack(t, w, w.size // BLOCK[t][1])
    for g, x in zip(got, want):
        assert np.array_equal(g, x)
    h.free()


def test_declines_and_errors_follow_the_reference_contract(dev):
    out = np.zeros(8, np.float32)
    x = np.zeros(100, np.float32)
    w = np.zeros(4096, np.uint8)
    assert not dev.MatVec(out, 3, w, x, 8, 64)          # Q4_1: unsupported type declines
    assert dev.last_status == DECLINED and "not served" in dev.Err()
    assert not dev.MatVec(out, Q4_K, w, x, 8, 100)      # ragged k declines
    assert dev.last_status == DECLINED
    assert not dev.MatVec(out, Q4_K, w[:100], x, 8, 256)  # short weight is an error, not a decline
    assert dev.last_status < 0


def test_residency_is_keyed_on_the_host_pointer_and_forget_drops_it(orc):
    rng = synth.rng_for(3)
    w = synth.q4k_matrix(rng, 64, 512)
    x = synth.activations(rng, 1, 512)[0]
    out = np.zeros(64, np.float32)
    with Device(0) as d:
        assert d.MatVec(out, Q4_K, w, x, 64, 512)
        assert d.MatVec(out, Q4_K, w, x, 64, 512)
        s = d.Stats()
        assert s.uploads == 1 and s.served == 2 and s.resident_bytes == w.nbytes
        first = out.copy()
        # the caller rewrites the bytes in place and says so
        w[:] = synth.q4k_matrix(rng, 64, 512)
        d.Forget(w)
        assert d.Stats().resident_bytes == 0 and d.Stats().forgets == 1
        assert d.MatVec(out, Q4_K, w, x, 64, 512)
        assert d.Stats().uploads == 2
        assert not np.array_equal(out, first)
        assert parity_err(out, orc.matmul_f64(Q4_K, w, x, 64, 512, 1)[0]) <= BAR


def test_min_weight_bytes_declines_small_weights():
    w = synth.q4k_matrix(synth.rng_for(1), 16, 256)
    with Device(0, min_weight_bytes=1 << 20) as d:
        assert not d.MatVec(np.zeros(16, np.float32), Q4_K, w, np.zeros(256, np.float32), 16, 256)
        assert d.last_status == DECLINED and "break-even" in d.Err()


def test_host_side_fault_injection(orc):
    # jit/gpu/tier/fault.go:12-58: fail the n-th call on the host; the caller sees an error and
    # the context stays usable.
    w = synth.q4k_matrix(synth.rng_for(1), 16, 256)
    x = synth.activations(synth.rng_for(2), 1, 256)[0]
    out = np.zeros(16, np.float32)
    with Device(0) as d:
        d.FailAt([2])
        assert d.MatVec(out, Q4_K, w, x, 16, 256)
        assert not d.MatVec(out, Q4_K, w, x, 16, 256)
        assert d.last_status == -4 and "injected" in d.Err()
        assert d.MatVec(out, Q4_K, w, x, 16, 256)
        assert d.Stats().injected == 1


@pytest.mark.parametrize("ntok", [1, 3, 4, 7, 8])
@pytest.mark.parametrize("nrows,k", [(16, 256), (5, 512), (100, 1024), (4096, 4096), (1024, 4096), (14336, 4096)])
def test_q8_0_tensor_core_decode_matches_oracle(orc, nrows, k, ntok):
    """Q8_0 decode: int8 codes straight into mma.sync.s8.s8, activations as two int8 digits."""
    if ntok > 1 and nrows > 4096:
        pytest.skip("the large shape is covered at one token")
    rng = synth.rng_for(0xB280 + nrows + k + ntok)
    w = synth.q8_0_matrix(rng, nrows, k)
    x = synth.activations(rng, ntok, k)
    with Device(0, pin_kernel=K_MMA) as d:
        ch = d.Select(Q8_0, nrows, k, ntok)
        assert ch is not None and ch.kernel == K_MMA and ch.tile_k == 32
        out = np.full((ntok, nrows), np.nan, np.float32)
        assert d.MatMul(out, Q8_0, w, x, nrows, k, ntok), d.Err()
        ref = orc.matmul_f64(Q8_0, w, x, nrows, k, ntok)
        assert np.isfinite(out).all()
        assert parity_err(out, ref) <= BAR, parity_err(out, ref)
        assert nmse(out, ref) < 1e-8
        out2 = np.empty_like(out)
        assert d.MatMul(out2, Q8_0, w, x, nrows, k, ntok)
        assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))      # fixed reduction order


def test_q8_0_decode_survives_extreme_activations(orc):
    rng = synth.rng_for(41)
    nrows, k = 64, 1024
    w = synth.q8_0_matrix(rng, nrows, k)
    for scale in (1e-30, 1.0, 1e30):
        x = (synth.activations(rng, 1, k) * np.float32(scale)).astype(np.float32)
        x[0, 5] = 0.0
        with Device(0) as d:
            out = np.full((1, nrows), np.nan, np.float32)
            assert d.MatMul(out, Q8_0, w, x, nrows, k, 1), d.Err()
        ref = orc.matmul_f64(Q8_0, w, x, nrows, k, 1)
        assert parity_err(out, ref) <= BAR
    with Device(0) as d:
        out = np.full((1, nrows), np.nan, np.float32)
        assert d.MatMul(out, Q8_0, w, np.zeros((1, k), np.float32), nrows, k, 1)
        assert not out.any()


@pytest.mark.parametrize("nrows,k", [(16, 256), (100, 1024), (4096, 4096), (8192, 4096), (4096, 14336)])
def test_q4k_concurrent_variant_matches_oracle(orc, nrows, k):
    """JL_FLAG_DECODE_CONCURRENT: small CTAs, weight tiles only in shared memory, operand through L1."""
    from jitllm_b200._lib import FLAG_DECODE_CONCURRENT
    with Device(0, flags=FLAG_DECODE_CONCURRENT) as d:
        out, ref, w, x = _check(d, orc, Q4_K, nrows, k, 0xB2C0 + nrows + k)
        assert nmse(out, ref) < 1e-8
        out2 = np.empty_like(out)
        assert d.MatVec(out2, Q4_K, w, x, nrows, k)
        assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))
    with Device(0) as d:
        out3 = np.empty_like(out)
        assert d.MatVec(out3, Q4_K, w, x, nrows, k)
        assert parity_err(out3, out.astype(np.float64)) < 1e-5          # same arithmetic, summation order only


@pytest.mark.parametrize("ntok", [1, 3, 4, 8])
@pytest.mark.parametrize("nrows,k", [(16, 64), (5, 128), (100, 1024), (2880, 2880), (4096, 4096)])
def test_mxfp4_tensor_core_decode_matches_oracle(orc, nrows, k, ntok):
    """MXFP4 decode: e2m1 codes placed bit-wise into f16 A fragments (value * 2^-14, subnormals for 0 and 0.5),
    block scales folded in f32 after the MMAs. Exercises every code and scales 2^-8..2^0."""
    rng = synth.rng_for(0xB2F0 + nrows + k + ntok)
    w = synth.mxfp4_matrix(rng, nrows, k)
    x = synth.activations(rng, ntok, k)
    with Device(0, pin_kernel=K_MMA) as d:
        ch = d.Select(MXFP4, nrows, k, ntok)
        assert ch is not None and ch.kernel == K_MMA and ch.tile_k == 16
        out = np.full((ntok, nrows), np.nan, np.float32)
        assert d.MatMul(out, MXFP4, w, x, nrows, k, ntok), d.Err()
        ref = orc.matmul_f64(MXFP4, w, x, nrows, k, ntok)
        assert np.isfinite(out).all()
        assert parity_err(out, ref) <= BAR, parity_err(out, ref)
        assert nmse(out, ref) < 1e-8
        out2 = np.empty_like(out)
        assert d.MatMul(out2, MXFP4, w, x, nrows, k, ntok)
        assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))


def test_mxfp4_decode_half_codes_and_wide_scales(orc):
    """Only the codes +-0.5 (the f16-subnormal images) and +-6, with block scales from 2^-40 to 2^+40."""
    rng = synth.rng_for(17)
    nrows, k = 48, 256
    nb = nrows * k // 32
    codes = rng.choice(np.array([1, 9, 7, 15], np.uint8), (nb, 32))
    e = (127 + rng.integers(-40, 41, nb)).astype(np.uint8)
    w = synth.mxfp4_from_parts(e, codes).reshape(nrows, -1)
    x = synth.activations(rng, 2, k)
    with Device(0) as d:
        out = np.full((2, nrows), np.nan, np.float32)
        assert d.MatMul(out, MXFP4, w, x, nrows, k, 2), d.Err()
    ref = orc.matmul_f64(MXFP4, w, x, nrows, k, 2)
    assert parity_err(out, ref) <= BAR


# (form, warps, ring stages, 16-row groups per CTA) of pinned Q4_K decode variants
VARIANTS = [(FORM_WIDE, 16, 2, 4), (FORM_WIDE, 8, 3, 4), (FORM_WIDE, 8, 3, 2), (FORM_WIDE, 16, 2, 8),
            (FORM_L1, 4, 3, 0), (FORM_L1, 2, 3, 0), (FORM_SPLIT, 8, 4, 0), (FORM_SPLIT, 2, 8, 0), (FORM_FUSED, 16, 2, 0)]


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("nrows,k", [(16, 256), (100, 1024), (4096, 4096), (1030, 2048)])
def test_q4k_decode_variants_pinned_by_form(orc, variant, nrows, k):
    """Every form of the Q4_K tensor-core decode, pinned through jl_opts (decode_form, pin_warps, pin_stages,
    pin_row_groups): the single-launch wide forms (a CTA of 32..128 rows converts the activation row itself),
    the small-CTA forms that read the operand through L1, split and fused. jl_select reports the pinned
    variant, the result meets the oracle and repeats bit for bit."""
    form, warps, stages, rg = variant
    with Device(0, pin_kernel=K_MMA, decode_form=form, pin_warps=warps, pin_stages=stages, pin_row_groups=rg) as d:
        ch = d.Select(Q4_K, nrows, k, 1)
        assert (ch.kernel, ch.form, ch.warps, ch.stages) == (K_MMA, form, warps, stages)
        assert ch.rows_per_cta == 16 * max(rg, 1) and ch.grid == -(-(-(-nrows // 16)) // max(rg, 1))
        out, ref, w, x = _check(d, orc, Q4_K, nrows, k, 0xB2D0 + form * 100 + warps + nrows)
        assert nmse(out, ref) < 1e-8
        out2 = np.empty_like(out)
        assert d.MatVec(out2, Q4_K, w, x, nrows, k)
        assert np.array_equal(out.view(np.uint32), out2.view(np.uint32))


@pytest.mark.parametrize("t,nrows,k,ntok", [(Q4_K, 4096, 4096, 1), (Q4_K, 14336, 4096, 1), (Q4_K, 4096, 14336, 1),
                                             (Q4_K, 64, 512, 1), (Q4_K, 4096, 4096, 4), (Q8_0, 4096, 4096, 1),
                                             (Q8_0, 1024, 4096, 8), (MXFP4, 2880, 2880, 1), (MXFP4, 96, 576, 1),
                                             (Q4_K, 4096, 4096, 32), (Q8_0, 4096, 4096, 32)])
@pytest.mark.parametrize("flags", [0, 16])
def test_select_reports_what_launches(t, nrows, k, ntok, flags):
    """jl_select's answer and the launch share one selection: the number of kernels a device-pointer call adds
    to jl_stats.launches equals jl_choice.launches, and the default 4096x4096 decode reports the wide form
    that actually runs (64-row CTAs, one per row group of four), not a 16-row grid."""
    import torch
    rng = synth.rng_for(77)
    with Device(0, flags=flags) as d:
        d.Reserve(nrows, k, ntok)
        h = d.Upload(t, synth.matrix(rng, t, nrows, k), nrows, k)
        ch = d.Select(t, nrows, k, ntok)
        assert ch is not None and ch.launches >= 1 and ch.grid >= 1
        x = torch.randn(ntok, k, device="cuda")
        out = torch.empty(ntok, nrows, device="cuda")
        n0 = d.Stats().launches
        d.MatMulDev(out, h, x, ntok, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert d.Stats().launches - n0 == ch.launches
        if t == Q4_K and ch.kernel == K_MMA:
            assert ch.tile_k == 32 and ch.form in (FORM_SPLIT, FORM_FUSED, FORM_WIDE, FORM_L1)
            assert ch.launches == (2 if ch.form in (FORM_SPLIT, FORM_L1) else 1)
        if (t, nrows, k, ntok, flags) == (Q4_K, 4096, 4096, 1, 0):
            assert (ch.form, ch.warps, ch.rows_per_cta, ch.grid, ch.stages) == (FORM_WIDE, 16, 64, 64, 2)
        h.free()


def test_a_wait_that_runs_out_surfaces_as_etimedout_and_the_context_stays_usable(orc):
    """Every device-side wait is bounded by the GPU's global timer. A test kernel waits (limit 1 ms) on an
    mbarrier that expects bytes nobody sends; it records the timeout and returns. jl_status_poll reports
    JL_ETIMEDOUT once, then JL_OK, and the same context still serves a matvec. No GPU fault is involved."""
    import time
    from jitllm_b200 import _lib
    with Device(0) as d:
        assert d.StatusPoll()
        t0 = time.perf_counter()
        assert d.lib.jl_test_wait_timeout(d.ctx, 1000, None) == _lib.OK
        assert not d.StatusPoll()
        assert time.perf_counter() - t0 < 1.0                      # the wait gave up after about a millisecond
        assert d.last_status == _lib.ETIMEDOUT and "test wait" in d.Err()
        assert d.StatusPoll()                                      # cleared on read
        out, ref, _, _ = _check(d, orc, Q4_K, 256, 1024, 3)
        assert parity_err(out, ref) <= BAR
        assert d.lib.jl_noalloc_status(None) == _lib.OK


def test_eviction_under_a_cap_re_uploads_with_correct_results(orc):
    """max_resident_bytes: the least recently used copy makes room, a later call on the evicted tensor uploads
    it again and still matches the oracle."""
    rng = synth.rng_for(31)
    nrows, k = 512, 1024
    ws = [synth.q4k_matrix(rng, nrows, k) for _ in range(3)]
    x = synth.activations(rng, 1, k)[0]
    one = ws[0].nbytes
    with Device(0, max_resident_bytes=2 * one + 16) as d:
        out = np.empty(nrows, np.float32)
        for w in ws:
            assert d.MatVec(out, Q4_K, w, x, nrows, k), d.Err()
        st = d.Stats()
        assert st.uploads == 3 and st.resident_bytes == 2 * one
        assert d.MatVec(out, Q4_K, ws[0], x, nrows, k), d.Err()    # evicted above: uploaded again
        assert d.Stats().uploads == 4 and d.Stats().resident_bytes == 2 * one
        assert parity_err(out, orc.matmul_f64(Q4_K, ws[0], x, nrows, k, 1)[0]) <= BAR
        assert d.MatVec(out, Q4_K, ws[2], x, nrows, k) and d.Stats().uploads == 4   # still resident
    with Device(0, max_resident_bytes=one // 2) as d:              # a cap below one tensor: refused, not served wrongly
        assert not d.MatVec(out, Q4_K, ws[0], x, nrows, k)
        assert d.last_status == -3


def test_forget_unlinks_at_once_and_frees_on_the_next_serving_call(orc):
    rng = synth.rng_for(32)
    nrows, k = 256, 1024
    w, w2 = synth.q4k_matrix(rng, nrows, k), synth.q4k_matrix(rng, nrows, k)
    x = synth.activations(rng, 1, k)[0]
    out = np.empty(nrows, np.float32)
    with Device(0) as d:
        assert d.MatVec(out, Q4_K, w, x, nrows, k)
        d.Forget(w)
        st = d.Stats()
        assert st.forgets == 1 and st.resident_bytes == 0
        w[:] = w2                                                   # the caller may reuse the memory after Forget
        assert d.MatVec(out, Q4_K, w, x, nrows, k)
        assert d.Stats().uploads == 2
        assert parity_err(out, orc.matmul_f64(Q4_K, w2, x, nrows, k, 1)[0]) <= BAR


@pytest.mark.parametrize("t", [Q4_K, Q8_0, MXFP4])
@pytest.mark.parametrize("dist", ["uniform", "student_t", "one_huge_per_block", "saturating"])
def test_decode_reference_distributions_and_shapes(orc, t, dist):
    """The reference's kernel gate (jit/cpu/matvec_test.go:46-143): its four activation distributions -- uniform,
    heavy-tailed, one huge value per 32-block, alternating +-1 -- at its five shapes, for every decode kernel."""
    shapes = [(1, 256), (4, 512), (8, 1024), (32, 2048), (3, 768)]
    with Device(0) as d:
        for nrows, k in shapes:
            rng = synth.rng_for(nrows * 1000 + k)
            w = synth.matrix(rng, t, nrows, k)
            if dist == "uniform":
                x = rng.uniform(-1, 1, k)
            elif dist == "student_t":
                x = rng.standard_normal(k) / (0.1 + np.abs(rng.standard_normal(k)))
            elif dist == "one_huge_per_block":
                x = rng.uniform(0, 0.01, k); x[7::32] = 1000.0
            else:
                x = np.where(np.arange(k) % 2 == 0, 1.0, -1.0)
            x = x.astype(np.float32)
            out = np.full(nrows, np.nan, np.float32)
            assert d.MatVec(out, t, w, x, nrows, k), d.Err()
            ref = orc.matmul_f64(t, w, x, nrows, k, 1)[0]
            assert np.isfinite(out).all()
            assert parity_err(out, ref) <= BAR, (nrows, k, parity_err(out, ref))
            d.Forget(w)


def test_measured_selection_times_the_variants_persists_and_is_what_launches(orc, tmp_path):
    """With tuning on, the first upload of a shape runs the timed duel over the decode variants; the verdict is what
    jl_select reports AND what launches; it persists, a second context answers from the file without a single trial,
    a damaged entry is measured again and overwritten, and a context that pins its form does not tune."""
    import torch
    from jitllm_b200 import _lib
    rng = synth.rng_for(0x7E)
    nrows, k = 4096, 4096
    w = synth.q4k_matrix(rng, nrows, k)
    x = synth.activations(rng, 1, k)
    ref = orc.matmul_f64(Q4_K, w, x, nrows, k, 1)
    cache = str(tmp_path / "tune")

    def serve(d, h):
        ch = d.Select(Q4_K, nrows, k, 1)
        xd, out = torch.from_numpy(x).cuda(), torch.empty(1, nrows, device="cuda")
        n0 = d.Stats().launches
        d.MatMulDev(out, h, xd, 1, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert d.Stats().launches - n0 == ch.launches
        assert parity_err(out.cpu().numpy(), ref) <= 2e-3
        return (ch.form, ch.warps, ch.stages, ch.rows_per_cta, ch.grid)

    with Device(0) as d:
        d.WithTune(_lib.TUNE_ON, cache)
        n0 = d.Stats().launches
        h = d.Upload(Q4_K, w, nrows, k)
        ts = d.TuneStats()
        assert ts["trials"] >= 2 * 11 and ts["measured"] + (1 if ts["refused"] else 0) >= 1
        assert d.Stats().launches == n0                              # trials are not served work
        first = serve(d, h)
        h2 = d.Upload(Q4_K, w, nrows, k)                             # the same shape again: no new trials
        assert d.TuneStats()["trials"] == ts["trials"]
        h.free(); h2.free()
    measured = ts["measured"] == 1
    if measured:
        line = open(cache + "/jl_select1").read()
        assert f"/12-{nrows}x{k}x1 " in line and line.count("\n") == 1
        with Device(0) as d:                                         # a later process: answered from the file
            d.WithTune(_lib.TUNE_ON, cache)
            h = d.Upload(Q4_K, w, nrows, k)
            ts2 = d.TuneStats()
            assert ts2["trials"] == 0 and ts2["cached"] == 1
            assert serve(d, h) == first
            h.free()
        key = line.split(" ")[0]
        open(cache + "/jl_select1", "w").write(f"{key} 9 9 9 9 9\n")  # names no variant: measured again, overwritten
        with Device(0) as d:
            d.WithTune(_lib.TUNE_ON, cache)
            h = d.Upload(Q4_K, w, nrows, k)
            ts3 = d.TuneStats()
            assert ts3["trials"] > 0 and ts3["cached"] == 0
            serve(d, h)
            h.free()
        if ts3["measured"]:
            assert " 9 9 9 9 9" not in open(cache + "/jl_select1").read()
    with Device(0, decode_form=FORM_SPLIT) as d:                     # the caller chose already
        d.WithTune(_lib.TUNE_FORCE, cache)
        h = d.Upload(Q4_K, w, nrows, k)
        assert d.TuneStats()["trials"] == 0
        assert d.Select(Q4_K, nrows, k, 1).form == FORM_SPLIT
        h.free()
    with Device(0) as d:                                             # explicit call on a context with tuning off
        h = d.Upload(Q4_K, w, nrows, k)
        assert d.TuneStats()["trials"] == 0
        ch = d.Tune(h, 2)
        assert ch is not None and d.TuneStats()["trials"] > 0
        assert (ch.form, ch.warps, ch.stages) == (lambda c: (c.form, c.warps, c.stages))(d.Select(Q4_K, nrows, k, 2))
        h.free()
