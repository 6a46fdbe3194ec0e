"""The decode kernels' activation representation, restated in numpy and checked on the CPU: every activation is
scaled by s = 32512 / amax of its group and written as two int8 digits, x * s ~ 256 q1 + q2. This file pins the
claims the kernels rely on: both digits fit int8, the representation error is at most half a unit (1.5e-5 of the
group's amax; one unit, 3.1e-5, in the rare case that the second digit saturates at +-127), the integer sums stay inside int32, and a Q8_0 matvec built from the digits sits far inside the
2e-3 output bar for the reference's four test distributions (jit/cpu/matvec_test.go:56-115)."""
import numpy as np
import pytest

from jitllm_b200 import synth
from jitllm_b200._lib import Q8_0


def digits(x: np.ndarray, group: int):
    """(q1, q2, inv_s) of x [k] with one scale per `group` elements, exactly as the prep kernels compute them."""
    g = x.reshape(-1, group).astype(np.float32)
    amax = np.max(np.abs(g), axis=1, keepdims=True)
    live = (amax > 0) & np.isfinite(amax)
    scale = np.where(live, np.float32(32512.0) / np.where(live, amax, 1), 0).astype(np.float32)
    xs = (g * scale).astype(np.float32)
    q1 = np.rint(xs * np.float32(1.0 / 256.0))
    q2 = np.clip(np.rint(xs - np.float32(256.0) * q1), -127, 127)
    inv_s = np.where(live, amax / np.float32(32512.0), 0).astype(np.float32)
    return q1.astype(np.int32).reshape(-1), q2.astype(np.int32).reshape(-1), inv_s.reshape(-1), xs.reshape(-1)


DISTS = {
    "uniform": lambda rng, k: rng.uniform(-1, 1, k),
    "student_t": lambda rng, k: rng.standard_normal(k) / (0.1 + np.abs(rng.standard_normal(k))),
    "one_huge_per_block": lambda rng, k: np.where(np.arange(k) % 32 == 7, 1000.0, rng.uniform(0, 0.01, k)),
    "saturating": lambda rng, k: np.where(np.arange(k) % 2 == 0, 1.0, -1.0),
    "tiny": lambda rng, k: rng.standard_normal(k) * 1e-30,
    "huge": lambda rng, k: rng.standard_normal(k) * 1e30,
}


@pytest.mark.parametrize("dist", sorted(DISTS))
@pytest.mark.parametrize("group", [32, 256])
def test_two_digits_hold_the_activation(dist, group):
    rng = np.random.default_rng(5)
    x = DISTS[dist](rng, 2048).astype(np.float32)
    q1, q2, inv_s, xs = digits(x, group)
    assert np.abs(q1).max() <= 127 and np.abs(q2).max() <= 127            # both digits are int8
    err = np.abs(xs - (256 * q1 + q2))
    assert np.max(err) <= 1.0 + 1e-3                                     # one unit of 1/s at worst ...
    assert np.all(err[np.abs(q2) < 127] <= 0.5 + 2e-3)                   # ... half a unit unless the second digit saturates
    back = (256 * q1 + q2).reshape(-1, group) * inv_s[:, None]
    amax = np.max(np.abs(x.reshape(-1, group)), axis=1, keepdims=True)
    assert np.all(np.abs(back - x.reshape(-1, group)) <= 3.2e-5 * amax + 1e-45)


@pytest.mark.parametrize("dist", ["uniform", "student_t", "one_huge_per_block", "saturating"])
def test_q8_0_matvec_from_digits_meets_the_output_bar(orc, dist):
    """Integer dot of int8 codes with each digit, 256 * S1 + S2 folded with d and 1/s per 32-block: the Q8_0 decode
    kernel's arithmetic, against the exact dot."""
    rng = synth.rng_for(11)
    nrows, k = 64, 1024
    w = synth.q8_0_matrix(rng, nrows, k)
    x = DISTS[dist](np.random.default_rng(3), k).astype(np.float32)
    q, d_bits, _, _, _ = orc.unpack(Q8_0, w, nrows * k // 32)
    codes = np.asarray(q, np.int64).reshape(nrows, k // 32, 32)
    d = np.asarray(d_bits, np.uint16).view(np.float16).astype(np.float64).reshape(nrows, k // 32)
    q1, q2, inv_s, _ = digits(x, 32)
    s1 = np.einsum("rbi,bi->rb", codes, q1.reshape(-1, 32).astype(np.int64))
    s2 = np.einsum("rbi,bi->rb", codes, q2.reshape(-1, 32).astype(np.int64))
    assert np.abs(256 * s1 + s2).max() < 2 ** 31                            # the kernel's int32 never overflows
    got = np.sum(d * inv_s[None, :].astype(np.float64) * (256 * s1 + s2), axis=1)
    ref = orc.matmul_f64(Q8_0, w, x, nrows, k, 1)[0]
    err = np.max(np.abs(got - ref) / np.maximum(np.abs(ref), np.sqrt(np.mean(ref * ref))))
    assert err <= 2e-4, err
