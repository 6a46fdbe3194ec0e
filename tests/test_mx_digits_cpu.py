"""The e4m3-digit arithmetic the block-scaled mixture arms rest on, checked on the CPU against its float64
restatement (the one the GPU tests hold the kernels to): how much each further digit leaves, and that two digits hold
a bf16 row."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from test_gpu_moe_bs import _mx8


def _rel_to_block_max(x, q):
    n, k = x.shape
    xb, qb = x.reshape(n, k // 32, 32).astype(np.float64), q.reshape(n, k // 32, 32)
    blk = np.abs(xb).max(-1, keepdims=True)
    return float((np.abs(qb - xb) / np.where(blk > 0, blk, 1.0)).max())


def test_each_digit_adds_four_bits():
    rng = np.random.default_rng(0x3D)
    x = (rng.standard_normal((16, 2880 // 32 * 32)) * rng.lognormal(0, 2, (16, 1))).astype(np.float32)
    errs = [_rel_to_block_max(x, _mx8(x, nd)) for nd in (1, 2, 3)]
    # e4m3 keeps 4 significant bits: half a unit of the last place is 2^-4 of the element, and an element is at
    # most its block's largest
    assert errs[0] <= 2.0 ** -4 and errs[1] <= 2.0 ** -8 and errs[2] <= 2.0 ** -12
    assert errs[0] > 16 * errs[1] * 0.25 and errs[1] > 16 * errs[2] * 0.25       # and not much better than that


def test_two_digits_hold_a_bf16_row_up_to_the_subnormal_step():
    rng = np.random.default_rng(0x2D)
    x = rng.standard_normal((32, 1024)).astype(np.float32)
    xb = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    q = _mx8(xb, 2)
    diff = np.abs(q - xb.astype(np.float64)).reshape(32, 32, 32)
    blk = np.abs(xb).reshape(32, 32, 32).max(-1, keepdims=True)
    # the scaled block maximum lies in (224, 448]; a remainder finer than e4m3's subnormal step 2^-9 belongs to an
    # element whose scaled magnitude is under 2^-2, i.e. under 2^-2 / 224 of its block's largest
    small = np.abs(xb).reshape(32, 32, 32) < blk * (0.25 / 224)
    assert np.all(diff[~small] == 0.0)                                   # exact wherever the remainder is representable
    assert float((diff / blk).max()) <= 2.0 ** -17                       # and negligible where it is not


def test_all_zero_and_single_spike_blocks():
    x = np.zeros((2, 64), np.float32)
    x[1, 5] = 3.0e4
    for nd in (1, 2, 3):
        q = _mx8(x, nd)
        assert np.all(q[0] == 0) and q[1, 5] == pytest.approx(3.0e4, rel=2.0 ** -4 if nd == 1 else 2.0 ** -8)
        assert np.all(np.delete(q[1], 5) == 0)
