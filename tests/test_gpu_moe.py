"""Mixture-of-experts layer (router, token lists, grouped tcgen05 GEMMs, ascending-id combine)
on a B200 through the C ABI, against the CPU oracle of State.moeBatch."""
import numpy as np
import pytest

from conftest import nmse, parity_err
from jitllm_b200 import ACT_SILU, ACT_SWIGLU_OAI, MXFP4, Device, synth

pytestmark = pytest.mark.gpu
BAR = 2e-3


def _layer(rng, E, hidden, ffn):
    return (synth.mxfp4_matrix(rng, E * ffn, hidden), synth.mxfp4_matrix(rng, E * ffn, hidden),
            synth.mxfp4_matrix(rng, E * hidden, ffn))


def _oracle(orc, h, logits, gate, up, down, E, topk, hidden, ffn, act=0, **bias):
    ntok = h.shape[0]
    sel = np.zeros((ntok, topk), np.int32)
    wt = np.zeros((ntok, topk), np.float32)
    lg = logits + bias["router_bias"][None, :] if bias.get("router_bias") is not None else logits
    for i in range(ntok):
        s, _, w, _, _ = orc.moe_router(orc.softmax(lg[i].astype(np.float32)), topk)
        sel[i], wt[i] = s, w
    out = orc.moe_layer(h, MXFP4, gate, up, down, sel, wt, E, hidden, ffn, act_kind=act,
                        bgate=bias.get("gate_bias"), bup=bias.get("up_bias"), bdown=bias.get("down_bias"))
    return out, sel, wt


@pytest.mark.parametrize("E,topk,hidden,ffn,ntok", [(8, 2, 128, 192, 20), (4, 4, 64, 64, 3), (16, 4, 256, 320, 70),
                                                     (8, 1, 192, 128, 9),
                                                     (4, 2, 64, 64, 600)])
@pytest.mark.parametrize("h_bf16", [True, False])
def test_moe_layer_matches_oracle(dev, orc, E, topk, hidden, ffn, ntok, h_bf16):
    rng = synth.rng_for(1000 + E + hidden + ntok)
    gate, up, down = _layer(rng, E, hidden, ffn)
    h = synth.activations(rng, ntok, hidden) * np.float32(0.25)
    logits = synth.activations(rng, ntok, E)
    if h_bf16:
        hin = synth.to_bf16_bits(h)
        h = synth.bf16_bits_to_f32(hin)
    else:
        hin = h
    out = np.zeros((ntok, hidden), np.float32)
    sel = np.full((ntok, topk), -7, np.int32)
    wt = np.full((ntok, topk), np.nan, np.float32)
    assert dev.MoeHost(out, hin, logits, gate, up, down, E, topk, hidden, ffn, sel_out=sel, wt_out=wt), dev.Err()
    ref, rsel, rwt = _oracle(orc, h, logits, gate, up, down, E, topk, hidden, ffn)
    assert np.array_equal(sel, rsel), "selected experts and their order"
    assert np.allclose(wt, rwt, rtol=2e-6, atol=0)
    assert np.isfinite(out).all()
    assert parity_err(out, ref) <= BAR, (parity_err(out, ref), nmse(out, ref))
    for w in (gate, up, down):
        dev.Forget(w)


def test_router_ties_go_to_the_lowest_id_and_out_is_added_to(dev, orc):
    rng = synth.rng_for(4)
    E, topk, hidden, ffn, ntok = 8, 3, 64, 64, 5
    gate, up, down = _layer(rng, E, hidden, ffn)
    h = synth.activations(rng, ntok, hidden)
    logits = np.zeros((ntok, E), np.float32)       # a fresh router emits identical logits
    logits[1, 5] = 1.0
    base = synth.activations(rng, ntok, hidden)
    out = base.copy()
    sel = np.zeros((ntok, topk), np.int32)
    assert dev.MoeHost(out, h, logits, gate, up, down, E, topk, hidden, ffn, sel_out=sel), dev.Err()
    assert list(sel[0]) == [0, 1, 2] and list(sel[1]) == [5, 0, 1]
    ref, _, _ = _oracle(orc, h, logits, gate, up, down, E, topk, hidden, ffn)
    assert parity_err(out - base, ref) <= BAR
    out2 = base.copy()
    assert dev.MoeHost(out2, h, logits, gate, up, down, E, topk, hidden, ffn)
    assert np.array_equal(out.view(np.uint32), out2.view(np.uint32)), "fixed combine order: same bits twice"
    for w in (gate, up, down):
        dev.Forget(w)


def test_swiglu_oai_with_biases(dev, orc):
    rng = synth.rng_for(6)
    E, topk, hidden, ffn, ntok = 8, 2, 128, 128, 17
    gate, up, down = _layer(rng, E, hidden, ffn)
    h = synth.activations(rng, ntok, hidden) * np.float32(0.1)
    logits = synth.activations(rng, ntok, E)
    b = dict(gate_bias=synth.activations(rng, E, ffn), up_bias=synth.activations(rng, E, ffn),
             down_bias=synth.activations(rng, E, hidden), router_bias=synth.activations(rng, 1, E)[0])
    out = np.zeros((ntok, hidden), np.float32)
    assert dev.MoeHost(out, h, logits, gate, up, down, E, topk, hidden, ffn, act=ACT_SWIGLU_OAI, **b), dev.Err()
    ref, _, _ = _oracle(orc, h, logits, gate, up, down, E, topk, hidden, ffn, act=1, **b)
    assert parity_err(out, ref) <= BAR
    for w in (gate, up, down):       # residency is keyed on the host address: forget before the arrays are freed
        dev.Forget(w)


def test_config3_gpt_oss_shape(dev, orc):
    """The gpt-oss-shaped mixture workload: hidden = ffn = 2880, 32 experts, top-4, 256 tokens, bf16 activations."""
    rng = synth.rng_for(0xB203)
    E, topk, hidden, ffn, ntok = 32, 4, 2880, 2880, 256
    gate, up, down = _layer(rng, E, hidden, ffn)
    hin = synth.to_bf16_bits(synth.activations(rng, ntok, hidden))
    h = synth.bf16_bits_to_f32(hin)
    logits = synth.activations(rng, ntok, E)
    out = np.zeros((ntok, hidden), np.float32)
    sel = np.zeros((ntok, topk), np.int32)
    assert dev.MoeHost(out, hin, logits, gate, up, down, E, topk, hidden, ffn, sel_out=sel), dev.Err()
    ref, rsel, _ = _oracle(orc, h, logits, gate, up, down, E, topk, hidden, ffn)
    assert np.array_equal(sel, rsel)
    assert parity_err(out, ref) <= BAR, (parity_err(out, ref), nmse(out, ref))
    for w in (gate, up, down):
        dev.Forget(w)


def test_declines(dev):
    z = np.zeros(17 * 64, np.uint8)
    out = np.zeros((1, 32), np.float32)
    assert not dev.MoeHost(out, np.zeros((1, 32), np.float32), np.zeros((1, 2), np.float32), z, z, z, 2, 1, 32, 32)
    assert dev.last_status == 1   # hidden not a multiple of 64: declined, not an error


@pytest.mark.parametrize("e_lo,e_hi", [(-23, -10), (-6, 1), (2, 12), (-20, 10)])
def test_moe_scale_ranges_cover_both_dequant_forms(dev, orc, e_lo, e_hi):
    """Block scales up to 2^1 take the conversion-free dequant (code bits read as an f16, one multiply); larger
    ones the e2m1 conversion. Both must be exact in f16, down to the subnormal end of the range."""
    rng = synth.rng_for(4000 + e_hi)
    E, topk, hidden, ffn, ntok = 4, 2, 128, 128, 12
    gate, up, down = (synth.mxfp4_matrix(rng, E * ffn, hidden, e_lo, e_hi), synth.mxfp4_matrix(rng, E * ffn, hidden, e_lo, e_hi),
                      synth.mxfp4_matrix(rng, E * hidden, ffn, e_lo, e_hi))
    # keep the layer's output in f32 range whatever the scales are
    h = synth.activations(rng, ntok, hidden) * np.float32(2.0 ** (-(e_lo + e_hi) // 2 - 2))
    logits = synth.activations(rng, ntok, E)
    out = np.zeros((ntok, hidden), np.float32)
    assert dev.MoeHost(out, h, logits, gate, up, down, E, topk, hidden, ffn), dev.Err()
    ref, _, _ = _oracle(orc, h, logits, gate, up, down, E, topk, hidden, ffn)
    assert np.isfinite(out).all() and np.isfinite(ref).all()
    assert parity_err(out, ref) <= BAR, (parity_err(out, ref), nmse(out, ref))
    for w in (gate, up, down):
        dev.Forget(w)


def test_selection_only_bias_changes_the_choice_not_the_weights(dev, orc):
    """MoEGate.Bias (internal/oracle/moe.go:204-262): added to the gated scores for the selection only; the
    weights come from the unbiased scores. Compared with the oracle's bias path."""
    rng = synth.rng_for(41)
    E, topk, hidden, ffn, ntok = 16, 4, 128, 128, 33
    gate, up, down = _layer(rng, E, hidden, ffn)
    h = synth.activations(rng, ntok, hidden) * np.float32(0.25)
    logits = synth.activations(rng, ntok, E)
    sel_bias = (rng.standard_normal(E) * 0.2).astype(np.float32)
    rsel = np.zeros((ntok, topk), np.int32)
    rwt = np.zeros((ntok, topk), np.float32)
    plain = np.zeros((ntok, topk), np.int32)
    for i in range(ntok):
        sc = orc.softmax(logits[i])
        rsel[i], _, rwt[i], _, _ = orc.moe_router(sc, topk, bias=sel_bias)
        plain[i] = orc.moe_router(sc, topk)[0]
    assert not np.array_equal(rsel, plain), "the bias must change at least one selection for this test to mean anything"
    ref = orc.moe_layer(h, MXFP4, gate, up, down, rsel, rwt, E, hidden, ffn)
    out = np.zeros((ntok, hidden), np.float32)
    sel = np.full((ntok, topk), -7, np.int32)
    wt = np.full((ntok, topk), np.nan, np.float32)
    assert dev.MoeHost(out, h, logits, gate, up, down, E, topk, hidden, ffn, sel_bias=sel_bias, sel_out=sel, wt_out=wt), dev.Err()
    assert np.array_equal(sel, rsel)
    assert np.allclose(wt, rwt, rtol=2e-6, atol=0)
    assert parity_err(out, ref) <= BAR
    for w in (gate, up, down):
        dev.Forget(w)


def test_a_row_of_nan_logits_gets_no_contribution_and_the_rest_still_match(dev, orc):
    """A row whose logits are all NaN selects nothing (sel = -1 in every slot): its output row is left as it was,
    every other row matches the oracle, and nothing reads outside the activation rows (the unused tail of the
    per-expert token lists names row 0)."""
    rng = synth.rng_for(43)
    E, topk, hidden, ffn, ntok = 8, 2, 128, 128, 12
    gate, up, down = _layer(rng, E, hidden, ffn)
    h = synth.activations(rng, ntok, hidden) * np.float32(0.25)
    logits = synth.activations(rng, ntok, E)
    bad = [3, 11]
    logits[bad] = np.nan
    good = [i for i in range(ntok) if i not in bad]
    before = synth.activations(rng, ntok, hidden)
    out = before.copy()
    sel = np.full((ntok, topk), -7, np.int32)
    wt = np.full((ntok, topk), np.nan, np.float32)
    assert dev.MoeHost(out, h, logits, gate, up, down, E, topk, hidden, ffn, sel_out=sel, wt_out=wt), dev.Err()
    assert (sel[bad] == -1).all()
    assert np.array_equal(out[bad], before[bad])
    ref, rsel, _ = _oracle(orc, h[good], logits[good], gate, up, down, E, topk, hidden, ffn)
    assert np.array_equal(sel[good], rsel)
    assert parity_err(out[good] - before[good], ref) <= BAR
    for w in (gate, up, down):
        dev.Forget(w)


def test_banks_stay_pinned_while_a_capped_context_fetches_all_three(orc):
    """With max_resident_bytes below the three banks' total the call is refused (JL_ENOMEM) instead of running on a
    bank that fetching the next one evicted; with room for exactly three it is served."""
    rng = synth.rng_for(44)
    E, topk, hidden, ffn, ntok = 4, 2, 64, 64, 6
    gate, up, down = _layer(rng, E, hidden, ffn)
    h = synth.activations(rng, ntok, hidden) * np.float32(0.25)
    logits = synth.activations(rng, ntok, E)
    out = np.zeros((ntok, hidden), np.float32)
    with Device(0, max_resident_bytes=gate.nbytes * 2 + 8) as d:
        assert not d.MoeHost(out, h, logits, gate, up, down, E, topk, hidden, ffn)
        assert d.last_status == -3
    with Device(0, max_resident_bytes=gate.nbytes * 3) as d:
        assert d.MoeHost(out, h, logits, gate, up, down, E, topk, hidden, ffn), d.Err()
        ref, _, _ = _oracle(orc, h, logits, gate, up, down, E, topk, hidden, ffn)
        assert parity_err(out, ref) <= BAR
