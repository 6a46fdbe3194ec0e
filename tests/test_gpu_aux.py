"""The decode-step neighbour kernels (jl_aux_*) one by one on a B200, through the C ABI, against float64
restatements: residual add + RMSNorm, SiLU(gate)*up, argmax, RoPE + KV-cache append, single-query attention.
The f32 kernels are held to 1e-5 of the row's scale; the bf16 stores to one bf16 rounding of the f32 value; the
prepared-operand outputs are checked through the matvec that consumes them."""
import numpy as np
import pytest

from conftest import parity_err
from jitllm_b200 import Q4_K, Device, _lib, synth

pytestmark = pytest.mark.gpu
F32_BAR = 1e-5


def _bf16_round(t):
    import torch
    return t.to(torch.bfloat16).double()


@pytest.mark.parametrize("n,h", [(1, 4096), (3, 512), (64, 4096), (2, 100), (5, 14336)])
@pytest.mark.parametrize("with_delta,with_w", [(True, True), (False, True), (True, False)])
def test_add_rmsnorm(n, h, with_delta, with_w):
    import torch
    L = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(n * 7 + h)
    x = torch.randn(n, h, device="cuda", generator=g) * 3
    delta = torch.randn(n, h, device="cuda", generator=g) if with_delta else None
    w = (torch.rand(h, device="cuda", generator=g) + 0.5) if with_w else None
    eps = 1e-5
    xs = x.double() + (delta.double() if with_delta else 0)
    ref = xs * torch.rsqrt((xs * xs).mean(-1, keepdim=True) + eps) * (w.double() if with_w else 1)
    x_io = x.clone()
    out = torch.full_like(x, float("nan"))
    rc = L.jl_aux_add_rmsnorm(x_io.data_ptr(), delta.data_ptr() if with_delta else None, w.data_ptr() if with_w else None,
                              eps, out.data_ptr(), None, n, h, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.OK
    torch.cuda.synchronize()
    assert torch.equal(x_io, (x + delta) if with_delta else x)           # the residual stream is updated in place
    err = ((out.double() - ref).abs() / ref.abs().amax(-1, keepdim=True)).max()
    assert float(err) <= F32_BAR


@pytest.mark.parametrize("n,ffn", [(1, 14336), (4, 1024), (64, 1792), (2, 100)])
def test_silu_mul(n, ffn):
    import torch
    L = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(ffn)
    gu = torch.randn(n, 2 * ffn, device="cuda", generator=g) * 4
    out = torch.full((n, ffn), float("nan"), device="cuda")
    assert L.jl_aux_silu_mul(out.data_ptr(), None, gu.data_ptr(), n, ffn, torch.cuda.current_stream().cuda_stream) == _lib.OK
    torch.cuda.synchronize()
    gd, ud = gu[:, :ffn].double(), gu[:, ffn:].double()
    ref = gd / (1 + torch.exp(-gd)) * ud
    err = ((out.double() - ref).abs() / torch.maximum(ref.abs(), ref.pow(2).mean().sqrt())).max()
    assert float(err) <= F32_BAR


def test_argmax_first_maximum_wins():
    import torch
    L = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(7, 128256, device="cuda", generator=g)
    x[1, 70000] = x[1, 123] = 9.0                                        # a tie: the lower index
    x[2, :] = -float("inf")
    x[3, 128255] = 50.0
    out = torch.full((7,), -1, device="cuda", dtype=torch.int64)
    assert L.jl_aux_argmax(out.data_ptr(), x.data_ptr(), 7, 128256, torch.cuda.current_stream().cuda_stream) == _lib.OK
    torch.cuda.synchronize()
    want = x.argmax(-1)
    want[1], want[2] = 123, 0
    assert torch.equal(out, want)


@pytest.mark.parametrize("n,hq,hkv,pos", [(1, 32, 8, 2048), (3, 4, 2, 0), (64, 4, 1, 17)])
def test_rope_and_cache_append(n, hq, hkv, pos):
    import torch
    L = _lib.load()
    d, max_len = 128, pos + 8
    g = torch.Generator(device="cuda").manual_seed(pos + n)
    qkv = torch.randn(n, (hq + 2 * hkv) * d, device="cuda", generator=g)
    inv = 1.0 / (500000.0 ** (torch.arange(0, d, 2, device="cuda").double() / d))
    ang = torch.arange(max_len, device="cuda").double()[:, None] * inv[None, :]
    cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    kc = torch.full((n, hkv, max_len, d), 7.0, device="cuda", dtype=torch.bfloat16)
    vc = torch.full_like(kc, 7.0)
    qb = torch.full((n, hq, d), float("nan"), device="cuda", dtype=torch.bfloat16)
    pos_dev = torch.tensor([pos], device="cuda")
    assert L.jl_aux_rope_kv(qb.data_ptr(), qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos_dev.data_ptr(), cos.data_ptr(),
                            sin.data_ptr(), n, hq, hkv, d, max_len, torch.cuda.current_stream().cuda_stream) == _lib.OK
    torch.cuda.synchronize()

    def rot(t):                                                          # adjacent-pair rotation, f64 on the f32 tables
        a, b = t[..., 0::2].double(), t[..., 1::2].double()
        c, s = cos[pos].double(), sin[pos].double()
        return torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
    q_ref = rot(qkv[:, :hq * d].view(n, hq, d))
    k_ref = rot(qkv[:, hq * d:(hq + hkv) * d].view(n, hkv, d))
    v_ref = qkv[:, (hq + hkv) * d:].view(n, hkv, d).double()
    # the stored value is the bf16 rounding of an f32 result: within one bf16 ulp (2^-8 relative) of the f64 value
    for got, ref in ((qb.double(), q_ref), (kc[:, :, pos].double(), k_ref)):
        assert float(((got - ref).abs() / ref.abs().clamp_min(1e-3)).max()) <= 2.0 ** -8
    assert torch.equal(vc[:, :, pos].double(), _bf16_round(v_ref.float()))   # v is only rounded
    keep = torch.ones(max_len, dtype=torch.bool, device="cuda")
    keep[pos] = False
    assert bool((kc[:, :, keep] == 7.0).all()) and bool((vc[:, :, keep] == 7.0).all())   # nothing else was touched


@pytest.mark.parametrize("n,hq,hkv,pos,max_len", [(1, 32, 8, 2048, 2064), (2, 8, 2, 63, 64), (2, 8, 2, 64, 200),
                                                   (64, 4, 1, 300, 320), (1, 2, 2, 0, 16), (1, 16, 2, 9000, 9100)])
def test_attention_decode(n, hq, hkv, pos, max_len):
    """Single-query attention over the bf16 cache, positions 0..pos, all query heads of a kv head together.
    The kernel takes bf16 q, K, V exactly and works in f32 (fast exp): 1e-4 of the largest output."""
    import torch
    L = _lib.load()
    d, g = 128, hq // hkv
    gen = torch.Generator(device="cuda").manual_seed(pos * 3 + n)
    q = torch.randn(n, hq, d, device="cuda", generator=gen).to(torch.bfloat16)
    kc = torch.randn(n, hkv, max_len, d, device="cuda", generator=gen).to(torch.bfloat16)
    vc = torch.randn(n, hkv, max_len, d, device="cuda", generator=gen).to(torch.bfloat16)
    kc[:, :, pos + 1:] = float("nan")                                    # beyond the sequence: must not be read
    vc[:, :, pos + 1:] = float("nan")
    scratch = torch.zeros(L.jl_aux_attn_scratch_bytes(n, hq, hkv, max_len), device="cuda", dtype=torch.uint8)
    pos_dev = torch.tensor([pos], device="cuda")
    out = torch.full((n, hq * d), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):                                                   # twice: the tickets must reset themselves
        out.fill_(float("nan"))
        assert L.jl_aux_attn_decode(out.data_ptr(), None, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos_dev.data_ptr(),
                                    scratch.data_ptr(), n, hq, hkv, d, max_len, st) == _lib.OK
        torch.cuda.synchronize()
        qd = q.double().view(n, hkv, g, d)
        kd, vd = kc[:, :, :pos + 1].double(), vc[:, :, :pos + 1].double()
        sc = torch.einsum("nkgd,nksd->nkgs", qd, kd) / d ** 0.5
        ref = torch.einsum("nkgs,nksd->nkgd", sc.softmax(-1), vd).reshape(n, hq * d)
        assert torch.isfinite(out).all()
        assert float((out.double() - ref).abs().max() / ref.abs().max()) <= 1e-4


@pytest.mark.parametrize("producer", ["norm", "silu", "attn"])
def test_producers_write_the_operand_the_matvec_consumes(orc, producer):
    """operand_out: the neighbour kernel writes the Q4_K decode kernel's prepared activation operand itself and
    jl_matvec_dev_prepared consumes it; the result equals the matvec over the kernel's f32 output."""
    import torch
    L = _lib.load()
    rng = synth.rng_for(61)
    nrows, k = 512, 4096 if producer != "silu" else 1792
    w = synth.q4k_matrix(rng, nrows, k)
    st = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(9)
    with Device(0) as d:
        d.Reserve(nrows, k, 1)
        h = d.Upload(Q4_K, w, nrows, k)
        op = L.jl_decode_operand(d.ctx, h.handle, 1)
        assert op
        f32 = torch.full((1, k), float("nan"), device="cuda")
        if producer == "norm":
            x = torch.randn(1, k, device="cuda", generator=gen)
            wn = torch.rand(k, device="cuda", generator=gen) + 0.5
            x2 = x.clone()
            assert L.jl_aux_add_rmsnorm(x.data_ptr(), None, wn.data_ptr(), 1e-5, f32.data_ptr(), None, 1, k, st) == 0
            assert L.jl_aux_add_rmsnorm(x2.data_ptr(), None, wn.data_ptr(), 1e-5, None, op, 1, k, st) == 0
        elif producer == "silu":
            gu = torch.randn(1, 2 * k, device="cuda", generator=gen)
            assert L.jl_aux_silu_mul(f32.data_ptr(), None, gu.data_ptr(), 1, k, st) == 0
            assert L.jl_aux_silu_mul(None, op, gu.data_ptr(), 1, k, st) == 0
        else:
            hq, hkv, dd, pos, ml = 32, 8, 128, 100, 128
            q = torch.randn(1, hq, dd, device="cuda", generator=gen).to(torch.bfloat16)
            kc = torch.randn(1, hkv, ml, dd, device="cuda", generator=gen).to(torch.bfloat16)
            vc = torch.randn(1, hkv, ml, dd, device="cuda", generator=gen).to(torch.bfloat16)
            scr = torch.zeros(L.jl_aux_attn_scratch_bytes(1, hq, hkv, ml), device="cuda", dtype=torch.uint8)
            pd = torch.tensor([pos], device="cuda")
            args = (q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pd.data_ptr(), scr.data_ptr(), 1, hq, hkv, dd, ml, st)
            assert L.jl_aux_attn_decode(f32.data_ptr(), None, *args) == 0
            assert L.jl_aux_attn_decode(None, op, *args) == 0
        got = torch.full((1, nrows), float("nan"), device="cuda")
        assert L.jl_matvec_dev_prepared(d.ctx, got.data_ptr(), h.handle, 1, st) == 0
        torch.cuda.synchronize()
        assert d.StatusPoll()
        ref = orc.matmul_f64(Q4_K, w, f32.cpu().numpy(), nrows, k, 1)
        assert parity_err(got.cpu().numpy(), ref) <= 2e-3
        h.free()


@pytest.mark.parametrize("ntok,nrows,k,delta", [(64, 512, 4096, True), (33, 256, 1024, False)])
def test_norm_writes_the_gemm_operand(orc, ntok, nrows, k, delta):
    """The batched counterpart: jl_aux_add_rmsnorm_gemm writes the tcgen05 GEMM's activation operand (f16 hi / lo rows
    and the per-row scale) and jl_matmul_dev_prepared consumes it. The result carries the same bits as the norm's f32
    output through jl_matmul_dev, whose conversion kernel the producer replaces; and x_io is updated alike."""
    import ctypes as C

    import torch
    L = _lib.load()
    rng = synth.rng_for(77 + ntok)
    w = synth.q4k_matrix(rng, nrows, k)
    st = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(10)
    with Device(0) as d:
        d.Reserve(nrows, k, ntok)
        h = d.Upload(Q4_K, w, nrows, k)
        rows, inv = C.c_void_p(), C.c_void_p()
        assert L.jl_gemm_operand(d.ctx, h.handle, ntok, C.byref(rows), C.byref(inv)) == 0
        x = torch.randn(ntok, k, device="cuda", generator=gen) * 3
        dl = torch.randn(ntok, k, device="cuda", generator=gen) if delta else None
        wn = torch.rand(k, device="cuda", generator=gen) + 0.5
        x2 = x.clone()
        f32 = torch.full((ntok, k), float("nan"), device="cuda")
        dp = dl.data_ptr() if delta else None
        assert L.jl_aux_add_rmsnorm(x.data_ptr(), dp, wn.data_ptr(), 1e-5, f32.data_ptr(), None, ntok, k, st) == 0
        ref = torch.full((ntok, nrows), float("nan"), device="cuda")
        d.MatMulDev(ref, h, f32, ntok, st)
        assert L.jl_aux_add_rmsnorm_gemm(x2.data_ptr(), dp, wn.data_ptr(), 1e-5, rows, inv, ntok, k, st) == 0
        got = torch.full((ntok, nrows), float("nan"), device="cuda")
        assert L.jl_matmul_dev_prepared(d.ctx, got.data_ptr(), 0, h.handle, ntok, st) == 0
        torch.cuda.synchronize()
        assert d.StatusPoll()
        assert torch.equal(x, x2)
        assert torch.equal(got, ref)
        exact = orc.matmul_f64_blas(Q4_K, w, f32.cpu().numpy(), nrows, k, ntok)
        assert parity_err(got.cpu().numpy(), exact) <= 2e-3
        # a token count the decode kernels serve has no GEMM operand
        assert L.jl_gemm_operand(d.ctx, h.handle, 1, C.byref(rows), C.byref(inv)) != 0
        h.free()
