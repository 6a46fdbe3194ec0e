"""CPU oracle for the quantized-matmul path -- TEST INFRASTRUCTURE ONLY.

ctypes front end of ``jl_oracle.c`` (see that file's header for what it restates
and how it is pinned). The library, its Python host layer and the benchmark's
GPU arm never import this package; only ``tests/``, the smoke check and the
benchmark's CPU-baseline leg do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libjl_oracle.so")

F32, F16, Q8_0, Q4_K, BF16, MXFP4 = 0, 1, 8, 12, 30, 39
Q4_0, Q5_0, Q5_1, Q5_K, Q6_K = 2, 6, 7, 13, 14


def build(force: bool = False) -> str:
    """Compile the C restatement with the committed Makefile."""
    src = os.path.join(_HERE, "jl_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.orc_half_decode.restype = C.c_double
        L.orc_half_decode.argtypes = [C.c_uint16]
        L.orc_half_encode.restype = C.c_uint16
        L.orc_half_encode.argtypes = [C.c_float]
        L.orc_bias_c.restype = C.c_double
        L.orc_bias_c.argtypes = [C.c_uint32]
        L.orc_silu.restype = C.c_double
        L.orc_silu.argtypes = [C.c_double]
        L.orc_swiglu_oai.restype = C.c_double
        L.orc_swiglu_oai.argtypes = [C.c_double, C.c_double]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _bytes(w) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(w, dtype=np.uint8) if not isinstance(w, np.ndarray) else w.view(np.uint8).reshape(-1))


def block_elems(t: int) -> int:
    return lib().orc_block_elems(C.c_uint32(t))


def block_bytes(t: int) -> int:
    return lib().orc_block_bytes(C.c_uint32(t))


def row_bytes(t: int, k: int) -> int:
    return k // block_elems(t) * block_bytes(t)


def half_decode(u: int) -> float:
    return lib().orc_half_decode(C.c_uint16(u))


def half_encode(f: float) -> int:
    return lib().orc_half_encode(C.c_float(f))


def dequant32(t: int, src, n: int) -> np.ndarray:
    s = _bytes(src)
    out = np.empty(n, dtype=np.float32)
    rc = lib().orc_dequant_f32(C.c_uint32(t), _p(s), C.c_size_t(n), _p(out))
    if rc:
        raise ValueError(f"orc_dequant_f32 rc={rc}")
    return out


def dequant64(t: int, src, n: int) -> np.ndarray:
    s = _bytes(src)
    out = np.empty(n, dtype=np.float64)
    rc = lib().orc_dequant_f64(C.c_uint32(t), _p(s), C.c_size_t(n), _p(out))
    if rc:
        raise ValueError(f"orc_dequant_f64 rc={rc}")
    return out


def unpack(t: int, src, nblocks: int):
    """Integer view of the blocks: (q[int8, one per element], d_bits, dmin_bits, sc, m), one record per 32-element
    sub-block (Q6_K: per 16 elements, as the reference's extract has it)."""
    s = _bytes(src)
    sub = 16 if t == Q6_K else 32
    nsub = nblocks * (block_elems(t) // sub)
    q = np.empty(nsub * sub, dtype=np.int8)
    d = np.empty(nsub, dtype=np.uint16)
    dmin = np.empty(nsub, dtype=np.uint16)
    sc = np.empty(nsub, dtype=np.uint8)
    m = np.empty(nsub, dtype=np.uint8)
    rc = lib().orc_unpack(C.c_uint32(t), _p(s), C.c_size_t(nblocks), _p(q), _p(d), _p(dmin), _p(sc), _p(m))
    if rc:
        raise ValueError(f"orc_unpack rc={rc}")
    return q, d, dmin, sc, m


def pack_weights(t: int, src, nrows: int, k: int, row0: int = 0, stride: int | None = None, into=None):
    """kernels.PackWeights: the container / device planes (qs, d, sc as uint32 arrays) of a raw tensor. With `into` =
    (qs, d, sc) the rows are ORed into an existing buffer of `stride` rows starting at `row0` (a bank's experts)."""
    s = _bytes(src)
    stride = stride or nrows
    nq, nd, ns = C.c_size_t(), C.c_size_t(), C.c_size_t()
    if lib().orc_packed_words(C.c_uint32(t), stride, k, C.byref(nq), C.byref(nd), C.byref(ns)):
        raise ValueError("orc_packed_words: type or k not packable")
    qs, d, sc = into if into is not None else (np.zeros(nq.value, np.uint32), np.zeros(nd.value, np.uint32),
                                                np.zeros(ns.value, np.uint32))
    rc = lib().orc_pack_weights(C.c_uint32(t), _p(s), nrows, k, row0, stride, _p(qs), _p(d), _p(sc) if sc.size else None)
    if rc:
        raise ValueError(f"orc_pack_weights rc={rc}")
    return qs, d, sc


def matvec(t: int, w, x: np.ndarray, nrows: int, k: int) -> np.ndarray:
    """oracle.MatVec: compensated f32 dot of Dequant32 rows."""
    s = _bytes(w)
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(nrows, dtype=np.float32)
    rc = lib().orc_matvec(_p(out), C.c_uint32(t), _p(s), _p(x), nrows, k)
    if rc:
        raise ValueError(f"orc_matvec rc={rc}")
    return out


def matmul_f64(t: int, w, x: np.ndarray, nrows: int, k: int, ntok: int, nthreads: int = 0) -> np.ndarray:
    """f64 dot of Dequant32(W) with f32 x[ntok][k]; returns [ntok][nrows] f64."""
    s = _bytes(w)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(ntok, k)
    out = np.empty((ntok, nrows), dtype=np.float64)
    rc = lib().orc_matmul_f64(_p(out), C.c_uint32(t), _p(s), _p(x), nrows, k, ntok, nthreads or (os.cpu_count() or 1))
    if rc:
        raise ValueError(f"orc_matmul_f64 rc={rc}")
    return out


def matmul_f64_blas(t: int, w, x: np.ndarray, nrows: int, k: int, ntok: int, chunk: int = 2048) -> np.ndarray:
    """Same quantity as matmul_f64 through numpy's f64 GEMM (fast at full sizes)."""
    s = _bytes(w)
    rb = row_bytes(t, k)
    x64 = np.ascontiguousarray(x, dtype=np.float32).reshape(ntok, k).astype(np.float64)
    out = np.empty((ntok, nrows), dtype=np.float64)
    for r0 in range(0, nrows, chunk):
        r1 = min(nrows, r0 + chunk)
        wr = dequant32(t, s[r0 * rb:r1 * rb], (r1 - r0) * k).reshape(r1 - r0, k).astype(np.float64)
        out[:, r0:r1] = x64 @ wr.T
    return out


def quantize_q8_window(x: np.ndarray, bias_c: float, window: int = 32):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.size
    q = np.empty(n, dtype=np.int8)
    pairs = np.empty(2 * (n // 32), dtype=np.float32)
    lib().orc_quantize_q8_window(_p(q), _p(pairs), _p(x), n, C.c_double(bias_c), window)
    return q, pairs


def bias_c(t: int) -> float:
    return lib().orc_bias_c(C.c_uint32(t))


def simd_level() -> int:
    return lib().orc_simd_level()


def matmul_int8(t: int, w, x: np.ndarray, nrows: int, k: int, ntok: int = 1, window: int = 32,
                nthreads: int = 0, simd: int = -1) -> np.ndarray:
    """The reference CPU JIT's arithmetic (int8 activations, integer dot, f32 fold)."""
    s = _bytes(w)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(ntok, k)
    out = np.empty((ntok, nrows), dtype=np.float32)
    rc = lib().orc_matmul_int8(_p(out), C.c_uint32(t), _p(s), _p(x), nrows, k, ntok, window,
                               nthreads or (os.cpu_count() or 1), simd)
    if rc:
        raise ValueError(f"orc_matmul_int8 rc={rc}")
    return out


def softmax(logits: np.ndarray) -> np.ndarray:
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    sc = np.empty_like(lg)
    lib().orc_softmax(_p(sc), _p(lg), lg.size)
    return sc


def moe_router(scores: np.ndarray, k: int, norm: bool = True, scale: float = 1.0,
               bias: np.ndarray | None = None, exp_scale: np.ndarray | None = None):
    """oracle.MoERouter over gated scores. Returns (sel, ord, wt, owt, sum)."""
    sc = np.ascontiguousarray(scores, dtype=np.float32)
    n = sc.size
    sel = np.empty(k, np.int32); ordv = np.empty(k, np.int32)
    wt = np.empty(k, np.float32); owt = np.empty(k, np.float32)
    sm = np.empty(1, np.float32)
    b = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
    es = np.ascontiguousarray(exp_scale, dtype=np.float32) if exp_scale is not None else None
    got = lib().orc_moe_router(_p(sc), n, k, int(norm), C.c_float(scale),
                               _p(b) if b is not None else None, _p(es) if es is not None else None,
                               _p(sel), _p(ordv), _p(wt), _p(owt), _p(sm))
    if got < 0:
        raise ValueError("orc_moe_router: bad shape")
    return sel[:got], ordv[:got], wt[:got], owt[:got], float(sm[0])


def silu(x: float) -> float:
    return lib().orc_silu(C.c_double(x))


def swiglu_oai(g: float, u: float) -> float:
    return lib().orc_swiglu_oai(C.c_double(g), C.c_double(u))


def moe_layer(h: np.ndarray, t: int, gate, up, down, sel: np.ndarray, wt: np.ndarray, n_expert: int,
              hidden: int, ffn: int, act_kind: int = 0, bgate=None, bup=None, bdown=None,
              out: np.ndarray | None = None, nthreads: int = 0) -> np.ndarray:
    """Expert-major mixture layer (moeBatch). sel/wt [ntok][top_k] selection order. Adds into out."""
    h = np.ascontiguousarray(h, dtype=np.float32)
    ntok = h.shape[0]
    sel = np.ascontiguousarray(sel, dtype=np.int32).reshape(ntok, -1)
    wt = np.ascontiguousarray(wt, dtype=np.float32).reshape(ntok, -1)
    top_k = sel.shape[1]
    if out is None:
        out = np.zeros((ntok, hidden), dtype=np.float32)
    g, u, d = _bytes(gate), _bytes(up), _bytes(down)

    def opt(a):
        return None if a is None else np.ascontiguousarray(a, dtype=np.float32)
    bg, bu, bd = opt(bgate), opt(bup), opt(bdown)
    rc = lib().orc_moe_layer(_p(out), _p(h), C.c_uint32(t), _p(g), _p(u), _p(d),
                             _p(bg) if bg is not None else None, _p(bu) if bu is not None else None,
                             _p(bd) if bd is not None else None, _p(sel), _p(wt), ntok, n_expert, top_k,
                             hidden, ffn, act_kind, nthreads or (os.cpu_count() or 1))
    if rc:
        raise ValueError(f"orc_moe_layer rc={rc}")
    return out
