"""Host-side mirror of the reference's accelerator seam.

`Device` has the methods jitllm's `nn.Device`, `CopyForgetter`, `ErrReporter`
and `Reserve` declare (engine/nn/device.go:23-31,1169-1175,1570-1593) with the
same argument meaning and the same error behaviour -- `MatVec`/`MatMul` return
False to decline, and `Err()` says why -- so a test written against the
reference's interface reads the same here. Every method is one call into
libjitllm_b200.so; nothing is computed in Python.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import Choice, LayersBlock, LayersDesc, MoeDesc, Opts, Packed, Stats


class DeviceError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"jitllm_b200: status {status}: {msg}")
        self.status = status


def _ptr(a) -> int:
    """Address of a numpy array, a torch tensor, a ctypes buffer or a raw int."""
    if a is None:
        return 0
    if isinstance(a, int):
        return a
    if isinstance(a, np.ndarray):
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        if not a.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return a.data_ptr()
    return C.addressof(a)


def _nbytes(a) -> int:
    if isinstance(a, np.ndarray):
        return a.nbytes
    if hasattr(a, "element_size"):
        return a.numel() * a.element_size()
    return C.sizeof(a)


def _dtype_code(a) -> int:
    name = str(a.dtype)
    if name.endswith("float32"):
        return _lib.DT_F32
    if name.endswith("bfloat16"):
        return _lib.DT_BF16
    if name.endswith("float16"):
        return _lib.DT_F16
    raise ValueError(f"unsupported element type {a.dtype}")


class Weight:
    """A weight (or expert bank) resident on the device: jl_weight."""

    def __init__(self, dev: "Device", handle: int, t: int, nrows: int, k: int, n_expert: int = 1):
        self.dev, self.handle, self.type, self.nrows, self.k, self.n_expert = dev, handle, t, nrows, k, n_expert

    def free(self) -> None:
        if self.handle and self.dev.ctx:
            self.dev.lib.jl_weight_free(self.dev.ctx, self.handle)
        self.handle = 0

    def unpack(self):
        """Integer view of the RESIDENT copy: (q, d_bits, dmin_bits, sc, m), a record per 32 elements (Q6_K: per 16)."""
        sub = 16 if self.type == _lib.Q6_K else 32
        nsub = self.n_expert * self.nrows * (self.k // sub)
        q = np.empty(nsub * sub, np.int8)
        d = np.empty(nsub, np.uint16)
        dm = np.empty(nsub, np.uint16)
        sc = np.empty(nsub, np.uint8)
        m = np.empty(nsub, np.uint8)
        self.dev._check(self.dev.lib.jl_unpack_resident(self.dev.ctx, self.handle, _ptr(q), _ptr(d), _ptr(dm),
                                                        _ptr(sc), _ptr(m)))
        return q, d, dm, sc, m


def packed_desc(qs, d, sc=None, row: int = 0, stride: int = 0) -> Packed:
    """nn.Packed over three numpy uint32 planes (sc None for formats without a sub-block scale table)."""
    return Packed(qs=_ptr(qs), d=_ptr(d), sc=_ptr(sc) if sc is not None and sc.size else None, qs_bytes=qs.nbytes, d_bytes=d.nbytes,
                  sc_bytes=sc.nbytes if sc is not None else 0, row=row, stride=stride)


def packed_to_blocks(t: int, p: Packed, nrows: int, k: int) -> np.ndarray:
    """The raw ggml blocks a packed weight was made from (the inverse of kernels.PackWeights)."""
    out = np.empty(nrows * _lib.row_bytes(t, k), np.uint8)
    rc = _lib.load().jl_packed_to_blocks(t, C.byref(p), nrows, k, _ptr(out), out.nbytes)
    if rc != _lib.OK:
        raise DeviceError(rc, "jl_packed_to_blocks")
    return out


class Layers:
    """Blocks prepared for whole-step submissions: the reference's nn.LayerDevice (PrepLayer / Layers / Head,
    engine/nn/device.go:1096-1176) over jl_layers_*. One decode step of one sequence is one kernel."""

    def __init__(self, dev: "Device", handle: int, rank: int, world: int, keep):
        self.dev, self.handle, self.rank, self.world, self._keep, self._peers = dev, handle, rank, world, keep, []

    def Run(self, tok, pos, logits=None, next_tok=None, advance: bool = False, stream: int = 0) -> None:
        """Layers(0, n_layer, pos, 1, ...) with the head: tok, pos are 1-element int64 DEVICE tensors."""
        self.dev._check(self.dev.lib.jl_layers_run(self.dev.ctx, self.handle, _ptr(tok), _ptr(pos), _ptr(logits),
                                                   _ptr(next_tok), int(advance), stream))

    def Profile(self, tok, pos, stream: int = 0):
        """One step with per-phase time stamps: uint64 array [2 (first / last CTA)][phases][4 (start, prologue done,
        work done, barrier passed)] in nanoseconds of the GPU's global timer."""
        n = self.dev.lib.jl_layers_phases(self.handle)
        out = np.zeros((2, n, 4), np.uint64)
        self.dev._check(self.dev.lib.jl_layers_profile(self.dev.ctx, self.handle, _ptr(tok), _ptr(pos), stream, _ptr(out), n))
        return out

    def Slot(self):
        """(device pointer, bytes) of this rank's tensor-parallel slot buffer."""
        p, n = C.c_void_p(), C.c_size_t()
        self.dev._check(self.dev.lib.jl_tp_slot(self.dev.ctx, self.handle, C.byref(p), C.byref(n)))
        return p.value, n.value

    def ExportHandle(self) -> bytes:
        buf = C.create_string_buffer(64)
        rc = self.dev.lib.jl_tp_ipc_export(self.Slot()[0], buf)
        if rc != _lib.OK:
            raise DeviceError(rc, "jl_tp_ipc_export")
        return buf.raw

    def Attach(self, handles) -> None:
        """handles[r]: rank r's 64-byte IPC handle (own entry ignored), or an int device pointer."""
        ptrs = (C.c_void_p * self.world)()
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs[r] = self.Slot()[0]
            elif isinstance(h, int):
                ptrs[r] = h
            else:
                p = C.c_void_p()
                rc = self.dev.lib.jl_tp_ipc_open(C.create_string_buffer(bytes(h), 64), C.byref(p))
                if rc != _lib.OK:
                    raise DeviceError(rc, "jl_tp_ipc_open")
                self._peers.append(p.value)
                ptrs[r] = p.value
        self.dev._check(self.dev.lib.jl_tp_attach(self.dev.ctx, self.handle, ptrs, self.world))

    def free(self) -> None:
        if self.handle and self.dev.ctx:
            self.dev.lib.jl_layers_free(self.dev.ctx, self.handle)
            for p in self._peers:
                self.dev.lib.jl_tp_ipc_close(p)
        self.handle, self._peers = 0, []


class Device:
    """One B200, behind the reference's `nn.Device` surface."""

    def __init__(self, device: int = 0, pin_kernel: int = _lib.K_AUTO, pin_warps: int = 0,
                 min_weight_bytes: int = 0, max_resident_bytes: int = 0, flags: int = 0,
                 decode_form: int = _lib.FORM_AUTO, pin_stages: int = 0, pin_row_groups: int = 0,
                 wait_limit_us: int = 0):
        self.lib = _lib.load()
        self.ctx = C.c_void_p()
        o = Opts(struct_size=C.sizeof(Opts), pin_kernel=pin_kernel, pin_warps=pin_warps,
                 min_weight_bytes=min_weight_bytes, max_resident_bytes=max_resident_bytes, flags=flags,
                 decode_form=decode_form, pin_stages=pin_stages, pin_row_groups=pin_row_groups,
                 wait_limit_us=wait_limit_us)
        rc = self.lib.jl_open(device, C.byref(o), C.byref(self.ctx))
        if rc != _lib.OK:
            self.ctx = None
            raise DeviceError(rc, "jl_open failed: no B200 (sm_100) visible as device %d; "
                                  "this path has no CPU fallback" % device)
        self.last_status = _lib.OK

    # -- lifetime -----------------------------------------------------------
    def Close(self) -> None:
        if self.ctx:
            self.lib.jl_close(self.ctx)
            self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.Close()

    def __del__(self):
        try:
            self.Close()
        except Exception:
            pass

    # -- reference surface ----------------------------------------------------
    def MatVec(self, out, t: int, w, x, nrows: int, k: int) -> bool:
        """nn.Device.MatVec: out[0:nrows] = W x, or False to decline. Host arrays."""
        self.last_status = self.lib.jl_matvec(self.ctx, _ptr(out), t, _ptr(w), _nbytes(w), _ptr(x), nrows, k)
        return self.last_status == _lib.OK

    def MatMul(self, out, t: int, w, x, nrows: int, k: int, ntok: int) -> bool:
        """JIT.MatMul: x [ntok][k] -> out [ntok][nrows], token-major. Host arrays; f32/f16/bf16
        (16-bit types as numpy uint16 views are passed with explicit dtype codes via MatMulRaw)."""
        return self.MatMulRaw(out, _dtype_code(out), t, w, x, _dtype_code(x), nrows, k, ntok)

    def MatMulRaw(self, out, out_dtype: int, t: int, w, x, x_dtype: int, nrows: int, k: int, ntok: int) -> bool:
        self.last_status = self.lib.jl_matmul(self.ctx, _ptr(out), out_dtype, t, _ptr(w), _nbytes(w), _ptr(x),
                                              x_dtype, nrows, k, ntok)
        return self.last_status == _lib.OK

    def MatVecPacked(self, out, t: int, p: Packed, x, nrows: int, k: int) -> bool:
        """JIT.MatVecPacked: the matvec on a weight in the container's planar layout. False = declined."""
        self.last_status = self.lib.jl_matvec_packed(self.ctx, _ptr(out), t, C.byref(p), _ptr(x), nrows, k)
        return self.last_status == _lib.OK

    def MatMulPacked(self, out, t: int, p: Packed, x, nrows: int, k: int, ntok: int) -> bool:
        """JIT.MatMulPacked: x [ntok][k] -> out [ntok][nrows] on a packed weight."""
        self.last_status = self.lib.jl_matmul_packed(self.ctx, _ptr(out), _dtype_code(out), t, C.byref(p), _ptr(x),
                                                     _dtype_code(x), nrows, k, ntok)
        return self.last_status == _lib.OK

    def UploadPacked(self, t: int, p: Packed, nrows: int, k: int) -> Weight:
        h = C.c_void_p()
        self._check(self.lib.jl_weight_upload_packed(self.ctx, t, C.byref(p), nrows, k, C.byref(h)))
        return Weight(self, h.value, t, nrows, k, 1)

    def Forget(self, p, n: int | None = None) -> None:
        """CopyForgetter.Forget: drop device copies of host bytes [p, p+n)."""
        self.lib.jl_forget(self.ctx, _ptr(p), _nbytes(p) if n is None else n)

    def Err(self) -> str:
        """ErrReporter.Err: why the last call declined or failed."""
        return self.lib.jl_last_error(self.ctx).decode()

    def Reserve(self, max_rows: int, max_k: int, max_tok: int = 1) -> None:
        self._check(self.lib.jl_reserve(self.ctx, max_rows, max_k, max_tok))

    # -- selection, statistics, fault injection --------------------------------
    def Select(self, t: int, nrows: int, k: int, ntok: int = 1) -> Choice | None:
        ch = Choice()
        rc = self.lib.jl_select(self.ctx, t, nrows, k, ntok, C.byref(ch))
        self.last_status = rc
        return ch if rc == _lib.OK else None

    def WithTune(self, mode: int = _lib.TUNE_ON, cache_dir: str | None = None) -> None:
        """Measured selection (the reference's WithTune / WithTuneCache, jit/gpu/tier/split.go:18-75): new shapes
        are timed at upload; verdicts persist under cache_dir keyed by GPU UUID + driver + library build."""
        self._check(self.lib.jl_tune_configure(self.ctx, mode, cache_dir.encode() if cache_dir else None))

    def Tune(self, weight: "Weight", ntok: int = 1) -> Choice | None:
        """Measure (or load) the verdict for this weight's shape now; returns what will run."""
        ch = Choice()
        rc = self.lib.jl_tune(self.ctx, weight.handle, ntok, C.byref(ch))
        self.last_status = rc
        return ch if rc == _lib.OK else None

    def TuneStats(self) -> dict:
        out = (C.c_int64 * 4)()
        self._check(self.lib.jl_tune_stats(self.ctx, C.byref(out)))
        return dict(trials=out[0], measured=out[1], cached=out[2], refused=out[3])

    def Stats(self) -> Stats:
        s = Stats()
        self._check(self.lib.jl_stats_get(self.ctx, C.byref(s)))
        return s

    def StatusPoll(self, stream: int = 0) -> bool:
        """True when no bounded device-side wait ran out since the last poll; False = JL_ETIMEDOUT (Err() says
        which wait). Synchronises `stream`."""
        self.last_status = self.lib.jl_status_poll(self.ctx, stream)
        if self.last_status not in (_lib.OK, _lib.ETIMEDOUT):
            raise DeviceError(self.last_status, self.Err())
        return self.last_status == _lib.OK

    def FailAt(self, ordinals) -> None:
        arr = (C.c_int * len(ordinals))(*ordinals)
        self._check(self.lib.jl_test_fail_at(self.ctx, arr, len(ordinals)))

    # -- device-pointer twins ----------------------------------------------------
    def Upload(self, t: int, w, nrows: int, k: int, n_expert: int = 1) -> Weight:
        h = C.c_void_p()
        self._check(self.lib.jl_weight_upload_bank(self.ctx, t, _ptr(w), _nbytes(w), n_expert, nrows, k,
                                                   C.byref(h)))
        return Weight(self, h.value, t, nrows, k, n_expert)

    def PrepLayers(self, blocks, hidden: int, n_head: int, n_kv: int, head_dim: int, ffn: int, max_len: int, eps: float,
                   cos, sin, emb, head: Weight | None = None, final_norm=None, rank: int = 0, world: int = 1):
        """nn.LayerDevice.PrepLayer for every block plus the head. blocks: dicts with qkv, o, gate_up, down (Weight),
        attn_norm, ffn_norm (device f32 or None), k_cache, v_cache (device bf16 [n_kv][max_len][head_dim]).
        n_head / n_kv / ffn and the head's rows are THIS rank's share. Returns None when the shape is declined."""
        arr = (LayersBlock * len(blocks))()
        for i, b in enumerate(blocks):
            arr[i] = LayersBlock(qkv=b["qkv"].handle, o=b["o"].handle, gate_up=b["gate_up"].handle, down=b["down"].handle,
                                 attn_norm=_ptr(b.get("attn_norm")), ffn_norm=_ptr(b.get("ffn_norm")),
                                 k_cache=_ptr(b["k_cache"]), v_cache=_ptr(b["v_cache"]))
        d = LayersDesc(struct_size=C.sizeof(LayersDesc), n_layer=len(blocks), hidden=hidden, n_head=n_head, n_kv=n_kv,
                       head_dim=head_dim, ffn=ffn, vocab=head.nrows if head else 0, max_len=max_len, eps=eps, blocks=arr,
                       head=head.handle if head else None, final_norm=_ptr(final_norm), emb_bf16=_ptr(emb),
                       cos_t=_ptr(cos), sin_t=_ptr(sin), rank=rank, world=world)
        h = C.c_void_p()
        rc = self.lib.jl_layers_prep(self.ctx, C.byref(d), C.byref(h))
        self.last_status = rc
        if rc == _lib.DECLINED:
            return None
        self._check(rc)
        return Layers(self, h.value, rank, world, keep=(arr, blocks, cos, sin, emb, final_norm))

    def MatVecDev(self, out, weight: Weight, x, ntok: int = 1, stream: int = 0) -> None:
        """Device tensors: x [ntok][k] f32 -> out [ntok][nrows] f32, on `stream`."""
        self._check(self.lib.jl_matvec_dev(self.ctx, _ptr(out), weight.handle, _ptr(x), ntok, stream))

    def MatMulDev(self, out, weight: Weight, x, ntok: int, stream: int = 0) -> None:
        self._check(self.lib.jl_matmul_dev(self.ctx, _ptr(out), _dtype_code(out), weight.handle, _ptr(x),
                                           _dtype_code(x), ntok, stream))

    def Moe(self, out, h, logits, ntok: int, desc: MoeDesc, sel_out=None, wt_out=None) -> bool:
        """State.moeBatch on host arrays. False = declined."""
        h_dtype = _lib.DT_BF16 if str(h.dtype) == "uint16" else _dtype_code(h)   # uint16 arrays carry bf16 bits
        self.last_status = self.lib.jl_moe(self.ctx, _ptr(out), _ptr(h), h_dtype, _ptr(logits), ntok,
                                           C.byref(desc), _ptr(sel_out), _ptr(wt_out))
        return self.last_status == _lib.OK

    def MoeHost(self, out, h, logits, gate, up, down, n_expert: int, top_k: int, hidden: int, ffn: int,
                act: int = _lib.ACT_SILU, norm: bool = True, scale: float = 1.0, t: int = _lib.MXFP4,
                gate_bias=None, up_bias=None, down_bias=None, router_bias=None, sel_out=None, wt_out=None,
                sel_bias=None, arm: int = _lib.MOE_ARM_EXACT) -> bool:
        """State.moeBatch with every operand in host memory (numpy). out is ADDED to. False = declined.
        arm = MOE_ARM_BLOCK_SCALED runs the expert GEMMs on the block-scaled tensor-core path (activations
        quantised to e4m3 per 32: faster, outside the parity bar)."""
        ntok = logits.shape[0]
        d = MoeDesc(struct_size=C.sizeof(MoeDesc), type=t, n_expert=n_expert, top_k=top_k, hidden=hidden, ffn=ffn,
                    act=act, norm=int(norm), scale=scale, gate=_ptr(gate), up=_ptr(up), down=_ptr(down),
                    gate_bytes=_nbytes(gate), up_bytes=_nbytes(up), down_bytes=_nbytes(down),
                    gate_bias=_ptr(gate_bias), up_bias=_ptr(up_bias), down_bias=_ptr(down_bias),
                    router_bias=_ptr(router_bias), sel_bias=_ptr(sel_bias), arm=arm)
        return self.Moe(out, h, logits, ntok, d, sel_out, wt_out)

    def MoeRouteDev(self, logits, ntok: int, desc: MoeDesc, sel_out, wt_out, stream: int = 0) -> None:
        """The router alone on device tensors: sel/wt [ntok][top_k] in selection order."""
        self._check(self.lib.jl_moe_route_dev(self.ctx, _ptr(logits), ntok, C.byref(desc), _ptr(sel_out), _ptr(wt_out),
                                              stream))

    def MoeExpertsDev(self, y, h, expert_ids, nrows: int, desc: MoeDesc, stream: int = 0) -> None:
        """The experts alone over already-routed rows (device tensors); y [nrows][hidden] f32 is written."""
        self._check(self.lib.jl_moe_experts_dev(self.ctx, _ptr(y), _ptr(h), _dtype_code(h), _ptr(expert_ids), nrows,
                                                C.byref(desc), stream))

    def MoeReserve(self, ntok: int, n_expert: int, top_k: int, hidden: int, ffn: int) -> None:
        self._check(self.lib.jl_moe_reserve(self.ctx, ntok, n_expert, top_k, hidden, ffn))

    def MoeDev(self, out, h, logits, ntok: int, desc: MoeDesc, sel_out=None, wt_out=None, stream: int = 0) -> None:
        self._check(self.lib.jl_moe_dev(self.ctx, _ptr(out), _ptr(h), _dtype_code(h), _ptr(logits), ntok,
                                        C.byref(desc), _ptr(sel_out), _ptr(wt_out), stream))

    def _check(self, rc: int) -> None:
        self.last_status = rc
        if rc != _lib.OK:
            raise DeviceError(rc, self.Err() if self.ctx else "")


def unpack_host(t: int, blocks, n_blocks: int):
    """jl_unpack: the host implementation of kernels.extract over raw blocks."""
    lib = _lib.load()
    sub = 16 if t == _lib.Q6_K else 32
    nsub = n_blocks * (_lib.BLOCK[t][0] // sub)
    q = np.empty(nsub * sub, np.int8)
    d = np.empty(nsub, np.uint16)
    dm = np.empty(nsub, np.uint16)
    sc = np.empty(nsub, np.uint8)
    m = np.empty(nsub, np.uint8)
    rc = lib.jl_unpack(t, _ptr(blocks), n_blocks, _ptr(q), _ptr(d), _ptr(dm), _ptr(sc), _ptr(m))
    if rc != _lib.OK:
        raise DeviceError(rc, "jl_unpack")
    return q, d, dm, sc, m
