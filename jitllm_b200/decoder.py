"""Llama-3-8B-shaped decoder harness for the quantized-matmul path.

Every matmul (q|k|v, o, gate|up, down, lm_head) goes through libjitllm_b200.so on Q4_K weights;
the steps around them -- RMSNorm, RoPE, the KV cache, attention, SiLU*up, the residual adds and
the greedy argmax -- are neighbours of the path: the prefill runs them as PyTorch ops, a decode
step runs the library's own short kernels between the matvecs (`decode_step`), and a decode step
of ONE sequence runs everything as one persistent kernel (`decode_step_block`: the reference's
LayerDevice seam). Weights are random-init Q4_K blocks of the right shapes (no checkpoint can be fetched);
q|k|v and gate|up are stored as one row-concatenated matrix each, as the reference's
`MatVecSegments` fuses them (docs/kernel-inventory.md:83).

Tensor parallel over `world` ranks: q|k|v and gate|up are column-parallel (whole heads / matching
gate-up rows per rank), o and down are row-parallel followed by an all-reduce of the [batch][4096]
f32 partial sums, lm_head is column-parallel with an all-gather before the argmax.
"""
from __future__ import annotations

import numpy as np

from . import parallel, synth
from ._lib import Q4_K


class Config:
    def __init__(self, n_layer=32, hidden=4096, n_head=32, n_kv=8, head_dim=128, ffn=14336, vocab=128256,
                 rope_theta=500000.0, eps=1e-5):
        self.n_layer, self.hidden, self.n_head, self.n_kv, self.head_dim = n_layer, hidden, n_head, n_kv, head_dim
        self.ffn, self.vocab, self.rope_theta, self.eps = ffn, vocab, rope_theta, eps


def random_q4k(rng: np.random.Generator, nrows: int, k: int) -> np.ndarray:
    """Fast random Q4_K tensor: uniform random payload bytes (codes U{0..15}, 6-bit fields uniform),
    d and dmin = f16(|N(0, 0.02)|) -- the value distribution of the headline 4096x4096 workload."""
    nb = nrows * (k // 256)
    blk = rng.integers(0, 256, (nb, 144), dtype=np.uint8)
    dd = np.abs(rng.normal(0.0, 0.02, (nb, 2))).astype(np.float16).view(np.uint16)
    blk[:, 0:4] = dd.view(np.uint8).reshape(nb, 4)
    return blk.reshape(nrows, (k // 256) * 144)


class Decoder:
    def __init__(self, dev, cfg: Config, max_batch: int, max_len: int, rank: int = 0, world: int = 1, seed: int = 0xB204,
                 group=None, max_prefill: int = 2048, keep_host: bool = False, share_full: bool = False):
        import torch
        self.torch, self.dev, self.cfg, self.rank, self.world, self.group = torch, dev, cfg, rank, world, group
        c = cfg
        assert c.n_head % world == 0 and c.n_kv % world == 0 and c.ffn % (world * 256) == 0 and c.vocab % world == 0
        self.hq, self.hkv = c.n_head // world, c.n_kv // world
        self.ffn_l, self.vocab_l = c.ffn // world, c.vocab // world
        self.max_batch, self.max_len = max_batch, max_len
        self._att_scratch, self._att_scratch_rows = None, 0
        rng = synth.rng_for(seed if share_full else seed + rank)
        d = c.head_dim
        self.layers, self.host = [], []          # host: the raw blocks, kept only for tests
        w_ = world

        def make(segments, k_full, k_split=False):
            """One resident matrix. segments: row counts of the UNSHARDED matrix's parts (q|k|v, gate|up);
            each part is column-parallel (rows [rank/world) of the part), or with k_split the whole
            matrix is row-parallel (k-range [rank/world) of every row, cut at super-block boundaries).
            share_full: every rank draws the same unsharded matrix and keeps its slice (parity tests);
            otherwise each rank draws only its own slice."""
            if share_full:
                raw, nrows, k = parallel.shard_segments(random_q4k(rng, sum(segments), k_full), Q4_K, segments, k_full,
                                                        rank, w_, k_split)
            else:
                nrows = sum(segments) if k_split else sum(n // w_ for n in segments)
                k = k_full // w_ if k_split else k_full
                raw = random_q4k(rng, nrows, k)
            if keep_host:
                self.host.append(raw)
            return dev.Upload(Q4_K, raw, nrows, k)

        for _ in range(c.n_layer):
            self.layers.append(dict(qkv=make([c.n_head * d, c.n_kv * d, c.n_kv * d], c.hidden),
                                    o=make([c.hidden], c.n_head * d, k_split=True),
                                    gu=make([c.ffn, c.ffn], c.hidden), down=make([c.hidden], c.ffn, k_split=True)))
        self.head = make([c.vocab], c.hidden)
        g = torch.Generator(device="cuda").manual_seed(seed)       # same on every rank
        self.emb = (torch.randn(c.vocab, c.hidden, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.norm_w = torch.ones(c.hidden, device="cuda")
        self.k_cache = torch.zeros(c.n_layer, max_batch, self.hkv, max_len, d, device="cuda", dtype=torch.bfloat16)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, d, 2, device="cuda").float() / d))
        ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        dev.Reserve(max(2 * self.ffn_l, self.vocab_l, c.hidden), max(c.hidden, self.ffn_l, self.hq * d), max(max_batch, max_prefill))
        self.weight_bytes = sum(w.nrows * (w.k // 256) * 144 for l in self.layers for w in l.values()) + \
            self.head.nrows * (self.head.k // 256) * 144

    # -- the path -------------------------------------------------------------
    def mm(self, w, x):
        """x [n][k] f32 or bf16 -> [n][rows] f32 through the library (decode kernel for few rows, tcgen05 GEMM above)."""
        torch = self.torch
        n = x.shape[0]
        out = torch.empty(n, w.nrows, device="cuda", dtype=torch.float32)
        stream = torch.cuda.current_stream().cuda_stream
        if n == 1 and x.dtype == torch.float32:
            self.dev.MatVecDev(out, w, x.contiguous(), 1, stream)
        else:
            self.dev.MatMulDev(out, w, x.contiguous(), n, stream)      # the library picks the kernel by n
        return out

    def _allreduce(self, t):
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.group)
        return t

    # -- neighbours of the path (PyTorch) ---------------------------------------
    def _rms(self, x):
        return x * self.torch.rsqrt((x * x).mean(-1, keepdim=True) + self.cfg.eps) * self.norm_w

    def _rope(self, t, pos):
        """t [n][heads][d]; pos [n] int64 positions."""
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        a, b = t[..., 0::2], t[..., 1::2]
        return self.torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)

    def _layers(self, x, pos, attend):
        """The layer stack over n rows x [n][hidden] f32. pos [n] int64 gives each row's position (RoPE);
        attend(li, q [n][hq][d], k [n][hkv][d], v [n][hkv][d]) -> [n][hq*d] stores k, v and attends."""
        torch, c = self.torch, self.cfg
        import torch.nn.functional as F
        n, d = x.shape[0], c.head_dim
        for li, l in enumerate(self.layers):
            qkv = self.mm(l["qkv"], self._rms(x))
            q = self._rope(qkv[:, :self.hq * d].view(n, self.hq, d), pos)
            k = self._rope(qkv[:, self.hq * d:(self.hq + self.hkv) * d].view(n, self.hkv, d), pos)
            v = qkv[:, (self.hq + self.hkv) * d:].view(n, self.hkv, d)
            att = attend(li, q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16))
            x = x + self._allreduce(self.mm(l["o"], att.float()))
            gu = self.mm(l["gu"], self._rms(x))
            x = x + self._allreduce(self.mm(l["down"], F.silu(gu[:, :self.ffn_l]) * gu[:, self.ffn_l:]))
        return x

    def _argmax(self, x):
        torch = self.torch
        logits = self.last_logits = self.mm(self.head, self._rms(x))
        if self.world > 1:
            import torch.distributed as dist
            parts = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(parts, logits, group=self.group)
            logits = torch.cat(parts, dim=-1)
        return logits.argmax(-1)

    def prefill(self, tokens):
        """One prompt tokens [T] int64, causal attention; its keys/values are written to EVERY
        sequence slot of the cache (all sequences of the batch share the prompt). Returns the next token."""
        torch = self.torch
        import torch.nn.functional as F
        T = tokens.shape[0]
        pos = torch.arange(T, device="cuda")
        g = self.hq // self.hkv

        def attend(li, q, k, v):
            self.k_cache[li, :, :, :T] = k.transpose(0, 1)[None]
            self.v_cache[li, :, :, :T] = v.transpose(0, 1)[None]
            o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                               is_causal=True, enable_gqa=True)       # query head h uses kv head h // g
            return o[0].transpose(0, 1).reshape(T, -1)

        x = self._layers(self.emb[tokens].float(), pos, attend)
        return self._argmax(x[-1:])

    def decode_step(self, tokens, pos_dev):
        """tokens [B] int64, one per sequence, all at position pos_dev (a 1-element int64 DEVICE tensor,
        so that the step can be replayed from a CUDA graph). Returns the next tokens [B].
        Between two matmuls runs ONE library kernel (jl_aux_*: add+RMSNorm, RoPE+cache append,
        attention over the cache, SiLU*up), all on the matvec kernels' dependent-launch chain."""
        torch, c, lib = self.torch, self.cfg, self.dev.lib
        B, d = tokens.shape[0], c.head_dim
        st = torch.cuda.current_stream().cuda_stream
        f32 = dict(device="cuda", dtype=torch.float32)
        if self._att_scratch is None or self._att_scratch_rows < B:
            nbytes = lib.jl_aux_attn_scratch_bytes(B, self.hq, self.hkv, self.max_len)
            self._att_scratch, self._att_scratch_rows = torch.zeros(nbytes, device="cuda", dtype=torch.uint8), B

        def ok(rc):
            if rc != 0:
                raise RuntimeError(f"jl_aux call failed with status {rc}")

        ctx = self.dev.ctx
        l0 = self.layers[0]
        # With few sequences every producer writes the next matvec's prepared activation operand itself
        # (no conversion launch in between); otherwise f32 rows go to the GEMM path.
        ops = [lib.jl_decode_operand(ctx, w.handle, B) for w in (l0["qkv"], l0["o"], l0["gu"], l0["down"], self.head)]
        prep = B <= 8 and all(ops) and (self.hq // self.hkv) % 2 == 0
        op = ops[0] if prep else None

        # With many sequences the norm writes the tcgen05 GEMM's activation operand (f16 hi / lo rows + per-row scale)
        # for its consumers (q|k|v, gate|up, the head: all of width hidden, so one place serves the three), again with
        # no conversion launch in between.
        import ctypes as C
        g_rows, g_inv = C.c_void_p(), C.c_void_p()
        gemm_prep = (not prep) and c.hidden % 256 == 0 and all(
            lib.jl_gemm_operand(ctx, w.handle, B, C.byref(g_rows), C.byref(g_inv)) == 0 for w in (l0["qkv"], l0["gu"], self.head))

        def mv(w, x_f32):
            if gemm_prep and x_f32 is h:
                out = torch.empty(B, w.nrows, **f32)
                ok(lib.jl_matmul_dev_prepared(ctx, out.data_ptr(), 0, w.handle, B, st))     # 0 = JL_DT_F32
                return out
            if not prep:
                return self.mm(w, x_f32)
            out = torch.empty(B, w.nrows, **f32)
            ok(lib.jl_matvec_dev_prepared(ctx, out.data_ptr(), w.handle, B, st))
            return out

        def norm(delta):
            if gemm_prep:
                ok(lib.jl_aux_add_rmsnorm_gemm(x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                               self.norm_w.data_ptr(), c.eps, g_rows, g_inv, B, c.hidden, st))
                return
            ok(lib.jl_aux_add_rmsnorm(x.data_ptr(), delta.data_ptr() if delta is not None else None, self.norm_w.data_ptr(),
                                      c.eps, None if prep else h.data_ptr(), op, B, c.hidden, st))

        x = self.emb[tokens].float()
        h = torch.empty_like(x)
        qb = torch.empty(B, self.hq, d, device="cuda", dtype=torch.bfloat16)
        att = torch.empty(B, self.hq * d, **f32)
        a = torch.empty(B, self.ffn_l, **f32)
        norm(None)
        for li, l in enumerate(self.layers):
            qkv = mv(l["qkv"], h)
            kc, vc = self.k_cache[li], self.v_cache[li]
            ok(lib.jl_aux_rope_kv(qb.data_ptr(), qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos_dev.data_ptr(),
                                  self.cos.data_ptr(), self.sin.data_ptr(), B, self.hq, self.hkv, d, self.max_len, st))
            ok(lib.jl_aux_attn_decode(None if prep else att.data_ptr(), op, qb.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                      pos_dev.data_ptr(), self._att_scratch.data_ptr(), B, self.hq, self.hkv, d, self.max_len, st))
            norm(self._allreduce(mv(l["o"], att)))
            ok(lib.jl_aux_silu_mul(None if prep else a.data_ptr(), op, mv(l["gu"], h).data_ptr(), B, self.ffn_l, st))
            norm(self._allreduce(mv(l["down"], a)))             # also the next layer's (or the final) norm
        logits = self.last_logits = mv(self.head, h)
        if self.world > 1:
            import torch.distributed as dist
            parts = [torch.empty_like(logits) for _ in range(self.world)]
            dist.all_gather(parts, logits, group=self.group)
            logits = torch.cat(parts, dim=-1)
        nxt = torch.empty(B, device="cuda", dtype=torch.int64)
        ok(lib.jl_aux_argmax(nxt.data_ptr(), logits.data_ptr(), B, logits.shape[1], st))
        return nxt

    # -- whole step as one kernel (nn.LayerDevice) -----------------------------------
    def prep_block_kernel(self):
        """PrepLayer for every block + the head. Returns False when the library declines the shape (the per-matvec
        decode_step keeps working). Under tensor parallelism the ranks exchange their slot handles here."""
        c = self.cfg
        blocks = [dict(qkv=l["qkv"], o=l["o"], gate_up=l["gu"], down=l["down"], attn_norm=self.norm_w, ffn_norm=self.norm_w,
                       k_cache=self.k_cache[li, 0], v_cache=self.v_cache[li, 0]) for li, l in enumerate(self.layers)]
        self.block = self.dev.PrepLayers(blocks, c.hidden, self.hq, self.hkv, c.head_dim, self.ffn_l, self.max_len, c.eps,
                                         self.cos, self.sin, self.emb, head=self.head, final_norm=self.norm_w,
                                         rank=self.rank, world=self.world)
        if self.block is None:
            return False
        if self.world > 1:
            parallel.tp_attach(self.block, self.group)
        return True

    def decode_step_block(self, tok_dev, pos_dev, advance=False):
        """One decode step of ONE sequence as ONE kernel launch (plus, under tensor parallelism, the gather of the
        vocabulary shards and the argmax). tok_dev, pos_dev: 1-element int64 device tensors. Returns the next token
        [1]; with advance (single GPU) the kernel also stores it into tok_dev and increments pos_dev."""
        torch = self.torch
        st = torch.cuda.current_stream().cuda_stream
        nxt = torch.empty(1, device="cuda", dtype=torch.int64)
        logits = self.last_logits = torch.empty(1, self.vocab_l, device="cuda", dtype=torch.float32)
        if self.world == 1:
            self.block.Run(tok_dev, pos_dev, logits, nxt, advance, st)
            return nxt
        import torch.distributed as dist
        self.block.Run(tok_dev, pos_dev, logits, None, False, st)
        parts = [torch.empty_like(logits) for _ in range(self.world)]
        dist.all_gather(parts, logits, group=self.group)
        full = torch.cat(parts, dim=-1)
        rc = self.dev.lib.jl_aux_argmax(nxt.data_ptr(), full.data_ptr(), 1, full.shape[1], st)
        if rc != 0:
            raise RuntimeError(f"jl_aux_argmax failed with status {rc}")
        return nxt

    def decode_step_torch(self, tokens, pos_dev):
        """The same step with PyTorch ops between the matmuls (the check of decode_step)."""
        torch = self.torch
        import torch.nn.functional as F
        B = tokens.shape[0]
        g = self.hq // self.hkv
        mask = (torch.arange(self.max_len, device="cuda") <= pos_dev)[None, None, None, :]

        def attend(li, q, k, v):
            self.k_cache[li, :B].index_copy_(2, pos_dev, k[:, :, None, :])
            self.v_cache[li, :B].index_copy_(2, pos_dev, v[:, :, None, :])
            o = F.scaled_dot_product_attention(q.view(B, self.hkv, g, -1), self.k_cache[li, :B], self.v_cache[li, :B],
                                               attn_mask=mask)
            return o.reshape(B, -1)

        x = self._layers(self.emb[tokens].float(), pos_dev.expand(B), attend)
        return self._argmax(x)
