"""The Llama-shaped decoder harness on a tiny configuration: every matmul through the library, checked
against a float32 PyTorch restatement over the oracle-dequantized weights, and prefill/decode agreement
(the token after T prompt tokens is the same whether the last one went through the GEMM path with causal
attention or through the decode path with the KV cache)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ref_logits(torch, orc, dec, cfg, tokens):
    from jitllm_b200._lib import Q4_K
    F = torch.nn.functional
    it = iter(dec.host)
    T, d, g = tokens.shape[0], cfg.head_dim, cfg.n_head // cfg.n_kv

    def W(nrows, k):
        return torch.from_numpy(orc.dequant32(Q4_K, next(it), nrows * k).reshape(nrows, k)).cuda().double()

    def rms(x):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + cfg.eps)

    def rope(t):
        pos = torch.arange(T, device="cuda")
        cos, sin = dec.cos[pos][:, None, :].double(), dec.sin[pos][:, None, :].double()
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)

    x = dec.emb[tokens].double()
    for _ in range(cfg.n_layer):
        wqkv, wo = W((cfg.n_head + 2 * cfg.n_kv) * d, cfg.hidden), W(cfg.hidden, cfg.n_head * d)
        wgu, wdn = W(2 * cfg.ffn, cfg.hidden), W(cfg.hidden, cfg.ffn)
        qkv = rms(x) @ wqkv.T
        q = rope(qkv[:, :cfg.n_head * d].view(T, cfg.n_head, d))
        k = rope(qkv[:, cfg.n_head * d:(cfg.n_head + cfg.n_kv) * d].view(T, cfg.n_kv, d))
        v = qkv[:, (cfg.n_head + cfg.n_kv) * d:].view(T, cfg.n_kv, d)
        k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
        sc = torch.einsum("thd,shd->hts", q, k) / d ** 0.5
        sc = sc.masked_fill(torch.triu(torch.ones(T, T, device="cuda", dtype=torch.bool), 1), float("-inf"))
        att = torch.einsum("hts,shd->thd", sc.softmax(-1), v).reshape(T, -1)
        x = x + att @ wo.T
        gu = rms(x) @ wgu.T
        x = x + (F.silu(gu[:, :cfg.ffn]) * gu[:, cfg.ffn:]) @ wdn.T
    return rms(x) @ W(cfg.vocab, cfg.hidden).T


@pytest.mark.parametrize("T", [1, 5, 24])
def test_decoder_matches_float_restatement(dev, orc, T):
    import torch
    from jitllm_b200.decoder import Decoder, Config
    cfg = Config(n_layer=2, hidden=512, n_head=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    dec = Decoder(dev, cfg, max_batch=3, max_len=64, max_prefill=32, keep_host=True, seed=11)
    tokens = torch.randint(0, cfg.vocab, (T + 1,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(T))
    with torch.no_grad():
        ref = _ref_logits(torch, orc, dec, cfg, tokens)            # [T+1][vocab], row i = logits after token i
        dec.prefill(tokens[:T])
        got_prefill = dec.last_logits[0].double()
        assert torch.isfinite(got_prefill).all()
        scale = ref.abs().max()
        assert float((got_prefill - ref[T - 1]).abs().max() / scale) < 3e-2       # bf16 attention operands
        # the next token through the decode path, three sequences sharing the prompt
        pos = torch.tensor([T], device="cuda")
        nxt = dec.decode_step(tokens[T:T + 1].expand(3).contiguous(), pos)
        got_dec = dec.last_logits.double()
        assert torch.equal(nxt, dec.last_logits.argmax(-1))
        assert torch.isfinite(got_dec).all()
        assert float((got_dec - ref[T][None]).abs().max() / scale) < 3e-2
        assert float((got_dec[0] - got_dec[2]).abs().max()) == 0.0                 # same inputs, same bits
        # the PyTorch-glue form of the same step agrees with the fused-neighbour form
        dec.decode_step_torch(tokens[T:T + 1].expand(3).contiguous(), pos)
        assert float((dec.last_logits.double() - got_dec).abs().max() / scale) < 1e-2
