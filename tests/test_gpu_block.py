"""The block kernel (one persistent launch per decode step: the reference's nn.LayerDevice seam) on a B200,
through the C ABI: against the per-matvec decode path, against the float64 restatement, over several steps
with the kernel advancing token and position itself, and with a peer that never answers (bounded wait)."""
import numpy as np
import pytest

from conftest import parity_err
from test_gpu_decoder import _ref_decode_step, _ref_logits

pytestmark = pytest.mark.gpu


def _tiny(dev, **kw):
    from jitllm_b200.decoder import Config, Decoder
    cfg = Config(n_layer=2, hidden=512, n_head=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    return cfg, Decoder(dev, cfg, max_batch=1, max_len=96, max_prefill=64, keep_host=True, seed=11, **kw)


@pytest.mark.parametrize("T", [1, 5, 31, 32, 33, 70])
def test_block_kernel_matches_the_float_restatement_and_the_per_matvec_path(dev, orc, T):
    import torch
    cfg, dec = _tiny(dev)
    assert dec.prep_block_kernel(), dev.Err()
    tokens = torch.randint(0, cfg.vocab, (T + 1,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(T))
    with torch.no_grad():
        ref = _ref_logits(torch, orc, dec, cfg, tokens)[T]          # logits after token T, float64
        dec.prefill(tokens[:T])
        kc, vc = dec.k_cache.clone(), dec.v_cache.clone()
        pos = torch.tensor([T], device="cuda")
        tok = tokens[T:T + 1].clone()
        nxt = dec.decode_step_block(tok, pos)
        torch.cuda.synchronize()
        assert dev.StatusPoll(), dev.Err()
        got = dec.last_logits[0].double()
        assert torch.isfinite(got).all()
        assert int(nxt) == int(dec.last_logits.argmax(-1))
        scale = ref.abs().max()
        assert float((got - ref).abs().max() / scale) < 3e-2        # the prefill's keys went through bf16 SDPA
        k_new, v_new = dec.k_cache[:, 0, :, T].clone(), dec.v_cache[:, 0, :, T].clone()
        # the same step through the per-matvec path on the same cache: same arithmetic, different summation order
        dec.k_cache.copy_(kc); dec.v_cache.copy_(vc)
        dec.decode_step(tok, pos)
        chain = dec.last_logits[0].double()
        assert float((got - chain).abs().max() / scale) < 2e-4
        # the appended key / value rows: the same values up to one bf16 rounding of the rotation (v is only rounded)
        assert torch.allclose(dec.k_cache[:, 0, :, T].float(), k_new.float(), rtol=2.0 ** -7, atol=1e-3)
        assert torch.equal(dec.v_cache[:, 0, :, T], v_new)
        # the same bits twice
        dec.k_cache.copy_(kc); dec.v_cache.copy_(vc)
        dec.decode_step_block(tok, pos)
        assert torch.equal(dec.last_logits[0].double(), got)
    dec.block.free()


def test_block_kernel_advances_token_and_position_itself(dev):
    """advance: the kernel writes the next token into *tok and increments *pos, so a chain of steps (or a replayed
    graph) needs nothing from the host. Eight steps against eight steps of the per-matvec path."""
    import torch
    cfg, dec = _tiny(dev)
    assert dec.prep_block_kernel(), dev.Err()
    with torch.no_grad():
        prompt = torch.arange(9, device="cuda") * 131 % cfg.vocab
        first = dec.prefill(prompt)
        kc, vc = dec.k_cache.clone(), dec.v_cache.clone()
        tok, pos = first.clone(), torch.tensor([9], device="cuda")
        want = []
        for _ in range(8):
            tok = dec.decode_step(tok, pos)
            want.append(int(tok))
            pos += 1
        dec.k_cache.copy_(kc); dec.v_cache.copy_(vc)
        tok, pos = first.clone(), torch.tensor([9], device="cuda")
        got = []
        for _ in range(8):
            got.append(int(dec.decode_step_block(tok, pos, advance=True)))
        torch.cuda.synchronize()
        assert dev.StatusPoll(), dev.Err()
        assert int(pos) == 17 and int(tok) == got[-1]
        assert got == want
        # and replayed from a CUDA graph
        dec.k_cache.copy_(kc); dec.v_cache.copy_(vc)
        tok.copy_(first); pos.fill_(9)
        dec.decode_step_block(tok, pos, advance=True)               # warm-up outside the capture
        dec.k_cache.copy_(kc); dec.v_cache.copy_(vc)
        tok.copy_(first); pos.fill_(9)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = dec.decode_step_block(tok, pos, advance=True)
        replayed = []
        for _ in range(8):
            g.replay()
            replayed.append(int(out))
        assert dev.StatusPoll(), dev.Err()
        assert replayed == want
    dec.block.free()


def test_block_kernel_one_full_width_layer(orc):
    """One layer at Llama-3-8B's width with 2048 cached positions through the block kernel, against the float64
    restatement: 2e-3, the bar of every single kernel."""
    import torch
    from jitllm_b200 import Device
    from jitllm_b200.decoder import Config, Decoder
    cfg = Config(n_layer=1, vocab=4096)
    T = 2048
    with Device(0) as dev:
        dec = Decoder(dev, cfg, max_batch=1, max_len=T + 16, max_prefill=64, keep_host=True, seed=23)
        assert dec.prep_block_kernel(), dev.Err()
        g = torch.Generator(device="cuda").manual_seed(1)
        dec.k_cache[:, :, :, :T] = torch.randn(1, 1, cfg.n_kv, T, cfg.head_dim, device="cuda", generator=g).to(torch.bfloat16)
        dec.v_cache[:, :, :, :T] = torch.randn(1, 1, cfg.n_kv, T, cfg.head_dim, device="cuda", generator=g).to(torch.bfloat16)
        kc0, vc0 = dec.k_cache.clone(), dec.v_cache.clone()
        tokens = torch.randint(0, cfg.vocab, (1,), device="cuda", generator=g)
        pos = torch.tensor([T], device="cuda")
        with torch.no_grad():
            nxt = dec.decode_step_block(tokens.clone(), pos)
            torch.cuda.synchronize()
            assert dev.StatusPoll(), dev.Err()
            got = dec.last_logits.double()
            ref = _ref_decode_step(torch, orc, dec, cfg, tokens, T, kc0, vc0)
        assert torch.isfinite(got).all()
        assert int(nxt) == int(dec.last_logits.argmax(-1))
        err = parity_err(got.cpu().numpy(), ref.cpu().numpy())
        assert err <= 2e-3, err
        dec.block.free()


def test_a_peer_that_never_answers_ends_in_a_status_not_a_hang():
    """Tensor-parallel blocks whose second rank does not exist: rank 0's kernel stores its partial sums, raises
    its flag and waits for rank 1's -- which nothing ever writes. With a 2 ms limit the wait runs out, the kernel
    records code 5 and returns; jl_status_poll says JL_ETIMEDOUT and the context serves the next call. The
    'peer' is a second buffer on the same GPU: no second process, no fault."""
    import time

    import torch
    from jitllm_b200 import Q4_K, Device, _lib, synth
    rng = synth.rng_for(71)
    hidden, hq, hkv, ffn, vocab, max_len = 512, 2, 1, 512, 1024, 64
    with Device(0, wait_limit_us=2000) as dev:
        def up(rows, k):
            return dev.Upload(Q4_K, synth.q4k_matrix(rng, rows, k), rows, k)
        kc = torch.zeros(hkv, max_len, 128, device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        blocks = [dict(qkv=up((hq + 2 * hkv) * 128, hidden), o=up(hidden, hq * 128), gate_up=up(2 * ffn, hidden),
                       down=up(hidden, ffn), k_cache=kc, v_cache=vc)]
        head = up(vocab, hidden)
        ang = torch.zeros(max_len, 64, device="cuda")
        emb = torch.randn(vocab, hidden, device="cuda").to(torch.bfloat16)
        lay = dev.PrepLayers(blocks, hidden, hq, hkv, 128, ffn, max_len, 1e-5, ang.cos(), ang.sin(), emb, head=head, rank=0, world=2)
        assert lay is not None, dev.Err()
        nobody = torch.zeros(lay.Slot()[1], device="cuda", dtype=torch.uint8)
        lay.Attach([None, nobody.data_ptr()])
        tok, pos = torch.tensor([3], device="cuda"), torch.tensor([0], device="cuda")
        t0 = time.perf_counter()
        lay.Run(tok, pos, None, None, False, torch.cuda.current_stream().cuda_stream)
        assert not dev.StatusPoll()
        assert time.perf_counter() - t0 < 2.0
        assert dev.last_status == _lib.ETIMEDOUT and "peer" in dev.Err()
        assert dev.StatusPoll()
        # the context is intact: a plain matvec still runs and is right
        w = synth.q4k_matrix(rng, 256, 1024)
        x = synth.activations(rng, 1, 1024)[0]
        out = np.empty(256, np.float32)
        assert dev.MatVec(out, Q4_K, w, x, 256, 1024), dev.Err()
        assert np.isfinite(out).all()
        lay.free()
