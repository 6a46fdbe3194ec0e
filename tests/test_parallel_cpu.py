"""Host logic of the sharded path, on CPU: byte sharding against the oracle, and the column /
row / expert-parallel orchestration as two gloo ranks with the oracle standing in for the kernels."""
import os

import numpy as np
import pytest

from conftest import nmse
from jitllm_b200 import parallel, synth
from jitllm_b200._lib import MXFP4, Q4_K, Q8_0


@pytest.mark.parametrize("t,k", [(Q4_K, 1024), (Q8_0, 256), (MXFP4, 192)])
def test_byte_sharding_matches_the_unsharded_oracle(orc, t, k):
    rng = synth.rng_for(70 + t)
    nrows, world = 24, 4
    w = synth.matrix(rng, t, nrows, k)
    x = synth.activations(rng, 1, k)[0]
    ref = orc.matmul_f64(t, w, x, nrows, k, 1)[0]
    cols = [orc.matmul_f64(t, *parallel.shard_rows(w, t, nrows, k, r, world)[:1], x, nrows // world, k, 1)[0]
            for r in range(world)]
    assert np.array_equal(np.concatenate(cols), ref), "column shards are row slices: identical numbers"
    if (k // world) % orc.block_elems(t) == 0:
        parts = []
        for r in range(world):
            wr, kl = parallel.shard_k(w, t, nrows, k, r, world)
            parts.append(orc.matmul_f64(t, wr, x[r * kl:(r + 1) * kl], nrows, kl, 1)[0])
        assert nmse(np.sum(parts, axis=0), ref) < 1e-28
    with pytest.raises(ValueError):
        parallel.shard_k(w, t, nrows, k, 0, 5)


def _worker(rank, world, port, tmp):
    import torch
    import torch.distributed as dist

    import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = synth.rng_for(5)                        # same seed everywhere: every rank builds the same tensors
        nrows, k, ntok = 32, 512, 3
        w = synth.q4k_matrix(rng, nrows, k)
        x = synth.activations(rng, ntok, k)
        ref = oracle.matmul_f64(Q4_K, w, x, nrows, k, ntok)
        # column parallel + gather
        wr, n = parallel.shard_rows(w, Q4_K, nrows, k, rank, world)
        col = parallel.ColumnParallel(lambda xx: torch.from_numpy(
            oracle.matmul_f64(Q4_K, wr, xx.numpy(), n, k, ntok).astype(np.float32)), n)
        full = col.gather(col.forward(torch.from_numpy(x)))
        assert full.shape == (ntok, nrows) and nmse(full.numpy(), ref) < 1e-13
        # row parallel + all-reduce
        wk, kl = parallel.shard_k(w, Q4_K, nrows, k, rank, world)
        row = parallel.RowParallel(lambda xx: torch.from_numpy(
            oracle.matmul_f64(Q4_K, wk, xx.numpy(), nrows, kl, ntok).astype(np.float32)))
        out = row.forward(torch.from_numpy(np.ascontiguousarray(x[:, rank * kl:(rank + 1) * kl])))
        assert nmse(out.numpy(), ref) < 1e-12
        # expert parallel: tokens split across the ranks, experts too
        E, topk, hidden, ffn, ntok_all = 4, 2, 64, 64, 6
        gate = synth.mxfp4_matrix(rng, E * ffn, hidden)
        up = synth.mxfp4_matrix(rng, E * ffn, hidden)
        down = synth.mxfp4_matrix(rng, E * hidden, ffn)
        h = synth.activations(rng, ntok_all, hidden)
        logits = synth.activations(rng, ntok_all, E)
        sel_all = np.zeros((ntok_all, topk), np.int32)
        wt_all = np.zeros((ntok_all, topk), np.float32)
        for i in range(ntok_all):
            s_, _, w_, _, _ = oracle.moe_router(oracle.softmax(logits[i]), topk)
            sel_all[i], wt_all[i] = s_, w_
        want = oracle.moe_layer(h, MXFP4, gate, up, down, sel_all, wt_all, E, hidden, ffn)
        g_l, epr = parallel.shard_experts(gate, MXFP4, E, ffn, hidden, rank, world)
        u_l, _ = parallel.shard_experts(up, MXFP4, E, ffn, hidden, rank, world)
        d_l, _ = parallel.shard_experts(down, MXFP4, E, hidden, ffn, rank, world)
        lo, hi = rank * ntok_all // world, (rank + 1) * ntok_all // world

        def route(lg):
            return torch.from_numpy(sel_all[lo:hi]), torch.from_numpy(wt_all[lo:hi])

        def experts(rows, ids):
            n_ = rows.shape[0]
            y = oracle.moe_layer(rows.numpy(), MXFP4, g_l, u_l, d_l, ids.numpy().reshape(n_, 1),
                                 np.ones((n_, 1), np.float32), epr, hidden, ffn)
            return torch.from_numpy(y)

        moe = parallel.ExpertParallelMoE(route, experts, E, topk, hidden)
        got = moe.forward(torch.zeros(hi - lo, hidden), torch.from_numpy(h[lo:hi]), torch.from_numpy(logits[lo:hi]))
        assert nmse(got.numpy(), want[lo:hi]) < 1e-12
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_column_row_and_expert_parallel(orc, tmp_path):
    import torch.multiprocessing as mp
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_dispatch_plan_and_ascending_combine():
    import torch
    sel = torch.tensor([[3, 0], [1, 2], [2, 3]], dtype=torch.int32)
    order, counts, local = parallel.dispatch_plan(sel, 2, 2)        # experts 0,1 -> rank 0; 2,3 -> rank 1
    assert counts.tolist() == [2, 4]
    assert order.tolist() == [1, 2, 0, 3, 4, 5]                      # stable: pair order kept inside a rank
    assert local.tolist() == [0, 1, 1, 0, 0, 1]
    wt = torch.tensor([[0.25, 0.75]] * 3)
    y = torch.arange(3 * 2 * 4, dtype=torch.float32).view(3, 2, 4)
    out = parallel.combine_ascending(torch.zeros(3, 4), y, sel, wt)
    want0 = 0.75 * y[0, 1] + 0.25 * y[0, 0]                           # expert 0 (slot 1) first, then expert 3
    assert torch.equal(out[0], (torch.zeros(4) + 0.75 * y[0, 1]) + 0.25 * y[0, 0]) and torch.allclose(out[0], want0)


def test_shard_segments_reassembles_and_matches_the_dense_product(orc):
    """q|k|v-style row-concatenated matrices: every rank holds matching slices of all parts (column parallel) or a
    k-range of every row (row parallel); the shards reassemble to the full matrix and their products to the full
    product."""
    import numpy as np
    from jitllm_b200 import parallel, synth
    from jitllm_b200._lib import Q4_K, Q8_0
    rng = synth.rng_for(8)
    for t, k in ((Q4_K, 1024), (Q8_0, 256)):
        segments = [64, 16, 16]
        nrows = sum(segments)
        full = synth.matrix(rng, t, nrows, k)
        x = synth.activations(rng, 2, k)
        ref = orc.matmul_f64(t, full, x, nrows, k, 2)
        for world in (1, 2, 4):
            # column parallel: outputs of rank r are the r-th slice of every part
            outs = []
            for rank in range(world):
                raw, rows_l, k_l = parallel.shard_segments(full, t, segments, k, rank, world)
                assert k_l == k and rows_l == nrows // world
                outs.append(orc.matmul_f64(t, raw, x, rows_l, k, 2))
            got = np.empty_like(ref)
            r0 = 0
            for si, n in enumerate(segments):
                per = n // world
                o0 = sum(s // world for s in segments[:si])
                for rank in range(world):
                    got[:, r0 + rank * per:r0 + (rank + 1) * per] = outs[rank][:, o0:o0 + per]
                r0 += n
            assert np.array_equal(got, ref)
            # row parallel: partial products over the k-ranges add up (f64: exact enough to compare tightly)
            acc = np.zeros_like(ref)
            for rank in range(world):
                raw, rows_l, k_l = parallel.shard_segments(full, t, segments, k, rank, world, k_split=True)
                assert rows_l == nrows and k_l == k // world
                acc += orc.matmul_f64(t, raw, x[:, rank * k_l:(rank + 1) * k_l], nrows, k_l, 2)
            assert np.allclose(acc, ref, rtol=1e-12, atol=1e-9)
    with pytest.raises(ValueError):
        parallel.shard_segments(synth.q4k_matrix(rng, 6, 256), Q4_K, [6], 256, 0, 4)          # 6 rows over 4 ranks
    with pytest.raises(ValueError):
        parallel.shard_segments(synth.q4k_matrix(rng, 8, 256), Q4_K, [8], 256, 0, 2, k_split=True)   # 128 is not a block multiple
