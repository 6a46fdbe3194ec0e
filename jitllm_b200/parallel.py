"""Sharding of the quantized-matmul path across the GPUs of one box.

The reference has no tensor or expert parallelism (docs/perf/current.md:582,760: layer placement
only), so there is no reference interface to mirror here; parity of every sharded form is
defined against the UNSHARDED oracle. One process per GPU, `torch.distributed` for the plumbing
(NCCL on GPUs; the same code runs over gloo on CPU tensors, which is how the host logic is
tested without GPUs).

  column-parallel  (q/k/v, gate, up, lm_head)  rows N/g per rank, whole blocks; no collective
  row-parallel     (o, down)                   K/g per rank, cut at block boundaries; the
                                               partial outputs meet in an all-reduce (sum)
  expert-parallel  (mixture layer)             E/g experts per rank, tokens data-parallel;
                                               all-to-all dispatch of routed rows, local grouped
                                               GEMMs, all-to-all return, combine in ascending
                                               expert id on the token's home rank

The byte-level sharding helpers are pure numpy. The compute is injected (`matmul`, `experts`
callables), which on a GPU are thin wrappers over libjitllm_b200.so and in the CPU tests are the
oracle.
"""
from __future__ import annotations

import numpy as np

from ._lib import BLOCK, row_bytes


# ------------------------------------------------------------ byte sharding

def shard_rows(w: np.ndarray, t: int, nrows: int, k: int, rank: int, world: int) -> tuple[np.ndarray, int]:
    """Column-parallel shard: rows [rank*nrows/world, (rank+1)*nrows/world) of a raw ggml tensor."""
    if nrows % world:
        raise ValueError(f"{nrows} rows do not split over {world} ranks")
    rb = row_bytes(t, k)
    n = nrows // world
    flat = np.ascontiguousarray(w).reshape(-1).view(np.uint8)
    return flat[rank * n * rb:(rank + 1) * n * rb].copy(), n


def shard_k(w: np.ndarray, t: int, nrows: int, k: int, rank: int, world: int) -> tuple[np.ndarray, int]:
    """Row-parallel shard: for every row the blocks of k-range [rank*k/world, (rank+1)*k/world).
    The cut must fall on block boundaries (256 elements for Q4_K, 32 for Q8_0 / MXFP4)."""
    be, bb = BLOCK[t]
    if k % world or (k // world) % be:
        raise ValueError(f"k={k} does not split over {world} ranks at {be}-element block boundaries")
    kl = k // world
    per = kl // be * bb
    m = np.ascontiguousarray(w).reshape(-1).view(np.uint8).reshape(nrows, row_bytes(t, k))
    return np.ascontiguousarray(m[:, rank * per:(rank + 1) * per]).reshape(-1), kl


def shard_experts(bank: np.ndarray, t: int, n_expert: int, rows: int, k: int, rank: int, world: int):
    """Expert-parallel shard of a bank [n_expert][rows][row_bytes]: experts [rank*E/g, (rank+1)*E/g)."""
    if n_expert % world:
        raise ValueError(f"{n_expert} experts do not split over {world} ranks")
    per = n_expert // world
    eb = rows * row_bytes(t, k)
    flat = np.ascontiguousarray(bank).reshape(-1).view(np.uint8)
    return flat[rank * per * eb:(rank + 1) * per * eb].copy(), per


def shard_segments(full: np.ndarray, t: int, segments, k: int, rank: int, world: int, k_split: bool = False):
    """Shard of a row-concatenated matrix (q|k|v, gate|up): `segments` are the row counts of its parts. Column
    parallel (default): rows [rank/world) of EVERY part, concatenated in part order, so a rank holds matching
    slices of all parts. Row parallel (k_split): the k-range [rank/world) of every row, cut at block boundaries.
    Returns (bytes [rows_local][row_bytes_local], rows_local, k_local)."""
    be, bb = BLOCK[t]
    nrows = sum(segments)
    m = np.ascontiguousarray(full).reshape(-1).view(np.uint8).reshape(nrows, k // be, bb)
    if k_split:
        if k % world or (k // world) % be:
            raise ValueError(f"k={k} does not split over {world} ranks at {be}-element block boundaries")
        nb = k // be // world
        out = m[:, rank * nb:(rank + 1) * nb]
        return np.ascontiguousarray(out).reshape(nrows, nb * bb), nrows, k // world
    parts, r0 = [], 0
    for n in segments:
        if n % world:
            raise ValueError(f"a part of {n} rows does not split over {world} ranks")
        per = n // world
        parts.append(m[r0 + rank * per:r0 + (rank + 1) * per])
        r0 += n
    out = np.ascontiguousarray(np.concatenate(parts, axis=0))
    return out.reshape(out.shape[0], -1), out.shape[0], k


# -------------------------------------------------------------- dense layers

class ColumnParallel:
    """out_local[ntok][nrows/g] = x W_r^T. `matmul(x) -> out` is this rank's kernel call."""

    def __init__(self, matmul, nrows_local: int):
        self.matmul, self.nrows_local = matmul, nrows_local

    def forward(self, x):
        return self.matmul(x)

    def gather(self, out_local, group=None):
        """All ranks' slices side by side: [ntok][nrows] (for a consumer that needs the whole row)."""
        import torch
        import torch.distributed as dist
        world = dist.get_world_size(group)
        parts = [torch.empty_like(out_local) for _ in range(world)]
        dist.all_gather(parts, out_local.contiguous(), group=group)
        return torch.cat(parts, dim=-1)


class RowParallel:
    """out[ntok][nrows] = sum over ranks of x[:, k_r] W[:, k_r]^T: partial product + all-reduce."""

    def __init__(self, matmul, group=None):
        self.matmul, self.group = matmul, group

    def forward(self, x_local):
        import torch.distributed as dist
        out = self.matmul(x_local)          # f32 partial sums
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out


# ------------------------------------------------------------ expert parallel

def dispatch_plan(sel, experts_per_rank: int, world: int):
    """From this rank's routing `sel` [ntok][top_k] (torch int tensor): the order in which its
    (token, slot) pairs are sent -- grouped by destination rank, token order kept inside a group --
    and how many go to each rank. Returns (order [npairs] indices into the flattened pairs,
    send_counts [world], local_expert_ids [npairs] in send order)."""
    import torch
    flat = sel.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world)[:world]
    local_ids = (flat[order] - dest[order] * experts_per_rank).to(torch.int32)
    return order, counts, local_ids


def combine_ascending(out, y_pairs, sel, wt):
    """out[tok] += sum_j w_j * y_j with the token's experts taken in ASCENDING expert id
    (engine/model/moe.go:127-134), one addition at a time so the f32 sum has a fixed order.
    y_pairs is [ntok][top_k][hidden] in slot order."""
    import torch
    idx = torch.argsort(sel.to(torch.int64), dim=1, stable=True)          # slots by ascending expert id
    ys = torch.gather(y_pairs, 1, idx[:, :, None].expand_as(y_pairs))
    ws = torch.gather(wt, 1, idx)
    for j in range(sel.shape[1]):
        out += ws[:, j:j + 1] * ys[:, j]
    return out


class ExpertParallelMoE:
    """Mixture layer with experts sharded over ranks and tokens data-parallel.

    route(logits) -> (sel [ntok][k] int32, wt [ntok][k] f32)     this rank's router (replicated weights)
    experts(h_rows, local_ids) -> y_rows [n][hidden] f32          this rank's experts over routed rows
    """

    def __init__(self, route, experts, n_expert: int, top_k: int, hidden: int, group=None):
        import torch.distributed as dist
        self.route, self.experts = route, experts
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_expert % self.world:
            raise ValueError(f"{n_expert} experts do not split over {self.world} ranks")
        self.epr, self.top_k, self.hidden, self.group = n_expert // self.world, top_k, hidden, group

    def forward(self, out, h, logits, capacity: int | None = None):
        """out [ntok][hidden] f32 += layer(h); h [ntok][hidden] (f32 or bf16), logits [ntok][E] f32.

        Fixed-capacity exchange: every rank sends every other rank the same number of row slots (`capacity`,
        default ntok * top_k: the worst case, so nothing can overflow; every rank must pass the same value), unused
        slots carrying expert id -1, which the experts' token lists skip. No size crosses the host, so the whole
        layer is a fixed sequence of device operations (a CUDA graph can hold it); the price is padding on the wire.
        The reference's grouped launches read one word home per chunk instead (jit/gpu/tier/moegroup.go:10-19)."""
        import torch
        import torch.distributed as dist
        ntok, K, W = h.shape[0], self.top_k, self.world
        npairs = ntok * K
        cap = capacity or npairs
        sel, wt = self.route(logits)
        flat = sel.reshape(-1).to(torch.int64)
        valid = flat >= 0
        dest = torch.where(valid, torch.div(flat, self.epr, rounding_mode="floor"), torch.zeros_like(flat))
        # slot of each pair inside its destination's bucket: pairs keep their order (a stable rank by one-hot cumsum)
        onehot = torch.nn.functional.one_hot(dest, W) * valid[:, None]
        rank_in = (onehot.cumsum(0) - onehot).gather(1, dest[:, None])[:, 0]
        ok = valid & (rank_in < cap)
        send_idx = torch.where(ok, dest * cap + rank_in, torch.full_like(dest, W * cap))     # W*cap: a scratch slot for the unsent
        tok_of_pair = torch.arange(npairs, device=h.device) // K
        send_rows = torch.zeros((W * cap + 1, self.hidden), dtype=h.dtype, device=h.device)
        send_ids = torch.full((W * cap + 1,), -1, dtype=torch.int32, device=h.device)
        send_rows[send_idx] = h[tok_of_pair]
        send_ids[send_idx] = torch.where(ok, flat - dest * self.epr, torch.full_like(flat, -1)).to(torch.int32)
        recv_rows = torch.empty((W * cap, self.hidden), dtype=h.dtype, device=h.device)
        recv_ids = torch.empty(W * cap, dtype=torch.int32, device=h.device)
        dist.all_to_all_single(recv_rows, send_rows[:W * cap].contiguous(), group=self.group)
        dist.all_to_all_single(recv_ids, send_ids[:W * cap].contiguous(), group=self.group)
        y_recv = self.experts(recv_rows, recv_ids)                         # rows whose id is -1 are not computed
        y_back = torch.empty((W * cap + 1, self.hidden), dtype=torch.float32, device=h.device)
        dist.all_to_all_single(y_back[:W * cap], y_recv.contiguous(), group=self.group)
        y_back[W * cap] = 0
        y_pairs = y_back[send_idx]                                         # back to (token, slot) order
        y_pairs = torch.where(ok[:, None], y_pairs, torch.zeros_like(y_pairs))
        wt_eff = torch.where(ok.view(ntok, K), wt, torch.zeros_like(wt))
        return combine_ascending(out, y_pairs.view(ntok, K, self.hidden), sel, wt_eff)


# ------------------------------------------------------ tensor-parallel slot exchange

def tp_attach(block, group=None):
    """Every rank exports its slot buffer as a CUDA IPC handle, the handles travel over the process group (any
    backend: they are 64 host bytes), every rank opens its peers' slots and attaches them, then the ranks meet once
    so that no kernel stores into a slot that is not mapped yet. `block` is a device.Layers."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    handles = [None] * world
    dist.all_gather_object(handles, block.ExportHandle(), group=group)
    block.Attach(handles)
    dist.barrier(group=group)
