"""Seeded synthetic VSA2 workloads: training-shape activations and block selections with a chosen shape of imbalance.

They stand in for captured activations and router outputs (nothing here needs model weights): tokens of a T x H x W latent
grid in 4 x 4 x 4 tiles (64-token blocks), q, k, v = unit Gaussian noise plus a smooth low-frequency component, an upstream
gradient dO ~ N(0, 1), and a selection drawn from a seeded random-but-local score between tiles,

    score[i, j] = exp(-|c_i - c_j|^2 / (2 sigma^2)) * U(0, 1),        c = tile coordinates,

either as the exact global top-(NB * topk) of that score (lists vary a little around topk), or with the list LENGTHS
prescribed per query block and the entries of a list chosen by the score. The prescribed shapes play the role of the
reference's skew generators (benchmarks/vsa2_splitkv_bench.py:120-183): every case keeps NB * topk pairs per head, so the
arithmetic is the same and only its distribution over query / kv blocks changes.

  uniform      exact global top-k of the score
  tenth_x4     10 % of the query blocks select 4 x topk kv blocks each, the others share the rest evenly
  eighth_x4    NB / 8 query blocks with 4 x topk (the reference's "hotq_mixed")
  quarter      a quarter of the query blocks hold all pairs ("hotq")
  straggler    the last query block selects every kv block, the others share the rest
  hot_kv       NB / 16 kv blocks are hot: every query block takes half of its list from them ("hotkv")
"""
import math

import torch

from . import ops
from .layout import build_layout, to_blocked

CASES = ("uniform", "tenth_x4", "eighth_x4", "quarter", "straggler", "hot_kv")


def train_inputs(grid=(16, 32, 64), heads=12, seed=4000, device="cuda", dtype=torch.bfloat16):
    """(q, k, v, gate, dout, layout) of one layer, B = 1, head dim 128, block-major token order, on `device`."""
    T, H, W = grid
    g = torch.Generator(device="cpu").manual_seed(seed)
    lay = build_layout(grid, R=16)
    n = T * H * W
    t, y, x = torch.meshgrid(torch.arange(T) / T, torch.arange(H) / H, torch.arange(W) / W, indexing="ij")
    pos = torch.stack([t, y, x], -1).reshape(n, 3)
    qkv = []
    for _ in range(3):
        noise = torch.randn(1, heads, n, 128, generator=g)
        freq = torch.randn(4, 3, generator=g) * 2.0
        phase = torch.rand(4, 128, generator=g) * 2 * math.pi
        smooth = torch.cos(2 * math.pi * (pos @ freq.t())[:, :, None] + phase[None]).sum(1) * 0.75
        qkv.append(to_blocked((noise + smooth[None, None]).to(dtype), lay).to(device).contiguous())
    gate = to_blocked((torch.randn(1, heads, n, generator=g) * 1.5).to(dtype), lay).to(device).contiguous()
    dout = to_blocked(torch.randn(1, heads, n, 128, generator=g).to(dtype), lay).to(device).contiguous()
    return qkv[0], qkv[1], qkv[2], gate, dout, lay


def tile_grid(grid):
    T, H, W = grid
    return -(-T // 4), -(-H // 4), -(-W // 4)


def local_scores(grid, heads, seed=4001, sigma=3.0):
    """[1, heads, NB, NB] float32 on the CPU: Gaussian of the distance between tile centres times U(0, 1)."""
    nt, nh, nw = tile_grid(grid)
    nb = nt * nh * nw
    c = torch.stack(torch.meshgrid(torch.arange(nt), torch.arange(nh), torch.arange(nw), indexing="ij"), -1)
    c = c.reshape(nb, 3).float()
    near = torch.exp(-((c[:, None] - c[None]) ** 2).sum(-1) / (2 * sigma ** 2))
    g = torch.Generator().manual_seed(seed)
    return near[None, None] * torch.rand(1, heads, nb, nb, generator=g)


def _even(total, n):
    """`total` spread over n entries as evenly as integers allow (the first total % n get one more)."""
    out = torch.full((n,), total // n, dtype=torch.int64)
    out[: total % n] += 1
    return out


def list_lengths(case, nb, topk, gen):
    """(length of every query block's list taken from hot kv blocks, from the other kv blocks, mask of hot kv blocks).
    The lengths of a head always add up to nb * topk."""
    total = nb * topk
    order = torch.randperm(nb, generator=gen)
    hot = torch.zeros(nb, dtype=torch.bool)
    from_hot = torch.zeros(nb, dtype=torch.int64)
    cold = torch.zeros(nb, dtype=torch.int64)
    if case in ("tenth_x4", "eighth_x4"):
        n_long = max(1, round(0.10 * nb)) if case == "tenth_x4" else max(1, nb // 8)
        long_len = min(4 * topk, nb)
        cold[order[:n_long]] = long_len
        cold[order[n_long:]] = _even(total - n_long * long_len, nb - n_long)
    elif case == "quarter":
        cold[order[: nb // 4]] = _even(total, nb // 4)
    elif case == "straggler":
        cold[nb - 1] = nb
        cold[: nb - 1] = _even(total - nb, nb - 1)
    elif case == "hot_kv":
        hot[torch.randperm(nb, generator=gen)[: max(1, nb // 16)]] = True
        from_hot[:] = min(topk // 2, int(hot.sum()))
        cold[:] = topk - from_hot
    else:
        raise ValueError(f"unknown case {case!r}; have {CASES}")
    if int(cold.max()) > nb - int(hot.sum()) or int((from_hot + cold).sum()) != total:
        raise ValueError(f"{case}: the lists do not fit nb = {nb}, topk = {topk}")
    return from_hot, cold, hot


def _largest_per_row(scores, lengths):
    """Bool mask: in row r, the lengths[r] largest entries of scores[r] (ties to the smaller column)."""
    if scores.shape[1] == 0:
        return torch.zeros_like(scores, dtype=torch.bool)
    order = torch.sort(scores, dim=1, descending=True, stable=True).indices
    rank = torch.empty_like(order)
    rank.scatter_(1, order, torch.arange(scores.shape[1]).expand_as(order))
    return rank < lengths[:, None]


def selection_mask(case, grid, heads, topk, seed=4001):
    """Bool [1, heads, NB, NB] on the CPU."""
    scores = local_scores(grid, heads, seed)
    nb = scores.shape[-1]
    if case == "uniform":
        flat = scores.reshape(heads, nb * nb)
        order = torch.sort(flat, dim=1, descending=True, stable=True).indices[:, : nb * topk]
        return torch.zeros(heads, nb * nb, dtype=torch.bool).scatter_(1, order, True).reshape(1, heads, nb, nb)
    gen = torch.Generator().manual_seed(seed + 1)
    mask = torch.zeros(1, heads, nb, nb, dtype=torch.bool)
    for h in range(heads):
        from_hot, cold, hot = list_lengths(case, nb, topk, gen)
        hc, cc = hot.nonzero().flatten(), (~hot).nonzero().flatten()
        m = torch.zeros(nb, nb, dtype=torch.bool)
        m[:, hc] = _largest_per_row(scores[0, h][:, hc], from_hot)
        m[:, cc] = _largest_per_row(scores[0, h][:, cc], cold)
        mask[0, h] = m
    return mask


def selection(case, grid, heads, topk, device, seed=4001):
    """The case's selection as the kernels' CSR lists (both directions) on `device`, and NB."""
    mask = selection_mask(case, grid, heads, topk, seed)
    return ops.mask_to_selection(mask.to(device)), mask.shape[-1]


def fine_flops(sel, D=128):
    """Algorithmic FLOP of the fine branch: forward 4 * 64 * 64 * D per selected pair (QK^T and PV); the backward's five
    products per pair are 2.5 x that."""
    pairs = int(sel.row_counts().sum())
    fwd = 4.0 * 64 * 64 * D * pairs
    return fwd, 2.5 * fwd, pairs
