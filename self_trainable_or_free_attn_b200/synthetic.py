"""Seeded synthetic activations with the shapes of video-diffusion attention layers.

They stand in for real model activations (no weights or prompts are needed): a latent token grid T x H x W laid out
frame-major, a per-head base signal = unit Gaussian noise plus a smooth low-frequency component (a sum of four random
3-D cosines over (t, y, x), amplitude 1.5, which makes attention locality-biased), and Q, K, V as independent random
128 x 128 projections (entries N(0, 1/128)) of the base. The previous denoising step's Q', K' are Q, K plus N(0, 0.02^2)
noise. Any rank can regenerate exactly its own (branch, head) shard from the seeds.
"""
import math

import torch

WORKLOADS = {
    # name: (grid T, H, W), heads, CFG branches, density, text tokens
    "cpu_small": ((4, 8, 16), 2, 1, 0.25, 0),
    "wan_1_3b_480p": ((21, 30, 52), 12, 2, 0.15, 0),
    "wan_14b_720p": ((21, 45, 80), 40, 2, 0.10, 0),
    "hunyuan_720p": ((33, 45, 80), 24, 1, 0.12, 256),
}


def grid_tokens(grid):
    return grid[0] * grid[1] * grid[2]


def head_seed(config_id, branch, head):
    return 1000 * config_id + 10 * branch + head


def head_qkv(grid, config_id, branch, head, device, text_tokens=0, prev=False, dtype=torch.bfloat16):
    """q, k, v of one (branch, head): (L, 128) each. The smooth component and the projections depend on the head only,
    the noise on (branch, head), so the two CFG branches see related but different activations. With prev=True, q and k
    get the previous step's perturbation."""
    T, Hh, W = grid
    L = T * Hh * W
    gs = torch.Generator(device=device).manual_seed(head_seed(config_id, 0, head) + 7919)
    gn = torch.Generator(device=device).manual_seed(head_seed(config_id, branch, head))
    t = torch.arange(T, device=device, dtype=torch.float32)[:, None, None] / T
    y = torch.arange(Hh, device=device, dtype=torch.float32)[None, :, None] / Hh
    x = torch.arange(W, device=device, dtype=torch.float32)[None, None, :] / W
    smooth = torch.zeros(T, Hh, W, 128, device=device)
    for _ in range(4):
        f = torch.randint(0, 4, (3, 128), device=device, generator=gs).float()
        phase = torch.rand(128, device=device, generator=gs) * (2 * math.pi)
        arg = t[..., None] * f[0] + y[..., None] * f[1] + x[..., None] * f[2]
        smooth += torch.cos(2 * math.pi * arg + phase)
    base = torch.randn(L, 128, device=device, generator=gn) + 1.5 * smooth.view(L, 128)
    w = [torch.randn(128, 128, device=device, generator=gs) / math.sqrt(128.0) for _ in range(3)]
    q, k, v = (base @ wi for wi in w)
    if text_tokens:
        q, k, v = (torch.cat([a, torch.randn(text_tokens, 128, device=device, generator=gn)]) for a in (q, k, v))
    if prev:
        q = q + 0.02 * torch.randn(q.shape, device=device, generator=gn)
        k = k + 0.02 * torch.randn(k.shape, device=device, generator=gn)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def branch_qkv(grid, config_id, branch, heads, device, text_tokens=0, prev=False):
    """[1, L, len(heads), 128] bf16 q, k, v of the listed heads of one CFG branch."""
    L = grid_tokens(grid) + text_tokens
    out = [torch.empty(1, L, len(heads), 128, device=device, dtype=torch.bfloat16) for _ in range(3)]
    for i, h in enumerate(heads):
        for dst, src in zip(out, head_qkv(grid, config_id, branch, h, device, text_tokens, prev)):
            dst[0, :, i] = src
    return out


def shard_heads(heads, rank, world):
    """Contiguous, balanced range of heads for `rank`: both CFG branches of a head stay on one GPU, so the shared block
    selection never crosses GPUs."""
    base, extra = divmod(heads, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def step_flops(L, counts, blocks, refine, skip_bits, tiles=None):
    """Algorithmic FLOP of one fused sparse step of one branch: 4 * D * sum over tiles of rows x columns, with columns =
    tokens of the exact blocks + block-mean columns + 4 per refined block (real rows and lengths, no padding).
    counts (nq, H), blocks (nq, H, nb) ascending, refine (nq, H, rw) padded with nb, skip_bits (H, nq, nw).
    `tiles`: optional list of tile indices to count (default: all)."""
    nq, H = counts.shape
    nb = blocks.shape[-1]
    dev = counts.device
    rows = torch.full((nq,), 128.0, device=dev, dtype=torch.float64)
    rows[-1] = L - 128 * (nq - 1)
    last = torch.gather(blocks, 2, (counts.long() - 1).clamp_min(0)[..., None])[..., 0]
    has_tail = (counts > 0) & (last == nb - 1)                               # lists are ascending
    exact_tokens = counts.double() * 64 - has_tail.double() * (64 * nb - L)
    j = torch.arange(nb, device=dev)
    words = skip_bits.long() & 0xFFFFFFFF                                    # (H, nq, nw)
    skipped = ((words[:, :, j // 32] >> (j % 32)) & 1) != 0                   # (H, nq, nb)
    mean_cols = (~skipped).sum(-1).t().double()                               # (nq, H)
    refined = (refine < nb).sum(-1).double()                                  # (nq, H)
    per_tile = (rows[:, None] * (exact_tokens + mean_cols + 4.0 * refined)).sum(1)
    if tiles is not None:
        per_tile = per_tile[torch.as_tensor(tiles, device=dev, dtype=torch.long)]
    return float(4.0 * 128.0 * per_tile.sum())
