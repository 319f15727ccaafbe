"""The sparse step of a sample of query tiles, entirely on host cores: the timed CPU baseline of bench.py.

TEST / BENCHMARK INFRASTRUCTURE ONLY (like everything under oracle/): the product path never imports it.

For one head of one CFG branch of a named synthetic workload it builds, with the oracle alone: the previous step's dense
log2 LSE and block masses of the sampled tiles (exact, row block by row block), the block selection, the block means,
the representatives of the blocks the sampled tiles refine, and then times the fused fixed-offset softmax of those tiles
(`echosparse_ref.fixed_offset_attention`). Nothing here touches a GPU.
"""
import math
import time

import torch

from oracle import echosparse_ref as R
from self_trainable_or_free_attn_b200 import synthetic


def build_sample(workload, config_id, n_tiles, iters=6):
    grid, _, _, density, text = synthetic.WORKLOADS[workload]
    L = synthetic.grid_tokens(grid) + text
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    q, k, v = (x[:, None].contiguous() for x in synthetic.head_qkv(grid, config_id, 0, 0, "cpu", text))
    qp, kp, _ = (x[:, None].contiguous() for x in synthetic.head_qkv(grid, config_id, 0, 0, "cpu", text, prev=True))
    tiles = sorted(set(int(t) for t in torch.linspace(0, nq - 1, min(nq, n_tiles)).round().tolist()))
    c = R.LOG2E / math.sqrt(128.0)
    offset = torch.full((nq * 128, 1), 1e30)
    mass = torch.zeros(1, nq, nb)
    pad = nb * 64 - L
    kf = kp[:, 0].float()
    for t in tiles:
        rows = torch.arange(128 * t, min(128 * t + 128, L))
        s = (qp[rows, 0].float() @ kf.T) * c
        lse = torch.logsumexp(s * math.log(2.0), -1) / math.log(2.0)
        offset[rows, 0] = lse
        p = torch.exp2(s - lse[:, None]).sum(0)
        mass[0, t] = torch.cat([p, torch.zeros(pad)]).view(nb, 64).sum(1)
    top, refined = R.budget(density, nb)
    rw = -(-refined // 32) * 32
    ones = torch.ones(1, nq, nb, dtype=torch.uint8)
    scale = torch.full((1, nq), 1.0 / 128.0)
    keep, counts, blocks, bits, refine = R.select_blocks(mass, ones, scale, torch.ones(1, nq),
                                                        torch.zeros(nq, 1, dtype=torch.int32), top, refined, L, rw)
    k_mean, v_mean = R.block_means(k, v)
    _, metric, probes = R.query_metric(q)
    k_rep = torch.zeros(1, (nb + 1) * 4, 128, dtype=torch.bfloat16)
    v_rep = torch.zeros_like(k_rep)
    log_counts = torch.full((1, (nb + 1) * 4), float("-inf"))
    need = sorted({b for t in tiles for b in refine[t, 0].tolist() if b < nb})
    for b in need:
        sl = slice(64 * b, min(64 * b + 64, L))
        k4, v4, c4, _ = R.kmeans_block(k[sl, 0], v[sl, 0], metric[0], probes[0], iters)
        k_rep[0, 4 * b:4 * b + 4], v_rep[0, 4 * b:4 * b + 4], log_counts[0, 4 * b:4 * b + 4] = k4, v4, c4
    args = dict(counts=counts, blocks=blocks, offset=offset, k_mean=k_mean, v_mean=v_mean, skip_bits=bits, refine=refine,
                k_rep=k_rep, v_rep=v_rep, log_counts=log_counts)
    flop = synthetic.step_flops(L, counts, blocks, refine, bits, tiles=tiles)
    return dict(q=q, k=k, v=v, tiles=[(t, 0) for t in tiles], args=args, flop=flop, L=L, nq=nq)


def time_sample(job, threads):
    """Seconds of one pass of the fused step over the job's tiles with `threads` torch threads."""
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    R.fixed_offset_attention(job["q"], job["k"], job["v"], tiles=job["tiles"], **job["args"])
    return time.perf_counter() - t0
