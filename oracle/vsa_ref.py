"""CPU restatement of VSA2 (router, exact global top-k, fine / coarse attention, gate fusion, three-tier fine branch).

TEST INFRASTRUCTURE ONLY: imported by tests/, by `__graft_entry__.smoke()` and by the CPU-baseline leg of bench.py,
never by the product path. Everything here is plain torch on the CPU, written blockwise (one query block at a time)
from the definition of the method, and differentiable, so gradients come from autograd.

Follows the reference (shaoshitong/self_trainable_or_free_attn):
  tests/vsa_reference.py:28-52    token validity, group means, block means (optionally rounded to the token dtype)
  tests/vsa_reference.py:56-74    PSP router scores: softmax over all valid pooled keys, summed per block pair
  tests/vsa_reference.py:77-87    exact global top-`budget` per (b, h), ties to the smaller flat index
  tests/vsa_reference.py:90-108   fine attention on selected blocks; empty / padded rows give 0 and lse = -inf
  tests/vsa_reference.py:110-117  coarse attention over block means
  tests/vsa_reference.py:119-136  O = O_fine + act(gate) * O_coarse[block], padded rows zero
  experiments/vsa2_representative/vsa2_rep/reference.py:24-96  three tiers: tokens, group means (+ln c), block means (+ln c)
Pinned against outputs of those files on seeded inputs: tests/golden/vsa2.npz (tests/golden/make_golden_vsa.py).
"""
import math

import torch

BLOCK = 64


def token_valid(blk_cnt, L):
    """[L] bool: slot t of block t // 64 holds a real token (the valid tokens come first in a block)."""
    pos = torch.arange(L)
    return (pos % BLOCK) < blk_cnt.to(torch.int64)[pos // BLOCK]


def _round(x, dtype):
    return x if dtype is None else x.to(dtype).to(x.dtype)


def group_means(x, blk_cnt, R, round_to=None):
    """Means of the R-token groups over their valid tokens. x [B,H,L,D] -> ([B,H,L/R,D], [L/R] group has a token)."""
    B, H, L, D = x.shape
    ok = token_valid(blk_cnt, L).to(x.dtype)
    n = ok.reshape(L // R, R).sum(1)
    tot = (x * ok[None, None, :, None]).reshape(B, H, L // R, R, D).sum(3)
    return _round(tot / n.clamp(min=1)[None, None, :, None], round_to), n > 0


def block_means(x, blk_cnt, round_to=None):
    return group_means(x, blk_cnt, BLOCK, round_to)[0]


def psp_scores(q, k, blk_cnt, R, row_norm="paper", round_to=torch.bfloat16):
    """Block scores [B,H,NB,NB] fp32: pooled-query softmax over all valid pooled keys, summed over the G x G group
    pairs of a block pair, divided by G^2 ("paper") or by the number of valid query groups of the block."""
    B, H, L, D = q.shape
    NB, G = L // BLOCK, BLOCK // R
    qr, q_ok = group_means(q.float(), blk_cnt, R, round_to)
    kr, k_ok = group_means(k.float(), blk_cnt, R, round_to)
    out = torch.zeros(B, H, NB, NB)
    for i in range(NB):
        rows = qr[:, :, i * G:(i + 1) * G]                                     # [B,H,G,D]
        s = rows @ kr.transpose(-1, -2) / math.sqrt(D)                         # [B,H,G,NB*G]
        s = s.masked_fill(~k_ok[None, None, None, :], float("-inf"))
        a = torch.softmax(s, -1) * q_ok[i * G:(i + 1) * G].to(s.dtype)[None, None, :, None]
        out[:, :, i] = a.reshape(B, H, G, NB, G).sum((2, 4))
    if row_norm == "paper":
        return out / (G * G)
    groups = (blk_cnt.to(torch.int64) + R - 1) // R
    return out / groups.to(out.dtype)[None, None, :, None]


def global_topk_mask(scores, budget):
    """The `budget` largest entries of every (b, h) score matrix; equal scores go to the smaller flat index."""
    B, H, NB, _ = scores.shape
    flat = scores.reshape(B * H, NB * NB)
    n = max(0, min(int(budget), NB * NB))
    mask = torch.zeros(B * H, NB * NB, dtype=torch.bool)
    if n:
        order = torch.sort(flat, dim=1, descending=True, stable=True).indices[:, :n]
        mask.scatter_(1, order, True)
    return mask.reshape(B, H, NB, NB)


def fine_attention(q, k, v, blk_cnt, mask):
    """Token attention of every query block over the valid tokens of its selected kv blocks, in the dtype of q.
    Returns (O [B,H,L,D], lse [B,H,L] natural); rows without a key and padded rows give 0 and -inf."""
    B, H, L, D = q.shape
    NB = L // BLOCK
    ok = token_valid(blk_cnt, L)
    o_rows, lse_rows = [], []
    for b in range(B):
        for h in range(H):
            for i in range(NB):
                qi = q[b, h, i * BLOCK:(i + 1) * BLOCK]
                row_ok = ok[i * BLOCK:(i + 1) * BLOCK]
                cols = [torch.arange(j * BLOCK, j * BLOCK + int(blk_cnt[j])) for j in mask[b, h, i].nonzero().flatten().tolist()]
                if not cols:
                    o_rows.append(qi * 0)
                    lse_rows.append(torch.full((BLOCK,), float("-inf"), dtype=q.dtype))
                    continue
                idx = torch.cat(cols)
                s = qi @ k[b, h, idx].transpose(0, 1) / math.sqrt(D)
                lse = torch.logsumexp(s, -1)
                o = torch.softmax(s, -1) @ v[b, h, idx]
                o_rows.append(o * row_ok[:, None].to(o.dtype))
                lse_rows.append(torch.where(row_ok, lse, torch.full_like(lse, float("-inf"))))
    return torch.stack(o_rows).reshape(B, H, L, D), torch.stack(lse_rows).reshape(B, H, L)


def coarse_attention(q, k, v, blk_cnt, round_to=torch.bfloat16):
    """Dense attention of the block means: [B,H,NB,D]."""
    qc, kc, vc = (block_means(x.float(), blk_cnt, round_to) for x in (q, k, v))
    s = qc @ kc.transpose(-1, -2) / math.sqrt(q.shape[-1])
    return torch.softmax(s, -1) @ vc


def vsa2_output(q, k, v, gate, blk_cnt, mask, gate_act="tanh", round_pooled=True):
    """O = O_fine + act(gate) * O_coarse[block of the token]; gate [B,H,L] or [B,H,L,D] or None (weight 1)."""
    B, H, L, D = q.shape
    of, _ = fine_attention(q, k, v, blk_cnt, mask)
    oc = coarse_attention(q, k, v, blk_cnt, q.dtype if round_pooled else None)
    oc_tok = oc.repeat_interleave(BLOCK, dim=2)
    if gate is None:
        a = torch.ones(B, H, L, 1, dtype=of.dtype)
    else:
        a = torch.tanh(gate.float()) if gate_act == "tanh" else gate.float()
        a = a[..., None] if a.dim() == 3 else a
    return (of + a * oc_tok) * token_valid(blk_cnt, L)[None, None, :, None].to(of.dtype)


def mask_to_csr(mask):
    """Block mask [B,H,NB,NB] -> (q2k_ptr [B,H,NB+1], q2k_idx, k2q_ptr, k2q_idx), int32, absolute offsets, ascending."""
    def one(m):
        B, H, N, _ = m.shape
        cnt = m.reshape(-1, N).sum(-1)
        incl = torch.cumsum(cnt, 0)
        start = (incl - cnt).reshape(B * H, N)
        ptr = torch.cat([start, incl.reshape(B * H, N)[:, -1:]], 1).reshape(B, H, N + 1)
        return ptr.to(torch.int32).contiguous(), m.reshape(-1, N).nonzero()[:, 1].to(torch.int32).contiguous()
    qp, qi = one(mask)
    kp, ki = one(mask.transpose(-1, -2).contiguous())
    return qp, qi, kp, ki


# ------------------------------------------------------------------------------------------- three tiers (64 / RM / 1)
def tier_tables(k, v, blk_cnt, mid_reps, round_to=None):
    """Group means of the 64/mid_reps-token groups and block means, with their token counts.
    Returns (k_mid, v_mid [B,H,NB*RM,D], c_mid [NB*RM], k_tail, v_tail [B,H,NB,D], c_tail [NB])."""
    R = BLOCK // mid_reps
    k_mid, _ = group_means(k, blk_cnt, R, round_to)
    v_mid, _ = group_means(v, blk_cnt, R, round_to)
    L = k.shape[2]
    c_mid = token_valid(blk_cnt, L).reshape(L // R, R).sum(1)
    return k_mid, v_mid, c_mid, block_means(k, blk_cnt, round_to), block_means(v, blk_cnt, round_to), blk_cnt.to(torch.int64)


def tier_fine_attention(q, k, v, blk_cnt, tier_a, tier_ab, mid_reps=4, round_reps=True, dtype=torch.float64):
    """One softmax per query row over: the valid tokens of tier-A blocks, the non-empty group means of tier-B blocks
    (tier_ab & ~tier_a) with + ln(count), the block means of tier-C blocks (~tier_ab) with + ln(count).
    tier_a, tier_ab: bool [B,H,NB,NB]. Returns (O, lse natural) in `dtype`."""
    B, H, L, D = q.shape
    NB, RM = L // BLOCK, mid_reps
    qd, kd, vd = q.to(dtype), k.to(dtype), v.to(dtype)
    rt = q.dtype if round_reps else None
    k_mid, v_mid, c_mid, k_tail, v_tail, c_tail = tier_tables(kd, vd, blk_cnt, RM, rt)
    ok = token_valid(blk_cnt, L)
    o_all = torch.zeros(B, H, L, D, dtype=dtype)
    lse_all = torch.full((B, H, L), float("-inf"), dtype=dtype)
    for b in range(B):
        for h in range(H):
            for i in range(NB):
                a = tier_a[b, h, i]
                ab = tier_ab[b, h, i]
                keys, vals, bias = [], [], []
                for j in a.nonzero().flatten().tolist():
                    n = int(blk_cnt[j])
                    keys.append(kd[b, h, j * BLOCK:j * BLOCK + n]); vals.append(vd[b, h, j * BLOCK:j * BLOCK + n])
                    bias.append(torch.zeros(n, dtype=dtype))
                for j in (ab & ~a).nonzero().flatten().tolist():
                    c = c_mid[j * RM:(j + 1) * RM]
                    keep = c > 0
                    keys.append(k_mid[b, h, j * RM:(j + 1) * RM][keep]); vals.append(v_mid[b, h, j * RM:(j + 1) * RM][keep])
                    bias.append(c[keep].to(dtype).log())
                cj = (~ab).nonzero().flatten()
                if cj.numel():
                    keys.append(k_tail[b, h, cj]); vals.append(v_tail[b, h, cj]); bias.append(c_tail[cj].to(dtype).log())
                if not keys:
                    continue
                Kc, Vc, bc = torch.cat(keys), torch.cat(vals), torch.cat(bias)
                s = qd[b, h, i * BLOCK:(i + 1) * BLOCK] @ Kc.transpose(0, 1) / math.sqrt(D) + bc
                row_ok = ok[i * BLOCK:(i + 1) * BLOCK]
                o_all[b, h, i * BLOCK:(i + 1) * BLOCK] = (torch.softmax(s, -1) @ Vc) * row_ok[:, None].to(dtype)
                lse = torch.logsumexp(s, -1)
                lse_all[b, h, i * BLOCK:(i + 1) * BLOCK] = torch.where(row_ok, lse, torch.full_like(lse, float("-inf")))
    return o_all, lse_all


# ------------------------------------------------------------------------------------------- split-KV plan
def split_plan(ptr, chunk, max_slots, min_len=0, rel_mean=0.0, tail_frac=0.0, resident=1, budget=-1):
    """Task plan of a CSR list ptr [B,H,NB+1] (reference: csrc/vsa/split.cu:1-22; its own Python statement of the same
    contract is tests/test_vsa2_split.py:60-87). Returns (tasks [T,4], merges [M,4], info [8]) as int lists.

    A row of n edges is eligible when n >= max(chunk + 1, min_len, ceil(tail_frac * W / resident),
    ceil(rel_mean * edges of its (b, h) / NB)); eligible rows have ceil(n / chunk) chunks; nothing splits when more
    than `budget` rows are eligible; a row splits while the running chunk count of the eligible rows (whether they
    split or not) stays <= max_slots. Split chunks first (slot = task index), then one direct task per other row."""
    import numpy as np
    p = ptr.reshape(-1, ptr.shape[-1]).cpu().numpy().astype(np.int64)
    BH, nb = p.shape[0], p.shape[1] - 1
    W = int(p[-1, -1] - p[0, 0])
    gthr = max(chunk + 1, min_len)
    if tail_frac > 0:
        gthr = max(gthr, math.ceil(tail_frac * W / resident))
    budget = 2 ** 31 - 1 if budget < 0 else budget
    n = (p[:, 1:] - p[:, :-1]).reshape(-1)
    beg = p[:, :-1].reshape(-1)
    thr = np.full(BH, gthr, dtype=np.int64)
    if rel_mean > 0:
        thr = np.maximum(thr, np.ceil(rel_mean * (p[:, nb] - p[:, 0]) / nb).astype(np.int64))
    elig = n >= np.repeat(thr, nb)
    c = np.where(elig, -(-n // chunk), 0)
    E = int(elig.sum())
    split = (E <= budget) & (c > 0) & (np.cumsum(c) <= max_slots)
    tasks, merges = [], []
    slot = 0
    for r in np.nonzero(split)[0]:
        cr, nr, br = int(c[r]), int(n[r]), int(beg[r])
        merges.append([int(r), slot, cr, 0])
        tasks += [[int(r), br + j * nr // cr, br + (j + 1) * nr // cr, slot + j] for j in range(cr)]
        slot += cr
    t_split = slot
    tasks += [[int(r), int(beg[r]), int(beg[r] + n[r]), -1] for r in np.nonzero(~split)[0]]
    return tasks, merges, [len(tasks), len(merges), t_split, BH * nb, E, int(E <= budget), gthr, W]


# ------------------------------------------------------------------------------------------- original VSA
def vsa_block_scores(q, k, blk_cnt):
    """Whole-block router scores of the original VSA in the token dtype (reference: tests/vsa_reference.py:147-160, the
    kernel's rounding csrc/vsa/vsa2_kernels.h:243-253): block means rounded to the dtype, fp32 dot rounded once, times the
    fp32 reciprocal of sqrt(D), rounded again."""
    dt = q.dtype
    qc = block_means(q.float(), blk_cnt, dt)
    kc = block_means(k.float(), blk_cnt, dt)
    once = (qc @ kc.transpose(-1, -2)).to(dt).float()
    inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(q.shape[-1]) ** 0.5, dtype=torch.float32)
    return (once * inv).to(dt)


def row_topk_mask(scores, topk):
    """Exactly min(topk, NB) kv blocks per row: score descending, ties to the smaller kv index, -0 == +0
    (reference: tests/vsa_reference.py:163-168)."""
    n = max(0, min(int(topk), scores.shape[-1]))
    order = torch.sort(scores.float() + 0.0, dim=-1, descending=True, stable=True).indices[..., :n]
    return torch.zeros(scores.shape, dtype=torch.bool).scatter_(-1, order, True)


def vsa_output(q, k, v, weight, blk_cnt, mask):
    """Original VSA on a frozen mask: O = O_fine + W * O_coarse[block], W a full [B,H,L,D] weight or None (1). The same
    arithmetic as `vsa2_output` with an identity gate per element (reference: tests/vsa_reference.py:171-193 states it with
    the original's extra rounding points; its own test tests/test_vsa.py:87-107 shows both agree without rounding)."""
    return vsa2_output(q, k, v, weight, blk_cnt, mask, gate_act="identity")
