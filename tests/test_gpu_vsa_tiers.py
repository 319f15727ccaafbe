"""The 64 / RM / 1 tier kernels through the C ABI against the golden vectors of the reference's own torch reference
(experiments/vsa2_representative/vsa2_rep/reference.py -> tests/golden/vsa2.npz) and the CPU restatement with autograd
gradients (oracle/vsa_ref.py). Cases follow the reference's experiments/vsa2_representative/tests/test_gpu.py: hand-made
tier masks with rows without tier A and all-tier-C rows, ragged block counts (empty groups), phase subsets, tier A alone
equal to the plain VSA2 fine kernel, the two-budget router."""
import os

import numpy as np
import pytest
import torch

from golden_util import vsa_case, vsa_tiers
from oracle import vsa_ref as R
from test_gpu_vsa import close, make

pytestmark = pytest.mark.gpu
DEV = "cuda"
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "vsa2.npz"))


def mods():
    from self_trainable_or_free_attn_b200 import vsa as V
    from self_trainable_or_free_attn_b200.vsa import tiers as T
    return V, T


def test_golden_three_tiers():
    V, T = mods()
    q, k, v, _, cnt, _ = vsa_case("tiers")
    a, ab = vsa_tiers(cnt.numel())
    sel = T.selection_from_masks(a.to(DEV), ab.to(DEV))
    o, lse = T.rep_fine_attention(q.to(DEV), k.to(DEV), v.to(DEV), cnt.to(DEV), sel, mid_reps=4)
    o_ref, lse_ref = torch.from_numpy(G["tiers_o"].astype(np.float32)), torch.from_numpy(G["tiers_lse"])
    close("tiers_o", o, o_ref, 2e-2)
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert (lse.cpu()[fin] - lse_ref[fin]).abs().max() < 1e-2


def tier_masks(B, H, nb, seed):
    rs = np.random.RandomState(seed)
    u = torch.from_numpy(rs.random_sample((B, H, nb, nb)))
    a, ab = u < 0.25, u < 0.6
    a[:, :, 0] = False
    a[:, :, 1] = False
    ab[:, :, 1] = False
    if nb > 4:
        ab[:, :, 3] = True          # no tier C in this row
    return a, ab


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("mid_reps", [2, 4, 16])
@pytest.mark.parametrize("cnt_kind", ["full", "mixed"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tiers_forward_backward(D, mid_reps, cnt_kind, dtype):
    V, T = mods()
    B, H, nb = 1, 2, 9
    q, k, v, _, cnt, dout = make(B, H, nb, D, dtype, cnt_kind, seed=D + mid_reps)
    a, ab = tier_masks(B, H, nb, 3)
    sel = T.selection_from_masks(a.to(DEV), ab.to(DEV))
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)]
    o, lse = T.rep_fine_attention(*leaves, cnt.to(DEV), sel, mid_reps=mid_reps)
    g = torch.autograd.grad(o, leaves, dout.to(DEV))
    lf = [x.double().clone().requires_grad_(True) for x in (q, k, v)]
    o_r, lse_r = oracle_subset(lf, cnt, a, ab & ~a, ~(a | ab), mid_reps=mid_reps, dtype=dtype)
    g_r = torch.autograd.grad(o_r, lf, dout.double())
    rt = 2e-2 if dtype == torch.bfloat16 else 1e-2
    close("o", o, o_r, rt)
    fin = torch.isfinite(lse_r)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    close("lse", torch.where(fin, lse.cpu().double(), torch.zeros((), dtype=torch.float64)),
          torch.where(fin, lse_r, torch.zeros((), dtype=torch.float64)), 1e-2)
    for name, got, exp in zip(("dq", "dk", "dv"), g, g_r):
        close(name, got, exp, 2 * rt)
    pad = ~R.token_valid(cnt, nb * 64)
    if pad.any():
        for t in (o, g[0], g[1], g[2]):
            assert (t[:, :, pad.to(DEV)] == 0).all()


@pytest.mark.parametrize("phases", [1, 2, 4, 3, 6])
def test_phase_subsets(phases):
    V, T = mods()
    B, H, nb, D = 1, 2, 8, 128
    q, k, v, _, cnt, dout = make(B, H, nb, D, torch.bfloat16, "mixed", seed=50 + phases)
    a, ab = tier_masks(B, H, nb, 4)
    sel = T.selection_from_masks(a.to(DEV), ab.to(DEV))
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)]
    o, lse = T.rep_fine_attention(*leaves, cnt.to(DEV), sel, mid_reps=4, phases=phases)
    g = torch.autograd.grad(o, leaves, dout.to(DEV))
    z = torch.zeros_like(a)
    ta = a if phases & 1 else z
    tb = (ab & ~a) if phases & 2 else z
    tc = ~(a | ab) if phases & 4 else z
    # the oracle takes (tier A, tier A or B) and treats the rest as tier C: restrict it by masking the missing tiers' columns
    lf = [x.double().clone().requires_grad_(True) for x in (q, k, v)]
    o_r, lse_r = oracle_subset(lf, cnt, ta, tb, tc)
    g_r = torch.autograd.grad(o_r, lf, dout.double())
    close("o", o, o_r, 2e-2)
    assert torch.equal(torch.isfinite(lse.cpu()), torch.isfinite(lse_r))
    for name, got, exp in zip(("dq", "dk", "dv"), g, g_r):
        close(name, got, exp, 4e-2)
    if phases == 1:
        # tier A alone is the plain fine kernel, bit for bit
        o2, lse2 = V.fine_block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), cnt.to(DEV), V.mask_to_selection(a.to(DEV)))
        assert torch.equal(o2, o) and torch.equal(lse2, lse)


def oracle_subset(leaves, cnt, ta, tb, tc, mid_reps=4, dtype=torch.bfloat16):
    """Three-tier oracle with explicit masks of every tier (a pair may be in no tier)."""
    import math
    q, k, v = leaves
    B, H, L, D = q.shape
    nb = L // 64
    RM = mid_reps
    k_mid, v_mid, c_mid, k_tail, v_tail, c_tail = R.tier_tables(k, v, cnt, RM, None)
    rnd = lambda x: x + (x.to(dtype).double() - x).detach()
    k_mid, v_mid, k_tail, v_tail = rnd(k_mid), rnd(v_mid), rnd(k_tail), rnd(v_tail)
    ok = R.token_valid(cnt, L)
    o = torch.zeros(B, H, L, D, dtype=torch.float64)
    lse = torch.full((B, H, L), float("-inf"), dtype=torch.float64)
    for b in range(B):
        for h in range(H):
            for i in range(nb):
                keys, vals, bias = [], [], []
                for j in ta[b, h, i].nonzero().flatten().tolist():
                    n = int(cnt[j])
                    keys.append(k[b, h, j * 64:j * 64 + n]); vals.append(v[b, h, j * 64:j * 64 + n]); bias.append(torch.zeros(n, dtype=torch.float64))
                for j in tb[b, h, i].nonzero().flatten().tolist():
                    c = c_mid[j * RM:(j + 1) * RM]
                    keep = c > 0
                    keys.append(k_mid[b, h, j * RM:(j + 1) * RM][keep]); vals.append(v_mid[b, h, j * RM:(j + 1) * RM][keep])
                    bias.append(c[keep].double().log())
                cj = tc[b, h, i].nonzero().flatten()
                if cj.numel():
                    keys.append(k_tail[b, h, cj]); vals.append(v_tail[b, h, cj]); bias.append(c_tail[cj].double().log())
                if not keys:
                    continue
                Kc, Vc, bc = torch.cat(keys), torch.cat(vals), torch.cat(bias)
                s = q[b, h, i * 64:(i + 1) * 64] @ Kc.t() / math.sqrt(D) + bc
                rok = ok[i * 64:(i + 1) * 64]
                o[b, h, i * 64:(i + 1) * 64] = (torch.softmax(s, -1) @ Vc) * rok[:, None].double()
                l = torch.logsumexp(s, -1)
                lse[b, h, i * 64:(i + 1) * 64] = torch.where(rok, l, torch.full_like(l, float("-inf")))
    return o, lse


def test_route_tiers():
    V, T = mods()
    B, H, nb, D = 1, 3, 20, 128
    q, k, v, _, cnt, dout = make(B, H, nb, D, torch.bfloat16, "tail", seed=60)
    tiers = T.RepTiers(frac_full=0.1, frac_mid=0.25, mid_reps=4)
    sel = T.route_tiers(q.to(DEV), k.to(DEV), cnt.to(DEV), tiers, R=16)
    ba, bab = tiers.budgets(nb)
    a, b, c = (m.cpu() for m in sel.tier_masks(nb))
    assert a.reshape(B, H, -1).sum(-1).eq(ba).all() and (a | b).reshape(B, H, -1).sum(-1).eq(bab).all()
    assert not (a & b).any() and (a | b | c).all()
    from self_trainable_or_free_attn_b200.vsa import ops
    assert torch.equal(ops.Selection(sel.q2k_ptr, sel.q2k_idx, sel.k2q_ptr, sel.k2q_idx).to_mask(nb).cpu(), a)
    # the same scores through the oracle's exact top-k at both budgets
    S = ops.router_scores(*ops.pool_fwd(q.to(DEV), k.to(DEV), k.to(DEV), cnt.to(DEV), 16)[:2], cnt.to(DEV), 16, 1).cpu()
    assert torch.equal(R.global_topk_mask(S, ba), a) and torch.equal(R.global_topk_mask(S, bab), a | b)
    # and the routed selection through the operator
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)]
    o, lse = T.rep_fine_attention(*leaves, cnt.to(DEV), sel)
    g = torch.autograd.grad(o, leaves, dout.to(DEV))
    lf = [x.double().clone().requires_grad_(True) for x in (q, k, v)]
    o_r, _ = oracle_subset(lf, cnt, a, b, c)
    close("o", o, o_r, 2e-2)
    for got, exp in zip(g, torch.autograd.grad(o_r, lf, dout.double())):
        close("grad", got, exp, 4e-2)
    with pytest.raises(ValueError):
        T.RepTiers(frac_full=0.9, frac_mid=0.5)
    with pytest.raises(ValueError):
        T.rep_fine_attention(q.to(DEV), k.to(DEV), v.to(DEV), cnt.to(DEV), sel, mid_reps=3)
