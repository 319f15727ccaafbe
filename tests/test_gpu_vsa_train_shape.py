"""VSA2 at the training shape (B = 1, H = 12, head dim 128, 32,768 tokens of a 16 x 32 x 64 grid = 512 blocks, top-k 32
= 16,384 selected pairs per head), forward and backward, against the sampled float32 oracle (oracle/vsa_sampled.py, pinned
on the CPU against the dense oracle and through it against the reference's tests/vsa_reference.py):

 * one whole head: O, fine LSE, dQ, dgate of all 512 query blocks and dK, dV of all 512 kv blocks;
 * the other heads: the longest, the shortest and the last query block and two random ones; the most and the least
   selected kv block and a random one;
 * on the even selection (exact global top-k of a local score) and on the skewed one where 10 % of the query blocks
   select 4 x more kv blocks, without split-KV scheduling, with the planner's automatic policy and with every list longer
   than a chunk split; split and unsplit runs must agree with each other as well;
 * the three-tier fine branch (64 tokens / 4 group means / 1 block mean per kv block) of one whole head against the
   closed-form tier oracle (pinned on the CPU against the dense tier oracle, which is pinned against the reference's
   vsa2_rep/reference.py).

Tolerances are the reference's (tests/test_vsa2.py:82-93): |error| <= 2e-2 (forward) or 4e-2 (gradients) of the largest
reference value; LSE 2e-2 absolute."""
import pytest
import torch

from oracle import vsa_ref as R
from oracle.vsa_sampled import SampledTiers, SampledVSA2, lists_from_csr

pytestmark = pytest.mark.gpu
DEV = "cuda"
GRID, HEADS, TOPK, NB = (16, 32, 64), 12, 32, 512


@pytest.fixture(scope="module")
def layer():
    from self_trainable_or_free_attn_b200.vsa import workloads
    q, k, v, gate, dout, lay = workloads.train_inputs(GRID, HEADS, device=DEV)
    assert q.shape == (1, HEADS, NB * 64, 128) and int(lay.blk_cnt.min()) == 64
    return q, k, v, gate, dout, lay.blk_cnt.to(DEV)


def _run(layer, sel, split):
    from self_trainable_or_free_attn_b200 import _native, vsa
    q, k, v, gate, dout, cnt = layer
    leaves = [x.detach().clone().requires_grad_(True) for x in (q, k, v, gate)]
    o = vsa.vsa2_attention(*leaves, cnt, R=16, selection=sel, split_kv=split)
    grads = torch.autograd.grad(o, leaves, dout)
    assert _native.device_status() == 0
    return [o.detach()] + [g.detach() for g in grads]


def _fine_lse(layer, sel):
    from self_trainable_or_free_attn_b200.vsa import ops
    q, k, v, _, _, cnt = layer
    return ops.attn_fwd(q, k, v, sel.q2k_ptr, sel.q2k_idx, cnt)[1]


def _oracle(layer, sel, h):
    q, k, v, gate, dout, cnt = (x.cpu() for x in layer)
    q2k = lists_from_csr(sel.q2k_ptr[0, h].cpu(), sel.q2k_idx.cpu(), NB)
    k2q = lists_from_csr(sel.k2q_ptr[0, h].cpu(), sel.k2q_idx.cpu(), NB)
    return SampledVSA2(q[0, h], k[0, h], v[0, h], gate[0, h], dout[0, h], cnt, q2k, k2q), q2k, k2q


def _check(got, lse, layer, sel, heads_whole=(0,), seed=0):
    o, dq, dk, dv, dgate = (x.float().cpu() for x in got)
    lse = lse.float().cpu()
    g = torch.Generator().manual_seed(seed)
    worst = dict(o=0.0, lse=0.0, dq=0.0, dk=0.0, dv=0.0, dgate=0.0)
    scale = dict(o=0.0, dq=0.0, dk=0.0, dv=0.0, dgate=0.0)
    for h in range(HEADS):
        ora, q2k, k2q = _oracle(layer, sel, h)
        row_len = torch.tensor([len(x) for x in q2k])
        col_len = torch.tensor([len(x) for x in k2q])
        if h in heads_whole:
            q_blocks, kv_blocks = range(NB), range(NB)
        else:
            nz = (row_len > 0).nonzero().flatten()
            q_blocks = sorted({int(row_len.argmax()), int(nz[row_len[nz].argmin()]), NB - 1,
                               *torch.randint(0, NB, (2,), generator=g).tolist()})
            kv_blocks = sorted({int(col_len.argmax()), int(col_len.argmin()), int(torch.randint(0, NB, (1,), generator=g))})
        for i in q_blocks:
            sl = slice(64 * i, 64 * (i + 1))
            o_r, lse_r, dq_r, dg_r = ora.query_block(i)
            for name, a, b in (("o", o[0, h, sl], o_r), ("dq", dq[0, h, sl], dq_r), ("dgate", dgate[0, h, sl], dg_r)):
                worst[name] = max(worst[name], float((a - b).abs().max()))
                scale[name] = max(scale[name], float(b.abs().max()))
            both_inf = torch.isinf(lse[0, h, sl]) & torch.isinf(lse_r)
            worst["lse"] = max(worst["lse"], float(torch.where(both_inf, torch.zeros(64), lse[0, h, sl] - lse_r).abs().max()))
        for j in kv_blocks:
            sl = slice(64 * j, 64 * (j + 1))
            dk_r, dv_r = ora.kv_block(j)
            for name, a, b in (("dk", dk[0, h, sl], dk_r), ("dv", dv[0, h, sl], dv_r)):
                worst[name] = max(worst[name], float((a - b).abs().max()))
                scale[name] = max(scale[name], float(b.abs().max()))
    assert worst["o"] <= 2e-2 * scale["o"], (worst, scale)
    assert worst["lse"] <= 2e-2, worst
    for name in ("dq", "dk", "dv", "dgate"):
        assert worst[name] <= 4e-2 * scale[name], (name, worst, scale)


def _splits():
    from self_trainable_or_free_attn_b200 import vsa
    return {"none": None, "auto": vsa.SplitKV.auto(), "manual": vsa.SplitKV(chunk=64)}


@pytest.mark.parametrize("case", ["uniform", "tenth_x4"])
def test_operator_matches_the_sampled_oracle_with_and_without_split_kv(layer, case):
    from self_trainable_or_free_attn_b200.vsa import workloads
    sel, nb = workloads.selection(case, GRID, HEADS, TOPK, DEV)
    rows = sel.row_counts().reshape(HEADS, NB)
    assert nb == NB and bool((rows.sum(1) == NB * TOPK).all())
    if case == "tenth_x4":
        assert int((rows == 4 * TOPK).sum()) == HEADS * 51 and int(rows.max()) == 4 * TOPK
    base = _run(layer, sel, None)
    _check(base, _fine_lse(layer, sel), layer, sel, heads_whole=(0,) if case == "uniform" else (5,))
    for name, split in _splits().items():
        if split is None:
            continue
        got = _run(layer, sel, split)
        for what, a, b in zip(("o", "dq", "dk", "dv", "dgate"), got, base):
            err = float((a.float() - b.float()).abs().max())
            assert err <= 1e-2 * float(b.float().abs().max()), (case, name, what, err)
        if name == "manual":
            _check(got, _fine_lse(layer, sel), layer, sel, heads_whole=(), seed=1)


@pytest.mark.parametrize("case", ["hot_kv", "straggler"])
def test_hot_kv_blocks_and_a_straggler_row_under_the_automatic_split(layer, case):
    """NB / 16 kv blocks that every query block selects (long kv->q lists: the backward's kv pass) and one query block that
    selects every kv block (one long q->kv list): the automatic split policy against the unsplit kernels and, on sampled
    blocks of every head (the longest lists among them), against the sampled oracle."""
    from self_trainable_or_free_attn_b200 import vsa
    from self_trainable_or_free_attn_b200.vsa import workloads
    sel, nb = workloads.selection(case, GRID, HEADS, TOPK, DEV)
    rows = sel.row_counts().reshape(HEADS, NB)
    assert nb == NB and bool((rows.sum(1) == NB * TOPK).all())
    if case == "straggler":
        assert bool((rows[:, NB - 1] == NB).all())
    base = _run(layer, sel, None)
    got = _run(layer, sel, vsa.SplitKV.auto())
    for what, a, b in zip(("o", "dq", "dk", "dv", "dgate"), got, base):
        err = float((a.float() - b.float()).abs().max())
        assert err <= 1e-2 * float(b.float().abs().max()), (case, what, err)
    _check(got, _fine_lse(layer, sel), layer, sel, heads_whole=(), seed=2)


def test_three_tier_fine_branch_matches_the_dense_tier_oracle_at_512_blocks(layer):
    """Tier A = the even selection (32 / 512 of the pairs), tier B the next 20 % of the same score, tier C the rest: two
    heads on the GPU, every query block and every kv block of head 1 against the closed-form tier oracle."""
    from self_trainable_or_free_attn_b200 import _native
    from self_trainable_or_free_attn_b200.vsa import tiers, workloads
    q, k, v, _, dout, cnt = (x[:, :2].contiguous() if x.dim() > 1 else x for x in layer)
    scores = workloads.local_scores(GRID, 2)
    flat = scores.reshape(2, NB * NB)
    order = torch.sort(flat, dim=1, descending=True, stable=True).indices
    na = NB * TOPK
    nab = na + int(round(0.20 * NB * NB))
    tier_a = torch.zeros(2, NB * NB, dtype=torch.bool).scatter_(1, order[:, :na], True).reshape(1, 2, NB, NB)
    tier_ab = torch.zeros(2, NB * NB, dtype=torch.bool).scatter_(1, order[:, :nab], True).reshape(1, 2, NB, NB)
    tsel = tiers.selection_from_masks(tier_a.to(DEV), tier_ab.to(DEV))
    leaves = [x.detach().clone().requires_grad_(True) for x in (q, k, v)]
    o, lse = tiers.rep_fine_attention(*leaves, cnt, tsel, mid_reps=4)
    grads = torch.autograd.grad(o, leaves, dout)
    assert _native.device_status() == 0
    h = 1
    ora = SampledTiers(q[0, h].cpu(), k[0, h].cpu(), v[0, h].cpu(), dout[0, h].cpu(), cnt.cpu(), tier_a[0, h], tier_ab[0, h],
                       mid_reps=4)
    o, lse = o.float().cpu(), lse.float().cpu()
    dq, dk, dv = (x.float().cpu() for x in grads)
    worst, scale = dict(o=0.0, lse=0.0, dq=0.0), dict(o=0.0, dq=0.0)
    for i in range(NB):
        sl = slice(64 * i, 64 * (i + 1))
        o_r, lse_r, dq_r = ora.query_block(i)
        worst["o"] = max(worst["o"], float((o[0, h, sl] - o_r).abs().max()))
        worst["lse"] = max(worst["lse"], float((lse[0, h, sl] - lse_r).abs().max()))
        worst["dq"] = max(worst["dq"], float((dq[0, h, sl] - dq_r).abs().max()))
        scale["o"], scale["dq"] = max(scale["o"], float(o_r.abs().max())), max(scale["dq"], float(dq_r.abs().max()))
    assert worst["o"] <= 2e-2 * scale["o"] and worst["lse"] <= 2e-2 and worst["dq"] <= 4e-2 * scale["dq"], (worst, scale)
    dk_r, dv_r = ora.kv_gradients()
    assert float((dk[0, h] - dk_r).abs().max()) <= 4e-2 * float(dk_r.abs().max())
    assert float((dv[0, h] - dv_r).abs().max()) <= 4e-2 * float(dv_r.abs().max())
