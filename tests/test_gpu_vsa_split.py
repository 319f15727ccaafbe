"""Split-KV scheduling of VSA2 on the GPU: the task plan bit for bit against the reference's Python planner (golden) and the
CPU restatement; the split forward / backward against the unsplit kernels and the oracle. Cases follow the reference's
tests/test_vsa2_split.py (skewed masks, chunk sizes, slot caps, automatic policy)."""
import os

import numpy as np
import pytest
import torch

from golden_util import POLICY, SPLIT_CASES, split_mask
from oracle import vsa_ref as R
from test_gpu_vsa import close, make, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda"
S = np.load(os.path.join(os.path.dirname(__file__), "golden", "vsa2_split.npz"))


def vsa():
    from self_trainable_or_free_attn_b200 import vsa as V
    return V


@pytest.mark.parametrize("name", sorted(SPLIT_CASES))
def test_plan_matches_golden_and_oracle(name):
    from self_trainable_or_free_attn_b200.vsa import ops
    kind, nb, heads, chunk, slots, policy = SPLIT_CASES[name]
    mask = split_mask(kind, heads, nb)
    sel = ops.mask_to_selection(mask.to(DEV))
    for d, ptr, idx in (("q2k", sel.q2k_ptr, sel.q2k_idx), ("k2q", sel.k2q_ptr, sel.k2q_idx)):
        cap = min(slots, ops.split_slots(idx.numel(), chunk, 1, 1 << 40))
        tasks, merges, info = ops.split_plan(ptr, chunk, cap, **policy)
        t_ref, m_ref, i_ref = R.split_plan(ptr, chunk, cap, **policy)
        info = info.cpu().tolist()
        assert info == i_ref, (name, d)
        assert tasks[: info[0]].cpu().tolist() == t_ref and merges[: info[1]].cpu().tolist() == m_ref, (name, d)
        assert tasks.shape[0] == heads * nb + cap


@pytest.mark.parametrize("name", ["random_c2", "hotq_c1_cap3", "policy_hotq", "policy_cap40", "full_c3"])
def test_plan_equals_golden_at_the_golden_cap(name):
    """The planner called exactly as the golden run was (same max_slots), compared with the stored plan."""
    from self_trainable_or_free_attn_b200.vsa import ops
    kind, nb, heads, chunk, slots, policy = SPLIT_CASES[name]
    sel = ops.mask_to_selection(split_mask(kind, heads, nb).to(DEV))
    for d, ptr in (("q2k", sel.q2k_ptr), ("k2q", sel.k2q_ptr)):
        cap = min(slots, 4096)                     # a cap far above what any of these plans uses behaves like 10**6
        tasks, merges, info = ops.split_plan(ptr, chunk, cap, **policy)
        info = info.cpu().tolist()
        assert info == S[f"{name}_{d}_info"].tolist(), (name, d)
        assert tasks[: info[0]].cpu().tolist() == S[f"{name}_{d}_tasks"].tolist()
        assert merges[: info[1]].cpu().tolist() == S[f"{name}_{d}_merges"].tolist()


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("mask_kind", ["random", "full", "hotq", "hotkv", "hotqkv"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("chunk", [1, 3])
def test_split_fine_frozen(D, mask_kind, dtype, chunk):
    V = vsa()
    B, H, nb = 1, 2, 13
    q, k, v, _, cnt, dout = make(B, H, nb, D, dtype, "mixed", seed=D + chunk)
    mask = split_mask(mask_kind, H, nb)
    sel = V.mask_to_selection(mask.to(DEV))
    res = []
    for split in (None, V.SplitKV(chunk=chunk)):
        leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)]
        of, lse = V.fine_block_sparse_attention(*leaves, cnt.to(DEV), sel, split_kv=split)
        res.append([of, lse] + list(torch.autograd.grad(of, leaves, dout.to(DEV))))
    lf = [x.float().clone().requires_grad_(True) for x in (q, k, v)]
    of_r, lse_r = R.fine_attention(*lf, cnt, mask)
    g_r = torch.autograd.grad(of_r, lf, dout.float())
    rt = 2e-2 if dtype == torch.bfloat16 else 1e-2
    fin = torch.isfinite(lse_r)
    for of, lse, dq, dk, dv in res:
        close("o", of, of_r, rt)
        assert torch.equal(torch.isfinite(lse.cpu()), fin)
        close("lse", torch.where(fin, lse.cpu(), torch.zeros(())), torch.where(fin, lse_r, torch.zeros(())), 1e-2)
        for name, got, exp in zip(("dq", "dk", "dv"), (dq, dk, dv), g_r):
            close(name, got, exp, 2 * rt)
        pad = ~R.token_valid(cnt, nb * 64)
        for t in (of, dq, dk, dv):
            assert (t[:, :, pad.to(DEV)] == 0).all()
    # split and unsplit agree far more closely than either does with the fp32 oracle
    for a, b in zip(res[0], res[1]):
        fa, fb = a.float(), b.float()
        ok = torch.isfinite(fa)
        assert torch.equal(ok, torch.isfinite(fb))
        assert (fa[ok] - fb[ok]).abs().max() <= 2e-2 * fa[ok].abs().max().clamp(min=1e-6)


@pytest.mark.parametrize("gate_mode", ["token", "none"])
@pytest.mark.parametrize("cap_bytes", [0, 3 * 64 * 129 * 4, 1 << 30])
def test_split_full_frozen_and_scratch_cap(gate_mode, cap_bytes):
    """The full operator with split lists; a scratch cap of zero or a few slots splits nothing or a prefix of the rows."""
    V = vsa()
    B, H, nb, D = 2, 2, 12, 128
    q, k, v, gate, cnt, dout = make(B, H, nb, D, torch.bfloat16, "tail", seed=31, gate_mode=gate_mode)
    mask = torch.cat([split_mask("hotqkv", H, nb), split_mask("hotq", H, nb)])
    sel = V.mask_to_selection(mask.to(DEV))
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)] + \
             ([gate.to(DEV).clone().requires_grad_(True)] if gate is not None else [])
    o = V.vsa2_attention(leaves[0], leaves[1], leaves[2], leaves[3] if gate is not None else None, cnt.to(DEV),
                         selection=sel, split_kv=V.SplitKV(chunk=2, max_scratch_bytes=cap_bytes))
    grads = torch.autograd.grad(o, leaves, dout.to(DEV))
    lf = [x.float().clone().requires_grad_(True) for x in (q, k, v)] + \
         ([gate.float().clone().requires_grad_(True)] if gate is not None else [])
    o_r = R.vsa2_output(lf[0], lf[1], lf[2], lf[3] if gate is not None else None, cnt, mask)
    grads_r = torch.autograd.grad(o_r, lf, dout.float())
    close("o", o, o_r, 2e-2)
    for name, g_, gr in zip(["dq", "dk", "dv", "dgate"], grads, grads_r):
        close(name, g_, gr, 4e-2)


def test_split_auto_policy_and_determinism():
    V = vsa()
    from self_trainable_or_free_attn_b200.vsa import ops
    B, H, nb, D = 1, 3, 24, 128
    q, k, v, gate, cnt, dout = make(B, H, nb, D, torch.bfloat16, "tail", seed=41)
    mask = split_mask("hotq", H, nb, seed=9)
    mask |= torch.eye(nb, dtype=torch.bool)
    sel = V.mask_to_selection(mask.to(DEV))
    auto = V.SplitKV.auto(chunk=2, policy=V.SplitPolicy(resident_ctas=4, fwd_waves=4, bwd_waves=4))
    d = V.describe_split(q.to(DEV), sel, auto)
    assert d["fwd"]["info"]["split_rows"] > 0 and d["bwd_kv"]["info"]["split_rows"] == 0, d
    runs = []
    for rep in range(2):
        leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v, gate)]
        o = V.vsa2_attention(*leaves, cnt.to(DEV), selection=sel, split_kv=auto)
        runs.append([o] + list(torch.autograd.grad(o, leaves, dout.to(DEV))))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    lf = [x.float().clone().requires_grad_(True) for x in (q, k, v, gate)]
    o_r = R.vsa2_output(*lf, cnt, mask)
    close("o", runs[0][0], o_r, 2e-2)
    for got, exp in zip(runs[0][1:], torch.autograd.grad(o_r, lf, dout.float())):
        close("grad", got, exp, 4e-2)
    # the string form and option checks
    o2 = V.vsa2_attention(q.to(DEV), k.to(DEV), v.to(DEV), gate.to(DEV), cnt.to(DEV), selection=sel, split_kv="auto")
    close("auto string", o2, o_r, 2e-2)
    with pytest.raises(TypeError):
        V.vsa2_attention(q.to(DEV), k.to(DEV), v.to(DEV), None, cnt.to(DEV), selection=sel, split_kv=3)
    with pytest.raises(ValueError):
        V.SplitKV(chunk=0)
    with pytest.raises(ValueError):
        V.SplitPolicy(rel_mean=-1.0)
