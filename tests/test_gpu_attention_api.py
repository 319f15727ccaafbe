"""The attention processor on a GPU, pinned the way the reference pins its own (tests/test_attention.py:103-149): full
density equals dense attention, CFG branches share the selection, a sparse step equals the one-softmax formula over
exact tokens + block means + representatives, and a far-off offset goes through the fallback."""
import math

import pytest
import torch

from oracle import echosparse_ref as R

pytestmark = pytest.mark.gpu
L, H, D = 4152, 2, 128          # 65 kv blocks (the last has 56 tokens), 33 query tiles (the last has 56 rows)


def steps(n, seed=0):
    """Inputs of n consecutive denoising steps: a fixed base plus a small change per step, with local structure."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    pos = torch.arange(L, device="cuda", dtype=torch.float32)[:, None, None] / 300.0
    freq = torch.randn(1, H, D, device="cuda", generator=g)
    base = [torch.sin(pos * freq + torch.randn(1, H, D, device="cuda", generator=g)) * 3.0 for _ in range(3)]
    return [[(b + 0.05 * torch.randn(b.shape, device="cuda", generator=g)).to(torch.bfloat16)[None] for b in base]
            for _ in range(n)]


def rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def dense(q, k, v):
    return R.dense_attention(q[0], k[0], v[0])[0][None]


def make(**kw):
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    return EchoSparseAttention(dense_steps=2, dense_layers=(), **kw)


def run(attn, inputs, branches=1):
    return [attn(q, k, v, step, branch, layer=1) for step, (q, k, v) in enumerate(inputs) for branch in range(branches)]


def check_formula(out, qkv, st, buf):
    out = out[0].float()
    q, k, v = (x[0].float() for x in qkv)
    nb = buf.k_mean.shape[0]
    block_len = torch.full((nb,), 64.0, device="cuda")
    block_len[-1] = L - 64 * (nb - 1)
    for h in range(H):
        for t in (0, 7, 32):
            exact = st.blocks[t, h, :st.counts[t, h]].tolist()
            refined = [b for b in st.refine[t, h].tolist() if b < nb]
            means = sorted(set(range(nb)) - set(exact) - set(refined))
            rows = torch.arange(128 * t, min(128 * t + 128, L), 9, device="cuda")
            keys, vals, bias = [], [], []
            for b in exact:
                tok = torch.arange(64 * b, min(64 * b + 64, L), device="cuda")
                keys.append(k[tok, h]); vals.append(v[tok, h]); bias.append(torch.zeros(len(tok), device="cuda"))
            keys.append(buf.k_mean[means, h].float()); vals.append(buf.v_mean[means, h].float())
            bias.append(block_len[means].log())
            for b in refined:
                sl = slice(4 * b, 4 * b + 4)
                keys.append(buf.reps.k[h, sl].float()); vals.append(buf.reps.v[h, sl].float())
                bias.append(buf.reps.log_counts[h, sl] * math.log(2))
            logits = q[rows, h] @ torch.cat(keys).T * D ** -0.5 + torch.cat(bias)
            ref = torch.softmax(logits, -1) @ torch.cat(vals)
            assert rel_err(out[rows, h], ref) < 1e-2, (h, t)


def test_dense_attention_and_lse():
    from self_trainable_or_free_attn_b200.attention import dense_attention
    q, k, v = steps(1)[0]
    out, lse = dense_attention(q, k, v, return_lse=True)
    ref, lse2 = R.dense_attention(q[0], k[0], v[0])
    assert rel_err(out[0], ref) < 1e-2
    assert (lse[0].t() * R.LOG2E - lse2).abs().max() < 1e-4


def test_dense_steps_after_the_first_run_on_the_previous_lse_and_stay_exact():
    """The first step of a video runs online softmax; the dense steps that follow take the previous step's LSE as a fixed
    offset over every block. Both are exact attention, and the stored offset is the step's own log2 LSE."""
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    inputs = steps(4, seed=7)
    attn = EchoSparseAttention(density=0.1, dense_steps=5, dense_layers=())
    for step, (q, k, v) in enumerate(inputs):
        out = attn(q, k, v, step, 0, layer=1)
        ref, lse2 = R.dense_attention(q[0], k[0], v[0])
        assert rel_err(out[0], ref) < 1e-2, step
        br = attn._states.record(1).branches[0]
        assert br.seeded and (br.offset[:L] - lse2).abs().max() < 2e-3, step
    attn.reset()
    assert not attn._states.record(1).branches[0].seeded


def test_full_density_matches_dense():
    inputs = steps(4)
    outs = run(make(density=1.0), inputs)
    for (q, k, v), out in zip(inputs, outs):
        assert rel_err(out, dense(q, k, v)) < 1e-2


def test_cfg_branches_share_selection():
    inputs = steps(4)
    outs = run(make(density=1.0), inputs, branches=2)
    for i, (q, k, v) in enumerate(inputs):
        ref = dense(q, k, v)
        assert rel_err(outs[2 * i], ref) < 1e-2 and rel_err(outs[2 * i + 1], ref) < 1e-2


def test_sparse_step_matches_formula():
    inputs = steps(3)
    attn = make(density=0.1)
    run(attn, inputs[:2])
    out = attn(*inputs[2], 2, 0, layer=1)
    check_formula(out, inputs[2], attn._states[(0, 1)], attn._buffers)
    assert rel_err(out, dense(*inputs[2])) < 5e-2         # and it is a usable approximation of dense attention


def test_second_cfg_branch_matches_formula():
    cond, uncond = steps(3, seed=1), steps(3, seed=2)
    attn = make(density=0.1)
    for step in range(2):
        attn(*cond[step], step, 0, layer=1)
        attn(*uncond[step], step, 1, layer=1)
    attn(*cond[2], 2, 0, layer=1)
    st = attn._states[(0, 1)]
    first = (st.counts.clone(), st.blocks.clone(), st.refine.clone())
    out = attn(*uncond[2], 2, 1, layer=1)
    assert all(torch.equal(a, b) for a, b in zip(first, (st.counts, st.blocks, st.refine)))
    check_formula(out, uncond[2], st, attn._buffers)


def test_fallback_tiles():
    inputs = steps(4)
    attn = make(density=1.0)
    run(attn, inputs[:3])
    attn._states[(0, 1)].offset[:L] += 200.0
    q, k, v = inputs[3]
    out = attn(q, k, v, 3, 0, layer=1)
    assert int(attn._states[(0, 1)].flags.sum()) == 33 * H
    assert rel_err(out, dense(q, k, v)) < 1e-2


def test_many_sparse_steps_stay_close_to_dense_and_keep_state_finite():
    """Ten sparse steps in a row: offsets track the LSE, masses stay finite (padding rows of the last tile included)."""
    inputs = steps(12)
    attn = make(density=0.1)
    outs = run(attn, inputs)
    st = attn._states[(0, 1)]
    assert torch.isfinite(st.mass).all() and torch.isfinite(st.scale_exact).all() and torch.isfinite(st.scale_skip).all()
    assert (st.offset[L:] == 1e30).all()
    assert rel_err(outs[-1], dense(*inputs[-1])) < 5e-2
    assert int(st.flags.sum()) == 0


def test_short_sequences_run_dense_and_reset_forgets():
    attn = make(density=0.1)
    q = torch.randn(1, 1024, H, D, device="cuda").to(torch.bfloat16)
    assert rel_err(attn(q, q, q, 5, 0, layer=1), dense(q, q, q)) < 1e-2 and not attn._states
    inputs = steps(3)
    run(attn, inputs)
    assert attn._states[(0, 1)].ready
    attn.reset()
    assert not attn._states[(0, 1)].ready
    out = attn(*inputs[2], 2, 0, layer=1)                   # not ready: dense again
    assert rel_err(out, dense(*inputs[2])) < 1e-2


def test_compact_plan_state_matches_the_layer_state():
    """The compact state (offsets + bit-mask plans per layer, lists rebuilt every step; reference attention.py:272-330)
    goes through the same kernels with the same selections as the per-(branch, layer) state: identical outputs over
    several steps and both CFG branches, with 25 x less resident state."""
    inputs = steps(6, seed=4)
    a, b = make(density=0.2), make(density=0.2, state="compact")
    outs_a, outs_b = run(a, inputs, branches=2), run(b, inputs, branches=2)
    for i, (x, y) in enumerate(zip(outs_a, outs_b)):
        assert torch.equal(x, y), f"call {i}: compact state differs"
    st = b._states[1]
    assert sorted(st.offsets) == [0, 1] and len(st.plans) == 2 and st.pending == (1 - st.current[0], 6)
    resident = sum(t.numel() * t.element_size() for p in st.plans for t in p) + sum(t.numel() * 4 for t in st.offsets.values())
    la = a._states[(0, 1)]
    layer = 2 * sum(t.numel() * t.element_size() for t in (la.mass, *la.keeps, la.blocks, *la.offsets, la.skip_bits))
    assert resident * 3 < layer          # 3.1 x at this small shape (the offsets dominate), 25 x at 75,600 tokens and 40 heads
    # a sink block and a reset
    c = make(density=0.2, state="compact")
    d = make(density=0.2)
    for step, (q, k, v) in enumerate(inputs[:4]):
        assert torch.equal(c(q, k, v, step, 0, layer=1, sink=60), d(q, k, v, step, 0, layer=1, sink=60))
    c.reset()
    q, k, v = inputs[0]
    assert rel_err(c(q, k, v, 5, 0, layer=1), dense(q, k, v)) < 1e-2          # not ready: dense
