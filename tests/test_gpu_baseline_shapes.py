"""Parity with the oracle at the token counts of the stated configurations: Wan2.1-1.3B 480p (32,760 tokens, 12 heads, two
CFG branches), Wan2.1-14B 720p (75,600 tokens, 40 heads, with tiles pushed into the online-softmax fallback) and HunyuanVideo
720p (118,800 video + 256 text tokens, the text blocks as a sink).

The oracle cannot run a whole head of these sizes in seconds, so every test runs the whole step on the GPU for a few heads
(dense pass -> every block at the fixed offset -> selection -> block means -> representatives -> fused sparse step ->
fallback of flagged tiles -> estimates) and then checks, with the kernels' OWN intermediate tables as the oracle's inputs:

 * whole heads, bit for bit: the selection (keep mask, lists, skip bit mask, refine list) the oracle makes from the
   kernel's mass map and scales; the plan round trip;
 * whole heads, float: block means, the query metric and probes, the estimates and scales;
 * sampled (tile, head) pairs spread over the sequence (first, last ragged tile, tiles next to the sink, injected
   fallback tiles): the dense LSE, the full step's LSE and block masses, the fused sparse step's output / LSE / flag /
   block masses, the fallback recomputation and compensation, and the representatives of the blocks those tiles refine.

Tolerances as everywhere: outputs relative L2 <= 1e-2 and max-abs <= 3e-2 (or one bf16 step of the largest value);
LSE and float32 tables <= 1e-4; integer results identical."""
import math

import pytest
import torch

from oracle import echosparse_ref as R
from golden_util import rel_l2
from test_gpu_kernels import _outputs, _same_selection, _select

pytestmark = pytest.mark.gpu
DEV = "cuda"
CONFIG_IDS = {"wan_1_3b_480p": 1, "wan_14b_720p": 2, "hunyuan_720p": 3}
ITERS = 6


@pytest.fixture(scope="module")
def K():
    from self_trainable_or_free_attn_b200 import _native, backends
    mod = backends.kernels(backends.resolve("auto", DEV))
    yield mod
    assert _native.device_status() == 0, "a bounded wait inside a kernel gave up"


def _workload(name):
    from self_trainable_or_free_attn_b200 import synthetic
    grid, heads, branches, density, text = synthetic.WORKLOADS[name]
    L = synthetic.grid_tokens(grid) + text
    sink = synthetic.grid_tokens(grid) // 64 if text else 1 << 30
    return synthetic, grid, heads, branches, density, text, L, sink


def gpu_step(K, name, heads, branch, selection=None, inject=()):
    """The whole schedule of one (branch, layer) on the GPU through the kernel-set module, every intermediate kept.
    `selection`: lists of another branch to reuse (the later CFG branches share branch 0's). `inject`: (tile, head index)
    pairs whose Q rows are scaled by 3 in the sparse step, which pushes them through the fallback."""
    synthetic, grid, _, _, density, text, L, sink = _workload(name)
    cid = CONFIG_IDS[name]
    H = len(heads)
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    s = dict(L=L, H=H, nq=nq, nb=nb, sink=sink, density=density)
    qp, kp, vp = (x[0].contiguous() for x in synthetic.branch_qkv(grid, cid, branch, heads, DEV, text, prev=True))
    q, k, v = (x[0].contiguous() for x in synthetic.branch_qkv(grid, cid, branch, heads, DEV, text))
    for t, h in inject:
        q[128 * t:128 * (t + 1), h] *= 3.0
    all_counts = torch.full((nq, H), nb, device=DEV, dtype=torch.int32)
    all_blocks = torch.arange(nb, device=DEV, dtype=torch.int32).expand(nq, H, nb).contiguous()
    # dense pass on the previous step's inputs: the online-softmax kernel over every block
    out, offset0, flags = _outputs(L, H, qp)
    flags.fill_(1)
    K.exact_fallback(qp, kp, vp, out, all_counts, all_blocks, offset0, flags)
    # every block at that offset: exact LSE, first mass map, scales
    out_full, lse1, flags1 = _outputs(L, H, qp)
    mass = torch.zeros(H, nq, nb, device=DEV)
    K.block_attention(qp, kp, vp, out_full, all_counts, all_blocks, offset0, lse1, flags1, mass=mass)
    se, ss = torch.empty(H, nq, device=DEV), torch.empty(H, nq, device=DEV)
    K.full_step_scales(offset0, lse1, se, ss, L)
    s.update(qp=qp, kp=kp, q=q, k=k, v=v, offset0=offset0, lse1=lse1, mass_full=mass.clone(), se=se.clone(), ss=ss.clone(),
             flags_full=flags1.clone())
    top, refined = R.budget(density, nb)
    rw = -(-refined // 32) * 32
    s.update(top=top, refined=refined, rw=rw)
    if selection is None:
        ones = torch.ones(H, nq, nb, device=DEV, dtype=torch.uint8)
        selection = _select(K, mass, ones, se, ss, flags1, top, refined, L, H, rw, sink=sink)
    keep, counts, blocks, bits, refine = selection
    s["selection"] = selection
    km = torch.empty(nb, H, 128, device=DEV, dtype=torch.bfloat16)
    vm = torch.empty_like(km)
    K.block_means(k, v, km, vm)
    reps = K.Representatives(L, H, 128, DEV, iters=ITERS)
    reps.build(q, k, v)
    out2, lse2, flags2 = _outputs(L, H, q)
    mass2 = torch.zeros(H, nq, nb, device=DEV)
    K.sparse_attention(q, k, v, km, vm, bits, out2, counts, blocks, lse1, lse2, flags2, refine, reps.k, reps.v,
                       reps.log_counts, mass=mass2)
    s.update(km=km, vm=vm, reps=reps, out_fused=out2.clone(), lse_fused=lse2.clone(), flags=flags2.clone(), mass2=mass2.clone())
    K.exact_fallback(q, k, v, out2, counts, blocks, lse2, flags2)
    K.compensate_fallback(q, km, vm, keep, lse2, out2, flags2)
    mass3, se3, ss3 = mass2.clone(), torch.empty_like(se), torch.empty_like(ss)
    K.estimate_skipped(q, km, keep, lse1, lse2, mass3, se3, ss3)
    s.update(out=out2, lse2=lse2, mass3=mass3, se3=se3, ss3=ss3)
    return s


def _close(got, want):
    assert rel_l2(got, want) <= 1e-2
    # values reach 4 .. 8 at these shapes, where one bf16 step is 2^-5: a rounding tie may move a value by one step
    assert (got.float() - want.float()).abs().max() <= max(3e-2, float(want.float().abs().max()) * 2.0 ** -7)


def check_whole_heads(K, s, own_selection=True):
    L, H, nq, nb = s["L"], s["H"], s["nq"], s["nb"]
    keep, counts, blocks, bits, refine = s["selection"]
    if own_selection:
        want = R.select_blocks(s["mass_full"].cpu(), torch.ones(H, nq, nb, dtype=torch.uint8), s["se"].cpu(), s["ss"].cpu(),
                               s["flags_full"].cpu(), s["top"], s["refined"], L, s["rw"], sink=s["sink"])
        _same_selection(s["selection"], want)
        assert int(counts.min()) >= s["top"]
        if s["sink"] < nb:
            assert bool((keep[:, :, s["sink"]:] == 1).all()), "every tile keeps the sink blocks"
        # the plan (two bit masks per tile) gives the same lists back
        exact = torch.empty_like(bits)
        K.pack_plan(keep, exact)
        assert torch.equal(exact.cpu(), R.pack_plan(keep.cpu()))
        got = [torch.empty_like(keep), torch.empty_like(counts), torch.zeros_like(blocks), torch.empty_like(refine),
               torch.empty_like(counts), torch.zeros_like(blocks), torch.empty_like(counts)]
        K.rebuild_plan(exact, bits, *got)
        rb = R.rebuild_plan(exact.cpu(), bits.cpu(), nb, s["rw"])
        for i, (a, b) in enumerate(zip(got, rb)):
            if i in (2, 5):                 # lists: compare the used part
                n = got[1] if i == 2 else got[6]
                j = torch.arange(nb, device=DEV)
                assert torch.equal(torch.where(j < n[..., None], a, 0).cpu(), b), i
            else:
                assert torch.equal(a.cpu(), b), i
        assert torch.equal(got[0], keep) and torch.equal(got[1], counts) and torch.equal(got[3], refine)
    km_r, vm_r = R.block_means(s["k"].cpu(), s["v"].cpu())
    assert rel_l2(s["km"].cpu(), km_r) <= 1e-3 and rel_l2(s["vm"].cpu(), vm_r) <= 1e-3
    _, metric_r, probes_r = R.query_metric(s["q"].cpu())
    assert rel_l2(s["reps"]._metric.cpu(), metric_r) <= 5e-3 and rel_l2(s["reps"]._probes.cpu(), probes_r) <= 1e-3
    # invariants of every block's representatives (the reference's own test: tests/test_sm120.py:65-83)
    reps = s["reps"]
    cnt = torch.exp2(reps.log_counts[:, :nb * 4]).view(H, nb, 4)
    assert torch.equal(cnt.sum(-1).round().long().cpu(), R.block_len(L, nb).long().expand(H, nb))
    assert torch.isinf(reps.log_counts[:, nb * 4:]).all() and bool((reps.k[:, nb * 4:] == 0).all())


def check_estimates(s):
    m3_r, se3_r, ss3_r = R.estimate_skipped(s["q"].cpu(), s["km"].cpu(), s["selection"][0].cpu(), s["lse1"].cpu(),
                                            s["lse2"].cpu(), s["mass2"].cpu())
    assert rel_l2(s["mass3"].cpu(), m3_r) <= 1e-4
    assert rel_l2(s["se3"].cpu(), se3_r) <= 1e-4 and rel_l2(s["ss3"].cpu(), ss3_r) <= 1e-4


def check_tiles(s, tiles, rep_tiles=2):
    """The sampled (tile, head index) pairs against the oracle, which gets the kernels' own tables."""
    L, H, nq, nb = s["L"], s["H"], s["nq"], s["nb"]
    c = R.LOG2E / math.sqrt(128.0)
    keep, counts, blocks, bits, refine = (x.cpu() for x in s["selection"])
    qp, kp, q, k, v = (s[x].cpu() for x in ("qp", "kp", "q", "k", "v"))
    offset0, lse1 = s["offset0"].cpu(), s["lse1"].cpu()
    pad = nb * 64 - L
    for t, h in tiles:
        rows = torch.arange(128 * t, min(128 * t + 128, L))
        sc = (qp[rows, h].float() @ kp[:, h].float().T) * c
        dense = torch.logsumexp(sc * math.log(2.0), -1) / math.log(2.0)
        assert (offset0[rows, h] - dense).abs().max() <= 1e-4, ("dense LSE", t, h)
        p = torch.exp2(sc - offset0[rows, h][:, None])
        assert (lse1[rows, h] - (offset0[rows, h] + torch.log2(p.sum(1)))).abs().max() <= 1e-4, ("full-step LSE", t, h)
        col = torch.cat([p.sum(0), torch.zeros(pad)]).view(nb, 64).sum(1)
        assert rel_l2(s["mass_full"][h, t].cpu(), col) <= 1e-4, ("full-step masses", t, h)
    km, vm = s["km"].cpu(), s["vm"].cpu()
    reps = s["reps"]
    k_rep, v_rep, log_counts = reps.k.cpu(), reps.v.cpu(), reps.log_counts.cpu()
    mass_r = torch.zeros(H, nq, nb)
    out_r, lse_r, flags_r = R.fixed_offset_attention(q, k, v, counts, blocks, lse1, mass=mass_r, k_mean=km, v_mean=vm,
                                                     skip_bits=bits, refine=refine, k_rep=k_rep, v_rep=v_rep,
                                                     log_counts=log_counts, tiles=tiles)
    flags = s["flags"].cpu()
    out_fused, lse_fused, mass2 = s["out_fused"].cpu(), s["lse_fused"].cpu(), s["mass2"].cpu()
    for t, h in tiles:
        rows = torch.arange(128 * t, min(128 * t + 128, L))
        assert int(flags[t, h]) == int(flags_r[t, h]), ("flag", t, h)
        if int(flags_r[t, h]) == 0:
            _close(out_fused[rows, h], out_r[rows, h])
            assert (lse_fused[rows, h] - lse_r[rows, h]).abs().max() <= 1e-4, ("fused LSE", t, h)
        n = int(counts[t, h])
        ids = blocks[t, h, :n].long()
        assert rel_l2(mass2[h, t][ids], mass_r[h, t][ids]) <= 1e-4, ("fused masses", t, h)
    # fallback of the flagged sampled tiles: online softmax over the list, then block-mean compensation
    only = torch.zeros_like(flags_r)
    for t, h in tiles:
        only[t, h] = flags_r[t, h]
    out_fb, lse_fb = out_r.clone(), lse_r.clone()
    R.exact_fallback(q, k, v, out_fb, counts, blocks, lse_fb, only)
    R.compensate_fallback(q, km, vm, keep, lse_fb, out_fb, only)
    out, lse2 = s["out"].cpu(), s["lse2"].cpu()
    for t, h in tiles:
        rows = torch.arange(128 * t, min(128 * t + 128, L))
        _close(out[rows, h], out_fb[rows, h])
        assert (lse2[rows, h] - lse_fb[rows, h]).abs().max() <= 1e-4, ("final LSE", t, h)
        assert bool((lse2[128 * t + len(rows):128 * (t + 1), h] == 1e30).all())
    # representatives of the blocks the first `rep_tiles` sampled tiles refine, from the kernel's metric and probes
    metric, probes = reps._metric.cpu(), reps._probes.cpu()
    total = same = 0
    for t, h in tiles[:rep_tiles]:
        for b in [b for b in refine[t, h].tolist() if b < nb]:
            sl = slice(64 * b, min(64 * b + 64, L))
            k4, v4, c4, _ = R.kmeans_block(k[sl, h], v[sl, h], metric[h], probes[h], ITERS)
            got_c = log_counts[h, 4 * b:4 * b + 4]
            total += 1
            if bool(((got_c == c4) | ((got_c - c4).abs() < 1e-6)).all()):
                same += 1
                assert rel_l2(k_rep[h, 4 * b:4 * b + 4], k4) <= 5e-3 and rel_l2(v_rep[h, 4 * b:4 * b + 4], v4) <= 5e-3
    # cluster labels are decided by float32 comparisons: a near-tie may move a token in a few blocks
    assert total == 0 or same >= 0.9 * total, (same, total)
    return flags_r


def _spread(nq, n, extra=()):
    tiles = sorted(set(int(round(x)) for x in torch.linspace(0, nq - 1, n).tolist()) | set(extra))
    return tiles


def test_wan_1_3b_480p_both_branches_share_the_selection(K):
    """32,760 tokens (512 kv blocks, the last with 56 tokens; 256 tiles, the last with 120 rows), 15 % of the blocks
    kept; three of the 12 heads. Branch 1 runs with branch 0's lists and its own offsets."""
    heads = [0, 5, 11]
    b0 = gpu_step(K, "wan_1_3b_480p", heads, 0)
    assert (b0["L"], b0["nb"], b0["nq"], b0["top"], b0["refined"]) == (32760, 512, 256, 77, 145)
    check_whole_heads(K, b0)
    check_estimates(b0)
    tiles0 = [(t, h) for h in range(3) for t in _spread(256, 6)]
    check_tiles(b0, tiles0)
    b1 = gpu_step(K, "wan_1_3b_480p", heads, 1, selection=b0["selection"])
    assert all(torch.equal(x, y) for x, y in zip(b0["selection"], b1["selection"]))
    check_whole_heads(K, b1, own_selection=False)
    check_tiles(b1, [(t, h) for h in range(3) for t in _spread(256, 4)], rep_tiles=1)
    # a second run of branch 0 gives the same bits: masses are stored in a fixed order, not added atomically
    again = gpu_step(K, "wan_1_3b_480p", heads, 0)
    for key in ("mass_full", "mass2", "mass3", "out", "lse2"):
        assert torch.equal(b0[key], again[key]), key
    assert all(torch.equal(x, y) for x, y in zip(b0["selection"], again["selection"]))


def test_wan_14b_720p_sampled_tiles_of_four_heads_with_fallback(K):
    """75,600 tokens (1,182 kv blocks, the last with 16 tokens; 591 tiles, the last with 80 rows), 10 % kept; four of the
    40 heads, nine tiles each; two tiles per head have their Q scaled by 3 and must go through the fallback."""
    heads = [0, 13, 26, 39]
    inject = [(t, h) for h in range(4) for t in (100 + 37 * h, 500 - 41 * h)]
    s = gpu_step(K, "wan_14b_720p", heads, 0, inject=inject)
    assert (s["L"], s["nb"], s["nq"], s["top"], s["refined"], s["rw"]) == (75600, 1182, 591, 118, 355, 384)
    check_whole_heads(K, s)
    check_estimates(s)
    tiles = [(t, h) for h in range(4) for t in _spread(591, 7, extra=[t for t, hh in inject if hh == h])]
    assert len(tiles) >= 32
    flags_r = check_tiles(s, tiles)
    assert all(int(flags_r[t, h]) == 1 for t, h in inject), "the injected tiles leave the safe range"
    assert len(inject) <= int(s["flags"].sum()) <= 2 * len(inject), "and hardly any other tile does"


def test_hunyuan_720p_text_blocks_as_sink(K):
    """118,800 video tokens + 256 text rows = 119,056 tokens (1,861 kv blocks, the last with 16 tokens; 931 tiles, the
    last with 16 rows); sink = block 1,856: every tile keeps the five text blocks; 12 % kept. Two of the 24 heads."""
    heads = [2, 21]
    s = gpu_step(K, "hunyuan_720p", heads, 0)
    assert (s["L"], s["nb"], s["nq"], s["sink"], s["top"], s["refined"], s["rw"]) == (119056, 1861, 931, 1856, 223, 546, 576)
    check_whole_heads(K, s)
    check_estimates(s)
    # first tile, tiles spread over the video, the last video tiles (their forced neighbours touch the sink), text tiles
    tiles = [(t, h) for h in range(2) for t in _spread(931, 5, extra=[926, 927, 928, 930])]
    check_tiles(s, tiles)
