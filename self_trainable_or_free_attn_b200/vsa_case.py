"""The VSA2 training-shape layer as a self-ending case for timing or a profiler.

    python -m self_trainable_or_free_attn_b200.vsa_case [--heads 12] [--grid 16 32 64] [--topk 32] [--skew] [--repeat 5]

B = 1, `--heads` heads, head dim 128, the tokens of a T x H x W latent grid in 4 x 4 x 4 tiles (64-token blocks, R = 16
router groups), bf16. q, k, v = N(0, 1) plus a smooth low-frequency component; the selection is the exact global top-k of a
seeded local score (Gaussian of the distance between tile centres times U(0, 1)) with NB * topk pairs per head; `--skew`
gives 10 % of the query tiles 4 x the score so that they select about four times more pairs. Prints CUDA-event times of the
forward, the backward and the fine-branch kernels, with their algorithmic TFLOP/s (fine forward 4 * 64 * 64 * D FLOP per
selected pair; backward 2.5 x that: five products per pair).
"""
import argparse
import math

import torch

from . import _native
from .vsa import build_layout, ops, to_blocked


def build(grid, heads, seed=4000, device="cuda"):
    T, H, W = grid
    g = torch.Generator(device="cpu").manual_seed(seed)
    lay = build_layout(grid, R=16)
    n = T * H * W
    t, y, x = torch.meshgrid(torch.arange(T) / T, torch.arange(H) / H, torch.arange(W) / W, indexing="ij")
    pos = torch.stack([t, y, x], -1).reshape(n, 3)
    out = []
    for _ in range(3):
        base = torch.randn(1, heads, n, 128, generator=g)
        f = torch.randn(4, 3, generator=g) * 2.0
        ph = torch.rand(4, 128, generator=g) * 2 * math.pi
        smooth = torch.cos(2 * math.pi * (pos @ f.t())[:, :, None] + ph[None]).sum(1) * 0.75
        out.append(to_blocked((base + smooth[None, None]).to(torch.bfloat16), lay).to(device).contiguous())
    gate = to_blocked((torch.randn(1, heads, n, generator=g) * 1.5).to(torch.bfloat16), lay).to(device).contiguous()
    dout = to_blocked(torch.randn(1, heads, n, 128, generator=g).to(torch.bfloat16), lay).to(device).contiguous()
    return out[0], out[1], out[2], gate, dout, lay


def local_selection(grid, heads, topk, skew, device, seed=4001):
    """Exact global top-(NB * topk) of a seeded local score over the tiles."""
    T, H, W = grid
    nt, nh, nw = -(-T // 4), -(-H // 4), -(-W // 4)
    nb = nt * nh * nw
    c = torch.stack(torch.meshgrid(torch.arange(nt), torch.arange(nh), torch.arange(nw), indexing="ij"), -1).reshape(nb, 3).float()
    d2 = ((c[:, None] - c[None]) ** 2).sum(-1).to(device)
    g = torch.Generator(device=device).manual_seed(seed)
    s = torch.exp(-d2 / (2 * 3.0 ** 2))[None, None] * torch.rand(1, heads, nb, nb, generator=g, device=device)
    if skew:
        hot = torch.rand(nb, generator=g, device=device) < 0.10
        s = torch.where(hot[None, None, :, None], s * 4 + 1.0, s)
    return ops.global_topk(s.contiguous(), nb * topk), nb


def timed(fn, repeat):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(repeat):
        out = fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / repeat, out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--grid", type=int, nargs=3, default=[16, 32, 64])
    ap.add_argument("--topk", type=int, default=32)
    ap.add_argument("--skew", action="store_true")
    ap.add_argument("--repeat", type=int, default=5)
    ap.add_argument("--split", default="none", choices=["none", "auto", "manual"],
                    help="split-KV scheduling of the operator runs: none, the planner's automatic policy, or every list > 64")
    args = ap.parse_args()
    split = {"none": None, "auto": ops.SplitKV.auto(), "manual": ops.SplitKV(chunk=64)}[args.split]
    dev = torch.device("cuda", 0)
    q, k, v, gate, dout, lay = build(tuple(args.grid), args.heads, device=dev)
    cnt = lay.blk_cnt.to(dev)
    sel, nb = local_selection(tuple(args.grid), args.heads, args.topk, args.skew, dev)
    pairs = int(sel.row_counts().sum())
    rows = sel.row_counts().reshape(-1)
    flop_fwd = 4.0 * 64 * 64 * 128 * pairs
    print(f"vsa2 case: {q.shape[2]} padded tokens, {nb} blocks, {args.heads} heads, {pairs} selected pairs "
          f"(per query block: mean {rows.float().mean():.1f}, max {int(rows.max())}), fine forward {flop_fwd / 1e12:.3f} TFLOP")

    ms, (of, lse) = timed(lambda: ops.attn_fwd(q, k, v, sel.q2k_ptr, sel.q2k_idx, cnt), args.repeat)
    print(f"  fine forward kernel      {ms:8.3f} ms  {flop_fwd / ms / 1e9:7.1f} TFLOP/s")
    delta = (dout.float() * of.float()).sum(-1)
    ms_kv, _ = timed(lambda: ops._bwd_kv(q, k, v, dout, lse, delta, sel.k2q_ptr, sel.k2q_idx, cnt), args.repeat)
    ms_q, _ = timed(lambda: ops._bwd_q(q, k, v, dout, lse, delta, sel.q2k_ptr, sel.q2k_idx, cnt), args.repeat)
    print(f"  fine backward dK/dV      {ms_kv:8.3f} ms  {2.0 * flop_fwd / ms_kv / 1e9:7.1f} TFLOP/s (4 products per pair)")
    print(f"  fine backward dQ         {ms_q:8.3f} ms  {1.5 * flop_fwd / ms_q / 1e9:7.1f} TFLOP/s (3 products per pair)")
    print(f"  fine backward, both      {ms_kv + ms_q:8.3f} ms  {2.5 * flop_fwd / (ms_kv + ms_q) / 1e9:7.1f} TFLOP/s on the "
          f"algorithmic 5 products per pair")

    def fwd_bwd(routed):
        leaves = [x.detach().requires_grad_(True) for x in (q, k, v, gate)]
        kw = dict(topk=args.topk) if routed else dict(selection=sel)
        o = ops.vsa2_attention(*leaves, cnt, R=16, split_kv=split, **kw)
        return torch.autograd.grad(o, leaves, dout)

    def fwd_only(routed):
        with torch.no_grad():
            kw = dict(topk=args.topk) if routed else dict(selection=sel)
            return ops.vsa2_attention(q, k, v, gate, cnt, R=16, split_kv=split, **kw)

    if split is not None:
        ms_s, _ = timed(lambda: ops.split_fine_fwd(q, k, v, sel.q2k_ptr, sel.q2k_idx, cnt, split), args.repeat)
        print(f"  fine forward, split ({args.split}) {ms_s:8.3f} ms  {flop_fwd / ms_s / 1e9:7.1f} TFLOP/s (plan + tasks + merge)")
        print("  plans:", {k_: v_["info"] for k_, v_ in ops.describe_split(q, sel, split).items()})
    for routed in (False, True):
        name = "router + top-k" if routed else "frozen selection"
        ms_f, _ = timed(lambda: fwd_only(routed), args.repeat)
        ms_fb, _ = timed(lambda: fwd_bwd(routed), args.repeat)
        print(f"  operator, {name:16s} forward {ms_f:8.3f} ms, forward + backward {ms_fb:8.3f} ms")
    # the 64 / 4 / 1 tiers: tier A = the same budget (topk / NB of the pairs), tier B the next 20 %, tier C the rest
    from .vsa import tiers as T
    rt = T.RepTiers(frac_full=args.topk / nb, frac_mid=0.20, mid_reps=4)
    tsel = T.route_tiers(q, k, cnt, rt, R=16)
    a_m, b_m, c_m = tsel.tier_masks(nb)
    na, nbp, ncp = int(a_m.sum()), int(b_m.sum()), int(c_m.sum())
    flop_t = 4.0 * 64 * 128 * (64 * na + 4 * nbp + ncp)
    tab = T.rep_build(k, v, cnt, 4)
    ms_t, (ot, lset) = timed(lambda: T._tier_fwd(q, k, v, tab, tsel, cnt, 4, 7), args.repeat)
    print(f"  tiers (router selection): pairs A {na}, B {nbp}, C {ncp}; algorithmic {flop_t / 1e12:.3f} TFLOP forward")
    print(f"  three-tier forward kernel {ms_t:8.3f} ms  {flop_t / ms_t / 1e9:7.1f} TFLOP/s")
    for ph, name in ((1, "A"), (3, "A+B")):
        ms_p, _ = timed(lambda: T._tier_fwd(q, k, v, tab, tsel, cnt, 4, ph), args.repeat)
        print(f"    phases {name:4s}            {ms_p:8.3f} ms")
    delta_t = (dout.float() * ot.float()).sum(-1)
    ms_tb, _ = timed(lambda: T._tier_bwd(q, k, v, tab, dout, lset, delta_t, tsel, cnt, 4, 7), args.repeat)
    print(f"  three-tier backward (dQ pass + tier-A dK/dV + representative pass + unpool) {ms_tb:8.3f} ms")
    print("device status", _native.device_status(), "launches", _native.launch_count())


if __name__ == "__main__":
    main()
