"""A small, self-ending case of the hot path for a profiler (Nsight Compute) or a quick timing.

    python -m self_trainable_or_free_attn_b200.profile_case [--workload wan_1_3b_480p] [--heads 12] [--repeat 1]

It takes one CFG branch of the named synthetic workload (optionally only the first `--heads` heads) through the dense
step, the full step and `--repeat` sparse steps of the attention processor, then prints the per-kernel durations of the
last sparse step measured with CUDA events. Kernel launch order, for a profiler's skip count: the dense step launches
attention_kernel<true> once; the full step attention_kernel<false> once (every block) and attention_kernel<true> once
(no flagged tile: returns at once); every sparse step: block_mean, select, gram, metric, probe, kmeans,
attention_kernel<false> (the fused sparse step), attention_kernel<true>, compensate, estimate.
"""
import argparse

import torch

from . import _native, synthetic
from .attention import EchoSparseAttention
from .kernels import sm100 as K


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="wan_1_3b_480p", choices=sorted(synthetic.WORKLOADS))
    ap.add_argument("--heads", type=int, default=0, help="use only the first N heads (0 = all)")
    ap.add_argument("--repeat", type=int, default=1)
    ap.add_argument("--threshold", type=float, default=60.0)
    args = ap.parse_args()
    grid, heads_all, _, density, text = synthetic.WORKLOADS[args.workload]
    heads = list(range(args.heads or heads_all))
    cid = sorted(synthetic.WORKLOADS).index(args.workload)
    dev = torch.device("cuda", 0)
    attn = EchoSparseAttention(density=density, dense_steps=2, dense_layers=(), threshold=args.threshold, min_blocks=1)
    qp, kp, vp = synthetic.branch_qkv(grid, cid, 0, heads, dev, text, prev=True)
    attn(qp, kp, vp, 0, 0, layer=1)
    attn(qp, kp, vp, 1, 0, layer=1)
    del qp, kp, vp
    q, k, v = synthetic.branch_qkv(grid, cid, 0, heads, dev, text)
    names = ["block_means", "select_blocks", "sparse_attention", "exact_fallback", "compensate_fallback",
             "estimate_skipped"]
    timer = K.KernelTimer(names)
    for i in range(args.repeat):
        if i == args.repeat - 1:
            K.set_kernel_timer(timer)
        attn(q, k, v, 2 + i, 0, layer=1)
    K.set_kernel_timer(None)
    torch.cuda.synchronize()
    st = attn._states[(0, 1)]
    L = q.shape[1]
    flop = synthetic.step_flops(L, st.counts, st.blocks, st.refine, st.skip_bits)
    print(f"workload {args.workload}: {L} tokens, {len(heads)} heads, mean exact blocks per tile "
          f"{st.counts.float().mean().item():.1f}, algorithmic {flop / 1e12:.3f} TFLOP per sparse step")
    for n in names:
        ms = timer.ms(n)
        extra = f"  {flop / ms[-1] / 1e9:.1f} TFLOP/s" if n == "sparse_attention" else ""
        print(f"  {n}: {ms[-1]:.3f} ms{extra}")
    print("device status", _native.device_status())


if __name__ == "__main__":
    main()
