"""Generates the golden vectors of tests/golden/ by running the REFERENCE's own kernels on CPU.

The reference (shaoshitong/self_trainable_or_free_attn) has no CPU path: its small kernels and its RTX 5090 attention
kernels are Triton. Triton ships a CPU interpreter (TRITON_INTERPRET=1) that executes the unmodified kernel source with
numpy; this script drives the reference's kernel functions through it, in the order the reference's attention
processor calls them (echosparse/attention.py:215-330), and stores their outputs.

Two fixes are applied to the interpreter, not to the reference, so that it computes what the GPU computes. Triton 3.6's
interpreter keeps bf16 tensors as uint16 bit patterns, and (1) its `tl.dot` multiplies those patterns as integers:
`_patched_dot` converts bf16 operands to float32 first; (2) its float32 -> bf16 cast truncates the mantissa:
`_patched_cast` rounds to nearest even, as `cvt.rn.bf16.f32` does.

Run from the repository root, in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

Inputs are produced by `golden_inputs` (numpy PCG64, stable across platforms) and are NOT stored; tests regenerate
them. Outputs are stored in `echosparse_step.npz` next to this file.
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
L, H, D = 4152, 2, 128          # the reference's own test shape (tests/test_attention.py:17): 65 kv blocks, tail 56
DENSITY = 0.1
ITERS = 6


def golden_inputs(step, seed=0):
    """q, k, v of denoising step `step` as float32 arrays holding bf16-representable values: a fixed sinusoidal base
    per tensor plus a small per-step change (the recipe of the reference's tests/test_attention.py:20-30)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    pos = np.arange(L, dtype=np.float32)[:, None, None] / np.float32(300.0)
    out = []
    freq = rng.standard_normal((1, H, D)).astype(np.float32)
    bases = [np.sin(pos * freq + rng.standard_normal((1, H, D)).astype(np.float32)) * np.float32(3.0) for _ in range(3)]
    for s in range(step + 1):
        cur = [b + np.float32(0.05) * rng.standard_normal(b.shape).astype(np.float32) for b in bases]
        out = cur
    return [to_bf16_values(x) for x in out]


def to_bf16_values(x):
    """Round-to-nearest-even to bf16, returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def bf16_bits(t):
    """torch bf16 tensor -> uint16 numpy array of its bit patterns."""
    import torch
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main(reference_root):
    os.environ["TRITON_INTERPRET"] = "1"
    sys.path.insert(0, reference_root)
    import torch
    import triton
    from triton.runtime import interpreter

    def _as_f32(h):
        import triton.language as tl
        if h.dtype.scalar == tl.bfloat16:
            return (h.data.astype(np.uint32) << 16).view(np.float32)
        return h.data

    def _patched_dot(self, a, b, d, input_precision, max_num_imprecise_acc):
        return interpreter.TensorHandle(np.matmul(_as_f32(a), _as_f32(b), dtype=d.data.dtype) + d.data, d.dtype.scalar)

    interpreter.InterpreterBuilder.create_dot = _patched_dot
    _orig_cast = interpreter.InterpreterBuilder.cast_impl

    def _patched_cast(self, src, dst_type):
        import triton.language as tl
        if src.dtype.scalar == tl.float32 and dst_type.scalar == tl.bfloat16:
            bits = (to_bf16_values(src.data).view(np.uint32) >> 16).astype(np.uint16).reshape(src.data.shape)
            return interpreter.TensorHandle(bits, dst_type.scalar)
        return _orig_cast(self, src, dst_type)

    interpreter.InterpreterBuilder.cast_impl = _patched_cast
    interpreter.InterpreterBuilder.create_fp_to_fp = lambda self, src, dst_type, rounding_mode: \
        _patched_cast(self, src, dst_type)

    from echosparse.kernels import sm120 as S
    from echosparse.kernels import triton_ops as T
    from echosparse.kernels.representatives import Representatives

    nq, nb = -(-L // 128), -(-L // 64)
    words = max(triton.next_power_of_2(nb) // 32, 4 * triton.cdiv(nb, 128))
    top = max(1, int(round(DENSITY * nb)))
    refined = max(0, int(round((nb - top) / 3)))
    rw = -(-refined // 32) * 32
    G = {"L": L, "H": H, "top": top, "refined": refined, "rw": rw, "words": words, "iters": ITERS}

    def tensors(step):
        return [torch.from_numpy(x).to(torch.bfloat16) for x in golden_inputs(step)]

    # ---- step 0: dense log2 LSE of the inputs (plain torch) becomes the offset of the full step
    q, k, v = tensors(0)
    s = torch.einsum("ihd,jhd->hij", q.float(), k.float()) / math.sqrt(D)
    offset = torch.full((nq * 128, H), 1e30)
    offset[:L] = (torch.logsumexp(s, -1) * S.LOG2E).T
    G["offset0"] = offset.numpy().copy()

    # ---- step 1: the full step (every block at the fixed offset) -> exact output, first mass map, scales
    q, k, v = tensors(1)
    counts_all = torch.full((nq, H), nb, dtype=torch.int32)
    blocks_all = torch.arange(nb, dtype=torch.int32).expand(nq, H, nb).contiguous()
    out = torch.zeros_like(q)
    lse = torch.zeros(nq * 128, H)
    flags = torch.zeros(nq, H, dtype=torch.int32)
    mass = torch.zeros(H, nq, nb)
    S.block_attention(q, k, v, out, counts_all, blocks_all, offset, lse, flags, mass=mass, threshold=60.0)
    G["full_out"] = bf16_bits(out[::9])
    G["full_lse"] = lse.numpy().copy()
    G["full_flags"] = flags.numpy().copy()
    G["full_mass"] = mass.numpy().copy()
    scale_exact = torch.ones(H, nq)
    scale_skip = torch.ones(H, nq)
    T.full_step_scales(offset, lse, scale_exact, scale_skip, L)
    G["full_lse_reset"] = lse.numpy().copy()
    G["full_scale_exact"] = scale_exact.numpy().copy()
    G["full_scale_skip"] = scale_skip.numpy().copy()
    offset = lse.clone()

    # ---- step 2: select -> plan -> rebuild -> means + representatives -> fused sparse step -> estimates
    q, k, v = tensors(2)
    keep_prev = torch.ones(H, nq, nb, dtype=torch.uint8)
    keep = torch.zeros(H, nq, nb, dtype=torch.uint8)
    counts = torch.zeros(nq, H, dtype=torch.int32)
    blocks = torch.zeros(nq, H, nb, dtype=torch.int32)
    skip_bits = torch.full((H, nq, words), -1, dtype=torch.int32)
    refine = torch.zeros(nq, H, rw, dtype=torch.int32)
    T.select_blocks(mass, keep_prev, scale_exact, scale_skip, keep, counts, blocks, flags, skip_bits, refine, top,
                    refined, L)
    for name, t in (("sel_keep", keep), ("sel_counts", counts), ("sel_blocks", blocks), ("sel_bits", skip_bits),
                    ("sel_refine", refine)):
        G[name] = t.numpy().copy()
    exact_bits = torch.full((H, nq, words), -1, dtype=torch.int32)
    S.pack_plan(keep, exact_bits)
    G["plan_exact"] = exact_bits.numpy().copy()
    keep2 = torch.zeros_like(keep)
    counts2 = torch.zeros_like(counts)
    blocks2 = torch.zeros_like(blocks)
    refine2 = torch.zeros_like(refine)
    rcounts = torch.zeros_like(counts)
    means = torch.zeros_like(blocks)
    mcounts = torch.zeros_like(counts)
    S.rebuild_plan(exact_bits, skip_bits, keep2, counts2, blocks2, refine2, rcounts, means, mcounts)
    assert torch.equal(keep2, keep) and torch.equal(counts2, counts) and torch.equal(refine2, refine)
    G["plan_refine_counts"] = rcounts.numpy().copy()
    G["plan_means"] = means.numpy().copy()
    G["plan_mean_counts"] = mcounts.numpy().copy()

    k_mean = torch.zeros(nb, H, D, dtype=torch.bfloat16)
    v_mean = torch.zeros(nb, H, D, dtype=torch.bfloat16)
    T.block_means(k, v, k_mean, v_mean)
    G["k_mean"] = bf16_bits(k_mean)
    G["v_mean"] = bf16_bits(v_mean)
    reps = Representatives(L, H, D, "cpu", iters=ITERS)
    reps.build(q, k, v)
    G["gram"] = (reps._gram * (D ** -1.0 / L)).numpy().copy()        # before the regularisation
    G["metric"] = bf16_bits(reps._metric)
    G["probes"] = bf16_bits(reps._probes)
    G["k_rep"] = bf16_bits(reps.k)
    G["v_rep"] = bf16_bits(reps.v)
    G["log_counts"] = reps.log_counts.numpy().copy()

    out = torch.zeros_like(q)
    lse = torch.zeros(nq * 128, H)
    mass2 = torch.zeros(H, nq, nb)
    S.sparse_attention(q, k, v, k_mean, v_mean, means, mcounts, out, counts, blocks, offset, lse, flags, refine,
                       rcounts, reps.k, reps.v, reps.log_counts, mass=mass2, threshold=60.0)
    G["sparse_out"] = bf16_bits(out[::9])
    G["sparse_lse"] = lse.numpy().copy()
    G["sparse_flags"] = flags.numpy().copy()
    G["sparse_mass"] = mass2.numpy().copy()
    mass3 = mass2.clone()
    T.estimate_skipped(q, k_mean, keep, offset, lse, mass3, scale_exact, scale_skip)
    G["est_mass"] = mass3.numpy().copy()
    G["est_scale_exact"] = scale_exact.numpy().copy()
    G["est_scale_skip"] = scale_skip.numpy().copy()

    # ---- the next selection, from the map that mixes exact masses and estimates (ties, forced blocks, refine cut)
    keep3 = torch.zeros_like(keep)
    T.select_blocks(mass3, keep, scale_exact, scale_skip, keep3, counts2, blocks2, flags, skip_bits, refine2, top,
                    refined, L)
    G["sel2_keep"] = keep3.numpy().copy()
    G["sel2_counts"] = counts2.numpy().copy()
    G["sel2_bits"] = skip_bits.numpy().copy()
    G["sel2_refine"] = refine2.numpy().copy()

    # ---- selection corner cases on a synthetic map: NaN and inf masses, ties, a sink, fell-back tiles, r = 0
    rng = np.random.Generator(np.random.PCG64(7))
    cm = rng.random((H, nq, nb), dtype=np.float32)
    cm[:, :, 5] = cm[:, :, 9]                        # ties
    cm[0, 3, 11] = np.nan
    cm[1, 4, 12] = np.inf
    cm[:, 6, :] = 0.25                               # a whole tile of equal masses
    cmass = torch.from_numpy(cm)
    ckeep_prev = torch.from_numpy((rng.random((H, nq, nb)) < 0.2).astype(np.uint8))
    cse = torch.from_numpy(rng.random((H, nq), dtype=np.float32) + 0.5)
    css = torch.from_numpy(rng.random((H, nq), dtype=np.float32) + 0.5)
    cflags = torch.from_numpy((rng.random((nq, H)) < 0.2).astype(np.int32))
    for name, kk, rr, sink in (("c1", 7, 19, 1 << 30), ("c2", 1, 0, 60), ("c3", nb, 5, 1 << 30), ("c4", 13, 40, 63)):
        w = -(-rr // 32) * 32
        ck = torch.zeros_like(keep)
        cc = torch.zeros_like(counts)
        cb = torch.zeros_like(blocks)
        cbits = torch.full((H, nq, words), -1, dtype=torch.int32)
        cr = torch.zeros(nq, H, w, dtype=torch.int32)
        T.select_blocks(cmass, ckeep_prev, cse, css, ck, cc, cb, cflags, cbits, cr, kk, rr, L, sink=sink)
        G[f"{name}_keep"], G[f"{name}_counts"], G[f"{name}_bits"], G[f"{name}_refine"] = \
            ck.numpy().copy(), cc.numpy().copy(), cbits.numpy().copy(), cr.numpy().copy()
        G[f"{name}_args"] = np.array([kk, rr, sink, w], np.int64)

    # ---- fallback: a far-off offset flags every tile; online softmax over the list, then block-mean compensation
    bad = offset.clone()
    bad[:L] += 200.0
    out_f = torch.zeros_like(q)
    lse_f = torch.zeros(nq * 128, H)
    flags_f = torch.zeros(nq, H, dtype=torch.int32)
    S.sparse_attention(q, k, v, k_mean, v_mean, means, mcounts, out_f, counts, blocks, bad, lse_f, flags_f, refine,
                       rcounts, reps.k, reps.v, reps.log_counts, mass=None, threshold=60.0)
    G["fb_flags"] = flags_f.numpy().copy()
    S.exact_fallback(q, k, v, out_f, counts, blocks, lse_f, flags_f)
    G["fb_exact_out"] = bf16_bits(out_f[::9])
    G["fb_exact_lse"] = lse_f.numpy().copy()
    T.compensate_fallback(q, k_mean, v_mean, keep, lse_f, out_f, flags_f)
    G["fb_comp_out"] = bf16_bits(out_f[::9])
    G["fb_comp_lse"] = lse_f.numpy().copy()

    path = os.path.join(HERE, "echosparse_step.npz")
    np.savez_compressed(path, **{k: np.asarray(v) for k, v in G.items()})
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <reference checkout>")
    main(sys.argv[1])
