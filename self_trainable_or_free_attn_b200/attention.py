"""LSE-guided block-sparse self-attention: the attention processor and its step-to-step state.

Same public surface as the reference's `echosparse/attention.py` (`EchoSparseAttention.__init__/__call__/reset`,
attributes `.backend`, `.K`, `._states`, `._buffers`, `._budget`), same schedule per (CFG branch, layer):

    steps 0 .. dense_steps-2   dense attention; its log2 LSE becomes the stored offset      (attention.py:187-190)
    step  dense_steps-1        every block through the fixed-offset kernel: exact output, the first
                               block-probability map and the scales                          (attention.py:215-228)
    later steps, branch 0      select -> representatives -> fused sparse step -> fallback of flagged tiles ->
                               estimates for the next selection                              (attention.py:230-248)
    later steps, branch > 0    branch 0's selection with this branch's own offsets           (attention.py:250-255)

The dense steps use this library's own online-softmax kernel over all blocks instead of FlashAttention-4, so the whole
path runs on the one native library.
"""
import torch

from . import backends

BM = 128
BK = 64
LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453
MIN_BLOCKS = 64          # sequences shorter than 64 kv blocks (4096 tokens) run dense


def cdiv(a, b):
    return -(-a // b)


def next_power_of_2(n):
    return 1 << (max(n, 1) - 1).bit_length()


def dense_attention(q, k, v, return_lse=False, K=None):
    """Dense softmax attention of [1, L, H, 128] bf16 tensors; with return_lse also the natural-log LSE [1, H, L].
    Runs the online-softmax kernel over every block (all tiles flagged)."""
    if K is None:
        K = backends.kernels(backends.resolve("auto", q.device))
    B, L, H, D = q.shape
    if k.shape[1] != L:
        # cross-shaped calls (text rows against all tokens, video rows against text tokens) are outside the sparse path:
        # the reference sends them to its library dense kernel (FlashAttention-4, backends.py:50-59); here torch's is used
        assert not return_lse, "the LSE is only needed for self-attention"
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).contiguous()
    assert B == 1
    nq, nb = cdiv(L, BM), cdiv(L, BK)
    dev = q.device
    counts = torch.full((nq, H), nb, device=dev, dtype=torch.int32)
    blocks = torch.arange(nb, device=dev, dtype=torch.int32).expand(nq, H, nb).contiguous()
    flags = torch.ones(nq, H, device=dev, dtype=torch.int32)
    lse = torch.empty(nq * BM, H, device=dev)
    out = torch.empty_like(q[0])
    K.exact_fallback(q[0].contiguous(), k[0].contiguous(), v[0].contiguous(), out, counts, blocks, lse, flags)
    if return_lse:
        return out[None], (lse[:L].t() * LN2)[None]
    return out[None]


class _LayerState:
    """State of one (branch, layer) (reference: attention.py:38-69)."""

    def __init__(self, L, H, device):
        nq, nb = cdiv(L, BM), cdiv(L, BK)
        self.L = L
        self.offsets = [torch.full((nq * BM, H), 1e30, device=device) for _ in range(2)]
        self.cur = 0
        self.mass = torch.zeros(H, nq, nb, device=device)
        self.keeps = [torch.ones(H, nq, nb, device=device, dtype=torch.uint8) for _ in range(2)]
        self.kc = 0
        self.scale_exact = torch.ones(H, nq, device=device)
        self.scale_skip = torch.ones(H, nq, device=device)
        self.counts = torch.empty(nq, H, device=device, dtype=torch.int32)
        self.blocks = torch.zeros(nq, H, nb, device=device, dtype=torch.int32)
        self.flags = torch.zeros(nq, H, device=device, dtype=torch.int32)
        words = max(next_power_of_2(nb) // 32, 4 * cdiv(nb, 128))
        self.skip_bits = torch.full((H, nq, words), -1, device=device, dtype=torch.int32)
        self.refine = torch.empty(nq, H, 0, device=device, dtype=torch.int32)
        self.ready = False

    @property
    def offset(self):
        return self.offsets[self.cur]

    @property
    def next_offset(self):
        return self.offsets[1 - self.cur]

    @property
    def keep(self):
        return self.keeps[self.kc]


class _CompactState:
    """Compact state of one layer (reference: attention.py:72-97): the offsets of every branch and the plans, each a pair
    of bit masks (exact blocks, blocks skipped by the block-mean compensation), 2 x H x nq x words x 4 bytes: 12 MB per
    plan at 75,600 tokens and 40 heads against the 310 MB of a `_LayerState`. Branch 0 writes the other of two plans for
    the next step while later branches still read the current one."""

    def __init__(self, L, H, device):
        nb = cdiv(L, BK)
        self.L, self.H, self.device = L, H, device
        self.words = max(next_power_of_2(nb) // 32, 4 * cdiv(nb, 128))
        self.plans = []
        self.offsets = {}
        self.ready = set()          # branches that have run the full step
        self.current = None         # (plan, step) used by the branches of this step
        self.pending = None         # (plan, step) made by branch 0 for the next step

    def plan(self, i):
        while len(self.plans) <= i:
            shape = (self.H, cdiv(self.L, BM), self.words)
            self.plans.append(tuple(torch.full(shape, -1, device=self.device, dtype=torch.int32) for _ in range(2)))
        return self.plans[i]

    def offset(self, branch):
        if branch not in self.offsets:
            self.offsets[branch] = torch.full((cdiv(self.L, BM) * BM, self.H), 1e30, device=self.device)
        return self.offsets[branch]


class _PlanScratch:
    """Per-call tensors of the compact path, shared by all layers (reference: attention.py:99-117)."""

    def __init__(self, L, H, device, refine_width):
        nq, nb = cdiv(L, BM), cdiv(L, BK)
        self.shape = (L, H, refine_width)
        self.mass = torch.empty(H, nq, nb, device=device)
        self.keep = torch.empty(H, nq, nb, device=device, dtype=torch.uint8)
        self.next_keep = torch.empty(H, nq, nb, device=device, dtype=torch.uint8)
        self.scale_exact = torch.empty(H, nq, device=device)
        self.scale_skip = torch.empty(H, nq, device=device)
        self.counts = torch.empty(nq, H, device=device, dtype=torch.int32)
        self.blocks = torch.zeros(nq, H, nb, device=device, dtype=torch.int32)
        self.refine = torch.empty(nq, H, refine_width, device=device, dtype=torch.int32)
        self.refine_counts = torch.empty(nq, H, device=device, dtype=torch.int32)
        self.means = torch.empty(nq, H, nb, device=device, dtype=torch.int32)
        self.mean_counts = torch.empty(nq, H, device=device, dtype=torch.int32)
        self.next_offset = torch.empty(nq * BM, H, device=device)


class _Buffers:
    """Per-call scratch for one sequence shape (reference: attention.py:119-130)."""

    def __init__(self, L, H, D, device, refine_iters, K):
        nq, nb = cdiv(L, BM), cdiv(L, BK)
        self.shape = (L, H, D)
        self.k_mean = torch.empty(nb, H, D, device=device, dtype=torch.bfloat16)
        self.v_mean = torch.empty(nb, H, D, device=device, dtype=torch.bfloat16)
        self.flags = torch.empty(nq, H, device=device, dtype=torch.int32)
        self.all_counts = torch.full((nq, H), nb, device=device, dtype=torch.int32)
        self.all_blocks = torch.arange(nb, device=device, dtype=torch.int32).expand(nq, H, nb).contiguous()
        self.reps = K.Representatives(L, H, D, device, iters=refine_iters)


class EchoSparseAttention:
    """Self-attention for one video at a time; call `reset()` before each video.

    `__call__(q, k, v, step, branch, layer)` takes [1, L, H, 128] bf16 tensors. `branch` numbers the transformer
    forwards of a denoising step (0: conditional, 1: unconditional); later branches reuse branch 0's block
    selection of the same step and layer. `sink`: first kv block that every query tile computes exactly (text or
    other conditioning tokens placed after the video tokens). `rows` is accepted for signature compatibility.

    `gpu`: "auto" or "b200". `min_blocks`: sequences with fewer kv blocks run dense (the reference's constant 64).
    `state`: "layer" keeps the reference's B200 state per (branch, layer) (mass map, keep masks, lists); "compact" keeps
    only the offsets and the bit-mask plans per layer (the reference's state on its other GPUs, attention.py:272-330) and
    rebuilds the lists from the plan every step: 25 x less resident state for two more small kernels per call.
    """

    def __init__(self, density=0.10, dense_steps=10, dense_layers=(0,), refine_iters=6, threshold=60.0, gpu="auto",
                 min_blocks=MIN_BLOCKS, state="layer"):
        assert state in ("layer", "compact"), "state must be 'layer' or 'compact'"
        self.state = state
        assert dense_steps >= 2, "the first sparse step needs the LSE of a dense step and a full-block step"
        self.density = density
        self.dense_steps = dense_steps
        self.dense_layers = set(dense_layers)
        self.refine_iters = refine_iters
        self.threshold = threshold
        self.min_blocks = min_blocks
        backends.check_name(gpu)
        self.gpu = gpu
        self.backend = None             # resolved from the device of the first call
        self._device = None
        self.K = None
        self._states = {}
        self._buffers = None
        self._plan_scratch = None

    def reset(self):
        for st in self._states.values():
            if isinstance(st, _CompactState):
                st.ready.clear()
                st.current = st.pending = None
            else:
                st.ready = False

    def __call__(self, q, k, v, step, branch, layer, sink=None, rows=None):
        B, L, H, D = q.shape
        assert B == 1, "batch size 1 only"
        if q.device != self._device:
            self.backend = backends.resolve(self.gpu, q.device)
            self.K = backends.kernels(self.backend)
            self._states.clear()
            self._buffers = self._plan_scratch = None
            self._device = q.device
        if layer in self.dense_layers or cdiv(L, BK) < self.min_blocks:
            return dense_attention(q, k, v, K=self.K)
        if self.state == "compact":
            return self._call_compact(q, k, v, step, branch, layer, sink)
        return self._call_b200(q, k, v, step, branch, layer, sink)

    def _call_compact(self, q, k, v, step, branch, layer, sink):
        """The schedule of `_call_b200` on the compact state (reference: attention.py:272-330): a step reads its plan,
        rebuilds the lists, runs the fused kernels and, in branch 0, selects and packs the plan of the next step."""
        L, H, D = q[0].shape
        st = self._states.get(layer)
        if st is None or st.L != L:
            self._states[layer] = None
            st = self._states[layer] = _CompactState(L, H, q.device)
        offset = st.offset(branch)
        if branch == 0 and step >= self.dense_steps:
            st.current = st.pending if st.pending is not None and st.pending[1] == step else None
            st.pending = None
        full = step == self.dense_steps - 1
        sparse = step >= self.dense_steps and branch in st.ready and st.current is not None and st.current[1] == step
        if not (full or sparse):
            out, lse = dense_attention(q, k, v, return_lse=True, K=self.K)
            offset[:L].copy_(lse[0].t() * LOG2E)
            return out
        K = self.K
        q, k, v = q[0].contiguous(), k[0].contiguous(), v[0].contiguous()
        top, refined = self._budget(cdiv(L, BK))
        width = -(-refined // 32) * 32
        buf = self._scratch(L, H, D, q.device)
        ps = self._plan_scratch
        if ps is None or ps.shape != (L, H, width):
            self._plan_scratch = None
            ps = self._plan_scratch = _PlanScratch(L, H, q.device, width)
        out = torch.empty_like(q)
        if full:
            ps.keep.fill_(1)
            ps.mass.zero_()
            K.block_attention(q, k, v, out, buf.all_counts, buf.all_blocks, offset, ps.next_offset, buf.flags,
                              mass=ps.mass, threshold=self.threshold)
            K.exact_fallback(q, k, v, out, buf.all_counts, buf.all_blocks, ps.next_offset, buf.flags)
            K.full_step_scales(offset, ps.next_offset, ps.scale_exact, ps.scale_skip, L)
            st.ready.add(branch)
        else:
            exact, skip = st.plan(st.current[0])
            K.rebuild_plan(exact, skip, ps.keep, ps.counts, ps.blocks, ps.refine, ps.refine_counts, ps.means,
                           ps.mean_counts)
            K.block_means(k, v, buf.k_mean, buf.v_mean)
            buf.reps.build(q, k, v)
            if branch == 0:
                ps.mass.zero_()
            K.sparse_attention(q, k, v, buf.k_mean, buf.v_mean, skip, out, ps.counts, ps.blocks, offset, ps.next_offset,
                               buf.flags, ps.refine, buf.reps.k, buf.reps.v, buf.reps.log_counts,
                               mass=ps.mass if branch == 0 else None, threshold=self.threshold)
            K.exact_fallback(q, k, v, out, ps.counts, ps.blocks, ps.next_offset, buf.flags)
            K.compensate_fallback(q, buf.k_mean, buf.v_mean, ps.keep, ps.next_offset, out, buf.flags)
            if branch == 0:
                K.estimate_skipped(q, buf.k_mean, ps.keep, offset, ps.next_offset, ps.mass, ps.scale_exact, ps.scale_skip)
        if branch == 0:
            # the next step's plan, after this step's last use of the current one in a single branch
            plan = 0 if st.current is None else st.current[0] ^ (len(st.offsets) > 1)
            exact, skip = st.plan(plan)
            K.select_blocks(ps.mass, ps.keep, ps.scale_exact, ps.scale_skip, ps.next_keep, ps.counts, ps.blocks, buf.flags,
                            skip, ps.refine, top, refined, L, sink=1 << 30 if sink is None else sink)
            K.pack_plan(ps.next_keep, exact)
            st.pending = (plan, step + 1)
        offset.copy_(ps.next_offset)
        return out[None]

    def _call_b200(self, q, k, v, step, branch, layer, sink):
        L, H, D = q[0].shape
        st = self._state(branch, layer, L, H, q.device)
        if step < self.dense_steps - 1 or (step >= self.dense_steps and not st.ready):
            out, lse = dense_attention(q, k, v, return_lse=True, K=self.K)
            st.offset[:L].copy_(lse[0].t() * LOG2E)
            return out
        q, k, v = q[0].contiguous(), k[0].contiguous(), v[0].contiguous()
        buf = self._scratch(L, H, D, q.device)
        if step < self.dense_steps:
            out = self._full_step(q, k, v, st, buf)
        elif branch == 0:
            out = self._sparse_step(q, k, v, st, buf, sink)
        else:
            out = self._shared_step(q, k, v, st, self._states[(0, layer)], buf)
        st.cur ^= 1
        return out[None]

    def _state(self, branch, layer, L, H, device):
        st = self._states.get((branch, layer))
        if st is None or st.L != L:
            self._states[(branch, layer)] = None          # free the old buffers before allocating new ones
            st = self._states[(branch, layer)] = _LayerState(L, H, device)
        return st

    def _scratch(self, L, H, D, device):
        if self._buffers is None or self._buffers.shape != (L, H, D):
            self._buffers = None                           # one sequence shape at a time
            self._buffers = _Buffers(L, H, D, device, self.refine_iters, self.K)
        return self._buffers

    def _full_step(self, q, k, v, st, buf):
        """Every block at the fixed offset: exact output and the first block-probability map."""
        K = self.K
        out = torch.empty_like(q)
        st.kc ^= 1
        st.keep.fill_(1)
        st.mass.zero_()
        K.block_attention(q, k, v, out, buf.all_counts, buf.all_blocks, st.offset, st.next_offset, buf.flags,
                          mass=st.mass, threshold=self.threshold)
        K.exact_fallback(q, k, v, out, buf.all_counts, buf.all_blocks, st.next_offset, buf.flags)
        K.full_step_scales(st.offset, st.next_offset, st.scale_exact, st.scale_skip, st.L)
        st.flags.copy_(buf.flags)
        st.ready = True
        return out

    def _sparse_step(self, q, k, v, st, buf, sink):
        K = self.K
        L, H, _ = q.shape
        nq, nb = cdiv(L, BM), cdiv(L, BK)
        K.block_means(k, v, buf.k_mean, buf.v_mean)
        top, refined = self._budget(nb)
        width = -(-refined // 32) * 32
        if st.refine.shape[-1] != width:
            st.refine = torch.empty(nq, H, width, device=q.device, dtype=torch.int32)
        keep_prev = st.keep
        st.kc ^= 1
        K.select_blocks(st.mass, keep_prev, st.scale_exact, st.scale_skip, st.keep, st.counts, st.blocks, st.flags,
                        st.skip_bits, st.refine, top, refined, L, sink=1 << 30 if sink is None else sink)
        st.mass.zero_()
        out = torch.empty_like(q)
        self._attend(q, k, v, st, st, buf, out, mass=st.mass)
        st.flags.copy_(buf.flags)
        K.estimate_skipped(q, buf.k_mean, st.keep, st.offset, st.next_offset, st.mass, st.scale_exact, st.scale_skip)
        return out

    def _shared_step(self, q, k, v, st, sel, buf):
        """A later CFG branch: branch 0's block selection, this branch's own offsets."""
        self.K.block_means(k, v, buf.k_mean, buf.v_mean)
        out = torch.empty_like(q)
        self._attend(q, k, v, st, sel, buf, out)
        return out

    def _attend(self, q, k, v, st, sel, buf, out, mass=None):
        K, reps = self.K, buf.reps
        reps.build(q, k, v)
        K.sparse_attention(q, k, v, buf.k_mean, buf.v_mean, sel.skip_bits, out, sel.counts, sel.blocks, st.offset,
                           st.next_offset, buf.flags, sel.refine, reps.k, reps.v, reps.log_counts, mass=mass,
                           threshold=self.threshold)
        # tiles whose offset was too far off: online softmax over the same list, then block-mean compensation
        K.exact_fallback(q, k, v, out, sel.counts, sel.blocks, st.next_offset, buf.flags)
        K.compensate_fallback(q, buf.k_mean, buf.v_mean, sel.keep, st.next_offset, out, buf.flags)

    def _budget(self, nb):
        """Exactly computed blocks per tile, and refined blocks (four representatives each) per tile."""
        top = max(1, int(round(self.density * nb)))
        return top, max(0, int(round((nb - top) / 3)))
