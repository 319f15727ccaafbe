"""LSE-guided block-sparse self-attention on B200: the attention processor and what it keeps between denoising steps.

Public surface of the reference's `echosparse/attention.py` (`EchoSparseAttention.__init__/__call__/reset`, `dense_attention`,
attributes `.backend`, `.K`, `._states`, `._buffers`, `._plan_scratch`, `._budget`), rebuilt around this backend:

* What a layer keeps is a PLAN: two bit masks per (tile, head) -- the blocks computed exactly and the blocks the block-mean
  compensation leaves out -- plus one log2-LSE vector per CFG branch (two buffers that swap roles, so a step never copies
  its LSE). 12 MB per plan at 75,600 tokens x 40 heads, against 310 MB for the reference's B200 state per (branch, layer).
  Block lists are expanded from the plan into one workspace shared by all layers (`state="compact"`, the default), or kept
  expanded per layer to save that expansion (`state="layer"`).
* The plan of step s + 1 is made at the END of branch 0's call of step s, while the block-probability map is still in the
  workspace; the map is therefore scratch and never resident. The fused kernel stores the masses of the listed blocks and
  the estimate kernel those of all others, so the map needs no clearing between steps.
* One schedule for every state mode, as a small table of phases:

      DENSE    attention over every block: online softmax for the first step of a video, afterwards the previous step's LSE
               as a fixed offset (flagged tiles recomputed); the log2 LSE becomes the branch's offset
      FULL     every block at the fixed offset: exact output, first map, scales; branch 0 plans the next step
      SPARSE   plan -> lists, block means, representatives, fused step, recomputation + compensation of flagged tiles;
               branch 0 also estimates the skipped masses and plans the next step; later branches reuse branch 0's plan

  Steps 0 .. dense_steps-2 are DENSE, step dense_steps-1 is FULL, later steps SPARSE when the branch has run its FULL step
  and a plan for exactly this step exists, otherwise DENSE again (reference: attention.py:184-200, 272-330).
* The dense steps run this library's own kernel; nothing depends on FlashAttention.
* The kernels report a wait that gave up through a status word instead of hanging; `reset()` (once per video) and
  `check_status()` read it and raise, so a broken launch cannot hand back garbage silently for a whole video.
"""
import enum

import torch

from . import _native, backends

BM = 128                 # query rows per tile
BK = 64                  # tokens per kv block
LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453
MIN_BLOCKS = 64          # sequences shorter than 64 kv blocks (4096 tokens) run dense
NO_SINK = 1 << 30


def cdiv(a, b):
    return -(-a // b)


def next_power_of_2(n):
    return 1 << (max(n, 1) - 1).bit_length()


def plan_words(nb):
    """32-bit words of a tile's bit mask: a power of two of bits >= nb, and at least four words per 128 blocks (the fused
    kernel reads the skip mask four words per block-mean iteration)."""
    return max(next_power_of_2(nb) // 32, 4 * cdiv(nb, 128))


class Phase(enum.Enum):
    DENSE = 0
    FULL = 1
    SPARSE = 2


# ------------------------------------------------------------------------------------------------------------ scratch
class _Buffers:
    """Scratch of one sequence shape that every call uses: block means, representatives, flags, and the list of all
    blocks (full step, dense steps)."""

    def __init__(self, L, H, D, device, refine_iters, K):
        nq, nb = cdiv(L, BM), cdiv(L, BK)
        self.shape = (L, H, D)
        self.k_mean = torch.empty(nb, H, D, device=device, dtype=torch.bfloat16)
        self.v_mean = torch.empty(nb, H, D, device=device, dtype=torch.bfloat16)
        self.flags = torch.zeros(nq, H, device=device, dtype=torch.int32)
        self.every_tile = torch.ones(nq, H, device=device, dtype=torch.int32)
        self.all_counts = torch.full((nq, H), nb, device=device, dtype=torch.int32)
        self.all_blocks = torch.arange(nb, device=device, dtype=torch.int32).expand(nq, H, nb).contiguous()
        self.dense_lse = torch.empty(nq * BM, H, device=device)
        self.reps = K.Representatives(L, H, D, device, iters=refine_iters)


class _Lists:
    """A plan expanded for the kernels: keep mask, ascending block lists with their lengths, refine list."""

    def __init__(self, L, H, device, refine_width):
        nq, nb = cdiv(L, BM), cdiv(L, BK)
        self.keep = torch.ones(H, nq, nb, device=device, dtype=torch.uint8)
        self.counts = torch.zeros(nq, H, device=device, dtype=torch.int32)
        self.blocks = torch.zeros(nq, H, nb, device=device, dtype=torch.int32)
        self.refine = torch.full((nq, H, refine_width), nb, device=device, dtype=torch.int32)


class _PlanScratch:
    """Scratch of the sparse path, shared by all layers: the block-probability map and its scales, the lists the current
    call runs on and the lists the selection writes for the next step."""

    def __init__(self, L, H, device, refine_width):
        nq, nb = cdiv(L, BM), cdiv(L, BK)
        self.shape = (L, H, refine_width)
        self.mass = torch.zeros(H, nq, nb, device=device)
        self.scale_exact = torch.ones(H, nq, device=device)
        self.scale_skip = torch.ones(H, nq, device=device)
        self.lists = _Lists(L, H, device, refine_width)
        self.next_lists = _Lists(L, H, device, refine_width)
        self.refine_counts = torch.empty(nq, H, device=device, dtype=torch.int32)

    # the names the reference's scratch object has
    keep = property(lambda self: self.lists.keep)
    counts = property(lambda self: self.lists.counts)
    blocks = property(lambda self: self.lists.blocks)
    refine = property(lambda self: self.lists.refine)
    next_keep = property(lambda self: self.next_lists.keep)


# ------------------------------------------------------------------------------------------------------------ state
class _Branch:
    """Offsets of one CFG branch of one layer: two log2-LSE buffers, the kernel reads one and writes the other."""

    def __init__(self, L, H, device):
        self.buffers = [torch.full((cdiv(L, BM) * BM, H), 1e30, device=device) for _ in range(2)]
        self.cur = 0
        self.ready = False           # has run the FULL step of this video
        self.seeded = False          # `offset` holds the LSE of an earlier step of this video

    @property
    def offset(self):
        return self.buffers[self.cur]

    @property
    def next_offset(self):
        return self.buffers[self.cur ^ 1]


class _LayerRecord:
    """Everything one layer keeps between steps."""

    def __init__(self, L, H, device, keep_lists):
        self.L, self.H, self.device = L, H, device
        self.words = plan_words(cdiv(L, BK))
        self.branches = {}
        self.plans = []              # [(exact bits, skip bits)], each (H, nq, words) int32
        self.current = None          # (plan index, step) the branches of this step read
        self.pending = None          # (plan index, step) branch 0 made for the next step
        self.keep_lists = keep_lists
        self.expanded = {}           # plan index -> _Lists (state="layer" only)

    def branch(self, b):
        if b not in self.branches:
            self.branches[b] = _Branch(self.L, self.H, self.device)
        return self.branches[b]

    def plan(self, i):
        while len(self.plans) <= i:
            shape = (self.H, cdiv(self.L, BM), self.words)
            self.plans.append(tuple(torch.full(shape, -1, device=self.device, dtype=torch.int32) for _ in range(2)))
        return self.plans[i]

    def lists_of(self, i, refine_width):
        got = self.expanded.get(i)
        if got is None or got.refine.shape[-1] != refine_width:
            got = self.expanded[i] = _Lists(self.L, self.H, self.device, refine_width)
        return got

    # ---- what the reference's compact state exposes
    @property
    def offsets(self):
        return {b: br.offset for b, br in self.branches.items()}

    @property
    def ready(self):
        return {b for b, br in self.branches.items() if br.ready}

    def offset(self, branch):
        return self.branch(branch).offset


class _BranchView:
    """`attn._states[(branch, layer)]`: the tensors the last call of that layer ran on, under the names of the reference's
    per-(branch, layer) state. Lists, map, scales and flags live in the shared workspace unless the layer keeps its own."""

    def __init__(self, owner, record, branch):
        self._owner, self._record, self._branch = owner, record, record.branch(branch)

    L = property(lambda self: self._record.L)
    ready = property(lambda self: self._branch.ready)
    offset = property(lambda self: self._branch.offset)
    next_offset = property(lambda self: self._branch.next_offset)
    offsets = property(lambda self: list(self._branch.buffers))
    cur = property(lambda self: self._branch.cur)
    mass = property(lambda self: self._owner._plan_scratch.mass)
    scale_exact = property(lambda self: self._owner._plan_scratch.scale_exact)
    scale_skip = property(lambda self: self._owner._plan_scratch.scale_skip)
    flags = property(lambda self: self._owner._buffers.flags)

    def _used(self):
        return self._owner._used_lists

    keep = property(lambda self: self._used().keep)
    keeps = property(lambda self: [self._owner._plan_scratch.lists.keep, self._owner._plan_scratch.next_lists.keep])
    counts = property(lambda self: self._used().counts)
    blocks = property(lambda self: self._used().blocks)
    refine = property(lambda self: self._used().refine)

    @property
    def skip_bits(self):
        rec = self._record
        which = rec.current if rec.current is not None else rec.pending
        return rec.plan(which[0] if which is not None else 0)[1]


class _StateTable:
    """`attn._states`: layer -> record, and (branch, layer) -> view of one branch. Empty until a layer leaves the dense
    path; iterating gives the (branch, layer) pairs that exist."""

    def __init__(self, owner):
        self._owner = owner
        self._layers = {}

    def record(self, layer):
        return self._layers.get(layer)

    def put(self, layer, record):
        self._layers[layer] = record

    def __getitem__(self, key):
        if isinstance(key, tuple):
            branch, layer = key
            rec = self._layers[layer]
            if branch not in rec.branches:
                raise KeyError(key)
            return _BranchView(self._owner, rec, branch)
        return self._layers[key]

    def __contains__(self, key):
        if isinstance(key, tuple):
            return key[1] in self._layers and key[0] in self._layers[key[1]].branches
        return key in self._layers

    def __iter__(self):
        return iter(sorted((b, layer) for layer, rec in self._layers.items() for b in rec.branches))

    def __len__(self):
        return sum(len(rec.branches) for rec in self._layers.values())

    def values(self):
        return list(self._layers.values())

    def clear(self):
        self._layers.clear()


# ------------------------------------------------------------------------------------------------------------ dense
def _dense_into(K, q, k, v, buf, out, lse):
    """Online-softmax attention over every block: the recomputation kernel with every tile flagged."""
    K.exact_fallback(q, k, v, out, buf.all_counts, buf.all_blocks, lse, buf.every_tile)


def dense_attention(q, k, v, return_lse=False, K=None):
    """Dense softmax attention of [1, L, H, 128] bf16 tensors; with return_lse also the natural-log LSE [1, H, L]."""
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
    buf = _Buffers.__new__(_Buffers)
    nq, nb = cdiv(L, BM), cdiv(L, BK)
    dev = q.device
    buf.all_counts = torch.full((nq, H), nb, device=dev, dtype=torch.int32)
    buf.all_blocks = torch.arange(nb, device=dev, dtype=torch.int32).expand(nq, H, nb).contiguous()
    buf.every_tile = torch.ones(nq, H, device=dev, dtype=torch.int32)
    lse = torch.empty(nq * BM, H, device=dev)
    out = torch.empty_like(q[0])
    _dense_into(K, q[0].contiguous(), k[0].contiguous(), v[0].contiguous(), buf, out, lse)
    if return_lse:
        return out[None], (lse[:L].t() * LN2)[None]
    return out[None]


# ------------------------------------------------------------------------------------------------------------ processor
class EchoSparseAttention:
    """Self-attention for one video at a time; call `reset()` before each video.

    `__call__(q, k, v, step, branch, layer)` takes [1, L, H, 128] bf16 tensors. `branch` numbers the transformer forwards
    of a denoising step (0: conditional, 1: unconditional); later branches reuse branch 0's block selection of the same
    step and layer. `sink`: first kv block that every query tile computes exactly (text or other conditioning tokens placed
    after the video tokens). `rows` is accepted for signature compatibility (every tile is computed).

    `gpu`: "auto" or "b200". `min_blocks`: sequences with fewer kv blocks run dense (the reference's constant 64).
    `state`: "compact" keeps per layer the offsets and the bit-mask plans and expands a plan into the shared workspace at
    every call; "layer" also keeps the expanded lists per layer.
    """

    def __init__(self, density=0.10, dense_steps=10, dense_layers=(0,), refine_iters=6, threshold=60.0, gpu="auto",
                 min_blocks=MIN_BLOCKS, state="compact"):
        if state not in ("layer", "compact"):
            raise ValueError("state must be 'layer' or 'compact'")
        assert dense_steps >= 2, "the first sparse step needs the LSE of a dense step and a full-block step"
        self.state = state
        self.density = density
        self.dense_steps = dense_steps
        self.dense_layers = set(dense_layers)
        self.refine_iters = refine_iters
        self.threshold = threshold
        self.min_blocks = min_blocks
        backends.check_name(gpu)
        self.gpu = gpu
        self.backend = None             # resolved from the device of the first call
        self.K = None
        self._device = None
        self._states = _StateTable(self)
        self._buffers = None
        self._plan_scratch = None
        self._used_lists = None         # the lists the last sparse / full call ran on

    # ---- housekeeping
    def reset(self):
        """Forget the previous video: every branch has to run its dense and full steps again. Also the place where the
        kernels' status word is read (one device synchronisation per video)."""
        for rec in self._states.values():
            for br in rec.branches.values():
                br.ready = br.seeded = False
            rec.current = rec.pending = None
        self.check_status()

    def check_status(self):
        """Raises NativeError if a kernel's bounded wait gave up since the last check (the word is cleared). Synchronises
        the device, so call it where that is cheap: between videos, or once per denoising step."""
        if self._device is None:
            return
        with torch.cuda.device(self._device):
            code = _native.device_status()
        if code != 0:
            raise _native.NativeError(f"an attention kernel gave up a wait (status {code}: wait {code % 1000} in CTA "
                                      f"{code // 1000}); the outputs since the last check are not valid")

    def _bind(self, device):
        self.backend = backends.resolve(self.gpu, device)
        self.K = backends.kernels(self.backend)
        self._states.clear()
        self._buffers = self._plan_scratch = self._used_lists = None
        self._device = device

    def _budget(self, nb):
        """Exactly computed blocks per tile, and refined blocks (four representatives each) per tile."""
        top = max(1, int(round(self.density * nb)))
        return top, max(0, int(round((nb - top) / 3)))

    def _scratch(self, L, H, D, device):
        if self._buffers is None or self._buffers.shape != (L, H, D):
            self._buffers = self._plan_scratch = self._used_lists = None       # one sequence shape at a time
            self._buffers = _Buffers(L, H, D, device, self.refine_iters, self.K)
        return self._buffers

    def _sparse_scratch(self, L, H, device, refine_width):
        ps = self._plan_scratch
        if ps is None or ps.shape != (L, H, refine_width):
            self._plan_scratch = self._used_lists = None
            ps = self._plan_scratch = _PlanScratch(L, H, device, refine_width)
        return ps

    def _record(self, layer, L, H, device):
        rec = self._states.record(layer)
        if rec is None or rec.L != L or rec.H != H:
            self._states.put(layer, None)                    # let the old buffers go before the new ones are made
            rec = _LayerRecord(L, H, device, keep_lists=self.state == "layer")
            self._states.put(layer, rec)
        return rec

    # ---- the schedule
    def _phase(self, rec, br, step, branch):
        if branch == 0 and step >= self.dense_steps:
            # the plan branch 0 made at the end of the previous step becomes this step's, if it was made for this step
            rec.current = rec.pending if rec.pending is not None and rec.pending[1] == step else None
            rec.pending = None
        if step == self.dense_steps - 1:
            return Phase.FULL
        if step >= self.dense_steps and br.ready and rec.current is not None and rec.current[1] == step:
            return Phase.SPARSE
        return Phase.DENSE

    def __call__(self, q, k, v, step, branch, layer, sink=None, rows=None):
        B, L, H, D = q.shape
        assert B == 1, "batch size 1 only"
        if q.device != self._device:
            self._bind(q.device)
        if cdiv(L, BK) < self.min_blocks:
            return dense_attention(q, k, v, K=self.K)
        if layer in self.dense_layers:
            # a full-length layer that always runs dense: the workspace already holds the list of all blocks
            buf = self._scratch(L, H, D, q.device)
            out = torch.empty_like(q[0])
            _dense_into(self.K, q[0].contiguous(), k[0].contiguous(), v[0].contiguous(), buf, out, buf.dense_lse)
            return out[None]
        with torch.cuda.device(q.device):
            return self._step(q[0].contiguous(), k[0].contiguous(), v[0].contiguous(), step, branch, layer,
                              NO_SINK if sink is None else sink)[None]

    def _step(self, q, k, v, step, branch, layer, sink):
        L, H, D = q.shape
        K = self.K
        rec = self._record(layer, L, H, q.device)
        br = rec.branch(branch)
        buf = self._scratch(L, H, D, q.device)
        phase = self._phase(rec, br, step, branch)
        out = torch.empty_like(q)
        if phase is Phase.DENSE:
            if br.seeded:
                # a dense step that follows another step of the same video: its LSE as a fixed offset over every block
                # (one sweep of QK^T instead of the two of the online-softmax kernel), tiles that leave the safe range
                # recomputed; exact attention either way
                K.block_attention(q, k, v, out, buf.all_counts, buf.all_blocks, br.offset, br.next_offset, buf.flags,
                                  mass=None, threshold=self.threshold)
                K.exact_fallback(q, k, v, out, buf.all_counts, buf.all_blocks, br.next_offset, buf.flags)
                br.cur ^= 1
            else:
                _dense_into(K, q, k, v, buf, out, br.offset)
                br.seeded = True
            return out
        top, refined = self._budget(cdiv(L, BK))
        ps = self._sparse_scratch(L, H, q.device, cdiv(refined, 32) * 32)
        if phase is Phase.FULL:
            lists = None
            ps.lists.keep.fill_(1)                           # "kept before": every block, for the first selection
            kept = ps.lists.keep
            K.block_attention(q, k, v, out, buf.all_counts, buf.all_blocks, br.offset, br.next_offset, buf.flags,
                              mass=ps.mass if branch == 0 else None, threshold=self.threshold)
            K.exact_fallback(q, k, v, out, buf.all_counts, buf.all_blocks, br.next_offset, buf.flags)
            if branch == 0:
                K.full_step_scales(br.offset, br.next_offset, ps.scale_exact, ps.scale_skip, L)
            br.ready = True
        else:
            exact, skip = rec.plan(rec.current[0])
            lists = self._expand(rec, rec.current[0], exact, skip, ps)
            kept = lists.keep
            K.block_means(k, v, buf.k_mean, buf.v_mean)
            buf.reps.build(q, k, v)
            K.sparse_attention(q, k, v, buf.k_mean, buf.v_mean, skip, out, lists.counts, lists.blocks, br.offset,
                               br.next_offset, buf.flags, lists.refine, buf.reps.k, buf.reps.v, buf.reps.log_counts,
                               mass=ps.mass if branch == 0 else None, threshold=self.threshold)
            # tiles whose offset was too far off: online softmax over the same list, then block-mean compensation
            K.exact_fallback(q, k, v, out, lists.counts, lists.blocks, br.next_offset, buf.flags)
            K.compensate_fallback(q, buf.k_mean, buf.v_mean, lists.keep, br.next_offset, out, buf.flags)
            if branch == 0:
                K.estimate_skipped(q, buf.k_mean, lists.keep, br.offset, br.next_offset, ps.mass, ps.scale_exact,
                                   ps.scale_skip)
        if lists is not None:
            self._used_lists = lists
        elif self._used_lists is None:
            self._used_lists = ps.lists
        if branch == 0:
            self._plan_next(rec, ps, kept, buf.flags, top, refined, L, sink, step)
        br.cur ^= 1
        br.seeded = True
        return out

    def _expand(self, rec, index, exact, skip, ps):
        """The lists of plan `index`: the layer's own copy (state="layer", filled when the plan was made) or the shared
        workspace, expanded from the two bit masks now."""
        if rec.keep_lists and index in rec.expanded and rec.expanded[index].refine.shape[-1] == ps.shape[2]:
            return rec.expanded[index]
        dst = ps.lists
        self.K.rebuild_plan(exact, skip, dst.keep, dst.counts, dst.blocks, dst.refine, ps.refine_counts)
        return dst

    def _plan_next(self, rec, ps, kept, flags, top, refined, L, sink, step):
        """Branch 0, end of a step: select the next step's blocks from the map in the workspace and pack them as a plan.
        The other of the layer's two plans is written: later branches of this step still read the current one, the
        selection reads the current keep mask while it writes the next, and the masks a step ran on stay readable until
        the next step has run."""
        index = 0 if rec.current is None else rec.current[0] ^ 1
        exact, skip = rec.plan(index)
        dst = rec.lists_of(index, ps.shape[2]) if rec.keep_lists else ps.next_lists
        self.K.select_blocks(ps.mass, kept, ps.scale_exact, ps.scale_skip, dst.keep, dst.counts, dst.blocks, flags, skip,
                             dst.refine, top, refined, L, sink=sink)
        self.K.pack_plan(dst.keep, exact)
        rec.pending = (index, step + 1)
