"""Pieces the model integrations share: the clock that turns a diffusers pipeline's own calls into (step, branch, layer),
the Morton order that makes a 64-token block a compact 3-D patch of the latent grid, the description of a token sequence
as [video tokens | conditioning tokens] with the one attention routine all model families use, and the registration of
the attention calls as torch custom ops (reference: echosparse/models/common.py and the three model files beside it)."""
import functools

import torch

from ..attention import BK, dense_attention


def _run_before(obj, name, hook):
    """Replaces obj.name by a function that runs `hook()` and then the original."""
    inner = getattr(obj, name)

    @functools.wraps(inner)
    def wrapped(*args, **kwargs):
        hook()
        return inner(*args, **kwargs)
    setattr(obj, name, wrapped)


class Clock:
    """Where a pipeline is: denoising `step`, transformer forward within the step (`branch`: 0 conditional, 1
    unconditional, ...) and attention `layer` within the forward. It listens to the pipeline's own calls:
    `scheduler.set_timesteps` begins a video (runs `on_reset`), `scheduler.step` ends a denoising step (runs `on_step`),
    a transformer forward begins a branch. The attention call of a layer reads the three numbers and advances `layer`."""

    def __init__(self, pipe, on_reset=(), on_step=()):
        self.step, self.branch, self.layer = 0, -1, 0
        self.on_reset, self.on_step = list(on_reset), list(on_step)
        _run_before(pipe.scheduler, "set_timesteps", self._video_begins)
        _run_before(pipe.scheduler, "step", self._step_ends)
        pipe.transformer.register_forward_pre_hook(self._forward_begins)

    def _video_begins(self):
        self.step, self.branch = 0, -1
        for fn in self.on_reset:
            fn()

    def _step_ends(self):
        self.step, self.branch = self.step + 1, -1
        for fn in self.on_step:
            fn()

    def _forward_begins(self, _module, _args):
        self.branch, self.layer = self.branch + 1, 0

    def tick(self):
        """(step, branch, layer) of the attention call that is about to run; the next call is the next layer."""
        now = (self.step, self.branch, self.layer)
        self.layer += 1
        return now


# ------------------------------------------------------------------------------------------------------------ Morton order
def _spread3(v):
    """Bits of v (up to 21) moved to every third position: bit i -> bit 3 i."""
    out = torch.zeros_like(v)
    for i in range(21):
        out |= ((v >> i) & 1) << (3 * i)
    return out


def morton_order(t, y, x):
    """Permutation that sorts tokens with integer coordinates (t, y, x) along a 3-D Morton curve (x in the lowest bit
    of every triple, then y, then t), and its inverse."""
    code = _spread3(x) | (_spread3(y) << 1) | (_spread3(t) << 2)
    perm = torch.argsort(code)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=perm.device)
    return perm, inv


@functools.lru_cache(maxsize=8)
def grid_morton_order(frames, height, width, device):
    """Morton order of a (frames, height, width) token grid stored in raster order: (perm, inverse) on `device`."""
    t, y, x = torch.meshgrid(torch.arange(frames), torch.arange(height), torch.arange(width), indexing="ij")
    perm, inv = morton_order(t.flatten(), y.flatten(), x.flatten())
    return perm.to(device), inv.to(device)


# ------------------------------------------------------------------------------------------------------------ sequences
class VideoFirst:
    """A model's token sequence seen as [video tokens in Morton order | conditioning tokens].

    `gather[i]` is the position, in the model's own order, of the token that sits at place i of that arrangement; the
    first `video` places are the video tokens, the others (text, conditioning frames, audio) follow in their own order.
    The sparse kernels see the conditioning blocks as a sink every tile computes exactly, which needs the video part to
    fill whole 64-token blocks."""

    def __init__(self, gather, video):
        self.gather = gather
        self.scatter = torch.argsort(gather)
        self.video = int(video)
        self.total = int(gather.numel())

    @property
    def conditioning(self):
        return self.total - self.video


def attend(attention, clock, q, k, v, seq):
    """Self-attention of [1, L, H, 128] tensors whose first `seq.total` tokens follow `seq`; tokens past that are padding
    and come back as zeros. Video rows go through the sparse processor (conditioning blocks as the sink), conditioning
    rows attend densely to everything; rows return in the model's own order."""
    step, branch, layer = clock.tick()
    n, nv = seq.total, seq.video
    qg, kg, vg = (x[:, :n].index_select(1, seq.gather) for x in (q, k, v))
    sink = nv // BK if seq.conditioning else None
    o = attention(qg, kg, vg, step, branch, layer, sink=sink, rows=nv)
    if seq.conditioning:
        o = torch.cat([o[:, :nv], dense_attention(qg[:, nv:].contiguous(), kg, vg)], 1)
    out = torch.zeros_like(q) if q.shape[1] > n else torch.empty_like(q)
    out[:, :n] = o.index_select(1, seq.scatter)
    return out


# ------------------------------------------------------------------------------------------------------------ custom ops
def register_op(name, fn, n_tensors):
    """Registers `fn` (tensors in, one tensor shaped like the first out) as the torch custom op `echosparse::<name>`, the
    name the reference registers, so that code looking the op up finds it; when that name is taken (both packages in one
    process) the op goes to `echosparse_b200::<name>`. Returns the callable op."""
    args = ", ".join(f"Tensor a{i}" for i in range(n_tensors))
    for ns in ("echosparse", "echosparse_b200"):
        try:
            op = torch.library.custom_op(f"{ns}::{name}", fn, mutates_args=(), schema=f"({args}) -> Tensor")
        except RuntimeError:
            continue
        op.register_fake(lambda first, *rest: torch.empty_like(first))
        return op
    raise RuntimeError(f"could not register the custom op {name}")
