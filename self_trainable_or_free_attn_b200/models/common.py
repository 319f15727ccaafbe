"""Pieces shared by the model integrations (reference: echosparse/models/common.py): the clock that follows a diffusers
pipeline's calls, and the Morton order that makes a 64-token block a compact 3-D patch of the latent grid."""
import functools

import torch


class Clock:
    """Denoising step, transformer forward within the step (CFG branch) and attention layer of the current call.

    Follows the pipeline's own calls: `scheduler.set_timesteps` starts a video (and runs the `on_reset` callbacks),
    `scheduler.step` ends a step, every transformer forward starts a branch; the attention dispatch advances `layer`."""

    def __init__(self, pipe, on_reset=()):
        self.step, self.branch, self.layer = 0, -1, 0
        self._on_reset = list(on_reset)
        sched = pipe.scheduler
        inner_set, inner_step = sched.set_timesteps, sched.step

        @functools.wraps(inner_set)
        def set_timesteps(*args, **kwargs):
            self.step, self.branch = 0, -1
            for fn in self._on_reset:
                fn()
            return inner_set(*args, **kwargs)

        @functools.wraps(inner_step)
        def step(*args, **kwargs):
            self.step += 1
            self.branch = -1
            return inner_step(*args, **kwargs)

        sched.set_timesteps = set_timesteps
        sched.step = step
        pipe.transformer.register_forward_pre_hook(self._begin_forward)

    def _begin_forward(self, _module, _args):
        self.branch += 1
        self.layer = 0


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
