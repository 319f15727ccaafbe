"""Model-integration helpers that need neither a GPU nor diffusers: the Morton order (with the reference's golden vector,
tests/test_attention.py:152-155 of the reference), the clock on a fake pipeline, presets and family detection."""
import types

import pytest
import torch

from self_trainable_or_free_attn_b200 import models
from self_trainable_or_free_attn_b200.models import common


def test_morton_order_golden_vector_and_permutation():
    perm, inv = common.grid_morton_order(5, 6, 7, "cpu")
    assert torch.equal(perm[inv], torch.arange(5 * 6 * 7))
    assert perm[:8].tolist() == [0, 1, 7, 8, 42, 43, 49, 50]          # the 2 x 2 x 2 cube at the origin
    # codes ascend along the order
    t, y, x = torch.meshgrid(torch.arange(5), torch.arange(6), torch.arange(7), indexing="ij")
    code = common._spread3(x.flatten()) | (common._spread3(y.flatten()) << 1) | (common._spread3(t.flatten()) << 2)
    assert (code[perm][1:] > code[perm][:-1]).all()


class _Sched:
    def __init__(self):
        self.calls = []

    def set_timesteps(self, n):
        self.calls.append(("set", n))
        return n

    def step(self, x):
        self.calls.append(("step", x))
        return x


class WanTransformerFake(torch.nn.Module):
    def forward(self, x):
        return x


def test_clock_follows_the_pipeline():
    pipe = types.SimpleNamespace(scheduler=_Sched(), transformer=WanTransformerFake())
    resets = []
    clock = common.Clock(pipe, on_reset=[lambda: resets.append(1)])
    assert pipe.scheduler.set_timesteps(50) == 50 and resets == [1]
    for step in range(3):
        for branch in range(2):                       # two transformer forwards per step (CFG)
            pipe.transformer(torch.zeros(1))
            assert (clock.step, clock.branch, clock.layer) == (step, branch, 0)
            clock.layer += 5
        assert pipe.scheduler.step(7) == 7
    assert clock.step == 3 and clock.branch == -1
    pipe.scheduler.set_timesteps(10)
    assert clock.step == 0 and len(resets) == 2 and pipe.scheduler.calls[0] == ("set", 50)


def test_presets_and_family():
    pipe = types.SimpleNamespace(transformer=WanTransformerFake())
    WanTransformerFake.__name__ = "WanTransformer3DModel"
    assert models.model_family(pipe) == "wan"
    assert models.settings("wan", density=0.2) == dict(density=0.2, dense_steps=10, dense_layers=(0,))
    assert models.settings("hunyuan_video")["dense_layers"] == ()
    assert models.settings("minimax_h3") == dict(density=0.10, dense_steps=10, dense_layers=(0,))
    WanTransformerFake.__name__ = "MiniMaxH3Transformer3DModel"
    assert models.model_family(pipe) == "minimax_h3"
    with pytest.raises(ValueError, match="not a wan preset"):
        models.settings("wan", preset="hunyuan_video")
    pipe.transformer = torch.nn.Linear(1, 1)
    with pytest.raises(ValueError, match="unsupported transformer"):
        models.model_family(pipe)


def test_enable_needs_diffusers():
    pytest.importorskip("torch")
    try:
        import diffusers  # noqa: F401
        pytest.skip("diffusers is installed: the integration is exercised by its own pipelines")
    except ImportError:
        pass
    pipe = types.SimpleNamespace(scheduler=_Sched(), transformer=WanTransformerFake())
    WanTransformerFake.__name__ = "WanTransformer3DModel"
    with pytest.raises(ImportError):
        models.enable(pipe)


def test_minimax_h3_layout_brings_the_target_video_to_the_front_in_morton_order():
    """Packed sequence [text | conditioning frame | audio | target video]: the target video is the last run of
    consecutive video positions; its rotary t coordinate is strided and must be ranked before the Morton code."""
    from self_trainable_or_free_attn_b200.models.common import morton_order
    from self_trainable_or_free_attn_b200.models.minimax_h3 import SequenceLayout
    text, cond, audio, (f, h, w) = 5, 4, 3, (2, 2, 4)
    nv = f * h * w
    L = text + cond + audio + nv
    pos = torch.zeros(L, 3, dtype=torch.long)
    t, y, x = torch.meshgrid(torch.arange(f) * 4 + 7, torch.arange(h), torch.arange(w), indexing="ij")
    start = L - nv
    pos[start:] = torch.stack([t.flatten(), y.flatten(), x.flatten()], 1)
    video_indices = torch.cat([torch.arange(text, text + cond), torch.arange(start, L)])
    lay = SequenceLayout(pos, video_indices)
    assert (lay.L, lay.prefix, lay.video) == (L, start, nv)
    perm, _ = morton_order((t.flatten() - 7) // 4, y.flatten(), x.flatten())
    assert torch.equal(lay.gather[:nv], perm + start) and torch.equal(lay.gather[nv:], torch.arange(start))
    assert torch.equal(lay.gather[lay.scatter], torch.arange(L))
    # without conditioning frames the video positions are one run
    lay2 = SequenceLayout(pos, torch.arange(start, L))
    assert lay2.prefix == start and lay2.matches(pos) and not lay2.matches(pos[:-1])
