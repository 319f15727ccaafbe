"""The HunyuanVideo joint-attention path and the Wan self-attention path on fake pipelines (no diffusers needed): Morton
order in and out, text tokens as a sink block, cropped padding, clock-driven (step, branch, layer)."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


class _Sched:
    def set_timesteps(self, n):
        return n

    def step(self, x):
        return x


class _Transformer(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.config = types.SimpleNamespace(patch_size_t=1, patch_size=2, )

    def forward(self, hidden_states=None):
        return hidden_states


def _dense(q, k, v):
    s = torch.einsum("blhd,bmhd->bhlm", q.float(), k.float()) / q.shape[-1] ** 0.5
    return torch.einsum("bhlm,bmhd->blhd", torch.softmax(s, -1), v.float())


def test_hunyuan_joint_attention_on_a_fake_pipeline():
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    from self_trainable_or_free_attn_b200.models import hunyuan_video as hv
    pipe = types.SimpleNamespace(scheduler=_Sched(), transformer=_Transformer())
    attn = EchoSparseAttention(density=1.0, dense_steps=2, dense_layers=(), min_blocks=1)
    joint = hv.JointAttention(pipe, attn)
    f, h, w = 4, 32, 32                                   # latent grid -> 4 x 16 x 16 = 1024 video tokens
    vl, text_pad, text_valid, H, D = 1024, 40, 24, 2, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    pipe.scheduler.set_timesteps(4)
    for step in range(4):
        pipe.transformer(hidden_states=torch.zeros(1, 16, f, h, w, device="cuda"))
        assert joint.video_len == vl
        q, k, v = (torch.randn(1, vl + text_pad, H, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
        mask = torch.zeros(1, 1, 1, vl + text_pad, dtype=torch.bool, device="cuda")
        mask[..., : vl + text_valid] = True
        assert joint.is_joint(q, k, v, mask, 0.0, False, None, None)
        out = joint(q, k, v, mask)
        L = vl + text_valid
        ref = _dense(q[:, :L], k[:, :L], v[:, :L])
        err = ((out[:, :L].float() - ref).norm() / ref.norm()).item()
        assert err < 1e-2, (step, err)
        assert (out[:, L:] == 0).all(), "padded text rows stay zero"
        assert joint.clock.layer == 1 and joint.clock.step == step
        pipe.scheduler.step(0)
    assert joint.text_len == text_valid
    pipe.scheduler.set_timesteps(4)
    assert joint.text_len is None


def test_wan_self_attention_and_morton_hooks():
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    from self_trainable_or_free_attn_b200.models import common, wan
    pipe = types.SimpleNamespace(scheduler=_Sched(), transformer=_Transformer())
    attn = EchoSparseAttention(density=1.0, dense_steps=2, dense_layers=(), min_blocks=1)
    clock = common.Clock(pipe, on_reset=[attn.reset])
    call = wan.SelfAttention(attn, clock)
    g = torch.Generator(device="cuda").manual_seed(1)
    pipe.scheduler.set_timesteps(3)
    for step in range(3):
        for branch in range(2):
            pipe.transformer(hidden_states=torch.zeros(1))
            for layer in range(2):
                q, k, v = (torch.randn(1, 1024, 2, 128, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
                out = call(q, k, v)
                ref = _dense(q, k, v)
                assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
            assert clock.layer == 2 and clock.branch == branch
        pipe.scheduler.step(0)
    assert sorted(attn._states) == [(0, 0), (0, 1), (1, 0), (1, 1)]
    # Morton order as index_select on the token axis: restoring gives the input back
    perm, inv = common.grid_morton_order(4, 16, 16, torch.device("cuda"))
    x = torch.randn(1, 1024, 8, device="cuda")
    assert torch.equal(x.index_select(1, perm).index_select(1, inv), x)


class _H3Transformer(torch.nn.Module):
    def forward(self, hidden_states=None, position_ids=None, video_indices=None):
        return hidden_states


def test_minimax_h3_packed_sequence_on_a_fake_pipeline():
    """[text | conditioning | audio | target video]: video rows through the sparse path (every block kept, so the result
    must equal dense attention over the whole packed sequence), prefix rows dense, rows back in the model's order."""
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    from self_trainable_or_free_attn_b200.models import minimax_h3 as h3
    pipe = types.SimpleNamespace(scheduler=_Sched(), transformer=_H3Transformer())
    attn = EchoSparseAttention(density=1.0, dense_steps=2, dense_layers=(), min_blocks=1)
    video = h3.VideoAttention(pipe, attn)
    prefix, (f, h, w), H, D = 72, (4, 16, 16), 2, 128
    nv = f * h * w
    L = prefix + nv
    pos = torch.zeros(L, 3, dtype=torch.long, device="cuda")
    t, y, x = torch.meshgrid(torch.arange(f) * 3 + 2, torch.arange(h), torch.arange(w), indexing="ij")
    pos[prefix:] = torch.stack([t.flatten(), y.flatten(), x.flatten()], 1).cuda()
    video_indices = torch.cat([torch.arange(40, 56), torch.arange(prefix, L)]).cuda()
    g = torch.Generator(device="cuda").manual_seed(0)
    pipe.scheduler.set_timesteps(4)
    for step in range(4):
        pipe.transformer(hidden_states=torch.zeros(1, device="cuda"), position_ids=pos, video_indices=video_indices)
        assert video.seq_len == L and video.layout.prefix == prefix
        q, k, v = (torch.randn(1, L, H, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
        out = video(q, k, v)
        ref = _dense(q, k, v)
        err = ((out.float() - ref).norm() / ref.norm()).item()
        assert err < 1e-2, (step, err)
        assert video.clock.layer == 1 and video.clock.step == step
        pipe.scheduler.step(0)
