"""MiniMax-H3 text-to-video-and-audio (diffusers' minimax-h3 `ModularPipeline`; reference: echosparse/models/minimax_h3.py).

H3 attends without a mask over one packed sequence [text | conditioning | audio | target video]. The target video is the
contiguous tail of the video token positions; everything before it is the prefix. Per attention call the tokens are gathered
into [target video in Morton order | prefix]: the video query rows go through EchoSparse attention with the prefix keys as a
sink that every tile computes exactly, the prefix query rows attend densely to all keys, and the rows are scattered back to
H3's own order. The Morton order comes from the rotary (t, h, w) coordinates of the video tokens, ranked per axis because t is
strided. Calls of other lengths (text-only rows before packing) keep diffusers' dispatcher. The checkpoint is
guidance-distilled: one transformer forward per step. This is the reference's B200 path (per-layer gathers, diffusers' own
rotary embedding); its RTX 5090 path, which remaps the model's index arguments once per forward, is not part of this library.
"""
import torch

from ..attention import BK, dense_attention
from .common import Clock, morton_order

_video_impl = None
_original_dispatch = None


class SequenceLayout:
    """Where the target video sits in the packed sequence and the gather that brings it, Morton-ordered, to the front.

    `position_ids` [L, 3] are the rotary (t, y, x) coordinates of every token, `video_indices` the positions of all video
    tokens (conditioning frames first): the target video is the last run of consecutive positions in it."""

    def __init__(self, position_ids, video_indices):
        L = int(position_ids.shape[0])
        steps = video_indices[1:] - video_indices[:-1]
        jumps = (steps != 1).nonzero()
        first = int(jumps[-1]) + 1 if jumps.numel() else 0           # one host synchronisation per layout
        start = int(video_indices[first])
        axes = [torch.unique(position_ids[start:, a], return_inverse=True)[1].long() for a in range(3)]
        perm, _ = morton_order(*axes)
        self.L, self.prefix, self.video = L, start, L - start
        self.gather = torch.cat([perm + start, torch.arange(start, device=perm.device)])
        self.scatter = torch.argsort(self.gather)

    def matches(self, position_ids):
        return position_ids.shape[0] == self.L


class VideoAttention:
    """The attention call of a packed H3 sequence: `(q, k, v) [1, L, H, 128] -> out [1, L, H, 128]` in H3's token order."""

    def __init__(self, pipe, attention):
        self.attention = attention
        self.clock = Clock(pipe, on_reset=[attention.reset])
        self.layout = None
        pipe.transformer.register_forward_pre_hook(self._set_layout, with_kwargs=True)

    @property
    def seq_len(self):
        return None if self.layout is None else self.layout.L

    def _set_layout(self, _module, args, kwargs):
        pos = kwargs["position_ids"]
        if self.layout is None or not self.layout.matches(pos):
            self.layout = SequenceLayout(pos, kwargs["video_indices"])

    def __call__(self, q, k, v):
        lay, c = self.layout, self.clock
        nv, np_ = lay.video, lay.prefix
        o = self.attention(*(x.index_select(1, lay.gather) for x in (q, k, v)), c.step, c.branch, c.layer,
                           sink=nv // BK, rows=nv)
        out = torch.empty_like(q)
        out[:, np_:] = o[:, :nv].index_select(1, lay.scatter[np_:])
        if np_:
            out[:, :np_] = dense_attention(q[:, :np_].contiguous(), k, v)
        c.layer += 1
        return out


def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
             attention_kwargs=None, *, backend=None, parallel_config=None):
    if query.shape[1] != _video_impl.seq_len:
        return _original_dispatch(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                  scale=scale, enable_gqa=enable_gqa, attention_kwargs=attention_kwargs, backend=backend,
                                  parallel_config=parallel_config)
    if attn_mask is not None or dropout_p != 0.0 or is_causal or scale is not None or parallel_config is not None:
        raise ValueError("the packed H3 sequence is attended without mask, dropout, causality, custom scale or sharding")
    return _video_impl(query.contiguous(), key.contiguous(), value.contiguous())


def enable(pipe, attention):
    global _video_impl, _original_dispatch
    from diffusers.models.transformers import transformer_minimax_h3 as th3        # raises ImportError without diffusers
    if _original_dispatch is None:
        _original_dispatch = th3.dispatch_attention_fn
    _video_impl = VideoAttention(pipe, attention)
    th3.dispatch_attention_fn = dispatch
