"""MiniMax-H3 text-to-video-and-audio (diffusers' minimax-h3 `ModularPipeline`; reference: echosparse/models/minimax_h3.py).

H3 attends without a mask over one packed sequence [text | conditioning frames | audio | target video]. The target video is
the last run of consecutive positions among the video tokens; everything before it is the prefix. Per attention call the
tokens are gathered into [target video in Morton order | prefix] and handled by `common.attend`: video rows through the
sparse processor with the prefix as the sink, prefix rows densely, rows back in H3's order. The Morton code is taken from
the rotary (t, y, x) coordinates of the video tokens, ranked per axis because t is strided. Calls of other lengths keep
diffusers' dispatcher. The checkpoint is guidance-distilled: one transformer forward per step. This is the per-layer-gather
path; the reference's variant that remaps the model's index arguments once per forward is not part of this library."""
import torch

from . import common

_state = {}


class SequenceLayout(common.VideoFirst):
    """`position_ids` [L, 3]: rotary (t, y, x) of every token; `video_indices`: positions of all video tokens, the
    conditioning frames first. Attributes: L, prefix (tokens before the target video), video, gather, scatter."""

    def __init__(self, position_ids, video_indices):
        L = int(position_ids.shape[0])
        breaks = (video_indices[1:] - video_indices[:-1] != 1).nonzero().flatten()
        run = int(breaks[-1]) + 1 if breaks.numel() else 0               # one host synchronisation per layout
        start = int(video_indices[run])
        ranks = [torch.unique(position_ids[start:, axis], return_inverse=True)[1].long() for axis in range(3)]
        perm, _ = common.morton_order(*ranks)
        super().__init__(torch.cat([perm + start, torch.arange(start, device=perm.device)]), L - start)
        self.L, self.prefix = L, start

    def matches(self, position_ids):
        return int(position_ids.shape[0]) == self.L


class VideoAttention:
    """The attention call of a packed H3 sequence: (q, k, v) [1, L, H, 128] -> out [1, L, H, 128] in H3's token order."""

    def __init__(self, pipe, attention):
        self.attention = attention
        self.clock = common.Clock(pipe, on_reset=[attention.reset], on_step=[attention.check_status])
        self.layout = None
        pipe.transformer.register_forward_pre_hook(self._packing, with_kwargs=True)

    @property
    def seq_len(self):
        return self.layout.L if self.layout is not None else None

    def _packing(self, _module, args, kwargs):
        pos = kwargs["position_ids"]
        if self.layout is None or not self.layout.matches(pos):
            self.layout = SequenceLayout(pos, kwargs["video_indices"])

    def __call__(self, q, k, v):
        return common.attend(self.attention, self.clock, q, k, v, self.layout)


def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
             attention_kwargs=None, *, backend=None, parallel_config=None):
    video = _state["video"]
    if query.shape[1] != video.seq_len:
        return _state["diffusers"](query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                   scale=scale, enable_gqa=enable_gqa, attention_kwargs=attention_kwargs,
                                   backend=backend, parallel_config=parallel_config)
    if attn_mask is not None or dropout_p != 0.0 or is_causal or scale is not None or parallel_config is not None:
        raise ValueError("the packed H3 sequence is attended without mask, dropout, causality, custom scale or sharding")
    return video(query.contiguous(), key.contiguous(), value.contiguous())


def enable(pipe, attention):
    from diffusers.models.transformers import transformer_minimax_h3 as th3        # raises ImportError without diffusers
    _state.setdefault("diffusers", th3.dispatch_attention_fn)
    _state["video"] = VideoAttention(pipe, attention)
    th3.dispatch_attention_fn = dispatch
    return _state["video"]
