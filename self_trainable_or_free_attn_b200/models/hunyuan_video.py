"""HunyuanVideo text-to-video (diffusers `HunyuanVideoPipeline`; reference: echosparse/models/hunyuan_video.py).

Its dual- and single-stream blocks attend over [video tokens | text tokens padded to a fixed length] under a key-padding
mask. Here the padding is cut off (the number of valid text tokens is read from the mask once per video), the video tokens
are put in Morton order and the valid text tokens follow them as the sink every query tile computes exactly; text query rows
attend densely; padded rows come back as zeros (`common.attend`). Attention calls that are not this joint attention (the
token refiner) keep diffusers' own dispatcher. One transformer forward per step (embedded guidance)."""
import torch

from . import common

_state = {}


class JointAttention:
    def __init__(self, pipe, attention):
        self.attention = attention
        self.clock = common.Clock(pipe, on_reset=[attention.reset, self._forget_text], on_step=[attention.check_status])
        cfg = pipe.transformer.config
        self.patch = (cfg.patch_size_t, cfg.patch_size, cfg.patch_size)
        self.video_len = 0
        self.text_len = None                 # valid text tokens of this video, known after the first joint call
        self._perm = None
        self._seq = None
        pipe.transformer.register_forward_pre_hook(self._latent_shape, with_kwargs=True)

    def _forget_text(self):
        self.text_len, self._seq = None, None

    def _latent_shape(self, _module, args, kwargs):
        latent = kwargs.get("hidden_states", args[0] if args else None)
        grid = tuple(n // p for n, p in zip(latent.shape[2:], self.patch))
        n = grid[0] * grid[1] * grid[2]
        if n != self.video_len:
            self.video_len, self._seq = n, None
        self._perm = common.grid_morton_order(*grid, latent.device)[0]

    def is_joint(self, query, key, value, attn_mask, dropout_p, is_causal, scale, parallel_config):
        plain = dropout_p == 0.0 and not is_causal and scale is None and parallel_config is None
        return (plain and attn_mask is not None and query.shape == key.shape == value.shape
                and query.shape[1] > self.video_len)

    def sequence(self, mask, device):
        if self.text_len is None:
            m = mask.reshape(mask.shape[0], -1)
            valid = m if m.dtype == torch.bool else m > -1.0
            self.text_len = int(valid[0, self.video_len:].sum())         # one host synchronisation per video
            self._seq = None
        if self._seq is None:
            tail = torch.arange(self.video_len, self.video_len + self.text_len, device=device)
            self._seq = common.VideoFirst(torch.cat([self._perm, tail]), self.video_len)
        return self._seq

    def __call__(self, query, key, value, mask):
        return common.attend(self.attention, self.clock, query, key, value, self.sequence(mask, query.device))


def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
             attention_kwargs=None, *, backend=None, parallel_config=None):
    joint = _state["joint"]
    if joint.is_joint(query, key, value, attn_mask, dropout_p, is_causal, scale, parallel_config):
        return _state["op"](query.contiguous(), key.contiguous(), value.contiguous(), attn_mask)
    return _state["diffusers"](query, key, value, attn_mask, dropout_p, is_causal, scale, enable_gqa, attention_kwargs,
                               backend=backend, parallel_config=parallel_config)


def enable(pipe, attention):
    from diffusers.models.transformers import transformer_hunyuan_video as hv      # raises ImportError without diffusers
    _state.setdefault("diffusers", hv.dispatch_attention_fn)
    if "op" not in _state:
        _state["op"] = common.register_op("hunyuan_joint_attention", lambda q, k, v, m: _state["joint"](q, k, v, m), 4)
    _state["joint"] = JointAttention(pipe, attention)
    hv.dispatch_attention_fn = dispatch
    return _state["joint"]
