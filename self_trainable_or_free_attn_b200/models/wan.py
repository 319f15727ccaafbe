"""Wan2.1 text-to-video (diffusers `WanPipeline`; reference: echosparse/models/wan.py).

Every token of Wan's self-attention is a video token, so instead of reordering q, k, v in every layer the hidden states
(and the rotary embedding) are put in Morton order once, in front of the first transformer block, and put back behind the
last; a 64-token block then covers a compact 3-D patch instead of part of one image row. Self-attention goes through the
sparse processor, cross-attention (text keys) through the dense kernel."""
import torch

from ..attention import dense_attention
from . import common

_ops = {}


class SelfAttention:
    """One self-attention layer: the clock says which (step, branch, layer) it is."""

    def __init__(self, attention, clock):
        self.attention, self.clock = attention, clock

    def __call__(self, q, k, v):
        return self.attention(q, k, v, *self.clock.tick())


class MortonHooks:
    """Keeps the tokens in Morton order between the first and the last transformer block.

    The grid comes from the shape of the latent given to the transformer and its patch size; the permutation is applied
    to the hidden states entering block 0 and to the (cos, sin) rotary tables, and undone on the output of the last block."""

    def __init__(self, transformer):
        self.patch = tuple(transformer.config.patch_size)
        self.perm = self.inv = None
        rope = transformer.rope.forward
        transformer.rope.forward = lambda hidden: tuple(t.index_select(1, self.perm) for t in rope(hidden))
        transformer.register_forward_pre_hook(self._latent_shape, with_kwargs=True)
        transformer.blocks[0].register_forward_pre_hook(self._reorder_in)
        transformer.blocks[-1].register_forward_hook(self._reorder_out)

    def _latent_shape(self, _module, args, kwargs):
        latent = kwargs.get("hidden_states", args[0] if args else None)
        grid = tuple(n // p for n, p in zip(latent.shape[2:], self.patch))
        self.perm, self.inv = common.grid_morton_order(*grid, latent.device)

    def _reorder_in(self, _module, args):
        return (args[0].index_select(1, self.perm), *args[1:])

    def _reorder_out(self, _module, _args, out):
        return out.index_select(1, self.inv)


def dispatch(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False,
             attention_kwargs=None, *, backend=None, parallel_config=None):
    """Stands in for diffusers' `dispatch_attention_fn` inside the Wan transformer ([B, N, H, D] tensors): equal lengths
    are self-attention, anything else is cross-attention."""
    if attn_mask is not None or dropout_p != 0.0 or is_causal or scale is not None:
        raise ValueError("Wan attention is called without mask, dropout, causality or a custom scale")
    kind = "self" if key.shape[1] == query.shape[1] else "cross"
    return _ops[kind](query.contiguous(), key.contiguous(), value.contiguous())


def enable(pipe, attention, morton=True):
    from diffusers.models.transformers import transformer_wan       # raises ImportError without diffusers
    clock = common.Clock(pipe, on_reset=[attention.reset], on_step=[attention.check_status])
    layer = SelfAttention(attention, clock)
    if not _ops:
        _ops["self"] = common.register_op("wan_self_attention", lambda q, k, v: _ops["impl"](q, k, v), 3)
        _ops["cross"] = common.register_op("wan_cross_attention", lambda q, k, v: dense_attention(q, k, v), 3)
    _ops["impl"] = layer
    transformer_wan.dispatch_attention_fn = dispatch
    if morton:
        MortonHooks(pipe.transformer)
    return layer
