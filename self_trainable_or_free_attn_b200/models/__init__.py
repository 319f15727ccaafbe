"""Routing a diffusers pipeline's self-attention through `EchoSparseAttention` (reference: echosparse/models/__init__.py).

`enable(pipe)` picks the integration from the transformer's class name. The integrations themselves patch functions of
`diffusers`, which they import when they are used; without `diffusers` installed they raise ImportError."""
from ..attention import EchoSparseAttention

# Settings of the reported results; the same on every GPU generation of the reference.
PRESETS = {
    "wan": dict(density=0.10, dense_steps=10, dense_layers=(0,)),
    "hunyuan_video": dict(density=0.10, dense_steps=10, dense_layers=()),
    "minimax_h3": dict(density=0.10, dense_steps=10, dense_layers=(0,)),
}


def model_family(pipe):
    name = type(pipe.transformer).__name__
    for prefix, family in (("WanTransformer", "wan"), ("HunyuanVideoTransformer", "hunyuan_video"),
                           ("MiniMaxH3", "minimax_h3")):
        if name.startswith(prefix):
            return family
    raise ValueError(f"unsupported transformer {name}")


def settings(family, preset=None, **overrides):
    """Attention settings of a model family: its preset (or the named one) with `overrides` applied."""
    preset = preset or family
    if preset not in PRESETS or not preset.startswith(family):
        raise ValueError(f"preset {preset!r} is not a {family} preset; have "
                         f"{sorted(p for p in PRESETS if p.startswith(family))}")
    return {**PRESETS[preset], **overrides}


def enable(pipe, preset=None, gpu="auto", **overrides):
    """Routes the pipeline's self-attention through EchoSparse attention and returns the attention object. `preset` names
    an entry of PRESETS (default: the model's own); `overrides` replace its values (density, dense_steps, dense_layers,
    refine_iters, state). `gpu`: "auto" or "b200"."""
    family = model_family(pipe)
    attention = EchoSparseAttention(**settings(family, preset, **overrides), gpu=gpu)
    if family == "wan":
        from . import wan
        wan.enable(pipe, attention)
    elif family == "hunyuan_video":
        from . import hunyuan_video
        hunyuan_video.enable(pipe, attention)
    else:
        from . import minimax_h3
        minimax_h3.enable(pipe, attention)
    return attention
