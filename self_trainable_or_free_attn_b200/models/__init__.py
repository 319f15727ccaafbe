"""Routing a diffusers pipeline's self-attention through `EchoSparseAttention` (reference: echosparse/models/__init__.py).

`enable(pipe)` recognises the model family by the class name of the pipeline's transformer and installs that family's hooks.
The integrations patch functions of `diffusers` and import it when they are used; without it they raise ImportError."""
import importlib

from ..attention import EchoSparseAttention

# Settings of the reported results (the reference's table: the same on every GPU generation).
PRESETS = {
    "wan": dict(density=0.10, dense_steps=10, dense_layers=(0,)),
    "hunyuan_video": dict(density=0.10, dense_steps=10, dense_layers=()),
    "minimax_h3": dict(density=0.10, dense_steps=10, dense_layers=(0,)),
}

# class-name prefix of the transformer -> (family, module with that family's `enable(pipe, attention)`)
FAMILIES = {
    "WanTransformer": ("wan", "wan"),
    "HunyuanVideoTransformer": ("hunyuan_video", "hunyuan_video"),
    "MiniMaxH3": ("minimax_h3", "minimax_h3"),
}


def _lookup(pipe):
    cls = type(pipe.transformer).__name__
    for prefix, entry in FAMILIES.items():
        if cls.startswith(prefix):
            return entry
    raise ValueError(f"unsupported transformer {cls}: expected one of {sorted(FAMILIES)}")


def model_family(pipe):
    return _lookup(pipe)[0]


def settings(family, preset=None, **overrides):
    """Constructor arguments of the attention for a model family: the family's preset, or a named preset of that
    family, with `overrides` on top."""
    name = family if preset is None else preset
    mine = sorted(p for p in PRESETS if p.startswith(family))
    if name not in mine:
        raise ValueError(f"preset {name!r} is not a {family} preset; have {mine}")
    chosen = dict(PRESETS[name])
    chosen.update(overrides)
    return chosen


def enable(pipe, preset=None, gpu="auto", **overrides):
    """Routes the pipeline's self-attention through EchoSparse attention and returns the attention object. `preset` names
    an entry of PRESETS (default: the model's own); `overrides` replace its values (density, dense_steps, dense_layers,
    refine_iters, state). `gpu`: "auto" or "b200"."""
    family, module = _lookup(pipe)
    attention = EchoSparseAttention(gpu=gpu, **settings(family, preset, **overrides))
    importlib.import_module(f"{__name__}.{module}").enable(pipe, attention)
    return attention
