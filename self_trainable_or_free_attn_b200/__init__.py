"""B200-native implementation of EchoSparse's sparse attention step (shaoshitong/self_trainable_or_free_attn).

Public names of the reference's package root (echosparse/__init__.py:1-5): `EchoSparseAttention`, `PRESETS`, `enable`.
`offload_blocks` (weight offload for small GPUs) is outside this library: a B200 holds the models the presets name.
`kernels.sm100` is the kernel-set module the attention processor calls; the CUDA code lives in `csrc/` behind the C ABI
declared in `include/echosparse_sm100.h`; `vsa` holds the VSA2 entry points.
"""
__version__ = "0.2.0"
__all__ = ["EchoSparseAttention", "PRESETS", "enable"]


def __getattr__(name):
    # resolved on first use, so that `import self_trainable_or_free_attn_b200` alone needs neither torch nor the library
    if name == "EchoSparseAttention":
        from .attention import EchoSparseAttention
        return EchoSparseAttention
    if name in ("PRESETS", "enable"):
        from . import models
        return getattr(models, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
