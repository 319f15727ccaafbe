"""The one GPU backend: B200 (sm_100a), hand-written CUDA. Replaces the reference's multi-generation dispatch
(echosparse/backends.py:15-61): same function names, but anything that is not compute capability 10.0 raises; there is
no Triton path and no CPU fallback.
"""
import importlib

import torch

GPUS = {"b200": 10}                      # name -> compute capability major
_OTHER = ("h100", "rtx5090")             # names the reference accepts and this build refuses


def check_name(gpu):
    if gpu in _OTHER:
        raise ValueError(f"gpu={gpu!r}: this build only has the B200 (sm_100a) kernel set; use 'auto' or 'b200'")
    if gpu not in ("auto", *GPUS):
        raise ValueError(f"gpu must be 'auto' or 'b200', not {gpu!r}")


def resolve(gpu, device):
    """Backend name for `gpu` ("auto" or "b200") on `device`; raises if the device is not a compute-10.0 CUDA GPU."""
    check_name(gpu)
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError(f"EchoSparse runs on CUDA tensors; got a tensor on {device}")
    major, minor = torch.cuda.get_device_capability(device)
    if (major, minor) != (10, 0):
        # the library is compiled for sm_100a only: architecture-specific code, not forward compatible within 10.x
        raise RuntimeError(f"{device} has compute capability {major}.{minor}; this build needs a B200 (10.0)")
    return "b200"


def kernels(name):
    """Kernel module of the backend; importing it opens the native library (and raises if it was not built)."""
    if name != "b200":
        raise ValueError(f"unknown backend {name!r}")
    mod = importlib.import_module("self_trainable_or_free_attn_b200.kernels.sm100")
    from . import _native
    _native.load()
    return mod
