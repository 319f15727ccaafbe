"""Helpers shared by the tests that use tests/golden/echosparse_step.npz."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
import make_golden as MG  # noqa: E402


def qkv(step, device="cpu"):
    """Inputs of the golden run's denoising step `step` as (L, H, 128) bf16 tensors."""
    return [torch.from_numpy(x).to(torch.bfloat16).to(device) for x in MG.golden_inputs(step)]


def bf16_from_bits(a, device="cpu"):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).to(device)


def T(a, device="cpu"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()
