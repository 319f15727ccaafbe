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


# ---------------------------------------------------------------------------------------------- VSA2 golden cases
# Inputs of tests/golden/vsa2.npz, rebuilt from numpy's legacy RandomState (a stable stream) on both sides.
VSA_CASES = {   # name: (B, H, NB, seed, blk_cnt kind)
    "fine": (1, 1, 5, 11, "mixed"),
    "full": (1, 1, 5, 12, "tail"),
    "route": (1, 2, 12, 13, "mixed"),
    "tiers": (1, 1, 5, 14, "mixed"),
}


def vsa_counts(nb, kind, rs):
    c = np.full(nb, 64, dtype=np.int32)
    if kind == "tail":
        c[-1] = 37
    elif kind == "mixed":
        c = rs.randint(1, 65, size=nb).astype(np.int32)
        c[0] = 64
        if nb > 2:
            c[1] = 1
    return torch.from_numpy(c)


def vsa_case(name, D=128, dtype=torch.bfloat16):
    """(q, k, v, gate, blk_cnt, dout): q, k, v [B,H,NB*64,D] with zeroed padding slots, gate [B,H,L], dout like q."""
    B, H, nb, seed, kind = VSA_CASES[name]
    rs = np.random.RandomState(seed)
    cnt = vsa_counts(nb, kind, rs)
    L = nb * 64
    pos = np.arange(L)
    valid = torch.from_numpy((pos % 64) < cnt.numpy()[pos // 64])[None, None, :, None]
    mk = lambda: (torch.from_numpy(rs.standard_normal((B, H, L, D)).astype(np.float32)) * valid).to(dtype).contiguous()
    q, k, v = mk(), mk(), mk()
    gate = torch.from_numpy((rs.standard_normal((B, H, L)) * 1.5).astype(np.float32)).to(dtype)
    dout = (torch.from_numpy(rs.standard_normal((B, H, L, D)).astype(np.float32)) * valid).to(dtype)
    return q, k, v, gate, cnt, dout


def vsa_mask(name, nb):
    """Frozen block mask [B,H,NB,NB]: 30 % random, a query block without edges, one that sees everything, a single edge."""
    B, H, _, seed, _ = VSA_CASES[name]
    rs = np.random.RandomState(seed + 100)
    m = torch.from_numpy(rs.random_sample((B, H, nb, nb)) < 0.3)
    m[:, :, 0] = False
    m[:, :, -1] = True
    if nb > 3:
        m[:, :, 2] = False
        m[:, :, 2, 1] = True
    return m


def vsa_tiers(nb):
    """Tier masks (tier A, tier A or B) [1,1,NB,NB]: A 25 %, B a further 35 %; row 0 has no tier A, row 1 is all tier C."""
    rs = np.random.RandomState(77)
    u = torch.from_numpy(rs.random_sample((1, 1, nb, nb)))
    a, ab = u < 0.25, u < 0.6
    a[:, :, 0] = False
    a[:, :, 1] = False
    ab[:, :, 1] = False
    return a, ab


# ---------------------------------------------------------------------------------------------- split-KV plan cases
POLICY = dict(min_len=4, rel_mean=4.0, tail_frac=0.05, resident=4)
SPLIT_CASES = {   # name: (mask kind, NB, heads, chunk, max_slots, policy arguments)
    "random_c2": ("random", 13, 4, 2, 10 ** 6, {}),
    "random_c3_cap10": ("random", 13, 4, 3, 10, {}),
    "hotq_c1_cap3": ("hotq", 13, 4, 1, 3, {}),
    "hotkv_c64": ("hotkv", 13, 4, 64, 10 ** 6, {}),
    "hotqkv_c2_cap0": ("hotqkv", 13, 4, 2, 0, {}),
    "full_c3": ("full", 13, 4, 3, 10 ** 6, {}),
    "policy_hotq": ("hotq", 24, 3, 2, 10 ** 6, dict(budget=16, **POLICY)),
    "policy_hotkv": ("hotkv", 24, 3, 2, 10 ** 6, dict(budget=16, **POLICY)),
    "policy_over_budget": ("hotqkv", 32, 4, 2, 10 ** 6, dict(budget=3, **POLICY)),
    "policy_cap40": ("hotqkv", 32, 4, 2, 40, dict(budget=64, **POLICY)),
}


def split_mask(kind, heads, nb, seed=5):
    """Skewed block masks [1, heads, NB, NB]: hot query rows, hot kv columns, both, with empty and single-edge rows."""
    rs = np.random.RandomState(seed + nb)
    u = lambda *s: torch.from_numpy(rs.random_sample(s))
    m = torch.zeros(1, heads, nb, nb, dtype=torch.bool)
    if kind == "full":
        m[:] = True
    elif kind == "random":
        m = u(1, heads, nb, nb) < 0.3
        m[:, :, 0] = False
        m[:, :, -1] = True
    elif kind == "hotq":
        m[:, :, 1] = True
        m[:, :, nb - 2] = u(1, heads, nb) < 0.8
        m[:, :, 3, 5] = True
    elif kind == "hotkv":
        m = u(1, heads, nb, nb) < 2.0 / nb
        m[..., 0] = True
        m[..., nb - 1] = True
        m[:, :, 2] = False
    elif kind == "hotqkv":
        m[:, :, : nb // 4] = u(1, heads, nb // 4, nb) < 0.7
        m[..., 1] = True
        m[:, :, nb // 2] = False
    else:
        raise ValueError(kind)
    return m
