"""Real tokens <-> the block-padded token order that the VSA2 kernels consume.

Same contract as the reference's `echosparse/vsa/layout.py:1-128`: every 64-token block is one (tt, th, tw) tile of the
video, its valid tokens first and zero padding last; inside a tile the tokens are ordered sub-cube major ((st, sh, sw)
sub-cubes of R = st*sh*sw tokens in raster order, raster inside a sub-cube), so consecutive R tokens form one router
group; boundary tiles keep that order restricted to the tokens that exist. `gather` / `scatter` are the explicit
permutation; `to_blocked` and `from_blocked` apply it (differentiable indexing, padding stays constant zero).
"""
import math
from dataclasses import dataclass
from typing import Tuple

import torch

SUBCUBE_FOR_R = {4: (1, 2, 2), 8: (2, 2, 2), 16: (1, 4, 4), 32: (2, 4, 4)}


@dataclass
class BlockLayout:
    shape: Tuple[int, ...]
    tile: Tuple[int, ...]
    sub: Tuple[int, ...]
    gather: torch.Tensor    # [NB*64] raster token index of every padded slot, -1 for padding
    scatter: torch.Tensor   # [tokens] padded slot of every raster token
    blk_cnt: torch.Tensor   # [NB] int32

    @property
    def num_blocks(self):
        return self.blk_cnt.numel()

    @property
    def padded_len(self):
        return self.gather.numel()


def build_layout(shape, tile=(4, 4, 4), sub=None, R=8, device="cpu"):
    T, H, W = shape
    tt, th, tw = tile
    assert tt * th * tw == 64, "hardware block must hold 64 tokens"
    sub = tuple(sub) if sub is not None else SUBCUBE_FOR_R[R]
    st, sh, sw = sub
    assert tt % st == 0 and th % sh == 0 and tw % sw == 0, "sub-cube must tile the block"
    t, h, w = torch.meshgrid(torch.arange(T), torch.arange(H), torch.arange(W), indexing="ij")
    t, h, w = t.flatten(), h.flatten(), w.flatten()
    nH, nW = -(-H // th), -(-W // tw)
    block = ((t // tt) * nH + h // th) * nW + w // tw
    lt, lh, lw = t % tt, h % th, w % tw
    cube = ((lt // st) * (th // sh) + lh // sh) * (tw // sw) + lw // sw
    inner = ((lt % st) * sh + lh % sh) * sw + lw % sw
    order = torch.argsort(block * 64 + cube * (st * sh * sw) + inner)        # keys are unique
    nb = -(-T // tt) * nH * nW
    cnt = torch.bincount(block, minlength=nb)
    start = torch.cumsum(cnt, 0) - cnt
    sorted_block = block[order]
    slot = sorted_block * 64 + (torch.arange(order.numel()) - start[sorted_block])
    gather = torch.full((nb * 64,), -1, dtype=torch.int64)
    gather[slot] = order
    scatter = torch.empty(order.numel(), dtype=torch.int64)
    scatter[order] = slot
    return BlockLayout(tuple(shape), tuple(tile), sub, gather.to(device), scatter.to(device),
                       cnt.to(torch.int32).to(device))


def tail_block_counts(L_valid, device="cpu"):
    """Counts of a 1-D sequence cut into blocks of 64 consecutive tokens (the last one may be partial)."""
    nb = math.ceil(L_valid / 64)
    cnt = torch.full((nb,), 64, dtype=torch.int32)
    cnt[-1] = L_valid - 64 * (nb - 1)
    return cnt.to(device)


def sequence_layout(n, device="cpu"):
    cnt = tail_block_counts(n)
    gather = torch.full((cnt.numel() * 64,), -1, dtype=torch.int64)
    gather[:n] = torch.arange(n)
    return BlockLayout((n,), (64,), (), gather.to(device), torch.arange(n, device=device), cnt.to(device))


def to_blocked(x, lay):
    """[B, H, N, ...] real tokens -> [B, H, NB*64, ...] block-padded, padding zero."""
    out = x.new_zeros(*x.shape[:2], lay.padded_len, *x.shape[3:])
    out[:, :, lay.scatter] = x
    return out


def from_blocked(y, lay):
    """[B, H, NB*64, ...] -> [B, H, N, ...] real tokens in their original order."""
    return y[:, :, lay.scatter]


def pad_tail(x, L_valid):
    """[B, H, L_valid, D] -> zero-padded at the end to a multiple of 64 tokens."""
    nb = math.ceil(L_valid / 64)
    if nb * 64 == L_valid:
        return x.contiguous()
    out = x.new_zeros(*x.shape[:2], nb * 64, x.shape[3])
    out[:, :, :L_valid] = x
    return out
