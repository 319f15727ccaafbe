"""Sequence-sharded pipelines (Ulysses): all-to-all between the sequence-sharded layout of the surrounding transformer and
the head-sharded layout the attention kernels work on.

The attention path itself shards by head and needs no collective. A pipeline that keeps its activations sharded along the
sequence (rank r holds tokens [r L/P, (r + 1) L/P) of every head) exchanges q, k, v before the attention and the output
after it, as the reference's multi-GPU recipe for HunyuanVideo does around `EchoSparseAttention`
(`torch.distributed.all_to_all_single` over NCCL on NVLink / NVSwitch; on CPU ranks the same code runs over gloo). Both
exchanges are one `all_to_all_single` each: every rank sends each peer an equal, contiguous slab.
"""
import torch
import torch.distributed as dist


def _check(x, world, what):
    if x.dim() != 4 or x.shape[0] != 1:
        raise ValueError(f"{what} must be [1, L, H, D]")
    return x[0]


def seq_to_heads(x, group=None):
    """[1, L / P, H, D] (this rank's tokens, all heads) -> [1, L, H / P, D] (all tokens, this rank's heads).
    Tokens of rank p come p-th; heads of rank r are [r H / P, (r + 1) H / P)."""
    world = dist.get_world_size(group)
    t = _check(x, world, "x")
    Ll, H, D = t.shape
    if H % world != 0:
        raise ValueError(f"{H} heads cannot be divided over {world} ranks")
    if world == 1:
        return x
    send = t.reshape(Ll, world, H // world, D).permute(1, 0, 2, 3).contiguous()      # [P, L/P, H/P, D], slab p -> rank p
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.reshape(1, world * Ll, H // world, D)                                  # slab p = tokens of rank p


def heads_to_seq(y, group=None):
    """[1, L, H / P, D] (all tokens, this rank's heads) -> [1, L / P, H, D] (this rank's tokens, all heads)."""
    world = dist.get_world_size(group)
    t = _check(y, world, "y")
    L, Hl, D = t.shape
    if L % world != 0:
        raise ValueError(f"{L} tokens cannot be divided over {world} ranks")
    if world == 1:
        return y
    send = t.reshape(world, L // world, Hl, D).contiguous()                            # slab p = tokens of rank p
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)                                    # slab p = heads of rank p
    return recv.permute(1, 0, 2, 3).reshape(1, L // world, world * Hl, D)


class UlyssesAttention:
    """Wraps an attention callable `attn(q, k, v, step, branch, layer, ...)` working on [1, L, H_local, D] (for example
    `EchoSparseAttention`) for a sequence-sharded caller: three all-to-alls in, one out. The per-layer state of the wrapped
    processor lives on the head shard, so nothing else crosses ranks."""

    def __init__(self, attn, group=None):
        self.attn = attn
        self.group = group

    def __call__(self, q, k, v, *args, **kwargs):
        qh, kh, vh = (seq_to_heads(t, self.group) for t in (q, k, v))
        out = self.attn(qh, kh, vh, *args, **kwargs)
        return heads_to_seq(out, self.group)
