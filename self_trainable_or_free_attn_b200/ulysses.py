"""Sequence-sharded pipelines (Ulysses): the exchange between the sequence-sharded layout of the surrounding transformer
and the head-sharded layout the attention kernels work on.

The attention path itself shards by head and needs no collective. A pipeline that keeps its activations sharded along the
sequence (rank r holds tokens [r L/P, (r + 1) L/P) of every head) exchanges q, k, v before the attention and the output
after it, as the reference's multi-GPU recipe for HunyuanVideo does around `EchoSparseAttention` with
`torch.distributed.all_to_all_single`. Two ways to run an exchange:

* `seq_to_heads` / `heads_to_seq`: one `all_to_all_single` between two layout copies (NCCL on GPUs; gloo on CPU ranks, which
  is how the host logic is tested);
* `PeerExchange`: one kernel of this library per rank and exchange (`es_exchange_rows`): every rank's receive buffers live in
  symmetric memory, mapped on all GPUs of the group, and the kernel stores each peer's slab straight into its final place in
  that peer's buffer over NVLink / NVSwitch, so the two layout copies disappear (they cost as much HBM time as the transfer
  costs link time). The kernel waits on nobody; a 4-byte all-reduce on the same stream after it is the point behind which
  every rank's slabs have landed, and the same point in the NEXT exchange of the same buffer is what makes overwriting it
  safe, so there is one small collective per exchange.
"""
import ctypes
import os

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


def seq_to_heads_plan(rank, world, Ll, H, D, elem):
    """Arguments of `es_exchange_rows` for rank `rank`'s [Ll, H, D] tokens on the way to heads, in bytes:
    (src_slab_stride, src_row_stride, dst_offset, dst_row_stride, rows, row_bytes). Peer p takes columns
    [p Hl D, (p + 1) Hl D) of every row; they become rows [rank Ll, (rank + 1) Ll) of its [world Ll, Hl, D] buffer."""
    Hl = H // world
    return Hl * D * elem, H * D * elem, rank * Ll * Hl * D * elem, Hl * D * elem, Ll, Hl * D * elem


def heads_to_seq_plan(rank, world, L, Hl, D, elem):
    """The same for rank `rank`'s [L, Hl, D] heads on the way back: peer p takes rows [p Ll, (p + 1) Ll); they become
    columns [rank Hl D, (rank + 1) Hl D) of the rows of its [Ll, world Hl, D] buffer."""
    Ll = L // world
    return Ll * Hl * D * elem, Hl * D * elem, rank * Hl * D * elem, world * Hl * D * elem, Ll, Hl * D * elem


class PeerExchange:
    """The two exchanges through peer memory. One object per process group; receive buffers are made once per (role, shape)
    by a collective call (every rank must ask for the same roles and shapes in the same order) and are handed out as the
    results: a result is valid until the next exchange with the same role."""

    def __init__(self, group=None):
        if not dist.is_initialized():
            raise RuntimeError("PeerExchange needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self._buffers = {}
        self._token = None

    def _receive_buffer(self, role, shape, dtype, device):
        key = (role, tuple(shape), dtype)
        got = self._buffers.get(key)
        if got is None:
            # peer mappings only: nothing here uses the switch's multicast
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            local = symm.empty(*shape, dtype=dtype, device=device)
            handle = symm.rendezvous(local, self.group)
            ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in handle.buffer_ptrs])
            got = self._buffers[key] = (local, handle, ptrs)
        return got

    def _landed(self, device):
        """Behind this point of the stream every rank has run its exchange kernel."""
        if self._token is None:
            self._token = torch.zeros(1, device=device, dtype=torch.int32)
        dist.all_reduce(self._token, group=self.group)

    def _run(self, src, dst_ptrs, slab_stride, src_row, dst_offset, dst_row, rows, row_bytes):
        from . import _native
        with torch.cuda.device(src.device):
            rc = _native.load().es_exchange_rows(src.data_ptr(), slab_stride, src_row, dst_ptrs, dst_offset, dst_row,
                                                 self.world, rows, row_bytes, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise _native.NativeError(f"es_exchange_rows: {_native.last_error()}")

    def seq_to_heads(self, x, role):
        """As `seq_to_heads`; the result is this rank's receive buffer of `role`."""
        t = _check(x, self.world, "x")
        if not t.is_contiguous():
            t = t.contiguous()
        Ll, H, D = t.shape
        if H % self.world != 0:
            raise ValueError(f"{H} heads cannot be divided over {self.world} ranks")
        recv, _, ptrs = self._receive_buffer(role, (1, self.world * Ll, H // self.world, D), t.dtype, t.device)
        self._run(t, ptrs, *seq_to_heads_plan(self.rank, self.world, Ll, H, D, t.element_size()))
        self._landed(t.device)
        return recv

    def heads_to_seq(self, y, role):
        """As `heads_to_seq`; the result is this rank's receive buffer of `role`."""
        t = _check(y, self.world, "y")
        if not t.is_contiguous():
            t = t.contiguous()
        L, Hl, D = t.shape
        if L % self.world != 0:
            raise ValueError(f"{L} tokens cannot be divided over {self.world} ranks")
        recv, _, ptrs = self._receive_buffer(role, (1, L // self.world, self.world * Hl, D), t.dtype, t.device)
        self._run(t, ptrs, *heads_to_seq_plan(self.rank, self.world, L, Hl, D, t.element_size()))
        self._landed(t.device)
        return recv


class UlyssesAttention:
    """Wraps an attention callable `attn(q, k, v, step, branch, layer, ...)` working on [1, L, H_local, D] (for example
    `EchoSparseAttention`) for a sequence-sharded caller: three exchanges in, one out. The per-layer state of the wrapped
    processor lives on the head shard, so nothing else crosses ranks. `peer_memory=True` runs the exchanges through
    `PeerExchange` (GPUs of one node); the returned tensor is then a receive buffer that the next call overwrites."""

    def __init__(self, attn, group=None, peer_memory=False):
        self.attn = attn
        self.group = group
        self.peer = PeerExchange(group) if peer_memory else None

    def __call__(self, q, k, v, *args, **kwargs):
        if self.peer is not None:
            qh, kh, vh = (self.peer.seq_to_heads(t, role) for t, role in ((q, "q"), (k, "k"), (v, "v")))
            out = self.attn(qh, kh, vh, *args, **kwargs)
            return self.peer.heads_to_seq(out, "out")
        qh, kh, vh = (seq_to_heads(t, self.group) for t in (q, k, v))
        out = self.attn(qh, kh, vh, *args, **kwargs)
        return heads_to_seq(out, self.group)
