"""Head sharding across ranks, on CPU with 2 gloo processes: the heads are divided without overlap, every rank regenerates
exactly its own (branch, head) shard from the seeds, and the whole-job numbers that bench.py reports (sum of work, max of
time) come out of the collectives as expected. No GPU and no data-path collective is involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from self_trainable_or_free_attn_b200 import synthetic

GRID, HEADS = (2, 4, 8), 5           # 64 tokens, 5 heads: an uneven split over 2 ranks


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    heads = synthetic.shard_heads(HEADS, rank, world)
    q, k, v = synthetic.branch_qkv(GRID, 0, 1, heads, "cpu")
    # what bench.py reduces: per-rank work is summed, per-rank time is maximised
    stats = torch.tensor([float(len(heads)), 10.0 + rank], dtype=torch.float64)
    total, slowest = stats.clone(), stats.clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    gathered = [None] * world
    dist.all_gather_object(gathered, heads)
    torch.save({"heads": heads, "q": q, "k": k, "v": v, "total": total, "slowest": slowest, "all": gathered},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_cover_all_heads_and_regenerate_their_shards(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranks = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    assert ranks[0]["heads"] == [0, 1, 2] and ranks[1]["heads"] == [3, 4]
    assert ranks[0]["all"] == [[0, 1, 2], [3, 4]]
    full = synthetic.branch_qkv(GRID, 0, 1, list(range(HEADS)), "cpu")
    for name, ref in zip("qkv", full):
        got = torch.cat([r[name] for r in ranks], dim=2)
        assert torch.equal(got, ref)
    for r in ranks:
        assert r["total"].tolist() == [5.0, 21.0] and r["slowest"].tolist() == [3.0, 11.0]


@pytest.mark.parametrize("heads,world", [(40, 1), (40, 2), (40, 4), (40, 8), (12, 8), (24, 8), (3, 4)])
def test_shard_heads_is_a_balanced_partition(heads, world):
    parts = [synthetic.shard_heads(heads, r, world) for r in range(world)]
    assert sum(parts, []) == list(range(heads))
    sizes = [len(p) for p in parts]
    assert max(sizes) - min(sizes) <= 1


def test_branches_of_a_head_share_structure_but_not_noise():
    a = synthetic.head_qkv(GRID, 2, 0, 3, "cpu", dtype=torch.float32)
    b = synthetic.head_qkv(GRID, 2, 1, 3, "cpu", dtype=torch.float32)
    again = synthetic.head_qkv(GRID, 2, 0, 3, "cpu", dtype=torch.float32)
    assert all(torch.equal(x, y) for x, y in zip(a, again))
    assert not torch.equal(a[0], b[0])
    prev = synthetic.head_qkv(GRID, 2, 0, 3, "cpu", prev=True, dtype=torch.float32)
    assert 0 < (prev[0] - a[0]).abs().max() < 0.2 and torch.equal(prev[2], a[2])


# ---------------------------------------------------------------------------------------------- Ulysses exchange
def _ulysses_worker(rank, world, port, out_dir):
    from self_trainable_or_free_attn_b200 import ulysses
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L, H, D = 24, 4, 8
    g = torch.Generator().manual_seed(3)
    full = [torch.randn(1, L, H, D, generator=g) for _ in range(3)]                  # the same on every rank
    mine = [t[:, rank * L // world:(rank + 1) * L // world].contiguous() for t in full]
    heads = slice(rank * H // world, (rank + 1) * H // world)
    qh = ulysses.seq_to_heads(mine[0])
    ok_fwd = torch.equal(qh, full[0][:, :, heads])
    ok_back = torch.equal(ulysses.heads_to_seq(qh), mine[0])

    def attn(q, k, v, scale=2.0):                                                     # any per-head attention
        p = torch.softmax(torch.einsum("blhd,bmhd->bhlm", q, k) / scale, -1)
        return torch.einsum("bhlm,bmhd->blhd", p, v)

    out = ulysses.UlyssesAttention(attn)(*mine, scale=3.0)
    ref = attn(*full, scale=3.0)[:, rank * L // world:(rank + 1) * L // world]
    bad = None
    try:
        ulysses.seq_to_heads(torch.zeros(1, 4, 3, 8))
    except ValueError as e:
        bad = str(e)
    torch.save({"ok_fwd": ok_fwd, "ok_back": ok_back, "err": (out - ref).abs().max().item(), "bad": bad},
               os.path.join(out_dir, f"u{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_ulysses_exchange_round_trip_and_attention_equivalence(tmp_path):
    world = 2
    mp.spawn(_ulysses_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"u{r}.pt")
        assert res["ok_fwd"] and res["ok_back"], "exchange is not the head / sequence transposition"
        assert res["err"] < 1e-6, "sequence-sharded attention differs from the unsharded one"
        assert "cannot be divided" in res["bad"]


def _emulate_exchange_rows(src, bufs, slab_stride, src_row, dst_offset, dst_row, rows, row_bytes):
    """What es_exchange_rows does, on host byte arrays: for every peer, `rows` rows of `row_bytes`."""
    for p, dst in enumerate(bufs):
        for i in range(rows):
            a = p * slab_stride + i * src_row
            b = dst_offset + i * dst_row
            assert a + row_bytes <= src.size and b + row_bytes <= dst.size, "a row leaves its buffer"
            dst[b:b + row_bytes] = src[a:a + row_bytes]


@pytest.mark.parametrize("P,Ll,Hl", [(2, 6, 3), (4, 5, 2), (8, 3, 3), (8, 4, 1)])
def test_exchange_plans_address_exactly_the_all_to_all_transposition(P, Ll, Hl):
    """The byte addressing that PeerExchange hands to the exchange kernel (ulysses.seq_to_heads_plan / heads_to_seq_plan),
    replayed on the host for every rank: each receive buffer ends up as the head shard (and, on the way back, the token
    shard) of the unsharded tensor, every byte written exactly once."""
    import numpy as np
    from self_trainable_or_free_attn_b200 import ulysses
    D, es = 8, 2
    H, L = P * Hl, P * Ll
    full = np.arange(L * H * D, dtype=np.int16).reshape(L, H, D)
    seq = [np.ascontiguousarray(full[r * Ll:(r + 1) * Ll]) for r in range(P)]
    heads = [np.ascontiguousarray(full[:, r * Hl:(r + 1) * Hl]) for r in range(P)]
    recv = [np.full(L * Hl * D * es, 0xEE, dtype=np.uint8) for _ in range(P)]
    for r in range(P):
        _emulate_exchange_rows(seq[r].view(np.uint8).reshape(-1), recv, *ulysses.seq_to_heads_plan(r, P, Ll, H, D, es))
    for r in range(P):
        assert np.array_equal(recv[r].view(np.int16).reshape(L, Hl, D), heads[r]), r
    back = [np.full(Ll * H * D * es, 0xEE, dtype=np.uint8) for _ in range(P)]
    for r in range(P):
        _emulate_exchange_rows(heads[r].view(np.uint8).reshape(-1), back, *ulysses.heads_to_seq_plan(r, P, L, Hl, D, es))
    for r in range(P):
        assert np.array_equal(back[r].view(np.int16).reshape(Ll, H, D), seq[r]), r
    for plan in (ulysses.seq_to_heads_plan(P - 1, P, Ll, H, D, es), ulysses.heads_to_seq_plan(P - 1, P, L, Hl, D, es)):
        assert all(x % 16 == 0 for x in plan[:4]) and plan[5] % 16 == 0      # what the kernel requires of strides and rows
