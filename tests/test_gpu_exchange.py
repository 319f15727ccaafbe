"""The sequence <-> head exchange kernel (es_exchange_rows). One GPU stands in for all ranks: every "rank" has its source and
its receive buffer in this GPU's memory, the kernel is launched once per rank with the list of all receive buffers, and the
result must be the transposition that all_to_all_single between two layout copies gives (ulysses.seq_to_heads /
heads_to_seq). The addressing is the same when the buffers are peer mappings; the 2-GPU path is run by bench.py --ulysses."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _launch(src, bufs, slab_stride, src_row, dst_offset, dst_row, rows, row_bytes):
    from self_trainable_or_free_attn_b200 import _native
    ptrs = (ctypes.c_void_p * len(bufs))(*[b.data_ptr() for b in bufs])
    rc = _native.load().es_exchange_rows(src.data_ptr(), slab_stride, src_row, ptrs, dst_offset, dst_row, len(bufs), rows,
                                         row_bytes, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _native.last_error()


@pytest.mark.parametrize("P,Ll,Hl", [(2, 96, 3), (4, 50, 2), (8, 33, 1)])
def test_both_directions_equal_the_all_to_all_transposition(P, Ll, Hl):
    from self_trainable_or_free_attn_b200 import ulysses
    D, es = 128, 2
    H, L = P * Hl, P * Ll
    g = torch.Generator(device="cuda").manual_seed(P)
    full = torch.randn(L, H, D, device="cuda", generator=g).to(torch.bfloat16)         # the unsharded activations
    seq = [full[r * Ll:(r + 1) * Ll].contiguous() for r in range(P)]                    # rank r: its tokens, all heads
    heads = [full[:, r * Hl:(r + 1) * Hl].contiguous() for r in range(P)]               # rank r: all tokens, its heads
    # sequence -> heads
    recv = [torch.full((L, Hl, D), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(P)]
    for r in range(P):
        _launch(seq[r], recv, *ulysses.seq_to_heads_plan(r, P, Ll, H, D, es))
    for r in range(P):
        assert torch.equal(recv[r], heads[r]), r
    # heads -> sequence
    back = [torch.full((Ll, H, D), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(P)]
    for r in range(P):
        _launch(heads[r], back, *ulysses.heads_to_seq_plan(r, P, L, Hl, D, es))
    for r in range(P):
        assert torch.equal(back[r], seq[r]), r


def test_bad_arguments_are_rejected_before_any_launch():
    from self_trainable_or_free_attn_b200 import _native
    lib = _native.load()
    x = torch.zeros(64, 128, device="cuda", dtype=torch.bfloat16)
    ptrs = (ctypes.c_void_p * 1)(x.data_ptr())
    before = _native.launch_count()
    assert lib.es_exchange_rows(x.data_ptr(), 0, 256, ptrs, 0, 256, 1, 64, 250, None) < 0      # row not a multiple of 16 bytes
    assert lib.es_exchange_rows(x.data_ptr(), 0, 128, ptrs, 0, 256, 1, 64, 256, None) < 0      # stride shorter than a row
    assert lib.es_exchange_rows(x.data_ptr(), 0, 256, ptrs, 0, 256, 17, 64, 256, None) < 0     # too many peers
    assert lib.es_exchange_rows(None, 0, 256, ptrs, 0, 256, 1, 64, 256, None) < 0
    assert _native.launch_count() == before
