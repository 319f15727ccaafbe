"""Host-side logic that needs no GPU: backend resolution and errors, budgets, state shapes (the reference pins these in
tests/test_api.py:21-43, 56-62 and tests/test_attention.py:152-155)."""
import pytest
import torch

from self_trainable_or_free_attn_b200 import attention, backends
from self_trainable_or_free_attn_b200.attention import EchoSparseAttention


def test_backend_names():
    backends.check_name("auto")
    backends.check_name("b200")
    for other in ("h100", "rtx5090"):
        with pytest.raises(ValueError, match="only has the B200"):
            backends.check_name(other)
    with pytest.raises(ValueError, match="gpu must be"):
        backends.check_name("tpu")
    with pytest.raises(ValueError, match="CUDA tensors"):
        backends.resolve("auto", "cpu")


def test_resolve_needs_compute_10(monkeypatch):
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda device=None: (9, 0))
    with pytest.raises(RuntimeError, match="needs a B200"):
        backends.resolve("auto", "cuda:0")
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda device=None: (10, 0))
    assert backends.resolve("b200", "cuda:0") == "b200"


def test_cpu_tensors_are_refused():
    attn = EchoSparseAttention()
    q = torch.zeros(1, 8192, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA tensors"):
        attn(q, q, q, 0, 0, 1)


def test_budgets_follow_the_reference():
    attn = EchoSparseAttention(density=0.10)
    assert attn._budget(1182) == (118, 355)          # Wan2.1-14B 720p: 75,600 tokens
    assert attn._budget(512) == (51, 154)
    assert attn._budget(8) == (1, 2)
    assert EchoSparseAttention(density=0.15)._budget(512) == (77, 145)
    assert EchoSparseAttention(density=1.0)._budget(65) == (65, 0)


def test_constructor_contract():
    with pytest.raises(AssertionError):
        EchoSparseAttention(dense_steps=1)
    attn = EchoSparseAttention(dense_layers=(0, 3))
    assert attn.dense_layers == {0, 3} and attn.backend is None and attn.K is None and attn._states == {}
    attn.reset()


def test_layer_state_shapes():
    st = attention._LayerState(4152, 2, "cpu")
    assert st.offset.shape == (33 * 128, 2) and float(st.offset[0, 0]) > 9e29
    assert st.mass.shape == (2, 33, 65) and st.keep.shape == (2, 33, 65) and st.keep.dtype == torch.uint8
    assert st.skip_bits.shape == (2, 33, 4) and int(st.skip_bits[0, 0, 0]) == -1
    assert st.blocks.shape == (33, 2, 65) and st.refine.shape == (33, 2, 0) and not st.ready
    assert attention._LayerState(75600, 1, "cpu").skip_bits.shape[-1] == 64
