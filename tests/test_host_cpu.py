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
    assert attn.dense_layers == {0, 3} and attn.backend is None and attn.K is None and not attn._states and len(attn._states) == 0
    attn.reset()


def test_layer_record_shapes_and_plan_state():
    """What a layer keeps between steps: two swapping offset buffers per branch and bit-mask plans."""
    rec = attention._LayerRecord(4152, 2, "cpu", keep_lists=False)
    br = rec.branch(0)
    assert br.offset.shape == (33 * 128, 2) and float(br.offset[0, 0]) > 9e29 and br.offset is not br.next_offset
    br.cur ^= 1
    assert br.offset is br.buffers[1] and br.next_offset is br.buffers[0] and not br.ready
    exact, skip = rec.plan(1)
    assert len(rec.plans) == 2 and exact.shape == skip.shape == (2, 33, 4) and int(skip[0, 0, 0]) == -1
    assert rec.offsets.keys() == {0} and rec.ready == set() and rec.offset(1).shape == (33 * 128, 2)
    assert attention.plan_words(1182) == 64 and attention.plan_words(65) == 4 and attention.plan_words(8) == 4
    lists = attention._Lists(4152, 2, "cpu", 32)
    assert lists.keep.shape == (2, 33, 65) and lists.keep.dtype == torch.uint8 and lists.blocks.shape == (33, 2, 65)
    assert lists.refine.shape == (33, 2, 32) and int(lists.refine[0, 0, 0]) == 65


def test_state_table_views():
    attn = EchoSparseAttention()
    rec = attention._LayerRecord(4152, 2, "cpu", keep_lists=False)
    rec.branch(0), rec.branch(1)
    attn._states.put(3, rec)
    assert sorted(attn._states) == [(0, 3), (1, 3)] and (1, 3) in attn._states and (2, 3) not in attn._states
    assert attn._states[3] is rec and attn._states[(1, 3)].offset is rec.branches[1].offset
    with pytest.raises(KeyError):
        attn._states[(2, 3)]
    attn._states.clear()
    assert not attn._states


class _RecordingKernels:
    """A kernel set that only writes down which entry points the processor calls, in order."""

    def __init__(self):
        self.calls = []

        outer = self

        class Representatives:
            def __init__(self, L, H, D, device, iters=6):
                nb = -(-L // 64)
                self.k = torch.zeros(H, (nb + 1) * 4, D)
                self.v = torch.zeros(H, (nb + 1) * 4, D)
                self.log_counts = torch.zeros(H, (nb + 1) * 4)

            def build(self, q, k, v, k_mean=None, v_mean=None):
                outer.calls.append("reps.build")

        self.Representatives = Representatives

    def __getattr__(self, name):
        def record(*args, **kwargs):
            self.calls.append(name if name != "block_attention" or kwargs.get("mass") is None else "block_attention+mass")
        return record

    def take(self):
        got, self.calls = self.calls, []
        return got


def test_schedule_of_kernel_calls_over_a_video():
    """The processor's phases, seen as the sequence of kernel-set calls (no GPU: a recording kernel set on CPU tensors):
    first dense step = online softmax; later dense steps = fixed offset + recomputation; full step; sparse steps with the
    plan of branch 0 reused by branch 1, two plans alternating; a skipped step falls back to a dense step; reset() starts
    over."""
    L, H = 64 * 6, 1
    attn = EchoSparseAttention(density=0.25, dense_steps=3, dense_layers=())
    K = attn.K = _RecordingKernels()
    q = torch.zeros(L, H, 128, dtype=torch.bfloat16)
    run = lambda step, branch: (attn._step(q, q, q, step, branch, 7, attention.NO_SINK), K.take())[1]
    first_dense = ["exact_fallback"]
    later_dense = ["block_attention", "exact_fallback"]
    sparse = ["rebuild_plan", "block_means", "reps.build", "sparse_attention", "exact_fallback", "compensate_fallback"]
    plan = ["select_blocks", "pack_plan"]
    assert run(0, 0) == first_dense and run(0, 1) == first_dense
    assert run(1, 0) == later_dense and run(1, 1) == later_dense
    rec = attn._states.record(7)
    assert rec.current is None and rec.pending is None and not rec.ready
    assert run(2, 0) == ["block_attention+mass", "exact_fallback", "full_step_scales"] + plan
    assert rec.pending == (0, 3) and rec.ready == {0}
    assert run(2, 1) == later_dense and rec.ready == {0, 1}
    assert run(3, 0) == sparse + ["estimate_skipped"] + plan
    assert rec.current == (0, 3) and rec.pending == (1, 4)           # the other plan is written while this one is read
    assert run(3, 1) == sparse
    assert run(4, 0) == sparse + ["estimate_skipped"] + plan and rec.current == (1, 4) and rec.pending == (0, 5)
    # the offsets swap roles every step that writes an LSE
    br = rec.branches[0]
    assert br.cur == 0 and br.seeded                 # steps 1, 2, 3, 4 swapped four times
    # step 5 is skipped: the pending plan was made for step 5, not 6 -> a dense step on the previous LSE
    assert run(6, 0) == later_dense and rec.current is None and rec.pending is None
    assert run(6, 1) == later_dense
    attn.reset()
    assert not rec.ready and not br.seeded
    assert run(0, 0) == first_dense


def test_layer_state_keeps_its_lists_and_skips_the_rebuild():
    L, H = 64 * 6, 1
    attn = EchoSparseAttention(density=0.25, dense_steps=2, dense_layers=(), state="layer")
    K = attn.K = _RecordingKernels()
    q = torch.zeros(L, H, 128, dtype=torch.bfloat16)
    for step in range(2):
        attn._step(q, q, q, step, 0, 1, attention.NO_SINK)
    K.take()
    attn._step(q, q, q, 2, 0, 1, attention.NO_SINK)
    calls = K.take()
    assert "rebuild_plan" not in calls and calls[:3] == ["block_means", "reps.build", "sparse_attention"]
    assert sorted(attn._states.record(1).expanded) == [0, 1]
