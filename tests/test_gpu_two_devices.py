"""Tensors on a GPU that is not the calling thread's current device: the kernel-set module launches on the tensors' device
and stream (reference: the device guard of csrc/vsa/vsa2_api.cpp:64, 80 and the per-device re-resolution of
echosparse/attention.py:173-177), and the opt-in for large dynamic shared memory is made per device. Skipped with one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_processor_and_vsa_on_the_second_gpu_while_the_first_is_current():
    from oracle import echosparse_ref as R
    from self_trainable_or_free_attn_b200 import _native, vsa
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 1)
    L, H = 4152, 2
    g = torch.Generator(device=dev).manual_seed(0)
    pos = torch.arange(L, device=dev, dtype=torch.float32)[:, None, None] / 300.0
    freq = torch.randn(1, H, 128, device=dev, generator=g)
    base = [torch.sin(pos * freq + torch.randn(1, H, 128, device=dev, generator=g)) * 3.0 for _ in range(3)]
    attn = EchoSparseAttention(density=0.2, dense_steps=2, dense_layers=())
    for step in range(4):
        q, k, v = ((b + 0.05 * torch.randn(b.shape, device=dev, generator=g)).to(torch.bfloat16)[None] for b in base)
        out = attn(q, k, v, step, 0, layer=1)
        assert out.device == dev and torch.cuda.current_device() == 0
        ref, _ = R.dense_attention(q[0], k[0], v[0])
        assert ((out[0].float() - ref).norm() / ref.norm()).item() < 5e-2, step
    attn.check_status()
    # the same processor object moved to the first GPU re-resolves its backend and state
    q0, k0, v0 = (x.to("cuda:0") for x in (q, k, v))
    out0 = attn(q0, k0, v0, 0, 0, layer=1)
    assert out0.device.index == 0 and len(attn._states) == 1
    # VSA2 on the second GPU
    B, nb, D = 1, 6, 128
    cnt = torch.full((nb,), 64, dtype=torch.int32, device=dev)
    qq, kk, vv = (torch.randn(B, H, nb * 64, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True) for _ in range(3))
    gate = torch.randn(B, H, nb * 64, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    o = vsa.vsa2_attention(qq, kk, vv, gate, cnt, R=16, topk=2)
    o.float().sum().backward()
    assert o.device == dev and qq.grad is not None and torch.isfinite(qq.grad.float()).all()
    with torch.cuda.device(1):
        assert _native.device_status() == 0
