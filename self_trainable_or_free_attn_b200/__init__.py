"""B200-native implementation of EchoSparse's sparse attention step (shaoshitong/self_trainable_or_free_attn).

`kernels.sm100` is the kernel-set module the reference's attention processor calls; `attention.EchoSparseAttention` is
the processor itself with the reference's call signature. The CUDA code lives in `csrc/` behind the C ABI declared in
`include/echosparse_sm100.h`.
"""
__version__ = "0.1.0"
