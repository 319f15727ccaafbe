"""Kernel sets. `sm100` is the only one: hand-written CUDA for B200 behind the C ABI of libechosparse_sm100.so."""
