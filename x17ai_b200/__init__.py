"""B200-native drop-in for the quantized block-forward hot path of x17ai.

The product is `libx17ai_b200.so` (hand-written sm_100a CUDA behind a C ABI, see
`include/x17ai_b200.h`).  This package is the thin host-side mirror of the reference's Rust
launchers for that path, used by the tests and the benchmark:

    device.CudaDevice / CudaStream / CudaTimer     src/device/cuda.rs, cuda_shim.rs
    kernels.AttnKernel, GemmKernel, rms_norm, ...  src/device/cuda/attn.rs, gemm.rs

There is no CPU or PyTorch fallback: without the built library, or without an sm_100 GPU,
calls raise `X17Error`.
"""
from ._lib import X17Error, load  # noqa: F401
from . import device, kernels  # noqa: F401
