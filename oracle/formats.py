"""CPU restatement of the reference's number formats (TEST INFRASTRUCTURE ONLY).

This module is part of the oracle: only the tests, the smoke check and the
CPU-baseline leg of the benchmark may import it.  The product path never does.

Formats restated here (reference file:line):
  * FixedI8: code = rint(clamp(x, -127, +127)), value = code / 8
        cuda/utils_b8.cuh:7-10 (3 fractional bits), :629-632 (f32_to_fixedi8)
  * custom e4m3 encode: flush below 1.9375 * 2^-7 to +0, round half up in
    magnitude, saturate to 0x7E
        cuda/utils_b8.cuh:636-647 (f32_to_e4m3)
  * custom e4m3 decode through bf16 bits
        cuda/utils_b8.cuh:652-657 (e4m3_to_bf16)
  * the float64 PyTorch oracle's e4m3: FTZ below the same threshold, then
    torch's round-to-nearest-even cast
        block_utils.py:126-137 (e4m3_ftz), new_block.py:18-19 (quantize_e4m3)
"""
import numpy as np

FIXED_I8_SCALE = 8.0
F32 = np.float32


def f32_to_fixedi8(x):
    """cuda/utils_b8.cuh:629-632: clamp to +-127, then round half to even."""
    x = np.asarray(x, dtype=F32)
    return np.rint(np.clip(x, F32(-127.0), F32(127.0))).astype(np.int8)


def quantize_fixedi8(x):
    """value -> FixedI8 code (new_block.py:12-16, block_utils.py:163-166)."""
    x = np.asarray(x, dtype=np.float64)
    return np.clip(np.rint(x * 8.0), -127.0, 127.0).astype(np.int8)


def f32_to_e4m3(x):
    """cuda/utils_b8.cuh:636-647, bit-for-bit (integer arithmetic on the f32 bits)."""
    bits = np.ascontiguousarray(np.asarray(x, dtype=F32)).view(np.uint32)
    sign = (bits >> np.uint32(24)) & np.uint32(0x80)
    rest = bits & np.uint32(0x7FFFFFFF)
    lo = np.uint32((120 << 23) + (0xF << 19))
    hi = np.uint32((135 << 23) + (0xC << 19))
    # (rest + (1<<19) - (120<<23)) >> 20, in wrapping u32 arithmetic like the kernel
    rounded = ((rest.astype(np.uint64) + np.uint64((1 << 19)) + np.uint64((1 << 32) - (120 << 23)))
               & np.uint64(0xFFFFFFFF)).astype(np.uint32) >> np.uint32(20)
    clamped = np.where(rest > hi, np.uint32(0x7E), rounded)
    out = np.where(rest < lo, np.uint32(0), sign | clamped)
    return out.astype(np.uint8)


def e4m3_to_f32(code):
    """cuda/utils_b8.cuh:652-657: decode via bf16 bits; 0x00/0x80 -> 0."""
    c = np.asarray(code, dtype=np.uint8).astype(np.uint32)
    sign = (c & np.uint32(0x80)) << np.uint32(8)
    rest = (c & np.uint32(0x7F)) << np.uint32(4)
    bf16_bits = ((sign | rest) + np.uint32(120 << 7)) & np.uint32(0xFFFF)
    f32_bits = (bf16_bits << np.uint32(16)).astype(np.uint32)
    val = f32_bits.view(F32)
    return np.where(rest == 0, F32(0.0), val).astype(F32)


def e4m3_oracle_quantize(x):
    """The float64 oracle's e4m3 (block_utils.py:126-137 + torch RNE cast), as f64 values.

    Differs from f32_to_e4m3 only on exact ties (half-up vs half-even).
    """
    import torch
    t = torch.as_tensor(np.asarray(x, dtype=np.float64))
    thr = (1.0 + 15.0 / 16.0) * 2.0 ** -7
    t = torch.where(t.abs() < thr, torch.zeros_like(t), t)
    return t.to(torch.float8_e4m3fn).to(torch.float64).numpy()


def hw_e4m3_to_f32(code):
    """Standard OCP e4m3fn decode (used by the e4m3 x e4m3 tensor-core mode)."""
    import torch
    c = torch.as_tensor(np.ascontiguousarray(np.asarray(code, dtype=np.uint8)))
    return c.view(torch.float8_e4m3fn).to(torch.float32).numpy()


def hw_f32_to_e4m3(x):
    """Standard OCP e4m3fn encode, round-to-nearest-even, saturating (torch cast)."""
    import torch
    t = torch.as_tensor(np.ascontiguousarray(np.asarray(x, dtype=F32)))
    t = torch.clamp(t, -448.0, 448.0)
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
