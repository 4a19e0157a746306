"""CPU restatement of the reference's RMSNorm kernel (TEST INFRASTRUCTURE ONLY).

Reference: Rms_norm::kernel, rms_norm.cu:55-113 (sum_squares :39-46, normalize :48-53):
    y = f32_to_fixedi8(x * rsqrtf(mean(x^2) + eps) * 8),  x = e4m3 decoded exactly to f32.
The GPU sums squares in f32 (lane-local fma chain, then a butterfly); here the sum is taken
in float64 and rounded once, so results can differ from a GPU by one code on rare ties.

`rms_norm_bf16_i8_rowscale` is the additional mode the benchmark description asks for
(bf16 in, int8 out with a per-row absmax/127 scale); the reference has no such kernel, so
that mode is pinned by nothing but this restatement.
"""
import numpy as np

from . import formats

F32 = np.float32


def rms_norm_e4m3_i8(x_e4m3, eps=2.0 ** -70):
    x = formats.e4m3_to_f32(x_e4m3)
    d = x.shape[-1]
    ssum = np.sum(x.astype(np.float64) ** 2, axis=-1).astype(F32)
    mean = (ssum * F32(1.0 / d) + F32(eps)).astype(F32)
    rrms = (1.0 / np.sqrt(mean.astype(np.float64))).astype(F32)
    y = ((x * rrms[..., None]).astype(F32) * F32(8.0)).astype(F32)
    return formats.f32_to_fixedi8(y)


def bf16_bits_to_f32(bits_u16):
    b = np.asarray(bits_u16, dtype=np.uint16).astype(np.uint32) << np.uint32(16)
    return b.view(F32)


def rms_norm_bf16_i8_fixed(x_bf16_bits, eps=2.0 ** -70):
    """bf16 in, FixedI8 out (same arithmetic as the e4m3 form)."""
    x = bf16_bits_to_f32(x_bf16_bits)
    d = x.shape[-1]
    ssum = np.sum(x.astype(np.float64) ** 2, axis=-1).astype(F32)
    mean = (ssum * F32(1.0 / d) + F32(eps)).astype(F32)
    rrms = (1.0 / np.sqrt(mean.astype(np.float64))).astype(F32)
    y = ((x * rrms[..., None]).astype(F32) * F32(8.0)).astype(F32)
    return formats.f32_to_fixedi8(y)


def rms_norm_bf16_i8_rowscale(x_bf16_bits, eps=2.0 ** -70):
    """bf16 in -> (int8 codes, f32 per-row scale) with scale = absmax(y) / 127, y = x * rrms."""
    x = bf16_bits_to_f32(x_bf16_bits)
    d = x.shape[-1]
    ssum = np.sum(x.astype(np.float64) ** 2, axis=-1).astype(F32)
    mean = (ssum * F32(1.0 / d) + F32(eps)).astype(F32)
    rrms = (1.0 / np.sqrt(mean.astype(np.float64))).astype(F32)
    absmax = np.max(np.abs(x), axis=-1).astype(F32)
    scale = ((absmax * rrms).astype(F32) * F32(1.0 / 127.0)).astype(F32)
    inv = np.where(scale > 0, (rrms.astype(np.float64) / np.where(scale > 0, scale, 1)).astype(F32), F32(0))
    y = (x * inv[..., None]).astype(F32)
    return formats.f32_to_fixedi8(y), scale
