"""CPU restatement of the reference's int8 / e4m3 GEMMs and their fused epilogues.

TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the CPU-baseline
leg of the benchmark; never by the product path.

Reference functions restated (file:line):
  * b8::Gemm::run, int32 accumulation of A[M,K] * B[N,K]^T      cuda/gemm_b8.cuh:666-754
  * ScaledMatrixWriter<I8Store>                                  cuda/gemm_b8.cuh:291-339
  * L2NormMatrixWriter + kv_helpers::l2_norm / raw_output        cuda/gemm_b8.cuh:760-949
  * GeGluMatrixWriter + math::fast::gelu                         cuda/gemm_b8.cuh:341-441,
                                                                 cuda/utils_core.cuh:426-448
  * ResidualMatrixWriter::residual_gate, sigmoid_base4,
    imprecise_softplus_base4                                     cuda/gemm_b8.cuh:484-505,
                                                                 cuda/utils_core.cuh:397-405,468-483
  * b16::Gemm with E4m3MatrixLoader / I8MatrixLoader (e4m3 x i8 -> f32)
                                                                 cuda/gemm_b16.cuh:72-185,478-566
  * scale constants of the live kernels                          src/main.rs:412-421,464-476,
                                                                 548-557,599-608,650-660
Transcendentals use exact libm values where the kernels use the PTX `.approx`
forms, so results agree with a GPU to within the last quantisation step, not bit
for bit; everything integer is exact. Pinned against the fixtures of tests/golden and against
the reference's own kernels compiled for sm_100a (oracle/build_ref.py,
tests/test_gpu_reference_gemm.py: at most 1.4e-4 of the e4m3 bytes differ from them).
"""
import math

import numpy as np

from . import formats

F32 = np.float32
GELU_VAR_FIX_2 = 1.0 / ((1.0 / 3.0) + (0.5 / math.pi) * (1.0 / math.sqrt(3.0)))


def gemm_i32(a_i8, b_i8):
    """acc[M,N] = A[M,K] . B[N,K]^T with exact int32 accumulation (gemm_b8.cuh:666-754).

    Computed blockwise in float64 BLAS: every partial sum is an integer far below 2^53,
    so the result is exact.
    """
    a = np.asarray(a_i8, dtype=np.int8)
    b = np.asarray(b_i8, dtype=np.int8)
    assert a.shape[1] == b.shape[1]
    acc = a.astype(np.float64) @ b.astype(np.float64).T
    return acc.astype(np.int64).astype(np.int32)


def gemm_f32_e4m3_i8(a_e4m3, b_i8):
    """acc_f32 = bf16(A_e4m3) . bf16(B_i8)^T (gemm_b16.cuh:478-566).

    Both conversions are exact; the f32 accumulation order on a GPU is not
    reproducible, so this returns the float64 sum rounded once to f32.
    """
    a = formats.e4m3_to_f32(a_e4m3).astype(np.float64)
    b = np.asarray(b_i8, dtype=np.int8).astype(np.float64)
    return (a @ b.T).astype(F32)


def gemm_f32_e4m3_e4m3(a_e4m3, b_e4m3):
    """acc_f32 = A_e4m3fn . B_e4m3fn^T with standard OCP e4m3 decode (tensor-core f8 mode)."""
    a = formats.hw_e4m3_to_f32(a_e4m3).astype(np.float64)
    b = formats.hw_e4m3_to_f32(b_e4m3).astype(np.float64)
    return (a @ b.T).astype(F32)


# ---------------------------------------------------------------------------------------------
# epilogues

def scaled_i8(acc, inp_scale, out_scale):
    """ScaledMatrixWriter<I8Store> (gemm_b8.cuh:291-339): rint(clamp(f32(acc) * f32(scale)))."""
    scale = F32(float(inp_scale) * float(out_scale))
    return formats.f32_to_fixedi8(np.asarray(acc).astype(F32) * scale)


def l2norm_kv_i8(acc, head_dim, eps, inp_scale, out_scale):
    """L2NormMatrixWriter (gemm_b8.cuh:861-949) for raw columns laid out per head as [K(D) | V(D)].

    K: acc * rsqrt(sum(acc^2) + eps) * (out_scale * sqrt(D))   (gemm.rs:146)
    V: acc * (inp_scale * out_scale)                            (gemm.rs:152)
    Returns (kv_i8 [M, N], rrms f32 [M, N / 2D]) where rrms is the K multiplier
    (gemm_b8.cuh:807-812).
    """
    acc = np.asarray(acc)
    m, n = acc.shape
    d = head_dim
    assert n % (2 * d) == 0
    heads = n // (2 * d)
    a = acc.astype(F32).reshape(m, heads, 2, d)
    k = a[:, :, 0, :]
    v = a[:, :, 1, :]
    ssum = np.sum(k.astype(np.float64) ** 2, axis=-1).astype(F32)
    head_scale = F32(float(out_scale) * math.sqrt(d))
    scale = (F32(1.0) / np.sqrt((ssum + F32(eps)).astype(np.float64))).astype(F32) * head_scale
    k_out = k * scale[..., None]
    v_out = v * F32(float(inp_scale) * float(out_scale))
    out = np.stack((k_out, v_out), axis=2).reshape(m, n)
    return formats.f32_to_fixedi8(out), scale.astype(F32)


def _gelu_scaled(x, inp_scale_2, out_scale_2, var_fix_2):
    """math::fast::gelu<INP_SCALE_2, OUT_SCALE_2, VAR_FIX_2>(x).val (utils_core.cuh:426-448)."""
    k = math.sqrt(inp_scale_2)
    ck = math.sqrt(inp_scale_2 * 2.0 / math.pi)
    ck3 = 0.044715 * ck * inp_scale_2
    y_scale = 0.5 * math.sqrt(out_scale_2 * var_fix_2) * k
    x = x.astype(F32)
    x2 = x * x
    s = ((F32(ck3) * x).astype(np.float64) * x2 + (F32(ck) * x).astype(np.float64)).astype(F32)
    t = np.tanh(s.astype(np.float64)).astype(F32)
    yx = F32(y_scale) * x
    return (yx.astype(np.float64) * t + yx).astype(F32)


def geglu_val(acc, inp_scale, out_scale):
    """f32 value before the store conversion of GeGluMatrixWriter::geglu (gemm_b8.cuh:357-372)."""
    acc = np.asarray(acc)
    gate = acc[:, 0::2]
    lin = acc[:, 1::2].astype(F32)
    inp2 = float(inp_scale) ** 2
    out2 = float(out_scale) ** 2
    g = _gelu_scaled(gate, inp2, inp2 * out2, 1.0)
    return (g * lin).astype(F32)


def geglu_e4m3(acc, inp_scale, out_scale):
    """GeGluMatrixWriter<E4m3Store>: raw columns (2j, 2j+1) = (gate, lin) -> e4m3 byte j."""
    return formats.f32_to_e4m3(geglu_val(acc, inp_scale, out_scale))


def residual_val(acc, residual_i8, inp_scale, out_scale):
    """f32 value before the store conversion of ResidualMatrixWriter::residual_gate
    (gemm_b8.cuh:484-505). `acc` is int32 (i8 GEMM) or f32 (e4m3 x i8 GEMM); raw columns
    (2j, 2j+1) = (gate, value); residual is FixedI8 [M, N/2]."""
    acc = np.asarray(acc)
    gate = acc[:, 0::2].astype(F32)
    new_val = acc[:, 1::2].astype(F32)
    old_val = np.asarray(residual_i8, dtype=np.int8).astype(F32)
    inp = float(inp_scale)
    out = float(out_scale)
    # sigmoid_base4<-INP, 1/8>(gate) (utils_core.cuh:397-405)
    half = F32(0.5 * (1.0 / formats.FIXED_I8_SCALE))
    t = np.tanh((F32(math.log(2.0) * -inp) * gate).astype(np.float64)).astype(F32)
    old_w = (half.astype(np.float64) * t + half).astype(F32)
    # imprecise_softplus_base4<INP, INP*OUT>(gate) (utils_core.cuh:468-483)
    sp_in = F32(inp * 2.0)
    sp_out = F32(inp * out / 2.0)
    line_scale = F32(inp * inp * out)
    line = np.maximum(F32(0.0), gate)
    if line_scale != F32(1.0):
        line = line * line_scale
    e = np.exp2(-np.abs((gate * sp_in)).astype(np.float64)).astype(F32)
    lg = np.log2((F32(1.0) + e).astype(np.float64)).astype(F32)
    new_w = (lg.astype(np.float64) * sp_out + line).astype(F32)
    ow = (old_w * old_val).astype(F32)
    return (new_w.astype(np.float64) * new_val + ow).astype(F32)


def residual_e4m3(acc, residual_i8, inp_scale, out_scale):
    return formats.f32_to_e4m3(residual_val(acc, residual_i8, inp_scale, out_scale))


def residual_i8(acc, residual_i8_codes, inp_scale, out_scale):
    return formats.f32_to_fixedi8(residual_val(acc, residual_i8_codes, inp_scale, out_scale))


# ---------------------------------------------------------------------------------------------
# the live kernels of src/main.rs, with their scale constants

def attn_q_fwd(x_i8, wq_i8):
    """attn_q_fwd (main.rs:387-421): q = rint(clamp(acc * Dm^-1/2 / 64 * 8))."""
    dm = x_i8.shape[1]
    return scaled_i8(gemm_i32(x_i8, wq_i8), dm ** -0.5 / 64.0, 8.0)


def attn_kv_fwd(x_i8, wkv_i8, head_dim, eps=2.0 ** -70):
    """attn_kv_fwd (main.rs:440-491): per head [K|V], K L2-normalised, V scaled."""
    dm = x_i8.shape[1]
    return l2norm_kv_i8(gemm_i32(x_i8, wkv_i8), head_dim, eps, dm ** -0.5 / 64.0, 8.0)


def ffn_f_fwd(x_i8, wf_i8):
    """ffn_f_fwd (main.rs:575-640): GeGLU -> e4m3, INP = Dm^-1/2 / 64, OUT = 1."""
    dm = x_i8.shape[1]
    return geglu_e4m3(gemm_i32(x_i8, wf_i8), dm ** -0.5 / 64.0, 1.0)


def attn_y_fwd(attn_out_i8, wy_i8, x_i8):
    """attn_y_fwd (main.rs:523-572): i8 GEMM + gated residual -> e4m3, INP = A^-1/2 / 64."""
    a = attn_out_i8.shape[1]
    return residual_e4m3(gemm_i32(attn_out_i8, wy_i8), x_i8, a ** -0.5 / 64.0, 1.0)


def ffn_y_fwd_f8(f_e4m3, wy_i8, x_i8):
    """ffn_y_fwd_f8 (main.rs:620-675): e4m3 x i8 GEMM + gated residual -> e4m3,
    INP = sqrt(GELU_VAR_FIX_2 / F) / 8."""
    f = f_e4m3.shape[1]
    inp = math.sqrt(GELU_VAR_FIX_2 / f) / 8.0
    return residual_e4m3(gemm_f32_e4m3_i8(f_e4m3, wy_i8), x_i8, inp, 1.0)


def ffn_y_fwd_i8(f_i8, wy_i8, x_i8):
    """ffn_y_fwd_i8 (ffn_y_fwd_i8.cu, stale harness): i8 x i8 GEMM + gated residual -> i8,
    INP = sqrt(GELU_VAR_FIX_2 / F) / 64."""
    f = f_i8.shape[1]
    inp = math.sqrt(GELU_VAR_FIX_2 / f) / 64.0
    return residual_i8(gemm_i32(f_i8, wy_i8), x_i8, inp, 1.0)


# ---------------------------------------------------------------------------------------------
# the FFN with e4m3 weights and e4m3 activations, one f32 scale per tensor (the benchmark description's
# second FFN run).  No counterpart in the reference, whose "f8" GEMM (gemm_b16.cuh:72-185) keeps int8 weights
# and multiplies in bf16: parity of this mode is pinned by this restatement only.  The epilogues are the
# reference's (gemm_b8.cuh:357-372, 484-505); the tensor scales fold into their input scale.

def quantize_e4m3_per_tensor(x):
    """(OCP e4m3 bytes, scale) with x ~ scale * e4m3: scale = absmax / 448, the largest finite e4m3 value."""
    x = np.asarray(x, dtype=F32)
    amax = float(np.abs(x).max())
    scale = amax / 448.0 if amax > 0 else 1.0
    return formats.hw_f32_to_e4m3((x / F32(scale)).astype(F32)), scale


def ffn_f_fwd_e4m3(x_e4m3, x_scale, wf_e4m3, wf_scale):
    """GeGLU(x . Wf^T) -> e4m3 with INP = x_scale * wf_scale, OUT = 1: the pre-activations are the plain products of
    the values (weights drawn N(0, 0.02) carry their own 1/sqrt(fan-in); the reference's Dm^-1/2 belongs to its
    unit-variance FixedI8 weights)."""
    return geglu_e4m3(gemm_f32_e4m3_e4m3(x_e4m3, wf_e4m3), float(x_scale) * float(wf_scale), 1.0)


def ffn_y_fwd_e4m3(f_e4m3, wy_e4m3, wy_scale, x_i8):
    """f . Wy^T + gated residual (x as FixedI8, the block's residual stream) -> e4m3, INP = wy_scale."""
    return residual_e4m3(gemm_f32_e4m3_e4m3(f_e4m3, wy_e4m3), x_i8, float(wy_scale), 1.0)
