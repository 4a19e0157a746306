"""Host-side mirror of the reference's kernel launchers for the hot path.

AttnKernelConfig / AttnKernel   <- src/device/cuda/attn.rs:45-232, launch :353-447
GemmConfig / epilogue configs   <- src/device/cuda/gemm.rs:60-366, launch :591-641
shape checks                    <- src/device/cuda/tensor_check.rs:19-101 (same messages)
scale constants of the block    <- src/main.rs:412-421,464-476,548-557,599-608,650-660

Tensors are torch CUDA tensors used as plain device buffers (pointer, shape, dtype); all
arithmetic happens in libx17ai_b200.so.
"""
import ctypes
import math
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import X17Error, check

DTYPE_E4M3, DTYPE_INT8, DTYPE_BF16, DTYPE_F32, DTYPE_I32_RAW = 0x30, 0x31, 0x40, 0x50, 0x51
EPI_SCALE, EPI_RMS_NORM, EPI_GEGLU, EPI_RESIDUAL = 0, 1, 2, 3
RMS_E4M3_FIXED, RMS_BF16_FIXED, RMS_BF16_ROWSCALE = 0, 1, 2
FIXED_I8_SCALE = 8.0
GELU_VAR_FIX_2 = 1.0 / ((1.0 / 3.0) + (0.5 / math.pi) * (1.0 / math.sqrt(3.0)))

_TORCH_DTYPES = {
    DTYPE_INT8: (torch.int8,),
    DTYPE_E4M3: (torch.uint8, torch.float8_e4m3fn),
    DTYPE_BF16: (torch.bfloat16,),
    DTYPE_F32: (torch.float32,),
    DTYPE_I32_RAW: (torch.int32,),
}
_DTYPE_NAMES = {DTYPE_INT8: "i8", DTYPE_E4M3: "e4m3", DTYPE_BF16: "bf16", DTYPE_F32: "f32", DTYPE_I32_RAW: "i32"}


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def matrix_shape(op, name, t, expected, dtype):
    """tensor_check::matrix_shape (tensor_check.rs:19-60)."""
    shape = tuple(t.shape)
    if len(shape) != 2:
        raise X17Error(f"{op} input {name} must be 2D, got shape {list(shape)}")
    rows, cols = shape
    if rows == 0 or cols == 0:
        raise X17Error(f"{op} input {name} has zero size {list(shape)}")
    if expected[0] is not None and rows != expected[0]:
        raise X17Error(f"{op} input {name} has {rows} rows, but should have {expected[0]}")
    if expected[1] is not None and cols != expected[1]:
        raise X17Error(f"{op} input {name} has {cols} columns, but should have {expected[1]}")
    _dtype_and_device(op, name, t, dtype)
    return rows, cols


def vector_shape(op, name, t, expected_len, dtype):
    """tensor_check::vector_shape (tensor_check.rs:62-82)."""
    shape = tuple(t.shape)
    if shape not in ((expected_len,), (expected_len, 1)):
        raise X17Error(f"{op} input {name} must have shape [{expected_len}] or [{expected_len}, 1], got {list(shape)}")
    _dtype_and_device(op, name, t, dtype)


def _dtype_and_device(op, name, t, dtype):
    if t.dtype not in _TORCH_DTYPES[dtype]:
        raise X17Error(f"{op} input {name} has dtype {t.dtype}, but should have {_DTYPE_NAMES[dtype]}")
    if not t.is_cuda:
        raise X17Error(f"{op} input {name} is not on device cuda")
    if not t.is_contiguous():
        raise X17Error(f"{op} input {name} must be contiguous")


ATTN_PERSISTENT, ATTN_PER_TILE = 0, 1


GEMM_ONE_CTA, GEMM_CTA_PAIR = 0, 1


def set_gemm_tiling(tiling: int = GEMM_CTA_PAIR) -> None:
    """Process-wide tiling of GemmKernel.launch and qkvg_fwd (x17ai_b200_set_gemm_tiling): clusters of two CTAs with
    256 x 256 tiles (tcgen05.mma.cta_group::2, the default), or one CTA per SM with 128 x 256 tiles. Same bytes out."""
    if _lib.load().x17ai_b200_set_gemm_tiling(int(tiling)) != 0:
        raise X17Error(f"unknown GEMM tiling {tiling}")


def set_attn_schedule(schedule: int = ATTN_PER_TILE, tiles_per_item: int = 0) -> None:
    """Process-wide choice of the attention kernel (x17ai_b200_set_attn_schedule): the one-CTA-per-query-tile
    kernel (default, the one the kernel objects embed) or the persistent kernel (`tiles_per_item`
    consecutive query tiles per item, 0 = chosen per launch)."""
    if _lib.load().x17ai_b200_set_attn_schedule(int(schedule), int(tiles_per_item)) != 0:
        raise X17Error(f"unknown attention schedule {schedule} / tiles_per_item {tiles_per_item}")


@dataclass(frozen=True)
class AttnKernelConfig:
    """attn.rs:45-53 (dtype is always Int8)."""
    n_heads: int
    head_dim: int
    q_stride: int
    kv_stride: int
    o_stride: int

    def n_ops(self, seq_len: int, window_size: int) -> float:
        """The reference's own work count (attn.rs:72-84)."""
        attended = window_size + 1.0 if window_size > 0 else seq_len / 2.0 + 0.5
        return 4.0 * (self.n_heads * self.head_dim) * seq_len * attended

    def _c(self):
        return _lib.AttnConfig(self.n_heads, self.head_dim, self.q_stride, self.kv_stride, self.o_stride)


class AttnKernel:
    """AttnKernel::new + launch (attn.rs:171-232, 353-447). `q`, `kv`, `out` may carry a leading
    batch dimension ([B, S, cols]); the reference's 2-D call is batch 1."""

    def __init__(self, config: AttnKernelConfig):
        self.config = config
        self._lib = _lib.load()
        meta = _lib.AttnMeta()
        cfg = config._c()
        check(self._lib.x17ai_b200_attn_meta(ctypes.byref(cfg), ctypes.byref(meta)))
        self.THREADS_PER_BLOCK = int(meta.threads_per_block)
        self.SMEM_BYTES = int(meta.smem_bytes)
        self.Q_PER_BLOCK = int(meta.q_per_block)

    def _shapes(self, q, kv, sink_k, sink_v, attn_temperature, out, l):
        c = self.config
        batch = 1
        if q.dim() == 3:
            batch = q.shape[0]
            q2, kv2, out2 = q[0], kv[0], out[0]
            if kv.shape[0] != batch or out.shape[0] != batch:
                raise X17Error("attention inputs q, kv, out must share the batch dimension")
        else:
            q2, kv2, out2 = q, kv, out
        seq_len, _ = matrix_shape("attention", "q", q2, (None, c.q_stride), DTYPE_INT8)
        matrix_shape("attention", "kv", kv2, (seq_len, c.kv_stride), DTYPE_INT8)
        matrix_shape("attention", "sink_k", sink_k, (c.n_heads, c.head_dim), DTYPE_INT8)
        matrix_shape("attention", "sink_v", sink_v, (c.n_heads, c.head_dim), DTYPE_INT8)
        vector_shape("attention", "attn_temperature", attn_temperature, c.n_heads, DTYPE_F32)
        matrix_shape("attention", "out", out2, (seq_len, c.o_stride), DTYPE_INT8)
        if l is not None:
            l2 = l[0] if l.dim() == 3 else l
            matrix_shape("attention", "l", l2, (c.n_heads, seq_len), DTYPE_F32)
        for t in (q, kv, out):
            if not t.is_contiguous():
                raise X17Error("attention batched inputs must be contiguous")
        return batch, seq_len

    def launch(self, stream, q, kv, sink_k, sink_v, attn_temperature, out, l=None, window_size=0):
        batch, seq_len = self._shapes(q, kv, sink_k, sink_v, attn_temperature, out, l)
        cfg = self.config._c()
        check(self._lib.x17ai_b200_attn_fwd_i8(
            stream.handle, ctypes.byref(cfg), batch, seq_len, _ptr(q), _ptr(kv), _ptr(sink_k), _ptr(sink_v),
            _ptr(attn_temperature), _ptr(out), _ptr(l), window_size))

    def launch_head_block(self, stream, q, kv, sink_k, sink_v, attn_temperature, out, l, window_size, head_begin,
                          peer_outs=()):
        """A head-sharded launch: this kernel's `n_heads` heads starting at head `head_begin` of wider tensors.
        The reference kernel addresses a head group the same way, by column offset with explicit row strides
        (cuda/attn_fwd_i8.cuh:378-384). `q` [.., S, q_stride] and `kv` [.., S, kv_stride] are the full-width
        tensors of all heads, `sink_k` / `sink_v` [H_total, D] and `attn_temperature` [H_total] those of all
        heads; `out` [.., S, o_stride] and `l` [.., n_heads, S] belong to this block alone (column 0 of `out`
        is the block's first head). `peer_outs`: up to seven device addresses (int) of buffers with the layout of
        `out` in other GPUs' memory, mapped into this process; the kernel's epilogue stores the output there as
        well (x17ai_b200_attn_fwd_i8_to_peers), which replaces an all-gather of the shards' outputs."""
        c = self.config
        batch = q.shape[0] if q.dim() == 3 else 1
        q2, kv2, out2 = (q[0], kv[0], out[0]) if q.dim() == 3 else (q, kv, out)
        seq_len, _ = matrix_shape("attention", "q", q2, (None, c.q_stride), DTYPE_INT8)
        matrix_shape("attention", "kv", kv2, (seq_len, c.kv_stride), DTYPE_INT8)
        total = sink_k.shape[0]
        if head_begin < 0 or head_begin + c.n_heads > total:
            raise X17Error(f"attention head block [{head_begin}, {head_begin + c.n_heads}) lies outside the {total} heads")
        if (head_begin + c.n_heads) * c.head_dim > c.q_stride or 2 * (head_begin + c.n_heads) * c.head_dim > c.kv_stride:
            raise X17Error("attention head block lies outside the q / kv row")
        matrix_shape("attention", "sink_k", sink_k, (total, c.head_dim), DTYPE_INT8)
        matrix_shape("attention", "sink_v", sink_v, (total, c.head_dim), DTYPE_INT8)
        vector_shape("attention", "attn_temperature", attn_temperature, total, DTYPE_F32)
        matrix_shape("attention", "out", out2, (seq_len, c.o_stride), DTYPE_INT8)
        if l is not None:
            matrix_shape("attention", "l", l[0] if l.dim() == 3 else l, (c.n_heads, seq_len), DTYPE_F32)
        for t in (q, kv, out):
            if not t.is_contiguous():
                raise X17Error("attention batched inputs must be contiguous")
        cfg = c._c()
        hb, d = head_begin, c.head_dim
        if peer_outs:
            if len(peer_outs) > 7:
                raise X17Error("attention output can be copied to at most seven peers")
            arr = (ctypes.c_void_p * len(peer_outs))(*[int(a) for a in peer_outs])
            check(self._lib.x17ai_b200_attn_fwd_i8_to_peers(
                stream.handle, ctypes.byref(cfg), batch, seq_len, _ptr(q) + hb * d, _ptr(kv) + 2 * hb * d,
                _ptr(sink_k) + hb * d, _ptr(sink_v) + hb * d, _ptr(attn_temperature) + 4 * hb, _ptr(out), _ptr(l),
                window_size, ctypes.cast(arr, ctypes.c_void_p), len(peer_outs)))
            return
        check(self._lib.x17ai_b200_attn_fwd_i8(
            stream.handle, ctypes.byref(cfg), batch, seq_len, _ptr(q) + hb * d, _ptr(kv) + 2 * hb * d,
            _ptr(sink_k) + hb * d, _ptr(sink_v) + hb * d, _ptr(attn_temperature) + 4 * hb, _ptr(out), _ptr(l),
            window_size))

    def launch_from_host(self, streams, h_q, h_kv, sink_k, sink_v, attn_temperature, q, kv, out, h_out,
                         l=None, window_size=0):
        """Batched attention whose q, kv arrive from and whose out returns to pinned host memory.

        Sequences are independent, so sequence b goes through streams[b % len(streams)] as
        upload -> kernel -> download; with two or more streams the copies of one sequence overlap the
        kernel and the opposite-direction copy of its neighbours. `q`, `kv`, `out` ([B, S, cols]) are
        the device staging buffers, `h_q`, `h_kv`, `h_out` their pinned host counterparts. Returns
        after queueing; the caller synchronises every stream before reading `h_out`."""
        batch, seq_len = self._shapes(q, kv, sink_k, sink_v, attn_temperature, out, l)
        if q.dim() != 3:
            raise X17Error("launch_from_host wants batched [B, S, cols] tensors")
        for h, d, name in ((h_q, q, "q"), (h_kv, kv, "kv"), (h_out, out, "out")):
            if tuple(h.shape) != tuple(d.shape) or h.dtype != d.dtype or not h.is_contiguous():
                raise X17Error(f"host buffer {name} must match its device buffer in shape and dtype")
            if not h.is_pinned():
                raise X17Error(f"host buffer {name} must be pinned")
        cfg = self.config._c()
        for b in range(batch):
            st = streams[b % len(streams)]
            st.upload(h_q[b].data_ptr(), q[b].data_ptr(), 0, q[b].numel())
            st.upload(h_kv[b].data_ptr(), kv[b].data_ptr(), 0, kv[b].numel())
            check(self._lib.x17ai_b200_attn_fwd_i8(
                st.handle, ctypes.byref(cfg), 1, seq_len, _ptr(q[b]), _ptr(kv[b]), _ptr(sink_k), _ptr(sink_v),
                _ptr(attn_temperature), _ptr(out[b]), _ptr(l[b]) if l is not None else None, window_size))
            st.download(out[b].data_ptr(), h_out[b].data_ptr(), 0, out[b].numel())

    def launch_pv_fp8(self, stream, q, kv, sink_k, sink_v, attn_temperature, v_scale, out, l=None, window_size=0):
        """fp8 P.V variant: kv holds int8 K and e4m3 V bytes (int8 view), sink_v e4m3, out bf16."""
        c = self.config
        batch = q.shape[0] if q.dim() == 3 else 1
        q2, kv2, out2 = (q[0], kv[0], out[0]) if q.dim() == 3 else (q, kv, out)
        seq_len, _ = matrix_shape("attention", "q", q2, (None, c.q_stride), DTYPE_INT8)
        matrix_shape("attention", "kv", kv2, (seq_len, c.kv_stride), DTYPE_INT8)
        matrix_shape("attention", "sink_k", sink_k, (c.n_heads, c.head_dim), DTYPE_INT8)
        matrix_shape("attention", "sink_v", sink_v, (c.n_heads, c.head_dim), DTYPE_E4M3)
        vector_shape("attention", "attn_temperature", attn_temperature, c.n_heads, DTYPE_F32)
        vector_shape("attention", "v_scale", v_scale, c.n_heads, DTYPE_F32)
        matrix_shape("attention", "out", out2, (seq_len, c.o_stride), DTYPE_BF16)
        cfg = c._c()
        check(self._lib.x17ai_b200_attn_fwd_pv_fp8(
            stream.handle, ctypes.byref(cfg), batch, seq_len, _ptr(q), _ptr(kv), _ptr(sink_k), _ptr(sink_v),
            _ptr(attn_temperature), _ptr(v_scale), _ptr(out), _ptr(l), window_size))

    def launch_scaled(self, stream, q, q_scale, kv, k_scale, v_scale, sink_k, sink_v, attn_temperature, out, l=None,
                      window_size=0):
        """Inputs with one f32 scale per token and head (value = scale * code; `q_scale`, `k_scale`, `v_scale`
        f32 [B, H, S] or [H, S]), bf16 output: x17ai_b200_attn_fwd_i8_scaled."""
        c = self.config
        batch = q.shape[0] if q.dim() == 3 else 1
        q2, kv2, out2 = (q[0], kv[0], out[0]) if q.dim() == 3 else (q, kv, out)
        seq_len, _ = matrix_shape("attention", "q", q2, (None, c.q_stride), DTYPE_INT8)
        matrix_shape("attention", "kv", kv2, (seq_len, c.kv_stride), DTYPE_INT8)
        matrix_shape("attention", "sink_k", sink_k, (c.n_heads, c.head_dim), DTYPE_INT8)
        matrix_shape("attention", "sink_v", sink_v, (c.n_heads, c.head_dim), DTYPE_INT8)
        vector_shape("attention", "attn_temperature", attn_temperature, c.n_heads, DTYPE_F32)
        matrix_shape("attention", "out", out2, (seq_len, c.o_stride), DTYPE_BF16)
        for name, t in (("q_scale", q_scale), ("k_scale", k_scale), ("v_scale", v_scale)):
            t2 = t[0] if t.dim() == 3 else t
            if t.dim() == 3 and t.shape[0] != batch:
                raise X17Error(f"attention input {name} must share the batch dimension")
            matrix_shape("attention", name, t2, (c.n_heads, seq_len), DTYPE_F32)
            if not t.is_contiguous():
                raise X17Error(f"attention input {name} must be contiguous")
        if l is not None:
            matrix_shape("attention", "l", l[0] if l.dim() == 3 else l, (c.n_heads, seq_len), DTYPE_F32)
        cfg = c._c()
        check(self._lib.x17ai_b200_attn_fwd_i8_scaled(
            stream.handle, ctypes.byref(cfg), batch, seq_len, _ptr(q), _ptr(q_scale), _ptr(kv), _ptr(k_scale), _ptr(v_scale),
            _ptr(sink_k), _ptr(sink_v), _ptr(attn_temperature), _ptr(out), _ptr(l), window_size))

    def launch_debug(self, stream, q, kv, sink_k, sink_v, attn_temperature, out, l, window_size, dbg_s, dbg_p, dbg_o):
        batch, seq_len = self._shapes(q, kv, sink_k, sink_v, attn_temperature, out, l)
        cfg = self.config._c()
        check(self._lib.x17ai_b200_attn_fwd_i8_debug(
            stream.handle, ctypes.byref(cfg), batch, seq_len, _ptr(q), _ptr(kv), _ptr(sink_k), _ptr(sink_v),
            _ptr(attn_temperature), _ptr(out), _ptr(l), window_size, _ptr(dbg_s), _ptr(dbg_p), _ptr(dbg_o)))

    def decode(self, stream, q, kv_cache, kv_len, sink_k, sink_v, attn_temperature, out, l=None, window_size=0,
               kv_lens=None, n_splits=0, no_alloc=False):
        """One new token per sequence: q [B, q_stride], kv_cache [B, T, kv_stride], out [B, o_stride].
        `no_alloc=True` takes the entry point that keeps its split-KV partials in the library's built-in
        4 MiB scratch instead of allocating (see x17ai_b200_attn_decode_i8_noalloc in the header)."""
        c = self.config
        batch, _ = matrix_shape("decode", "q", q, (None, c.q_stride), DTYPE_INT8)
        if kv_cache.dim() != 3 or kv_cache.shape[0] != batch or kv_cache.shape[2] != c.kv_stride:
            raise X17Error(f"decode input kv_cache must have shape [{batch}, T, {c.kv_stride}], got {list(kv_cache.shape)}")
        _dtype_and_device("decode", "kv_cache", kv_cache, DTYPE_INT8)
        matrix_shape("decode", "sink_k", sink_k, (c.n_heads, c.head_dim), DTYPE_INT8)
        matrix_shape("decode", "sink_v", sink_v, (c.n_heads, c.head_dim), DTYPE_INT8)
        vector_shape("decode", "attn_temperature", attn_temperature, c.n_heads, DTYPE_F32)
        matrix_shape("decode", "out", out, (batch, c.o_stride), DTYPE_INT8)
        if l is not None:
            matrix_shape("decode", "l", l, (batch, c.n_heads), DTYPE_F32)
        if kv_lens is not None:
            # read on the device as u32 [batch]; lengths above the cache's capacity are clamped there
            if kv_lens.dtype not in (torch.int32, torch.uint32) or tuple(kv_lens.shape) != (batch,):
                raise X17Error(f"decode input kv_lens must be int32 [{batch}], got {kv_lens.dtype} {list(kv_lens.shape)}")
            if not kv_lens.is_cuda or not kv_lens.is_contiguous():
                raise X17Error("decode input kv_lens must be a contiguous tensor on device cuda")
        cfg = c._c()
        entry = self._lib.x17ai_b200_attn_decode_i8_noalloc if no_alloc else self._lib.x17ai_b200_attn_decode_i8
        check(entry(
            stream.handle, ctypes.byref(cfg), batch, _ptr(q), _ptr(kv_cache), kv_cache.shape[1], kv_len,
            _ptr(kv_lens), _ptr(sink_k), _ptr(sink_v), _ptr(attn_temperature), _ptr(out), _ptr(l), window_size,
            n_splits))


@dataclass(frozen=True)
class GemmConfig:
    """GemmConfig + one epilogue config (gemm.rs:60-366). b is [b_rows, a_cols] (trans = true)."""
    a_dtype: int
    b_dtype: int
    c_dtype: int
    epilogue: int
    a_cols: int
    b_rows: int
    inp_scale: float = 1.0
    out_scale: float = 1.0
    eps: float = 2.0 ** -70
    head_dim: int = 0

    def n_ops(self, a_rows: int) -> float:
        """gemm.rs:445-449."""
        return 2.0 * a_rows * self.a_cols * self.b_rows

    def _c(self):
        return _lib.GemmConfig(self.a_dtype, self.b_dtype, self.c_dtype, self.epilogue, self.a_cols, self.b_rows,
                               self.inp_scale, self.out_scale, self.eps, self.head_dim)


class GemmKernel:
    """GemmKernel<E>::new + launch (gemm.rs:368-443, 591-641)."""

    def __init__(self, config: GemmConfig):
        self.config = config
        self._lib = _lib.load()
        meta = _lib.GemmMeta()
        cfg = config._c()
        check(self._lib.x17ai_b200_gemm_meta(ctypes.byref(cfg), ctypes.byref(meta)))
        self.THREADS_PER_BLOCK = int(meta.threads_per_block)
        self.SMEM_BYTES = int(meta.smem_bytes)
        self.M_PER_BLOCK = int(meta.m_per_block)
        self.N_PER_BLOCK = int(meta.n_per_block)

    def launch(self, stream, a, b, c, rrms=None, residual=None):
        g = self.config
        a_rows = self.check_shapes(a, b, c, rrms, residual)
        cfg = g._c()
        check(self._lib.x17ai_b200_gemm_fwd(stream.handle, ctypes.byref(cfg), _ptr(a), a_rows, _ptr(b), g.b_rows,
                                            _ptr(c), _ptr(rrms), _ptr(residual)))

    def check_shapes(self, a, b, c, rrms=None, residual=None) -> int:
        """BasicGemmLauncher's argument checks (gemm.rs:591-641, tensor_check.rs:19-101); returns the row count."""
        g = self.config
        a_rows, _ = matrix_shape("gemm", "a", a, (None, g.a_cols), g.a_dtype)
        split = g.a_dtype == DTYPE_E4M3 and g.b_dtype == DTYPE_INT8
        if split:  # b is the [b_rows, 2 * a_cols] e4m3 buffer made by split_i8_weights
            matrix_shape("gemm", "b", b, (g.b_rows, 2 * g.a_cols), DTYPE_E4M3)
        else:
            matrix_shape("gemm", "b", b, (g.b_rows, g.a_cols), g.b_dtype)
        c_cols = g.b_rows if g.epilogue in (EPI_SCALE, EPI_RMS_NORM) else g.b_rows // 2
        matrix_shape("gemm", "c", c, (a_rows, c_cols), g.c_dtype)
        if g.epilogue == EPI_RMS_NORM:
            if rrms is None:
                raise X17Error("gemm rms-norm epilogue needs the rrms output")
            matrix_shape("gemm", "rrms", rrms, (a_rows, g.b_rows // (2 * g.head_dim)), DTYPE_F32)
        if g.epilogue == EPI_RESIDUAL:
            if residual is None:
                raise X17Error("gemm residual epilogue needs the residual input")
            matrix_shape("gemm", "residual", residual, (a_rows, g.b_rows // 2), DTYPE_INT8)
        return a_rows


def _proj_scale(inputs: int) -> float:
    """inv_sqrt(inputs) / FIXED_I8_SCALE**2 with the reference's operations (sqrt, reciprocal, divide:
    src/util.rs:20-24, src/main.rs:413-415), so that the constant is the same f64."""
    return 1.0 / math.sqrt(float(inputs)) / (FIXED_I8_SCALE * FIXED_I8_SCALE)


def qkvg_fwd_i8(stream, x, w_qkvg, n_heads, head_dim, q, kv, k_rrms, g=None, eps=2.0 ** -70):
    """Fused Q / KV / gate projection (attn_q_fwd + attn_kv_fwd of src/main.rs:387-491 in one launch)."""
    rows, model_dim = matrix_shape("qkvg", "x", x, (None, None), DTYPE_INT8)
    hd = n_heads * head_dim
    gate_cols = 0 if g is None else g.shape[1]
    matrix_shape("qkvg", "w_qkvg", w_qkvg, (3 * hd + gate_cols, model_dim), DTYPE_INT8)
    matrix_shape("qkvg", "q", q, (rows, hd), DTYPE_INT8)
    matrix_shape("qkvg", "kv", kv, (rows, 2 * hd), DTYPE_INT8)
    matrix_shape("qkvg", "k_rrms", k_rrms, (rows, n_heads), DTYPE_F32)
    if g is not None:
        matrix_shape("qkvg", "g", g, (rows, gate_cols), DTYPE_INT8)
    cfg = _lib.QkvgConfig(model_dim, n_heads, head_dim, gate_cols, _proj_scale(model_dim), FIXED_I8_SCALE, eps)
    check(_lib.load().x17ai_b200_qkvg_fwd_i8(stream.handle, ctypes.byref(cfg), _ptr(x), rows, _ptr(w_qkvg), _ptr(q),
                                              _ptr(kv), _ptr(k_rrms), _ptr(g)))


def split_i8_weights(stream, w):
    """int8 weights [rows, cols] -> e4m3 [rows, 2*cols] = [16*hi | lo] for e4m3-activation GEMMs."""
    rows, cols = matrix_shape("split_i8_weights", "w", w, (None, None), DTYPE_INT8)
    out = torch.empty((rows, 2 * cols), dtype=torch.uint8, device=w.device)
    check(_lib.load().x17ai_b200_split_i8_weights(stream.handle, _ptr(w), rows, cols, _ptr(out)))
    return out


def rms_norm(stream, mode, inp, out, row_scale=None, eps=2.0 ** -70):
    """Rms_norm::kernel (rms_norm.cu:55-113) and its bf16-input modes."""
    in_dtype = DTYPE_E4M3 if mode == RMS_E4M3_FIXED else DTYPE_BF16
    rows, cols = matrix_shape("rms_norm", "inp", inp, (None, None), in_dtype)
    matrix_shape("rms_norm", "out", out, (rows, cols), DTYPE_INT8)
    if mode == RMS_BF16_ROWSCALE:
        if row_scale is None:
            raise X17Error("rms_norm row-scale mode needs the row_scale output")
        vector_shape("rms_norm", "row_scale", row_scale, rows, DTYPE_F32)
    check(_lib.load().x17ai_b200_rms_norm(stream.handle, mode, _ptr(inp), rows, cols, _ptr(out), _ptr(row_scale), eps))


# ---- the live kernels of the reference's block (src/main.rs:387-675) with their scales ----------

def attn_q_fwd_config(model_dim, q_outputs):
    return GemmConfig(DTYPE_INT8, DTYPE_INT8, DTYPE_INT8, EPI_SCALE, model_dim, q_outputs,
                      inp_scale=_proj_scale(model_dim), out_scale=FIXED_I8_SCALE)


def attn_kv_fwd_config(model_dim, kv_outputs, head_dim, eps=2.0 ** -70):
    return GemmConfig(DTYPE_INT8, DTYPE_INT8, DTYPE_INT8, EPI_RMS_NORM, model_dim, kv_outputs,
                      inp_scale=_proj_scale(model_dim), out_scale=FIXED_I8_SCALE, eps=eps, head_dim=head_dim)


def attn_y_fwd_config(attn_width, model_dim, c_dtype=DTYPE_E4M3):
    return GemmConfig(DTYPE_INT8, DTYPE_INT8, c_dtype, EPI_RESIDUAL, attn_width, 2 * model_dim,
                      inp_scale=_proj_scale(attn_width), out_scale=1.0)


def ffn_f_fwd_config(model_dim, f_width):
    return GemmConfig(DTYPE_INT8, DTYPE_INT8, DTYPE_E4M3, EPI_GEGLU, model_dim, 2 * f_width,
                      inp_scale=_proj_scale(model_dim), out_scale=1.0)


def ffn_y_fwd_f8_config(f_width, model_dim, b_dtype=DTYPE_INT8, c_dtype=DTYPE_E4M3):
    return GemmConfig(DTYPE_E4M3, b_dtype, c_dtype, EPI_RESIDUAL, f_width, 2 * model_dim,
                      inp_scale=math.sqrt(GELU_VAR_FIX_2 / f_width) / 8.0, out_scale=1.0)


def ffn_f_fwd_e4m3_config(model_dim, f_width, x_scale, w_scale):
    """GeGLU FFN input projection with e4m3 activations and e4m3 weights, one f32 scale per tensor (value =
    scale * e4m3): the benchmark description's second FFN run; the reference has no such kernel (its "f8" GEMM,
    gemm_b16.cuh:72-185, keeps int8 weights). The tensor scales are the epilogue's input scale: the
    pre-activations are the plain products of the values (weights drawn N(0, 0.02) carry their own
    1/sqrt(fan-in); the reference's Dm^-1/2 belongs to its unit-variance FixedI8 weights)."""
    return GemmConfig(DTYPE_E4M3, DTYPE_E4M3, DTYPE_E4M3, EPI_GEGLU, model_dim, 2 * f_width,
                      inp_scale=float(x_scale) * float(w_scale), out_scale=1.0)


def ffn_y_fwd_e4m3_config(f_width, model_dim, w_scale, c_dtype=DTYPE_E4M3):
    """FFN output projection of the same run: e4m3 GeGLU output x e4m3 weights (scale w_scale), gated residual
    with the FixedI8 residual stream."""
    return GemmConfig(DTYPE_E4M3, DTYPE_E4M3, c_dtype, EPI_RESIDUAL, f_width, 2 * model_dim,
                      inp_scale=float(w_scale), out_scale=1.0)


def ffn_y_fwd_i8_config(f_width, model_dim, c_dtype=DTYPE_INT8):
    return GemmConfig(DTYPE_INT8, DTYPE_INT8, c_dtype, EPI_RESIDUAL, f_width, 2 * model_dim,
                      inp_scale=math.sqrt(GELU_VAR_FIX_2 / f_width) / 64.0, out_scale=1.0)
