"""CPU restatement of the reference's int8 sliding-window attention forward.

TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the CPU-baseline
leg of the benchmark; never by the product path.

Follows the reference *kernel* (not its float64 PyTorch model) step by step:
  AttnForward::run                 cuda/attn_fwd_i8.cuh:368-619
    window rounding, KV range      :408-422
    temperature (SSMax)            :444-450, :497
    sink seeding of max/sum/O      :489-517
    per-KV-tile loop               :520-606   (QK^T i32, scale, masks, online softmax,
                                               P -> u8, PV i32 -> f32 accumulate)
    online_softmax                 :208-291   (running max, lazy rescale, un-rounded sum)
    combine_and_store              :293-351   (out = rint(clamp(O / sum)), L = log2(sum) + max)
  masks: keys j with i - W' <= j <= i - 1  (:79-134, :540-567), W' = W rounded up to 16
Pinned twice: against the float64 model new_block.py:162-232 (attn_one_head) through the fixtures
of tests/golden, and, with `kv_tile=16`, bit for bit against the reference kernel itself compiled
for sm_100a (oracle/build_ref.py, tests/test_gpu_reference_kernel.py).

`kv_tile` is the number of keys per online-softmax step.  The reference kernel uses 16
(:65-66); a different tile changes when the running max moves and therefore which
probabilities round up or down, so out codes may differ by one step between tilings.
Integer parts (scores, P.V per tile) are exact for any tiling.
"""
import math

import numpy as np

F32 = np.float32
PROB_SCALE = F32(255.0)   # attn_fwd_i8.cuh:206
E_APPROX = 3              # attn_fwd_i8.cuh:446


def _round_window(window):
    """attn_fwd_i8.cuh:408-412: 0 = unbounded; otherwise round up to a multiple of 16."""
    if window == 0:
        return None
    return ((window - 1) // 16 + 1) * 16


def row_temperature(seq_len, head_dim, window, pos0=0):
    """f32 per-row temperature before the per-head factor (attn_fwd_i8.cuh:444-450)."""
    w = _round_window(window)
    i = np.arange(pos0, pos0 + seq_len, dtype=np.int64)
    n = i + 1 + E_APPROX if w is None else np.minimum(w + 1 + E_APPROX, i + 1 + E_APPROX)
    base = F32((1.0 / math.sqrt(head_dim)) / 64.0)
    return (base * np.log2(n.astype(F32)).astype(F32)).astype(F32)


def attn_head(q, k, v, sink_k, sink_v, head_temp, window, kv_tile=16, want_debug=False):
    """One head. q,k,v: int8 [S,D]; sink_k,sink_v: int8 [D]; head_temp: float.
    Returns out int8 [S,D], l f32 [S] (and optionally a dict of per-row stats)."""
    q = np.asarray(q, dtype=np.int8)
    k = np.asarray(k, dtype=np.int8)
    v = np.asarray(v, dtype=np.int8)
    s_len, d = q.shape
    w = _round_window(window)
    t = kv_tile
    qf = q.astype(F32)
    kf = k.astype(F32)
    vf = v.astype(F32)
    temp = (row_temperature(s_len, d, window) * F32(head_temp)).astype(F32)   # :497

    sink_score = (qf @ np.asarray(sink_k, dtype=np.int8).astype(F32)).astype(F32)  # exact ints
    m = (sink_score * temp).astype(F32)                        # :498-499
    ssum = np.full(s_len, PROB_SCALE, dtype=F32)               # :500 (4 x 0.25 x 255)
    o = np.tile(np.asarray(sink_v, dtype=np.int8).astype(F32) * PROB_SCALE, (s_len, 1))  # :505-517

    n_tiles = (s_len + t - 1) // t
    rows_all = np.arange(s_len, dtype=np.int64)
    for ti in range(n_tiles):
        k0 = ti * t
        k1 = min(k0 + t, s_len)
        # rows that attend at least one key of this tile: j <= i-1 and j >= i-w
        r0 = k0 + 1
        r1 = s_len if w is None else min(s_len, k1 - 1 + w + 1)
        if r0 >= r1:
            continue
        rows = rows_all[r0:r1]
        keys = np.arange(k0, k1, dtype=np.int64)
        acc = qf[r0:r1] @ kf[k0:k1].T                          # exact int32 values in f32
        s = (acc * temp[r0:r1, None]).astype(F32)              # :534-536
        mask = keys[None, :] >= rows[:, None]                  # causal, strict
        if w is not None:
            mask |= keys[None, :] < (rows[:, None] - w)
        s = np.where(mask, F32(-np.inf), s)
        tile_max = s.max(axis=1)
        new_m = np.maximum(m[r0:r1], tile_max)                 # :232-256
        rescale = np.exp2((m[r0:r1] - new_m).astype(F32)).astype(F32)
        p = (np.exp2((s - new_m[:, None]).astype(F32)).astype(F32) * PROB_SCALE).astype(F32)  # :265-277
        ssum[r0:r1] = (ssum[r0:r1] * rescale + p.sum(axis=1, dtype=np.float64)).astype(F32)    # :280-290
        p_u8 = np.rint(p)                                      # Round_cast<u8,f32>, utils_core.cuh:119-123
        pv = p_u8.astype(F32) @ vf[k0:k1]                      # exact ints (< 2^24)
        o[r0:r1] = (o[r0:r1] * rescale[:, None] + pv).astype(F32)   # :588-605
        m[r0:r1] = new_m

    recip = (F32(1.0) / ssum).astype(F32)                      # :325-326
    out = np.rint(np.clip((o * recip[:, None]).astype(F32), F32(-127), F32(127))).astype(np.int8)
    l = (np.log2(ssum).astype(F32) + m).astype(F32)            # :322-323
    if want_debug:
        return out, l, {"max": m, "sum": ssum, "o": o, "sink_score": sink_score, "temp": temp}
    return out, l


def attn_fwd_i8(q, kv, sink_k, sink_v, temperature, window, n_heads, head_dim, kv_tile=16):
    """Whole launch. q int8 [S, H*D]; kv int8 [S, H*2*D] with per-head [K(D)|V(D)]
    (attn_fwd_i8.cuh:383,475,528); sink_k/sink_v int8 [H,D]; temperature f32 [H].
    Returns out int8 [S, H*D], l f32 [H, S] (templates/attn/kernel.cu:9-20)."""
    q = np.asarray(q, dtype=np.int8)
    kv = np.asarray(kv, dtype=np.int8)
    s_len = q.shape[0]
    d = head_dim
    out = np.empty((s_len, n_heads * d), dtype=np.int8)
    l = np.empty((n_heads, s_len), dtype=F32)
    temperature = np.asarray(temperature, dtype=F32).reshape(-1)
    for h in range(n_heads):
        qh = q[:, h * d:(h + 1) * d]
        kh = kv[:, 2 * h * d:2 * h * d + d]
        vh = kv[:, 2 * h * d + d:2 * (h + 1) * d]
        o, lh = attn_head(qh, kh, vh, sink_k[h], sink_v[h], temperature[h], window, kv_tile)
        out[:, h * d:(h + 1) * d] = o
        l[h] = lh
    return out, l


def attn_decode_i8(q, kv_cache, kv_len, sink_k, sink_v, temperature, window, n_heads, head_dim,
                   kv_tile=16):
    """Single-query decode with the prefill semantics (no int8 decode exists in the reference:
    the stale attn_incremental.cu:329-481 is bf16).  The new token sits at position `kv_len`
    and attends keys [kv_len - W', kv_len - 1] of the cache plus the sink, exactly as row
    `kv_len` of attn_fwd_i8 would.
    q int8 [B, H*D]; kv_cache int8 [B, T, H*2*D]; returns out int8 [B, H*D], l f32 [B, H]."""
    q = np.asarray(q, dtype=np.int8)
    b = q.shape[0]
    d = head_dim
    out = np.empty((b, n_heads * d), dtype=np.int8)
    l = np.empty((b, n_heads), dtype=F32)
    temperature = np.asarray(temperature, dtype=F32).reshape(-1)
    w = _round_window(window)
    for bi in range(b):
        k_lo = 0 if w is None else max(0, kv_len - w)
        for h in range(n_heads):
            kh = kv_cache[bi, k_lo:kv_len, 2 * h * d:2 * h * d + d]
            vh = kv_cache[bi, k_lo:kv_len, 2 * h * d + d:2 * (h + 1) * d]
            o, lh = _decode_row(q[bi, h * d:(h + 1) * d], kh, vh, sink_k[h], sink_v[h],
                                temperature[h], kv_len, w, kv_tile, k_lo)
            out[bi, h * d:(h + 1) * d] = o
            l[bi, h] = lh
    return out, l


def _decode_row(q, k, v, sink_k, sink_v, head_temp, pos, w, kv_tile, k_lo):
    d = q.shape[0]
    qf = q.astype(F32)
    n = pos + 1 + E_APPROX if w is None else min(w + 1 + E_APPROX, pos + 1 + E_APPROX)
    temp = F32(F32((1.0 / math.sqrt(d)) / 64.0) * np.log2(F32(n)).astype(F32)) * F32(head_temp)
    temp = F32(temp)
    m = F32(F32(qf @ np.asarray(sink_k, dtype=np.int8).astype(F32)) * temp)
    ssum = PROB_SCALE
    o = np.asarray(sink_v, dtype=np.int8).astype(F32) * PROB_SCALE
    n_keys = k.shape[0]
    # tiles are aligned to absolute key positions, as in the prefill kernel
    first = (k_lo // kv_tile) * kv_tile
    for t0 in range(first, k_lo + n_keys, kv_tile):
        a = max(t0, k_lo) - k_lo
        b = min(t0 + kv_tile, k_lo + n_keys) - k_lo
        if a >= b:
            continue
        s = ((k[a:b].astype(F32) @ qf) * temp).astype(F32)
        new_m = max(m, F32(s.max()))
        rescale = F32(np.exp2(F32(m - new_m)))
        p = (np.exp2((s - new_m).astype(F32)).astype(F32) * PROB_SCALE).astype(F32)
        ssum = F32(F32(ssum * rescale) + F32(p.sum(dtype=np.float64)))
        pv = np.rint(p).astype(F32) @ v[a:b].astype(F32)
        o = (o * rescale + pv).astype(F32)
        m = new_m
    recip = F32(1.0) / F32(ssum)
    out = np.rint(np.clip((o * recip).astype(F32), F32(-127), F32(127))).astype(np.int8)
    return out, F32(np.log2(F32(ssum)) + m)


def attended_keys_total(seq_len, window):
    """Sum over queries of (min(i, W') + 1): attended keys including the sink."""
    w = _round_window(window)
    i = np.arange(seq_len, dtype=np.int64)
    n = i if w is None else np.minimum(i, w)
    return int((n + 1).sum())


def attn_ops(batch, n_heads, head_dim, seq_len, window):
    """Algorithmic operation count of one attention pass: 4 * B*H*D * sum_i (min(i,W')+1)."""
    return 4.0 * batch * n_heads * head_dim * attended_keys_total(seq_len, window)


def attn_fwd_pv_fp8(q, k, v_e4m3, sink_k, sink_v_e4m3, temperature, v_scale, window, n_heads, head_dim):
    """fp8 P.V variant described for the benchmark (no counterpart in the reference; its
    attn_y_fwd_fp8.cu:11-47 is a bf16 GEMM).  Scores, masks, sink, temperature and maximum as in
    attn_head (cuda/attn_fwd_i8.cuh:408-450, 489-517); then P = e4m3(256 * 2^(s - max)) with the OCP
    e4m3 encoding (round to nearest even), V = e4m3 * v_scale[h], O accumulated in float (float64 here,
    f32 on the tensor core), out = O / sum * v_scale with the un-rounded sum, L = log2(256 * sum) + max.
    q, k: int8 [S, H*D]; v_e4m3: uint8 [S, H*D]; returns out f32 [S, H*D] (before the bf16 cast), l [H, S]."""
    from . import formats
    q = np.asarray(q, dtype=np.int8)
    k = np.asarray(k, dtype=np.int8)
    s_len, d = q.shape[0], head_dim
    w = _round_window(window)
    out = np.empty((s_len, n_heads * d), dtype=F32)
    l = np.empty((n_heads, s_len), dtype=F32)
    i = np.arange(s_len)[:, None]
    j = np.arange(s_len)[None, :]
    mask = j >= i
    if w is not None:
        mask |= j < i - w
    for h in range(n_heads):
        sl = slice(h * d, (h + 1) * d)
        qf, kf = q[:, sl].astype(F32), k[:, sl].astype(F32)
        vf = formats.hw_e4m3_to_f32(v_e4m3[:, sl]).astype(np.float64)
        svf = formats.hw_e4m3_to_f32(sink_v_e4m3[h]).astype(np.float64)
        temp = (row_temperature(s_len, d, window) * F32(temperature[h])).astype(F32)
        sink_s = ((qf @ np.asarray(sink_k[h], dtype=np.int8).astype(F32)) * temp).astype(F32)
        acc = qf @ kf.T
        # the kernel evaluates fma(acc, temp, -max) with one rounding
        s64 = acc.astype(np.float64) * temp.astype(np.float64)[:, None]
        s32 = np.where(mask, -np.inf, (acc * temp[:, None]).astype(F32))
        m = np.maximum(sink_s, s32.max(axis=1)).astype(F32)
        x = np.where(mask, -np.inf, (s64 - m.astype(np.float64)[:, None])).astype(F32)
        p = np.exp2(x).astype(F32)
        sink_e = np.exp2((sink_s - m).astype(F32)).astype(F32)
        total = ((p.sum(axis=1, dtype=np.float64) + sink_e).astype(F32) * F32(256.0)).astype(F32)
        p8 = formats.hw_e4m3_to_f32(formats.hw_f32_to_e4m3((p * F32(256.0)).astype(F32))).astype(np.float64)
        o = p8 @ vf + (sink_e.astype(np.float64) * 256.0)[:, None] * svf[None, :]
        out[:, sl] = (o / total.astype(np.float64)[:, None] * float(v_scale[h])).astype(F32)
        l[h] = (np.log2(total) + m).astype(F32)
    return out, l


def quantize_per_token(x):
    """Symmetric int8 quantisation with one f32 scale per token and head (the benchmark description's input
    format): x [..., D] -> (codes int8 [..., D], scale f32 [...]) with scale = absmax / 127, x ~ scale * code."""
    x = np.asarray(x, dtype=np.float64)
    amax = np.abs(x).max(axis=-1)
    scale = np.where(amax > 0, amax / 127.0, 1.0).astype(F32)
    codes = np.clip(np.rint(x / scale[..., None].astype(np.float64)), -127, 127).astype(np.int8)
    return codes, scale


def attn_fwd_i8_scaled(q, q_scale, k, k_scale, v, v_scale, sink_k, sink_v, temperature, window, quantise_p=True):
    """The int8 attention on per-token-per-head scaled inputs with real-valued (bf16) output.  No counterpart in the
    reference (one global FixedI8 scale, cuda/utils_b8.cuh:7-10); masks, sink, temperature, maximum and normaliser
    follow the reference kernel as attn_head does (cuda/attn_fwd_i8.cuh:408-450, 489-517): parity of this mode is
    pinned by this restatement only, and by its case q_scale = k_scale = v_scale = 1/8, which is attn_head.
      q, k, v int8 [S, H, D]; q_scale, k_scale, v_scale f32 [H, S]; sink_k, sink_v int8 [H, D] (FixedI8, code / 8);
      returns out f64 [S, H, D] (before the bf16 cast) and l f32 [H, S].
    `quantise_p` models the kernel's u8 probabilities P = rint(255 * 2^(x - m) * v_scale / g), g the largest v_scale
    among the row's visible keys (so P <= 255 without a second maximum over the scores); without it the result is the
    plain float64 softmax attention of the dequantised inputs."""
    q = np.asarray(q, dtype=np.int8); k = np.asarray(k, dtype=np.int8); v = np.asarray(v, dtype=np.int8)
    s_len, n_heads, d = q.shape
    w = _round_window(window)
    i = np.arange(s_len)[:, None]
    j = np.arange(s_len)[None, :]
    mask = j >= i
    if w is not None:
        mask |= j < i - w
    out = np.zeros((s_len, n_heads, d), dtype=np.float64)
    l = np.zeros((n_heads, s_len), dtype=F32)
    for h in range(n_heads):
        temp = row_temperature(s_len, d, window).astype(np.float64) * float(temperature[h])     # includes the 1/64
        a_row = temp * 64.0 * q_scale[h].astype(np.float64)
        acc = q[:, h].astype(np.int64) @ k[:, h].astype(np.int64).T
        x = acc * a_row[:, None] * k_scale[h].astype(np.float64)[None, :]
        x = np.where(mask, -np.inf, x)
        sink_s = (q[:, h].astype(np.int64) @ np.asarray(sink_k[h], dtype=np.int64)) * a_row * 0.125
        m = np.maximum(sink_s, x.max(axis=1))
        e = np.exp2(x - m[:, None])
        sink_e = np.exp2(sink_s - m)
        total = e.sum(axis=1) + sink_e
        vs = v_scale[h].astype(np.float64)
        if quantise_p:
            wgt = e * vs[None, :]
            g = np.where(mask, 0.0, vs[None, :]).max(axis=1)       # the largest v_scale among the row's visible keys
            p8 = np.where(g[:, None] > 0, np.rint(255.0 * wgt / np.where(g > 0, g, 1.0)[:, None]), 0.0)
            o = (p8 @ v[:, h].astype(np.float64)) * (g / 255.0)[:, None]
        else:
            o = (e * vs[None, :]) @ v[:, h].astype(np.float64)
        o = o + sink_e[:, None] * (np.asarray(sink_v[h], dtype=np.float64) / 8.0)[None, :]
        out[:, h] = o / total[:, None]
        l[h] = (np.log2(255.0 * total) + m).astype(F32)
    return out, l
