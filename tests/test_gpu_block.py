"""The six kernels of the reference's block chained on the device (x17ai_b200/block.py, the launch
sequence of src/main.rs:193-255), every stage checked against the oracle applied to the tensor the
device actually fed it, and the ends against the reference model's own fixtures."""
import numpy as np
import pytest
import torch

from conftest import code_hist, load_golden
from oracle import attn as o_attn, gemm as o_gemm

pytestmark = pytest.mark.gpu


def _block(stream, g, c, fused):
    from x17ai_b200.block import BlockConfig, BlockForward
    S, Dm, D, H, F, W = c["S"], c["Dm"], c["D"], c["H"], c["F"], c["W"]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    blk = BlockForward(
        stream, BlockConfig(Dm, H, D, F, W),
        t(g["attn_q_weights_i8"].reshape(H * D, Dm)), t(g["attn_kv_weights_i8"].reshape(2 * H * D, Dm)),
        t(g["attn_y_weights_i8"].reshape(2 * Dm, H * D)), t(g["ffn_f_weights_i8"].reshape(2 * F, Dm)),
        t(g["ffn_y_weights_i8"].reshape(2 * Dm, F)), t(g["sinks_k_i8"].reshape(H, D)), t(g["sinks_v_i8"].reshape(H, D)),
        t(g["attn_temperature_f32"].reshape(H)), fused_qkv=fused)
    x = t(g["x_i8"].reshape(S, Dm))
    torch.cuda.synchronize()
    return blk, x


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128", "block_d32_w0"])
def test_block_forward_chain(stream, name, fused):
    from x17ai_b200 import X17Error
    g, c = load_golden(name)
    S, Dm, D, H, F, W = c["S"], c["Dm"], c["D"], c["H"], c["F"], c["W"]
    if fused and (H * D) % 256 != 0:   # the fused projection tiles the output by 256 columns
        with pytest.raises(X17Error, match="multiple of 256"):
            _block(stream, g, c, fused)
        return
    blk, x = _block(stream, g, c, fused)
    out = blk.forward(x, timed=True)
    got = {k: v.cpu().numpy() for k, v in out.items()}
    xs = g["x_i8"].reshape(S, Dm)

    # projections: the reference model's tensors themselves
    assert np.array_equal(got["q"], g["q_i8"].reshape(S, H * D))
    dd = np.abs(got["kv"].astype(np.int32) - g["kv_i8"].reshape(S, 2 * H * D).astype(np.int32))
    assert dd.max() <= 1 and (dd > 0).mean() <= 1e-4
    assert np.max(np.abs(got["k_rrms"] / g["k_rrms_f32"].reshape(S, H) - 1)) < 1e-6

    # attention on the q, kv the device produced: oracle with one KV tile (the kernel's schedule)
    ref_out, ref_l = o_attn.attn_fwd_i8(got["q"], got["kv"], g["sinks_k_i8"].reshape(H, D),
                                        g["sinks_v_i8"].reshape(H, D), g["attn_temperature_f32"].reshape(H), W, H, D,
                                        kv_tile=1 << 20)
    hist = code_hist(got["attn_out"], ref_out)
    assert hist[2:].sum() == 0 and hist[1] / got["attn_out"].size <= 0.02
    assert np.max(np.abs(got["attn_l"] - ref_l)) < 1e-3
    # and against the float64 model: the bar the reference's own kernel meets (expected.txt:65-99)
    hist = code_hist(got["attn_out"], g["attn_out_i8"].reshape(S, H * D))
    assert hist[1:].sum() / got["attn_out"].size <= 0.40 and hist[6:].sum() == 0

    # output projection with gated residual, on the attention output the device produced
    ref = o_gemm.attn_y_fwd(got["attn_out"], g["attn_y_weights_i8"].reshape(2 * Dm, H * D), xs)
    assert (got["attn_y"] != ref).mean() <= 2e-3
    # FFN: GeGLU on x, then the e4m3 x int8 projection on the GeGLU output the device produced
    assert (got["ffn_f"] != g["ffn_f_f8"].reshape(S, F)).mean() <= 2e-3
    ref = o_gemm.ffn_y_fwd_f8(got["ffn_f"], g["ffn_y_weights_i8"].reshape(2 * Dm, F), xs)
    assert (got["ffn_y"] != ref).mean() <= 2e-3
    assert (got["ffn_y"] != g["ffn_y_f8"].reshape(S, Dm)).mean() <= 5e-3

    # per-stage device times, like the reference's harness prints them
    assert set(blk.seconds) == set(blk.STAGES) and all(v >= 0.0 for v in blk.seconds.values())
    ops = blk.n_ops(S)
    assert ops["attn_q"] == 2.0 * S * Dm * H * D and ops["ffn_f"] == 2.0 * S * Dm * 2 * F


def test_block_forward_twice_is_stable(stream):
    """Buffers are reused: a second forward on the same input returns the same bytes."""
    g, c = load_golden("block_d64_w64")
    blk, x = _block(stream, g, c, False)
    first = {k: v.clone() for k, v in blk.forward(x).items()}
    stream.synchronize()
    second = blk.forward(x)
    stream.synchronize()
    for k in first:
        assert torch.equal(first[k], second[k]), k
