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


def test_block_from_reference_files(stream, tmp_path):
    """The block built from safetensors files named as the reference's harness names them
    (src/main.rs:39-71) equals the block built from the same tensors in memory."""
    from x17ai_b200 import tensor_io
    from x17ai_b200.block import BlockForward
    g, c = load_golden("block_d64_w64")
    S, Dm, D, H, F, W = c["S"], c["Dm"], c["D"], c["H"], c["F"], c["W"]
    shapes = {"x_i8": (S, Dm), "attn_q_weights_i8": (H * D, Dm), "attn_kv_weights_i8": (H, 2 * D, Dm),
              "attn_y_weights_i8": (2 * Dm, H * D), "ffn_f_weights_i8": (2 * F, Dm), "ffn_y_weights_i8": (2 * Dm, F),
              "sinks_k_i8": (H, D), "sinks_v_i8": (H, D), "attn_temperature_f32": (H,)}
    for name, shape in shapes.items():
        tensor_io.write_safetensors_file(tmp_path / f"{name}.safetensors", torch.from_numpy(g[name].reshape(shape)), name)
    blk, x = BlockForward.from_directory(stream, tmp_path, H, D, W)
    assert blk.config.model_dim == Dm and blk.config.ffn_width == F and tuple(x.shape) == (S, Dm)
    got = {k: v.clone() for k, v in blk.forward(x).items()}
    stream.synchronize()
    ref_blk, ref_x = _block(stream, g, c, False)
    want = ref_blk.forward(ref_x)
    stream.synchronize()
    for k in want:
        assert torch.equal(got[k], want[k]), k
    # the output files of the reference's harness (src/main.rs:273-280), read back with the safetensors package
    from safetensors.torch import load_file
    blk.save_outputs(tmp_path / "out", blk.forward(x))
    q = load_file(str(tmp_path / "out" / "q_i8.safetensors"))["tensor"]
    assert np.array_equal(q.numpy(), g["q_i8"].reshape(S, H * D))
    kv = load_file(str(tmp_path / "out" / "kv_i8.safetensors"))["tensor"]
    assert tuple(kv.shape) == (S, H, 2, D) and torch.equal(kv.reshape(S, -1), want["kv"].cpu())
    y = load_file(str(tmp_path / "out" / "ffn_y_f8.safetensors"))["tensor"]
    assert y.dtype == torch.float8_e4m3fn and torch.equal(y.view(torch.uint8), want["ffn_y"].cpu())
    with pytest.raises(Exception, match="requires a CPU tensor"):
        tensor_io.write_safetensors_file(tmp_path / "dev.safetensors", want["q"])


def test_block_harness_writes_what_it_reports(tmp_path):
    """`python -m x17ai_b200.block_main` on fixture files: the report names every launch of
    src/main.rs:355-372 and the stored files hold the fixtures' projections."""
    import io
    from safetensors.torch import load_file
    from x17ai_b200 import block_main, tensor_io
    g, c = load_golden("block_d128_w128")
    S, Dm, D, H, F, W = c["S"], c["Dm"], c["D"], c["H"], c["F"], c["W"]
    shapes = {"x_i8": (S, Dm), "attn_q_weights_i8": (H * D, Dm), "attn_kv_weights_i8": (2 * H * D, Dm),
              "attn_y_weights_i8": (2 * Dm, H * D), "ffn_f_weights_i8": (2 * F, Dm), "ffn_y_weights_i8": (2 * Dm, F),
              "sinks_k_i8": (H, D), "sinks_v_i8": (H, D), "attn_temperature_f32": (H,)}
    for name, shape in shapes.items():
        tensor_io.write_safetensors_file(tmp_path / "in" / f"{name}.safetensors", torch.from_numpy(g[name].reshape(shape)))
    for fused in (False, True):
        if fused and (H * D) % 256 != 0:
            continue
        text = io.StringIO()
        seconds = block_main.run(tmp_path / "in", tmp_path / "out", H, D, W, fused_qkv=fused, out=text)
        report = text.getvalue()
        for name in (("qkvg_fwd_i8",) if fused else ("attn_q_fwd", "attn_kv_fwd")) + ("attn_fwd_i8", "attn_y_fwd", "ffn_f_fwd", "ffn_y_fwd_f8"):
            assert f"\t{name} in " in report, report
        assert all(v > 0 for k, v in seconds.items() if not (fused and k == "attn_kv"))
        q = load_file(str(tmp_path / "out" / "q_i8.safetensors"))["tensor"].numpy()
        assert np.array_equal(q, g["q_i8"].reshape(S, H * D))
        f8 = load_file(str(tmp_path / "out" / "ffn_f_f8.safetensors"))["tensor"].view(torch.uint8).numpy()
        assert (f8 != g["ffn_f_f8"].reshape(S, F)).mean() <= 1e-3
    assert block_main.main([str(tmp_path / "nowhere"), str(tmp_path / "out"), "--heads", "2", "--head-dim", "128"]) == 1


def test_block_graph_replay(stream):
    """The six launches recorded once and replayed (x17ai_b200_graph_*): a replay on new input in the
    same buffer equals a plain forward on that input, and counts its kernels as launches."""
    import x17ai_b200
    from x17ai_b200 import X17Error
    from x17ai_b200.device import CudaGraph
    lib = x17ai_b200.load()
    g, c = load_golden("block_d128_w128")
    for fused in (False, True):
        blk, x = _block(stream, g, c, fused)
        with pytest.raises(X17Error, match="capture"):
            blk.replay()
        blk.capture(x)
        n = blk._graph.kernel_nodes
        assert n == (5 if fused else 6)
        x2 = torch.roll(x, shifts=3, dims=0).contiguous()
        want = {k: v.clone() for k, v in blk.forward(x2).items()}
        stream.synchronize()
        x.copy_(x2)
        torch.cuda.synchronize()
        before = lib.x17ai_b200_launch_count()
        blk.replay()
        stream.synchronize()
        assert lib.x17ai_b200_launch_count() - before == n
        for k, v in want.items():
            assert torch.equal(getattr(blk, k), v), k
    # a synchronising call inside the recording invalidates it; the error is reported, the stream stays usable
    with pytest.raises(X17Error):
        with CudaGraph(stream):
            blk.forward(x)
            stream.synchronize()
    out = blk.forward(x)
    stream.synchronize()
    assert torch.equal(out["q"], want["q"])


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128"])
def test_layer_sequential_form(stream, name):
    """forward_layer: RMSNorm -> attention sub-block -> RMSNorm -> FFN sub-block, two layers chained through
    the e4m3 hidden state; every stage against the oracle applied to the tensor the device fed it."""
    from oracle import rms_norm as o_rms
    g, c = load_golden(name)
    S, Dm, D, H, F, W = c["S"], c["Dm"], c["D"], c["H"], c["F"], c["W"]
    blk, _ = _block(stream, g, c, False)
    h = torch.from_numpy(g["ffn_y_f8"].reshape(S, Dm).copy()).cuda()   # an e4m3 hidden state of the model's own making
    torch.cuda.synchronize()
    for layer in range(2):
        out = blk.forward_layer(h)
        stream.synchronize()
        got = {k: v.cpu().numpy() for k, v in out.items()}
        h_np = h.cpu().numpy()
        ref = o_rms.rms_norm_e4m3_i8(h_np)
        dd = np.abs(got["x_attn"].astype(np.int32) - ref.astype(np.int32))
        assert dd.max() <= 1 and (dd > 0).mean() <= 2e-3
        x = got["x_attn"]
        assert np.array_equal(got["q"], o_gemm.attn_q_fwd(x, g["attn_q_weights_i8"].reshape(H * D, Dm)))
        kv_ref, _ = o_gemm.attn_kv_fwd(x, g["attn_kv_weights_i8"].reshape(2 * H * D, Dm), D)
        dd = np.abs(got["kv"].astype(np.int32) - kv_ref.astype(np.int32))
        assert dd.max() <= 1 and (dd > 0).mean() <= 1e-4
        ao, _ = o_attn.attn_fwd_i8(got["q"], got["kv"], g["sinks_k_i8"].reshape(H, D), g["sinks_v_i8"].reshape(H, D),
                                   g["attn_temperature_f32"].reshape(H), W, H, D, kv_tile=1 << 20)
        hist = code_hist(got["attn_out"], ao)
        assert hist[2:].sum() == 0 and hist[1] / ao.size <= 0.02
        ref = o_gemm.attn_y_fwd(got["attn_out"], g["attn_y_weights_i8"].reshape(2 * Dm, H * D), x)
        assert (got["attn_y"] != ref).mean() <= 2e-3
        ref = o_rms.rms_norm_e4m3_i8(got["attn_y"])
        dd = np.abs(got["x_ffn"].astype(np.int32) - ref.astype(np.int32))
        assert dd.max() <= 1 and (dd > 0).mean() <= 2e-3
        x2 = got["x_ffn"]
        ref = o_gemm.ffn_f_fwd(x2, g["ffn_f_weights_i8"].reshape(2 * F, Dm))
        assert (got["ffn_f"] != ref).mean() <= 2e-3
        ref = o_gemm.ffn_y_fwd_f8(got["ffn_f"], g["ffn_y_weights_i8"].reshape(2 * Dm, F), x2)
        assert (got["ffn_y"] != ref).mean() <= 2e-3
        h = out["ffn_y"].clone()   # the next layer's hidden state
        torch.cuda.synchronize()


@pytest.mark.parametrize("name", ["block_d64_w64", "block_d128_w128", "block_d32_w0"])
def test_block_through_kernel_objects(stream, name):
    """The block with its kernels loaded as kernel objects (kernel.cubin + meta.json through the generic shim
    calls, the reference's grids and argument lists) returns the bytes of the block on the entry points."""
    from x17ai_b200.block import BlockConfig, BlockForward
    g, c = load_golden(name)
    S, Dm, D, H, F, W = c["S"], c["Dm"], c["D"], c["H"], c["F"], c["W"]
    plain, x = _block(stream, g, c, False)
    want = {k: v.clone() for k, v in plain.forward(x).items()}
    stream.synchronize()
    obj = BlockForward(stream, BlockConfig(Dm, H, D, F, W), plain.w_q, plain.w_kv, plain.w_attn_y, plain.w_ffn_f, plain.w_ffn_y,
                       plain.sink_k, plain.sink_v, plain.attn_temperature, kernel_objects=True)
    got = obj.forward(x, timed=True)
    stream.synchronize()
    for k in want:
        assert torch.equal(got[k], want[k]), k
    assert np.array_equal(got["q"].cpu().numpy(), g["q_i8"].reshape(S, H * D))
    # six of six launches ran on kernel objects, and none of them gave up a wait
    from x17ai_b200 import kernel_objects as KO
    objs = [obj.k_q, obj.k_kv, obj.k_attn, obj.k_attn_y, obj.k_ffn_f, obj.k_ffn_y]
    assert all(isinstance(o, (KO.GemmObject, KO.AttnObject)) for o in objs)
    for o in objs:
        assert o.kernel.status(stream) == [0, 0, 0, 0]
