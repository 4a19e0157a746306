"""safetensors reader/writer of the host mirror (x17ai_b200/tensor_io.py) against the `safetensors`
package, and the errors the reference's loader raises (src/tensor.rs:155-179)."""
import numpy as np
import pytest
import torch


def _cases():
    g = torch.Generator().manual_seed(0)
    yield "i8", torch.randint(-127, 128, (37, 48), generator=g, dtype=torch.int8)
    yield "u8", torch.randint(0, 256, (5, 7, 3), generator=g, dtype=torch.uint8)
    yield "f32", torch.randn(11, generator=g)
    yield "bf16", torch.randn(4, 6, generator=g).to(torch.bfloat16)
    yield "e4m3", torch.randn(8, 16, generator=g).to(torch.float8_e4m3fn)


@pytest.mark.parametrize("name,t", list(_cases()))
def test_roundtrip_against_the_safetensors_package(tmp_path, name, t):
    from safetensors.torch import load_file, save_file
    from x17ai_b200 import tensor_io
    # ours -> theirs
    p = tmp_path / f"{name}_ours.safetensors"
    tensor_io.write_safetensors_file(p, t, name)
    theirs = load_file(str(p))
    assert list(theirs) == [name] and theirs[name].dtype == t.dtype and theirs[name].shape == t.shape
    assert torch.equal(theirs[name].view(torch.uint8), t.view(torch.uint8))
    # theirs -> ours
    q = tmp_path / f"{name}_theirs.safetensors"
    save_file({name: t}, str(q))
    back = tensor_io.read_safetensors_file(q)
    assert back.dtype == t.dtype and back.shape == t.shape and torch.equal(back.view(torch.uint8), t.view(torch.uint8))


def test_loader_errors(tmp_path):
    from safetensors.torch import save_file
    from x17ai_b200 import X17Error, tensor_io
    p = tmp_path / "two.safetensors"
    save_file({"a": torch.zeros(2), "b": torch.zeros(3)}, str(p))
    with pytest.raises(X17Error, match="expected exactly one tensor, found 2"):
        tensor_io.read_safetensors_file(p)
    (tmp_path / "short.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(X17Error, match="invalid safetensors file"):
        tensor_io.read_safetensors_file(tmp_path / "short.safetensors")
    (tmp_path / "long.safetensors").write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(X17Error, match="header length"):
        tensor_io.read_safetensors_file(tmp_path / "long.safetensors")
    p = tmp_path / "f64.safetensors"
    save_file({"a": torch.zeros(2, dtype=torch.float64)}, str(p))
    with pytest.raises(X17Error, match="unsupported safetensors dtype"):
        tensor_io.read_safetensors_file(p)


def test_writer_creates_the_directory_and_names_the_tensor(tmp_path):
    from safetensors.torch import load_file
    from x17ai_b200 import tensor_io
    p = tmp_path / "a" / "b" / "q_i8.safetensors"
    tensor_io.write_safetensors_file(p, torch.arange(6, dtype=torch.int8).reshape(2, 3))
    assert list(load_file(str(p))) == ["tensor"]   # the name the reference's writer uses (tensor.rs:247)
    empty = tmp_path / "empty.safetensors"
    tensor_io.write_safetensors_file(empty, torch.zeros(0, 4, dtype=torch.int8))
    assert tuple(tensor_io.read_safetensors_file(empty).shape) == (0, 4)


def test_named_tensor_files_bin_and_safetensors(tmp_path):
    """The name's tag declares the storage type (block_utils.py:51-83); raw files are the bytes alone."""
    from safetensors.torch import load_file
    from x17ai_b200 import X17Error, tensor_io
    g = torch.Generator().manual_seed(1)
    cases = {"q_i8": torch.randint(-127, 128, (6, 8), generator=g, dtype=torch.int8),
             "ffn_f_f8": torch.randn(6, 8, generator=g).to(torch.float8_e4m3fn),
             "attn_l_f32": torch.randn(2, 6, generator=g), "acc_i32": torch.randint(-9, 9, (3, 4), generator=g, dtype=torch.int32),
             "x_bf16": torch.randn(4, 4, generator=g).to(torch.bfloat16)}
    for stem, t in cases.items():
        for ext in (".bin", ".safetensors"):
            p = tmp_path / (stem + ext)
            assert tensor_io.storage_dtype(p) == t.dtype
            tensor_io.write_tensor_file(p, t)
            back = tensor_io.read_tensor_file(p, t.shape)
            assert back.dtype == t.dtype and torch.equal(back.view(torch.uint8), t.view(torch.uint8))
        assert (tmp_path / (stem + ".bin")).read_bytes() == t.view(torch.uint8).numpy().tobytes()
        # the reference's Python side names the tensor after the file without its tag (block_utils.py:104-107)
        assert list(load_file(str(tmp_path / (stem + ".safetensors")))) == [stem.rpartition("_")[0]]
    assert tuple(tensor_io.read_tensor_file(tmp_path / "q_i8.bin", (-1, 4)).shape) == (12, 4)
    with pytest.raises(X17Error, match="dtype tag"):
        tensor_io.storage_dtype("weights.bin")
    with pytest.raises(X17Error, match="extension"):
        tensor_io.storage_dtype("weights_i8.npy")
    with pytest.raises(X17Error, match="declares"):
        tensor_io.write_tensor_file(tmp_path / "q_f32.bin", cases["q_i8"])
    with pytest.raises(X17Error, match="do not fit"):
        tensor_io.read_tensor_file(tmp_path / "q_i8.bin", (5, 5))
    (tmp_path / "odd_f32.bin").write_bytes(b"\x00" * 6)
    with pytest.raises(X17Error, match="whole number"):
        tensor_io.read_tensor_file(tmp_path / "odd_f32.bin")
