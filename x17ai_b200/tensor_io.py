"""Tensors in and out of safetensors files, the way the reference's host reads its inputs
(Tensor::from_safetensors_file, src/tensor.rs:155-179: one tensor per file, uploaded as it is).

Raw `.bin` files (the bytes of the tensor and nothing else) follow the naming rule of the
reference's Python side: the storage type is the tag before the extension, `_i8`, `_f8`, `_f32`,
`_i32` or `_bf16` (block_utils.py:51-83), and the shape is the caller's.

The safetensors format is parsed here directly (8-byte little-endian header length, JSON header with dtype,
shape and byte offsets, raw little-endian data), so the package needs no extra dependency; the
tests check the reader and writer against the `safetensors` package.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

from ._lib import X17Error

# safetensors dtype names -> (numpy dtype of the raw bytes, torch dtype of the tensor)
_DTYPES = {
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "F32": (np.float32, torch.float32),
    "I32": (np.int32, torch.int32),
    "BF16": (np.uint16, torch.bfloat16),
    "F8_E4M3": (np.uint8, torch.float8_e4m3fn),
}
_NAMES = {torch.int8: "I8", torch.uint8: "U8", torch.float32: "F32", torch.int32: "I32", torch.bfloat16: "BF16",
          torch.float8_e4m3fn: "F8_E4M3"}


def read_safetensors_file(path) -> torch.Tensor:
    """The single tensor of a safetensors file as a host tensor (no copy of the data beyond the read)."""
    try:
        raw = Path(path).read_bytes()
    except OSError as e:
        raise X17Error(f"cannot read tensor file {path}: {e.strerror}") from e
    if len(raw) < 8:
        raise X17Error(f"invalid safetensors file {path}: shorter than its header length field")
    (hlen,) = struct.unpack("<Q", raw[:8])
    if 8 + hlen > len(raw):
        raise X17Error(f"invalid safetensors file {path}: header length {hlen} exceeds the file")
    header = json.loads(raw[8:8 + hlen])
    tensors = {k: v for k, v in header.items() if k != "__metadata__"}
    if len(tensors) != 1:
        raise X17Error(f"expected exactly one tensor, found {len(tensors)}")   # tensor.rs:164-170
    (info,) = tensors.values()
    if info["dtype"] not in _DTYPES:
        raise X17Error(f"unsupported safetensors dtype {info['dtype']} in {path}")
    np_dtype, torch_dtype = _DTYPES[info["dtype"]]
    begin, end = info["data_offsets"]
    shape = tuple(info["shape"])
    count = int(np.prod(shape, dtype=np.int64)) if shape else 1
    if end - begin != count * np.dtype(np_dtype).itemsize or 8 + hlen + end > len(raw):
        raise X17Error(f"invalid safetensors file {path}: data range does not match shape {list(shape)}")
    data = np.frombuffer(raw, dtype=np_dtype, count=count, offset=8 + hlen + begin).reshape(shape)
    t = torch.from_numpy(data.copy())
    return t.view(torch_dtype) if t.dtype != torch_dtype else t


def write_safetensors_file(path, tensor: torch.Tensor, name: str = "tensor") -> None:
    """One host tensor into a safetensors file under the name the reference's writer uses
    (Tensor::save_safetensors_file, src/tensor.rs:213-248); missing parent directories are created."""
    if tensor.dtype not in _NAMES:
        raise X17Error(f"unsupported tensor dtype {tensor.dtype}")
    if tensor.device.type != "cpu":   # tensor.rs:229-234: the caller downloads first
        raise X17Error("save_safetensors_file requires a CPU tensor; call to_cpu() first")
    Path(path).parent.mkdir(parents=True, exist_ok=True)   # tensor.rs:218-228
    t = tensor.detach().contiguous()
    payload = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.uint8 else t.numpy().tobytes()
    header = json.dumps({name: {"dtype": _NAMES[tensor.dtype], "shape": list(t.shape), "data_offsets": [0, len(payload)]}},
                        separators=(",", ":")).encode()
    header += b" " * (-len(header) % 8)   # the data starts on an 8-byte boundary, as the format asks
    Path(path).write_bytes(struct.pack("<Q", len(header)) + header + payload)


def load_to_device(path, stream, device: torch.device | None = None) -> torch.Tensor:
    """File -> device tensor, the bytes uploaded through the driver shim on `stream`
    (x17ai_cuda_upload_data); returns after the copy has completed."""
    host = read_safetensors_file(path).pin_memory()
    dev = torch.empty(host.shape, dtype=host.dtype, device=device or torch.device("cuda", torch.cuda.current_device()))
    torch.cuda.synchronize(dev.device)
    stream.upload(host.data_ptr(), dev.data_ptr(), 0, host.numel() * host.element_size())
    stream.synchronize()
    return dev


def download(tensor: torch.Tensor, stream) -> torch.Tensor:
    """Device tensor -> pinned host tensor through the driver shim (x17ai_cuda_download_data), the
    to_cpu() of src/tensor.rs:98-113; returns after the copy has completed."""
    src = tensor.contiguous()
    host = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
    stream.download(src.data_ptr(), host.data_ptr(), 0, src.numel() * src.element_size())
    stream.synchronize()
    return host


# storage type tag in a tensor file's name (block_utils.py:51-58)
_TAGS = {"i8": torch.int8, "f8": torch.float8_e4m3fn, "f32": torch.float32, "i32": torch.int32, "bf16": torch.bfloat16}


def storage_dtype(file_name) -> torch.dtype:
    """`attn_out_i8.safetensors` -> torch.int8: the tag after the last underscore of the stem names the
    storage type; `.bin` and `.safetensors` are the two extensions (block_utils.py:60-83)."""
    p = Path(file_name)
    if p.suffix not in (".bin", ".safetensors"):
        raise X17Error(f"unsupported tensor file extension {p.suffix!r} in {str(file_name)!r}")
    base, sep, tag = p.stem.rpartition("_")
    if not sep or not base or tag not in _TAGS:
        raise X17Error(f"tensor file name must end with a dtype tag (_i8, _f8, _f32, _i32, _bf16): {str(file_name)!r}")
    return _TAGS[tag]


def read_tensor_file(path, shape=None) -> torch.Tensor:
    """A `.safetensors` or raw `.bin` tensor file as a host tensor of the type its name declares. A raw
    file needs `shape` (one dimension may be -1); for a safetensors file `shape`, when given, reshapes."""
    dtype = storage_dtype(path)
    if Path(path).suffix == ".safetensors":
        t = read_safetensors_file(path)
        if t.dtype != dtype:
            raise X17Error(f"{path} declares {dtype} by name but holds {t.dtype}")
    else:
        try:
            raw = Path(path).read_bytes()
        except OSError as e:
            raise X17Error(f"cannot read tensor file {path}: {e.strerror}") from e
        item = torch.empty(0, dtype=dtype).element_size()
        if len(raw) % item != 0:
            raise X17Error(f"{path}: {len(raw)} bytes is not a whole number of {dtype} elements")
        t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dtype) if raw else torch.empty(0, dtype=dtype)
    if shape is not None:
        try:
            t = t.reshape(shape)
        except RuntimeError as e:
            raise X17Error(f"{path}: {t.numel()} elements do not fit shape {list(shape)}") from e
    return t


def write_tensor_file(path, tensor: torch.Tensor) -> None:
    """The counterpart of read_tensor_file: the extension picks the format, the name's tag must match
    the tensor's type (store_tensor_with_dtype, block_utils.py:139-186, refuses a mismatch too)."""
    dtype = storage_dtype(path)
    if tensor.dtype != dtype:
        raise X17Error(f"tensor file name {str(path)!r} declares {dtype}, the tensor is {tensor.dtype}")
    if Path(path).suffix == ".safetensors":
        write_safetensors_file(path, tensor, Path(path).stem.rpartition("_")[0])
        return
    if tensor.device.type != "cpu":
        raise X17Error("write_tensor_file requires a CPU tensor; download it first")
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    t = tensor.detach().contiguous()
    Path(path).write_bytes(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
