"""A small reader and writer for the safetensors file format.

Layout of a file: 8 bytes little-endian header length ``n``; ``n`` bytes of
JSON mapping tensor name -> {"dtype", "shape", "data_offsets": [begin, end]}
(plus an optional "__metadata__" entry); then the raw little-endian tensor
bytes, offsets relative to the end of the header.

The reference never reads a checkpoint file itself: it delegates to
``GPT2LMHeadModel.from_pretrained`` (reference: src/model/gpt2.py:92-93).  This
engine reads the file directly so that no model library is involved.
"""

from __future__ import annotations

import json
import struct
from typing import Dict

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Return {name: CPU tensor}.  Tensors are copies; the file is not kept open."""
    with open(path, "rb") as handle:
        head = handle.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (header_len,) = struct.unpack("<Q", head)
        file_size = handle.seek(0, 2)
        if header_len <= 0 or 8 + header_len > file_size:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file")
        handle.seek(8)
        try:
            header = json.loads(handle.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: header is not JSON ({error})") from error
        data_start = 8 + header_len
        data_size = file_size - data_start
        tensors: Dict[str, torch.Tensor] = {}
        for name, entry in header.items():
            if name == "__metadata__":
                continue
            dtype_name = entry.get("dtype")
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype_name!r}")
            dtype, width = _DTYPES[dtype_name]
            shape = [int(extent) for extent in entry["shape"]]
            begin, end = (int(offset) for offset in entry["data_offsets"])
            count = int(np.prod(shape)) if shape else 1
            if end - begin != count * width or begin < 0 or end > data_size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has offsets [{begin}, {end}) inconsistent with "
                    f"shape {shape} of {dtype_name}"
                )
            if count == 0:
                tensors[name] = torch.empty(shape, dtype=dtype)
                continue
            handle.seek(data_start + begin)
            raw = bytearray(end - begin)
            if handle.readinto(raw) != end - begin:
                raise SafetensorsError(f"{path}: short read of tensor {name!r}")
            tensors[name] = torch.frombuffer(raw, dtype=torch.uint8).view(dtype).reshape(shape)
    return tensors


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write {name: tensor} in name order; tensors are made contiguous on the CPU."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    payload = []
    for name in sorted(tensors):
        tensor = tensors[name].detach().to("cpu").contiguous()
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {tensor.dtype} cannot be written")
        raw = tensor.view(torch.uint8).numpy().tobytes() if tensor.numel() else b""
        header[name] = {
            "dtype": _NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + len(raw)],
        }
        offset += len(raw)
        payload.append(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for raw in payload:
            handle.write(raw)
