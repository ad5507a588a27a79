"""Checkpoint folders: config.json + model.safetensors.  The safetensors container is read directly (an 8-byte
little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw little-endian data), with
the file memory-mapped so that tensors are copied once, to the device."""
import json
import mmap
import os
import struct
import warnings
from typing import Dict

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64, "I8": torch.int8,
           "U8": torch.uint8, "I16": torch.int16, "I32": torch.int32, "I64": torch.int64, "BOOL": torch.bool}


def read_config(folder) -> dict:
    with open(os.path.join(str(folder), "config.json")) as f:
        return json.load(f)


def read_safetensors(path, device="cpu") -> Dict[str, torch.Tensor]:
    out = {}
    with open(str(path), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            lo, hi = meta["data_offsets"]
            dtype = _DTYPES[meta["dtype"]]
            if hi == lo:
                t = torch.empty(meta["shape"], dtype=dtype)
            else:
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore", UserWarning)   # read-only mapping: every tensor is copied below
                    t = torch.frombuffer(mm, dtype=dtype, count=(hi - lo) // dtype.itemsize, offset=base + lo)
                t = t.reshape(meta["shape"])
            out[name] = t.clone() if str(device) == "cpu" else t.to(device)
    return out


def is_checkpoint_folder(path) -> bool:
    p = str(path)
    return os.path.isdir(p) and os.path.isfile(os.path.join(p, "config.json")) and os.path.isfile(os.path.join(p, "model.safetensors"))
