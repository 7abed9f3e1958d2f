"""safetensors checkpoints (own parser over mmap, like blazr_b200/gguf_loader.py for GGUF; reference src/loader/safetensors/).

File layout: 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets), then the data.
Tensors come back as torch CPU tensors that alias the mapping (bfloat16 stays bfloat16: no widening copy on the host).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {"BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8), "I32": (torch.int32, 4),
           "I64": (torch.int64, 8), "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "I16": (torch.int16, 2), "BOOL": (torch.bool, 1)}


class Safetensors:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._mm[:8])
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file")
        try:
            head = json.loads(self._mm[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})")
        self.metadata = head.pop("__metadata__", {})
        self._base = 8 + n
        self._info: Dict[str, Tuple[str, List[int], int, int]] = {}
        for name, d in head.items():
            dt, shape, (a, b) = d["dtype"], list(d["shape"]), d["data_offsets"]
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {dt}")
            numel = int(np.prod(shape)) if shape else 1
            if b - a != numel * _DTYPES[dt][1] or self._base + b > size or a < 0:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")
            self._info[name] = (dt, shape, a, b)

    def names(self) -> List[str]:
        return list(self._info)

    def shape(self, name: str) -> List[int]:
        return self._info[name][1]

    def dtype(self, name: str) -> str:
        return self._info[name][0]

    def __contains__(self, name: str) -> bool:
        return name in self._info

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self._info:
            raise SafetensorsError(f"{self.path}: no tensor named {name}")
        dt, shape, a, b = self._info[name]
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=b - a, offset=self._base + a)
        return torch.from_numpy(buf.copy()).view(_DTYPES[dt][0]).reshape(shape)

    def close(self):
        self._mm.close()
        self._f.close()


def load_checkpoint(folder: str):
    """(config dict, Safetensors) of a model folder holding config.json and model.safetensors"""
    cfg_path = os.path.join(folder, "config.json")
    if not os.path.isfile(cfg_path):
        raise SafetensorsError(f"{folder}: no config.json")
    with open(cfg_path) as f:
        cfg = json.load(f)
    return cfg, Safetensors(os.path.join(folder, "model.safetensors"))
