"""Loading (and, for tests and tools, writing) quantized checkpoints in the reference's on-disk
format: safetensors shards + `model.safetensors.index.json` + `config.json` with a top-level
"quantization": {"group_size", "bits"} (generative-models/quantize/safetensors-writer.cc:127-279,
model-quantizer.cc:1265-1272,1991-1997; read by generative-models/llama3/metal-llama-weights.h:47-57).
The C++ twin for hosts that link the library is include/vpq_safetensors.hpp.

A quantized linear `<pfx>` is three tensors: `<pfx>.weight` U32 [N, K*bits/32], `<pfx>.scales` and
`<pfx>.biases` F16 [N, K/group]. `load_quant_linear` copies them to the device unchanged and
converts the two small ones to bf16 once, as the reference's loaders do
(generative-models/flux2/metal-flux2-transformer.cc:142-151)."""
from __future__ import annotations

import json
import os
import struct

import numpy as np

_DTYPES = {"U32": np.uint32, "F16": np.float16, "BF16": np.uint16, "F32": np.float32, "I32": np.int32,
           "U8": np.uint8, "I64": np.int64}


class Model:
    """Directory of shards; tensors are memory-mapped on demand."""

    def __init__(self, path: str):
        self.path = path
        self.tensors = {}          # name -> (file, dtype string, shape, begin, end) absolute offsets
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            shards = sorted(set(json.load(open(idx))["weight_map"].values()))
        else:
            shards = ["model.safetensors"]
        for name in shards:
            self._open_shard(os.path.join(path, name))
        cfg = os.path.join(path, "config.json")
        self.quantization = json.load(open(cfg)).get("quantization") if os.path.exists(cfg) else None

    def _open_shard(self, file: str) -> None:
        with open(file, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(hlen))
        size = os.path.getsize(file)
        for k, v in header.items():
            if k == "__metadata__":
                continue
            b0, b1 = v["data_offsets"]
            if b1 < b0 or 8 + hlen + b1 > size:
                raise ValueError(f"{file}: tensor {k} lies outside the file")
            self.tensors[k] = (file, v["dtype"], tuple(v["shape"]), 8 + hlen + b0, 8 + hlen + b1)

    def has(self, name: str) -> bool:
        return name in self.tensors

    def numpy(self, name: str) -> np.ndarray:
        file, dtype, shape, b0, b1 = self.tensors[name]
        return np.memmap(file, dtype=_DTYPES[dtype], mode="r", offset=b0, shape=shape)

    def quant_shape(self, pfx: str, group: int | None = None):
        """(N, K, bits, group) of a quantized linear, from shapes alone plus the group size."""
        group = group or (self.quantization or {}).get("group_size")
        if not group:
            raise ValueError("group size unknown: no config.json 'quantization' and none given")
        _, _, wshape, _, _ = self.tensors[pfx + ".weight"]
        _, _, sshape, _, _ = self.tensors[pfx + ".scales"]
        K = sshape[1] * group
        return wshape[0], K, wshape[1] * 32 // K, group


def load_quant_linear(model: Model, pfx: str, device, group: int | None = None):
    """(codes int32 [N, K/8], scales bf16, biases bf16) on `device`; w4 / group 64 only."""
    import torch
    from . import ops
    N, K, bits, group = model.quant_shape(pfx, group)
    if bits != 4 or group != 64:
        raise ValueError(f"{pfx}: w{bits} g{group}; this library computes w4 g64")
    codes = torch.from_numpy(np.array(model.numpy(pfx + ".weight")).view(np.int32)).to(device)
    s16 = torch.from_numpy(np.array(model.numpy(pfx + ".scales"))).to(device)
    b16 = torch.from_numpy(np.array(model.numpy(pfx + ".biases"))).to(device)
    return codes, ops.scales_to_bf16(s16), ops.scales_to_bf16(b16)


def write_model(path: str, tensors: dict, group: int, bits: int, shard_max_bytes: int = 5 << 30) -> None:
    """tensors: name -> numpy array (uint32 -> U32, float16 -> F16, float32 -> F32, uint16 -> BF16).
    Same layout rules as the reference's writer: header padded so the blob starts 16-byte aligned,
    ranges tile the blob, small tensors of odd size go last in their shard."""
    os.makedirs(path, exist_ok=True)
    names = {np.dtype(np.uint32): "U32", np.dtype(np.float16): "F16", np.dtype(np.float32): "F32",
             np.dtype(np.uint16): "BF16", np.dtype(np.int32): "I32"}
    shards, cur, cur_bytes = [], [], 0
    for k, a in tensors.items():
        a = np.ascontiguousarray(a)
        if cur and cur_bytes + a.nbytes > shard_max_bytes:
            shards.append(cur)
            cur, cur_bytes = [], 0
        cur.append((k, a))
        cur_bytes += a.nbytes
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, items in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        items = [it for it in items if it[1].nbytes % 16 == 0] + [it for it in items if it[1].nbytes % 16]
        header, off = {}, 0
        for k, a in items:
            header[k] = {"dtype": names[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
            off += a.nbytes
            weight_map[k] = fname
        text = json.dumps(header, separators=(",", ":")).encode()
        text += b" " * (-(8 + len(text)) % 16)
        with open(os.path.join(path, fname), "wb") as f:
            f.write(struct.pack("<Q", len(text)))
            f.write(text)
            for _, a in items:
                f.write(a.tobytes())
    json.dump({"metadata": {"total_size": 0}, "weight_map": weight_map},
              open(os.path.join(path, "model.safetensors.index.json"), "w"))
    cfg_path = os.path.join(path, "config.json")
    cfg = json.load(open(cfg_path)) if os.path.exists(cfg_path) else {}
    cfg["quantization"] = {"group_size": group, "bits": bits}
    json.dump(cfg, open(cfg_path, "w"))
