"""Expert banks straight from a GGUF file: the tensors of the MoE-FFN path
(`blk.N.ffn_gate_inp / ffn_gate_exps / ffn_up_exps / ffn_down_exps / ffn_norm`,
the names src/model/model.cpp:144-157 requires) are located by a small reader of
the GGUF v2/v3 container and handed to the kernels as they sit in the file --
quantised payloads are never re-encoded.

The reader covers what this path needs (header, metadata key/values, tensor
directory, data alignment); it is not a general GGUF library. Offsets can be
cross-checked against gguf-py with `verify_against_gguf_py`, the check
tools/q4k_job.py:51-68 makes before it trusts an offset.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

GGML_F32, GGML_F16, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 12, 14, 30
# ggml type -> (bytes per block, weights per block)
_BLOCK = {GGML_F32: (4, 1), GGML_F16: (2, 1), GGML_BF16: (2, 1), GGML_Q4_K: (144, 256), GGML_Q6_K: (210, 256)}
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


@dataclass
class TensorInfo:
    name: str
    dims: tuple        # ggml order: dims[0] is the fastest-varying (input) dimension
    ggml_type: int
    offset: int        # absolute byte offset in the file
    nbytes: int


class GgufFile:
    """Metadata and tensor directory of one GGUF file; payloads are memory-mapped."""

    def __init__(self, path: str):
        self.path = path
        self.data = np.memmap(path, dtype=np.uint8, mode="r")
        buf = memoryview(self.data)
        pos = 0

        def take(fmt):
            nonlocal pos
            v = struct.unpack_from(fmt, buf, pos)[0]
            pos += struct.calcsize(fmt)
            return v

        def take_str():
            nonlocal pos
            n = take("<Q")
            s = bytes(buf[pos:pos + n]).decode("utf-8")
            pos += n
            return s

        def take_value(t):
            if t in _SCALAR:
                return take(_SCALAR[t])
            if t == 8:
                return take_str()
            if t == 9:
                et, n = take("<I"), take("<Q")
                return [take_value(et) for _ in range(n)]
            raise ValueError(f"{path}: unknown GGUF value type {t}")

        if bytes(buf[0:4]) != b"GGUF":
            raise ValueError(f"{path}: not a GGUF file")
        pos = 4
        self.version = take("<I")
        if self.version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {self.version} is not supported")
        n_tensors, n_kv = take("<Q"), take("<Q")
        self.meta = {}
        for _ in range(n_kv):
            key = take_str()
            self.meta[key] = take_value(take("<I"))
        infos = []
        for _ in range(n_tensors):
            name = take_str()
            nd = take("<I")
            dims = tuple(take("<Q") for _ in range(nd))
            infos.append((name, dims, take("<I"), take("<Q")))
        align = int(self.meta.get("general.alignment", 32))
        data_start = (pos + align - 1) // align * align
        self.tensors = {}
        for name, dims, t, off in infos:
            if t not in _BLOCK:
                nbytes = -1  # a type this path does not read
            else:
                bpb, wpb = _BLOCK[t]
                n = int(np.prod(dims, dtype=np.int64))
                if dims[0] % wpb:
                    raise ValueError(f"{path}: {name}: row length {dims[0]} is not a multiple of {wpb}")
                nbytes = n // wpb * bpb
            self.tensors[name] = TensorInfo(name, dims, t, data_start + off, nbytes)

    def arch(self) -> str:
        return self.meta["general.architecture"]

    def meta_int(self, key: str) -> int:
        return int(self.meta[key])

    def require(self, name: str) -> TensorInfo:
        if name not in self.tensors:
            raise KeyError(f"{self.path}: tensor {name} is missing")
        return self.tensors[name]

    def payload(self, info: TensorInfo) -> np.ndarray:
        if info.nbytes < 0:
            raise ValueError(f"{info.name}: ggml type {info.ggml_type} is not read by this path")
        return self.data[info.offset:info.offset + info.nbytes]

    def n_layers(self) -> int:
        return self.meta_int(self.arch() + ".block_count")


def _bf16_bits(info: TensorInfo, raw: np.ndarray) -> np.ndarray:
    """Weights of an unquantised tensor as bf16 bit patterns (round to nearest even from f32 / f16)."""
    if info.ggml_type == GGML_BF16:
        return raw.view(np.uint16).copy()
    f = raw.view(np.float32) if info.ggml_type == GGML_F32 else raw.view(np.float16).astype(np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def layer_arrays(g: GgufFile, layer: int) -> dict:
    """Host arrays of one block's MoE-FFN tensors: gate/up/down payloads as uint8
    [E][rows][K/256][bytes per block], router and norm weights as bf16 bits."""
    p = g.arch() + "."
    E = g.meta_int(p + "expert_count")
    b = f"blk.{layer}."
    out = {"top_k": g.meta_int(p + "expert_used_count"),
           "rms_eps": float(g.meta.get(p + "attention.layer_norm_rms_epsilon", 1e-6))}
    for key, name in (("gate", "ffn_gate_exps"), ("up", "ffn_up_exps"), ("down", "ffn_down_exps")):
        info = g.require(b + name + ".weight")
        if info.ggml_type not in (GGML_Q4_K, GGML_Q6_K) or len(info.dims) != 3 or info.dims[2] != E:
            raise ValueError(f"{info.name}: expected a Q4_K / Q6_K tensor [in, out, {E}], got type {info.ggml_type} dims {info.dims}")
        if key != "down" and info.ggml_type != GGML_Q4_K:
            raise ValueError(f"{info.name}: gate and up must be Q4_K for this path")
        bpb, wpb = _BLOCK[info.ggml_type]
        n_in, n_out, _ = info.dims
        out[key] = np.asarray(g.payload(info)).reshape(E, n_out, n_in // wpb, bpb)
    r = g.require(b + "ffn_gate_inp.weight")
    out["router"] = _bf16_bits(r, np.asarray(g.payload(r))).reshape(r.dims[1], r.dims[0])
    out["router_exact"] = r.ggml_type == GGML_BF16  # f32 / f16 router weights were rounded to bf16
    n = g.tensors.get(b + "ffn_norm.weight")
    if n is not None:
        out["norm"] = _bf16_bits(n, np.asarray(g.payload(n)))
        out["norm_exact"] = n.ggml_type == GGML_BF16
    return out


def load_expert_bank(g: GgufFile, layer: int, device="cuda"):
    """`ExpertBank` of block `layer` on `device` plus the block's top-k."""
    import torch
    from .moe import ExpertBank
    a = layer_arrays(g, layer)

    def bf(bits):
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)
    bank = ExpertBank(gate=torch.from_numpy(np.ascontiguousarray(a["gate"])).to(device),
                      up=torch.from_numpy(np.ascontiguousarray(a["up"])).to(device),
                      down=torch.from_numpy(np.ascontiguousarray(a["down"])).to(device),
                      router=bf(a["router"]), norm_w=bf(a["norm"]) if "norm" in a else None, rms_eps=a["rms_eps"])
    return bank, a["top_k"]


def verify_against_gguf_py(path: str, names=None) -> int:
    """Every tensor this reader located holds the bytes gguf-py hands out for the same name; returns the
    number of tensors compared. Raises on the first mismatch."""
    import gguf
    mine = GgufFile(path)
    n = 0
    for t in gguf.GGUFReader(path).tensors:
        if names is not None and t.name not in names:
            continue
        info = mine.tensors[t.name]
        if info.nbytes < 0:
            continue
        theirs = memoryview(t.data).cast("B").tobytes()
        if bytes(mine.payload(info)) != theirs:
            raise ValueError(f"{path}: {t.name}: bytes at offset {info.offset} differ from gguf-py's")
        n += 1
    return n
