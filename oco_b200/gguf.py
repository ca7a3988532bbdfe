"""GGUF checkpoints -> the MoE layer's weight spans.

The reference maps the checkpoint file and hands the selected tensors' byte ranges to the GPU
unchanged (`src/gguf.rs`, selection in `src/weights/gpt_oss/load.rs:20-41,126-141` and
`src/weights/nemotron/load.rs:92-128`, upload in `src/gpu/buffer.rs:145-222`). This module does the
same for the tensors of the MoE path: it parses the directory of a GGUF file (v2 / v3), checks
what the reference checks for these operands (type codes, shapes, data inside the file, scalar
alignment) and returns a `synth.Layer` whose arrays are views into the memory map; uploading them
(`moe._Weights.from_layer`) copies the spans byte for byte, at whatever alignment the file gives.

`write()` produces a minimal GGUF file; the tests use it to stage synthetic layers through the
same reader a real checkpoint would go through.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import synth

MAGIC = 0x46554747          # "GGUF" little endian
MAX_ENTRIES = 100_000       # the reference's directory limits (src/gguf.rs:12-13)
MAX_VALUES = 10_000_000

# ggml type codes the MoE path reads (src/gguf.rs:540-555) -> (elements per block, bytes per block)
BLOCKS = {0: (1, 4), 1: (1, 2), 30: (1, 2), synth.FMT_Q4_0: (32, 18), synth.FMT_Q4_K: (256, 144), synth.FMT_MXFP4: (32, 17)}
F32 = 0
# scalar alignment the kernels' casts need, whatever the file declares (src/gguf.rs:44-60)
ALIGN = {0: 4, 1: 2, 30: 2, synth.FMT_Q4_0: 2, synth.FMT_Q4_K: 2, synth.FMT_MXFP4: 1}

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


class CheckpointError(ValueError):
    """The file is not a checkpoint this path can run (reference `Error::Checkpoint`)."""


@dataclass
class Entry:
    shape: Tuple[int, ...]   # GGUF order: innermost dimension first
    code: int
    offset: int              # absolute byte offset in the file
    nbytes: int


class _Reader:
    def __init__(self, buf):
        self.buf, self.at = buf, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.at + size > len(self.buf):
            raise CheckpointError("truncated GGUF directory")
        v = struct.unpack_from(fmt, self.buf, self.at)[0]
        self.at += size
        return v

    def string(self):
        n = self.take("<Q")
        if n > MAX_VALUES or self.at + n > len(self.buf):
            raise CheckpointError("GGUF string runs past the file")
        s = bytes(self.buf[self.at:self.at + n]).decode("utf-8", "replace")
        self.at += n
        return s

    def value(self, kind):
        if kind in _SCALARS:
            return self.take(_SCALARS[kind])
        if kind == _STRING:
            return self.string()
        if kind == _ARRAY:
            inner, n = self.take("<I"), self.take("<Q")
            if n > MAX_VALUES:
                raise CheckpointError("GGUF array too long")
            return [self.value(inner) for _ in range(n)]
        raise CheckpointError(f"unknown GGUF value type {kind}")


class GgufFile:
    """Memory-mapped GGUF file: `metadata` and the tensor `directory`."""

    def __init__(self, path: str):
        self._file = open(path, "rb")
        self.map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        r = _Reader(self.map)
        if r.take("<I") != MAGIC:
            raise CheckpointError("not a GGUF file")
        version = r.take("<I")
        if version not in (2, 3):
            raise CheckpointError(f"unsupported GGUF version {version}")
        tensors, pairs = r.take("<Q"), r.take("<Q")
        if tensors > MAX_ENTRIES or pairs > MAX_ENTRIES:
            raise CheckpointError("GGUF directory too large")
        self.metadata: Dict[str, object] = {}
        for _ in range(pairs):
            key = r.string()
            self.metadata[key] = r.value(r.take("<I"))
        infos = []
        for _ in range(tensors):
            name = r.string()
            rank = r.take("<I")
            if rank < 1 or rank > 4:
                raise CheckpointError(f"tensor {name}: rank {rank}")
            shape = tuple(r.take("<Q") for _ in range(rank))
            infos.append((name, shape, r.take("<I"), r.take("<Q")))
        alignment = int(self.metadata.get("general.alignment", 32))
        if alignment < 1 or alignment & (alignment - 1):
            raise CheckpointError("GGUF alignment is not a power of two")
        data0 = (r.at + alignment - 1) // alignment * alignment
        self.directory: Dict[str, Entry] = {}
        for name, shape, code, rel in infos:
            if name in self.directory:
                raise CheckpointError(f"duplicate tensor {name}")
            self.directory[name] = Entry(shape, code, data0 + rel, _extent(name, shape, code))

    def close(self):
        """Closes the file; the map itself goes when the last array viewing it has gone."""
        try:
            self.map.close()
        except BufferError:
            pass
        self._file.close()

    def tensor(self, name: str) -> Entry:
        """Directory entry of an operand the kernels will read: known type, whole blocks, data inside
        the file, scalar alignment (reference `Entry::select`, src/gguf.rs:40-80)."""
        if name not in self.directory:
            raise CheckpointError(f"missing tensor {name}")
        e = self.directory[name]
        if e.code not in BLOCKS:
            raise CheckpointError(f"unsupported GGUF tensor type {e.code} in {name}")
        if e.offset % ALIGN[e.code]:
            raise CheckpointError(f"unaligned tensor data in {name}")
        if e.offset + e.nbytes > len(self.map):
            raise CheckpointError(f"tensor {name} runs past the file")
        return e

    def bytes_of(self, e: Entry) -> np.ndarray:
        return np.frombuffer(self.map, dtype=np.uint8, count=e.nbytes, offset=e.offset)

    def floats(self, name: str, shape: Tuple[int, ...]) -> np.ndarray:
        """An f32 tensor with the given GGUF shape (innermost first), as a row-major array."""
        e = self.tensor(name)
        if e.code != F32 or e.shape != tuple(shape):
            raise CheckpointError(f"{name}: expected f32 {shape}, found type {e.code} {e.shape}")
        return self.bytes_of(e).view(np.float32).reshape(tuple(reversed(shape)))

    def packed(self, name: str, fmt: int, shape: Tuple[int, ...]) -> np.ndarray:
        """A block-quantised tensor as bytes `[..., rows, row_bytes]`, rows along the innermost dimension."""
        e = self.tensor(name)
        if e.code != fmt or e.shape != tuple(shape):
            raise CheckpointError(f"{name}: expected type {fmt} {shape}, found type {e.code} {e.shape}")
        return self.bytes_of(e).reshape(tuple(reversed(shape[1:])) + (synth.row_bytes(fmt, shape[0]),))


def _extent(name, shape, code) -> int:
    if code not in BLOCKS:
        return 0
    elems, size = BLOCKS[code]
    if shape[0] % elems:
        raise CheckpointError(f"tensor {name}: rows of {shape[0]} elements do not fill whole blocks")
    n = 1
    for d in shape:
        n *= d
    return n // elems * size


def moe_layer(f: GgufFile, index: int, arch: int, top_k: int, normalize: bool = False, scale: float = 1.0) -> synth.Layer:
    """The MoE operands of layer `index` as a `synth.Layer` over the file's bytes (no copy).
    gpt-oss: reference `Selection::expert` / `router` (src/weights/gpt_oss/load.rs:20-41,131-134);
    Nemotron: `relu_experts` (src/weights/nemotron/load.rs:92-128). Geometry comes from the tensors."""
    p = f"blk.{index}"
    router = f.tensor(f"{p}.ffn_gate_inp.weight")
    if router.code != F32 or len(router.shape) != 2:
        raise CheckpointError("router weights must be float32 [hidden, experts]")
    hidden, experts = router.shape
    if arch == synth.ARCH_GPT_OSS:
        fmt = synth.FMT_MXFP4
        up = f.tensor(f"{p}.ffn_up_exps.weight")
        if len(up.shape) != 3 or hidden % 64:
            raise CheckpointError(f"invalid expert coefficients {p}.ffn_up_exps")
        ffn = up.shape[1]
        L = synth.Layer(arch=arch, hidden=hidden, ffn=ffn, experts=experts, top_k=top_k, fmt=fmt, name=f"{p} (gguf)")
        L.router_w = f.floats(f"{p}.ffn_gate_inp.weight", (hidden, experts))
        L.router_b = f.floats(f"{p}.ffn_gate_inp.bias", (experts,))
        L.gate_w = f.packed(f"{p}.ffn_gate_exps.weight", fmt, (hidden, ffn, experts))
        L.up_w = f.packed(f"{p}.ffn_up_exps.weight", fmt, (hidden, ffn, experts))
        L.down_w = f.packed(f"{p}.ffn_down_exps.weight", fmt, (ffn, hidden, experts))
        L.gate_b = f.floats(f"{p}.ffn_gate_exps.bias", (ffn, experts))
        L.up_b = f.floats(f"{p}.ffn_up_exps.bias", (ffn, experts))
        L.down_b = f.floats(f"{p}.ffn_down_exps.bias", (hidden, experts))
        return L
    if arch == synth.ARCH_NEMOTRON:
        fmt = synth.FMT_Q4_0
        up = f.tensor(f"{p}.ffn_up_exps.weight")
        if len(up.shape) != 3:
            raise CheckpointError(f"unsupported expert up coefficients in {p}")
        ffn = up.shape[1]
        shared = f.directory.get(f"{p}.ffn_up_shexp.weight")
        shared_ffn = shared.shape[1] if shared is not None else 0
        L = synth.Layer(arch=arch, hidden=hidden, ffn=ffn, experts=experts, top_k=top_k, fmt=fmt, shared_ffn=shared_ffn,
                        normalize=normalize, scale=scale, name=f"{p} (gguf)")
        L.router_w = f.floats(f"{p}.ffn_gate_inp.weight", (hidden, experts))
        L.router_b = f.floats(f"{p}.exp_probs_b.bias", (experts,))
        L.up_w = f.packed(f"{p}.ffn_up_exps.weight", fmt, (hidden, ffn, experts))
        L.down_w = f.packed(f"{p}.ffn_down_exps.weight", fmt, (ffn, hidden, experts))
        if shared_ffn:
            L.shared_up_w = f.packed(f"{p}.ffn_up_shexp.weight", fmt, (hidden, shared_ffn))
            L.shared_down_w = f.packed(f"{p}.ffn_down_shexp.weight", fmt, (shared_ffn, hidden))
        return L
    raise CheckpointError("the reference has no MoE loader for this family")


# ---- writer (tests and synthetic checkpoints) ------------------------------------------------------

def _gguf_string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write(path: str, metadata: Dict[str, object], tensors: List[Tuple[str, int, Tuple[int, ...], np.ndarray]],
          alignment: int = 32, skew: int = 0) -> None:
    """Writes a GGUF v3 file. tensors: (name, type code, GGUF shape innermost first, bytes).
    `skew` extra bytes are put before every tensor's data, a multiple of the type's scalar alignment,
    so that spans start off the file alignment as they may in a real checkpoint."""
    head = struct.pack("<IIQQ", MAGIC, 3, len(tensors), len(metadata) + 1)
    head += _gguf_string("general.alignment") + struct.pack("<II", 4, alignment)
    for k, v in metadata.items():
        head += _gguf_string(k)
        if isinstance(v, str):
            head += struct.pack("<I", _STRING) + _gguf_string(v)
        elif isinstance(v, float):
            head += struct.pack("<If", 6, v)
        else:
            head += struct.pack("<II", 4, int(v))
    infos, blobs, at = b"", [], 0
    for name, code, shape, data in tensors:
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        pad = (-at) % alignment + skew
        at += pad
        infos += _gguf_string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        infos += struct.pack("<IQ", code, at)
        blobs.append((pad, raw))
        at += raw.size
    with open(path, "wb") as out:
        out.write(head + infos)
        out.write(b"\0" * ((-(len(head) + len(infos))) % alignment))
        for pad, raw in blobs:
            out.write(b"\0" * pad)
            out.write(raw.tobytes())


def layer_tensors(layer: synth.Layer, index: int):
    """The tensor list of `write()` for one synthetic layer, named as in the checkpoints."""
    p, H, F, E = f"blk.{index}", layer.hidden, layer.ffn, layer.experts
    t = [(f"{p}.ffn_gate_inp.weight", F32, (H, E), layer.router_w)]
    if layer.arch == synth.ARCH_GPT_OSS:
        t += [(f"{p}.ffn_gate_inp.bias", F32, (E,), layer.router_b),
              (f"{p}.ffn_gate_exps.weight", layer.fmt, (H, F, E), layer.gate_w), (f"{p}.ffn_gate_exps.bias", F32, (F, E), layer.gate_b),
              (f"{p}.ffn_up_exps.weight", layer.fmt, (H, F, E), layer.up_w), (f"{p}.ffn_up_exps.bias", F32, (F, E), layer.up_b),
              (f"{p}.ffn_down_exps.weight", layer.fmt, (F, H, E), layer.down_w), (f"{p}.ffn_down_exps.bias", F32, (H, E), layer.down_b)]
    else:
        t += [(f"{p}.exp_probs_b.bias", F32, (E,), layer.router_b),
              (f"{p}.ffn_up_exps.weight", layer.fmt, (H, F, E), layer.up_w),
              (f"{p}.ffn_down_exps.weight", layer.fmt, (F, H, E), layer.down_w)]
        if layer.shared_ffn:
            t += [(f"{p}.ffn_up_shexp.weight", layer.fmt, (H, layer.shared_ffn), layer.shared_up_w),
                  (f"{p}.ffn_down_shexp.weight", layer.fmt, (layer.shared_ffn, H), layer.shared_down_w)]
    return t
