"""On-disk container for packed W4A16 weights: the arrays exactly as the kernels consume them, plus a JSON header.

The reference quantizes in memory on every start (python/nanoserve/qwen.py:88-92: load bf16, call ns_w4_quantize) and
has no format of its own; this is the "quantize once, memory-map afterwards" counterpart.  Nothing is re-laid out:
``Wq [N, K/8]`` uint32 and ``S [N, K/G]`` bf16 are stored row-major, so a tensor-parallel rank reads only its rows
(``[r N/P, (r+1) N/P)`` is one contiguous byte range of each array) and the arrays can be handed to ``ns_w4_linear``
as they come.

File layout (little endian):
    bytes 0..7    magic  b"NSW4A16\\0"
    bytes 8..15   uint64 length H of the JSON header
    bytes 16..    H bytes of UTF-8 JSON:
                  {"version": 1, "tensors": {name: {"kind": "w4", "N":, "K":, "G":, "wq": [offset, nbytes],
                                                    "s": [offset, nbytes], "crc": [crc32(wq), crc32(s)]}
                                             | {"kind": "bf16", "shape": [...], "data": [offset, nbytes], "crc": [...]}},
                   "meta": {...}}
    data          every array starts on a 256-byte boundary; offsets are absolute file offsets
"""
import json
import struct
import zlib
from typing import Dict, Optional, Tuple

import numpy as np

MAGIC = b"NSW4A16\0"
VERSION = 1
ALIGN = 256


def _aligned(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def save(path: str, tensors: Dict[str, object], meta: Optional[dict] = None) -> None:
    """tensors: name -> (Wq uint32 [N, K/8], S uint16 (bf16 bits) [N, K/G]) for a quantized linear, or a uint16 array
    (bf16 bits, any shape) for a tensor kept in bf16 (embeddings, norms, lm_head)."""
    entries, blobs = {}, []
    for name, t in tensors.items():
        if isinstance(t, tuple):
            wq, s = (np.ascontiguousarray(a) for a in t)
            if wq.dtype != np.uint32 or s.dtype != np.uint16 or wq.ndim != 2 or s.ndim != 2 or wq.shape[0] != s.shape[0]:
                raise ValueError(f"{name}: expected (uint32 [N, K/8], uint16 [N, K/G])")
            N, K = wq.shape[0], wq.shape[1] * 8
            if s.shape[1] == 0 or K % s.shape[1]:
                raise ValueError(f"{name}: K = {K} is not a multiple of the number of groups {s.shape[1]}")
            G = K // s.shape[1]
            if G % 32:
                raise ValueError(f"{name}: group size {G} is not a multiple of 32")
            entries[name] = {"kind": "w4", "N": N, "K": K, "G": G, "wq": len(blobs), "s": len(blobs) + 1,
                             "crc": [zlib.crc32(wq.tobytes()), zlib.crc32(s.tobytes())]}
            blobs += [wq, s]
        else:
            a = np.ascontiguousarray(t)
            if a.dtype != np.uint16:
                raise ValueError(f"{name}: bf16 tensors are passed as uint16 bit patterns")
            entries[name] = {"kind": "bf16", "shape": list(a.shape), "data": len(blobs), "crc": [zlib.crc32(a.tobytes())]}
            blobs.append(a)

    def header_bytes(offsets):
        out = {}
        for name, e in entries.items():
            e = dict(e)
            for key in ("wq", "s", "data"):
                if key in e:
                    e[key] = [offsets[e[key]], int(blobs[e[key]].nbytes)]
            out[name] = e
        return json.dumps({"version": VERSION, "tensors": out, "meta": meta or {}}, sort_keys=True).encode()

    # the header's length depends on the offsets it contains: lay out with generous width, then fix the point
    offsets = [0] * len(blobs)
    for _ in range(4):
        hdr = header_bytes(offsets)
        pos = _aligned(16 + len(hdr) + 64)
        new = []
        for b in blobs:
            new.append(pos)
            pos = _aligned(pos + b.nbytes)
        if new == offsets:
            break
        offsets = new
    hdr = header_bytes(offsets)
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", len(hdr)))
        f.write(hdr)
        for off, b in zip(offsets, blobs):
            f.seek(off)
            f.write(b.tobytes())
        f.truncate(_aligned(f.tell()))


class PackedWeights:
    """Memory-mapped view of a weight file.  Arrays are numpy views into the mapping (no copy until they are uploaded)."""

    def __init__(self, path: str, verify: bool = False):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(16)
            if len(head) < 16 or head[:8] != MAGIC:
                raise ValueError(f"{path}: not a packed W4A16 weight file")
            (hlen,) = struct.unpack("<Q", head[8:])
            if hlen > (1 << 28):
                raise ValueError(f"{path}: implausible header length {hlen}")
            raw = f.read(hlen)
            if len(raw) != hlen:
                raise ValueError(f"{path}: truncated header")
        hdr = json.loads(raw.decode())
        if hdr.get("version") != VERSION:
            raise ValueError(f"{path}: version {hdr.get('version')} is not supported (this reader: {VERSION})")
        self.meta, self.tensors = hdr.get("meta", {}), hdr["tensors"]
        self._map = np.memmap(path, dtype=np.uint8, mode="r")
        for name, e in self.tensors.items():
            for key in ("wq", "s", "data"):
                if key in e and (e[key][0] % ALIGN or e[key][0] + e[key][1] > self._map.shape[0]):
                    raise ValueError(f"{path}: {name}.{key} lies outside the file or is misaligned")
        if verify:
            self.verify()

    def names(self):
        return list(self.tensors)

    def _view(self, span, dtype, shape):
        off, nbytes = span
        return self._map[off:off + nbytes].view(dtype).reshape(shape)

    def linear(self, name: str, rank: int = 0, world: int = 1) -> Tuple[np.ndarray, np.ndarray, int]:
        """(Wq, S, G) of a quantized linear; with world > 1 the rows [rank N/world, (rank+1) N/world) only."""
        e = self.tensors[name]
        if e["kind"] != "w4":
            raise KeyError(f"{name} is not a quantized linear")
        N, K, G = e["N"], e["K"], e["G"]
        wq = self._view(e["wq"], np.uint32, (N, K // 8))
        s = self._view(e["s"], np.uint16, (N, K // G))
        if world > 1:
            if N % world:
                raise ValueError(f"{name}: {N} rows do not split evenly over {world} ranks")
            lo, hi = rank * (N // world), (rank + 1) * (N // world)
            wq, s = wq[lo:hi], s[lo:hi]
        return wq, s, G

    def bf16(self, name: str) -> np.ndarray:
        e = self.tensors[name]
        if e["kind"] != "bf16":
            raise KeyError(f"{name} is not a bf16 tensor")
        return self._view(e["data"], np.uint16, tuple(e["shape"]))

    def verify(self) -> None:
        """Checks every array against the CRC32 recorded when the file was written."""
        for name, e in self.tensors.items():
            spans = [e["wq"], e["s"]] if e["kind"] == "w4" else [e["data"]]
            for (off, nbytes), crc in zip(spans, e["crc"]):
                if zlib.crc32(self._map[off:off + nbytes].tobytes()) != crc:
                    raise ValueError(f"{self.path}: checksum mismatch in {name}")

    def to_torch(self, name: str, device, rank: int = 0, world: int = 1):
        """Uploads a tensor: (Wq int32, S bfloat16) for a linear -- the dtypes the binding uses -- or a bfloat16 tensor."""
        import torch
        e = self.tensors[name]
        if e["kind"] == "w4":
            wq, s, _ = self.linear(name, rank, world)
            return (torch.from_numpy(np.ascontiguousarray(wq).view(np.int32)).to(device),
                    torch.from_numpy(np.ascontiguousarray(s).view(np.int16)).view(torch.bfloat16).to(device))
        return torch.from_numpy(np.ascontiguousarray(self.bf16(name)).view(np.int16)).view(torch.bfloat16).to(device)
