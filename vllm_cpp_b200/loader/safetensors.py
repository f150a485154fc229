"""safetensors reader / writer on ``mmap`` (no third-party dependency).

File layout: ``u64 little-endian header length | JSON header | raw tensor bytes``. The header
is untrusted input: every offset pair is bounds-checked against the data section, must match
``prod(shape) * itemsize`` and may not overlap its neighbours, before any tensor view is
handed out. Sharded checkpoints are resolved through ``model.safetensors.index.json``.

Reference: ``src/vllm/model_executor/model_loader/safetensors_reader.cpp`` (mmap reader with
header bounds checks, index.json, windowed release of consumed pages).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterator

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1), "F8_E5M2": (torch.float8_e5m2, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
MAX_HEADER_BYTES = 100 << 20


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: file too small for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} out of bounds")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: malformed JSON header: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.entries: dict[str, tuple] = {}
        spans = []
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], list(e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise SafetensorsError(f"{path}: bad entry for {name!r}") from ex
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: unsupported dtype {dt} for {name!r}")
            if not all(isinstance(d, int) and d >= 0 for d in shape):
                raise SafetensorsError(f"{path}: bad shape for {name!r}")
            n = 1
            for d in shape:
                n *= d
            if not (isinstance(b, int) and isinstance(en, int) and 0 <= b <= en <= data_len):
                raise SafetensorsError(f"{path}: data offsets of {name!r} out of bounds")
            if en - b != n * _DTYPES[dt][1]:
                raise SafetensorsError(f"{path}: size of {name!r} does not match its shape")
            self.entries[name] = (dt, shape, b, en)
            spans.append((b, en, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: tensors {n0!r} and {n1!r} overlap")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def keys(self):
        return self.entries.keys()

    def __contains__(self, name):
        return name in self.entries

    def get(self, name: str) -> torch.Tensor:
        """Zero-copy CPU view of one tensor (valid while the file object is alive)."""
        dt, shape, b, en = self.entries[name]
        tdt, _ = _DTYPES[dt]
        if en == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self.data_start + b: self.data_start + en]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # read-only mmap: tensors are never written
            t = torch.frombuffer(buf, dtype=torch.uint8).view(tdt)
        return t.reshape(shape)

    def release(self, name: str) -> None:
        """Tell the kernel the pages of a consumed tensor are no longer needed."""
        if self._mm is None or not hasattr(self._mm, "madvise"):
            return
        _, _, b, en = self.entries[name]
        page = mmap.PAGESIZE
        lo = (self.data_start + b + page - 1) // page * page
        hi = (self.data_start + en) // page * page
        if hi > lo:
            try:
                self._mm.madvise(mmap.MADV_DONTNEED, lo, hi - lo)
            except (OSError, ValueError):
                pass

    def close(self):
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass  # tensor views still alive; the OS unmaps at exit
        self._f.close()


def save_file(tensors: dict[str, torch.Tensor], path: str, metadata: dict | None = None) -> None:
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def open_shards(model_dir: str) -> list[SafetensorsFile]:
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        names = sorted(set(wm.values()))
    else:
        names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not names:
        raise FileNotFoundError(f"no *.safetensors files in {model_dir}")
    return [SafetensorsFile(os.path.join(model_dir, n)) for n in names]


def iter_tensors(model_dir: str) -> Iterator[tuple[str, torch.Tensor]]:
    for sf in open_shards(model_dir):
        for k in sf.keys():
            yield k, sf.get(k)
