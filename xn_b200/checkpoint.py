"""Quantized-weight checkpoints: the on-disk side of the int4 / int8 / fp8 linears.

The reference loads weights from safetensors files (xn-core/src/safetensors.rs:21-39 knows F32, F16,
BF16, I64 and U8; its VarBuilder keeps only the float types, xn-core/src/nn/var_builder.rs:53-58) and
has no quantized format.  This module defines one inside the same container, so that the reference's
own parser can open the file and a quantized model does not have to be re-quantized at every start:

* a linear `<name>` with int4 block weights is stored as `<name>.q4` -- a U8 tensor holding the q4 tiles
  of include/xn_mm.h exactly as the kernels read them;
* int8 block weights as `<name>.q8` (q8 tiles);
* fp8-e4m3 per-channel weights as `<name>.fp8` (U8 [n, k]) plus `<name>.fp8_scale` (F32 [n]);
* logical shapes and the format version travel in the header's `__metadata__` (string -> string, as the
  container requires) under `xn_mm.<name>`.

The quantizers here run on the host in numpy and produce bit-for-bit what the device quantizers
(`xn_mm_quantize_weights_q4/q8/fp8`) produce; the tile packing goes through the library's host packers
(`xn_mm_pack_q4_host`, `xn_mm_pack_q8_host`).  Everything else (float tensors, biases, norms) is stored
unchanged.
"""
from __future__ import annotations

import json
import struct

import numpy as np

from ._lib import check, lib

FORMAT_VERSION = "1"

_NP_TO_ST = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.uint8): "U8", np.dtype(np.int8): "I8",
             np.dtype(np.int64): "I64", np.dtype(np.int32): "I32"}
_ST_TO_NP = {v: k for k, v in _NP_TO_ST.items()}
_ST_TO_NP["BF16"] = np.dtype(np.uint16)  # numpy has no bfloat16: kept as raw 16-bit patterns


# ------------------------------------------------------------------------------------------------
# host quantizers (bit-exact with the device ones)
# ------------------------------------------------------------------------------------------------
def quantize_blocks_host(w: np.ndarray, block: int, qmax: int):
    """Symmetric block quantization: scale = max|w| / qmax per `block` consecutive k, q = rint(w / scale)
    clamped to [-qmax, qmax] (f32 arithmetic, round half to even)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    if k % block:
        raise ValueError(f"k={k} is not a multiple of the block size {block}")
    b = w.reshape(n, k // block, block)
    scale = (np.max(np.abs(b), axis=-1) / np.float32(qmax)).astype(np.float32)
    safe = np.where(scale == 0, np.float32(1), scale)
    q = np.rint(b / safe[..., None])
    q = np.where(scale[..., None] == 0, 0, np.clip(q, -qmax, qmax)).astype(np.int8)
    return q.reshape(n, k), scale


def f32_to_e4m3_host(x: np.ndarray) -> np.ndarray:
    """f32 -> e4m3 codes, round to nearest even, saturating to +-448 (NaN -> 0x7f | sign)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = ((x.view(np.uint32) >> 24) & 0x80).astype(np.uint8)
    a = np.abs(x)
    nan = np.isnan(a)
    a = np.where(nan, np.float32(0), a)
    _, e = np.frexp(a)                       # a = f * 2^e, f in [0.5, 1): leading bit at e - 1
    lead = np.maximum(e - 1, -6)              # subnormal grid below 2^-6: spacing 2^-9
    q = np.rint(np.ldexp(a, 3 - lead)).astype(np.int32)   # grid units: 8..16 for normals, 0..8 below
    carry = q == 16
    q = np.where(carry, 8, q)
    lead = np.where(carry, lead + 1, lead)
    code = np.where(q < 8, q, ((lead + 7) << 3) | (q - 8))
    sat = (a >= 448) | (lead > 8) | ((lead == 8) & (q > 14))
    code = np.where(sat, 0x7E, code)
    code = np.where(a == 0, 0, code)
    code = np.where(nan, 0x7F, code)
    return (sign | code.astype(np.uint8)).astype(np.uint8)


def quantize_fp8_channel_host(w: np.ndarray):
    """Per-output-channel e4m3: scale[n] = max_k |w| / 448, q = e4m3(w / scale)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    scale = (np.max(np.abs(w), axis=1) / np.float32(448)).astype(np.float32)
    safe = np.where(scale == 0, np.float32(1), scale)
    q = f32_to_e4m3_host((w / safe[:, None]).astype(np.float32))
    q = np.where(scale[:, None] == 0, np.uint8(0), q).astype(np.uint8)
    return q, scale


def _pack(fn_bytes, fn_pack, q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    n, k = q.shape
    if k % 128:
        raise ValueError(f"k={k} must be a multiple of 128 for the tiled formats")
    packed = np.zeros(fn_bytes(n, k), dtype=np.uint8)
    q = np.ascontiguousarray(q, dtype=np.int8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    check(fn_pack(packed.ctypes.data, q.ctypes.data, scales.ctypes.data, n, k))
    return packed


def pack_q4_host(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    return _pack(lib().xn_mm_q4_packed_bytes, lib().xn_mm_pack_q4_host, q, scales)


def pack_q8_host(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    return _pack(lib().xn_mm_q8_packed_bytes, lib().xn_mm_pack_q8_host, q, scales)


def quantize_linear_host(w: np.ndarray, scheme: str) -> dict:
    """One weight [n, k] (f32) -> the tensors stored for it and its metadata entry."""
    n, k = w.shape
    if scheme == "q4":
        q, s = quantize_blocks_host(w, 32, 7)
        return {"tensors": {"q4": pack_q4_host(q, s)}, "meta": {"scheme": "q4", "n": n, "k": k, "block": 32}}
    if scheme == "q8":
        q, s = quantize_blocks_host(w, 32, 127)
        return {"tensors": {"q8": pack_q8_host(q, s)}, "meta": {"scheme": "q8", "n": n, "k": k, "block": 32}}
    if scheme == "fp8":
        q, s = quantize_fp8_channel_host(w)
        return {"tensors": {"fp8": q, "fp8_scale": s}, "meta": {"scheme": "fp8", "n": n, "k": k}}
    raise ValueError(f"unknown scheme {scheme!r}")


# ------------------------------------------------------------------------------------------------
# container
# ------------------------------------------------------------------------------------------------
def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Minimal writer of the safetensors container: u64 header length, JSON header, raw little-endian data.
    `tensors` maps names to numpy arrays (uint16 arrays given with dtype tag via a (array, "BF16") pair)."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        t = tensors[name]
        tag = None
        if isinstance(t, tuple):
            t, tag = t
        t = np.ascontiguousarray(t)
        tag = tag or _NP_TO_ST.get(t.dtype)
        if tag is None:
            raise ValueError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.tobytes()
        header[name] = {"dtype": tag, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)  # keep the data 8-byte aligned
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


def read_safetensors(path: str):
    """-> (tensors: name -> numpy array (BF16 as uint16 bit patterns), metadata: dict)."""
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: truncated header")
        (hl,) = struct.unpack("<Q", head)
        if hl > (100 << 20):
            raise ValueError(f"{path}: header length {hl} is not plausible")
        header = json.loads(f.read(hl).decode("utf-8"))
        data = f.read()
    meta = header.pop("__metadata__", {})
    out = {}
    for name, info in header.items():
        dt = _ST_TO_NP.get(info["dtype"])
        if dt is None:
            raise ValueError(f"{path}: {name} has unsupported dtype {info['dtype']}")
        b, e = info["data_offsets"]
        if not (0 <= b <= e <= len(data)):
            raise ValueError(f"{path}: {name} points outside the file")
        count = int(np.prod(info["shape"])) if info["shape"] else 1
        if (e - b) != count * dt.itemsize:
            raise ValueError(f"{path}: {name} size does not match its shape")
        out[name] = np.frombuffer(data, dtype=dt, count=count, offset=b).reshape(info["shape"])
    return out, meta


def save_quantized(path: str, weights: dict, schemes: dict, extra: dict | None = None) -> None:
    """weights: name -> f32 [n, k]; schemes: name -> "q4" | "q8" | "fp8" (names absent from `schemes` are stored
    as they are); extra: further tensors stored unchanged (biases, norms...)."""
    tensors, meta = {}, {"xn_mm.format_version": FORMAT_VERSION}
    for name, w in weights.items():
        sch = schemes.get(name)
        if sch is None:
            tensors[name] = np.ascontiguousarray(w)
            continue
        ql = quantize_linear_host(np.asarray(w, dtype=np.float32), sch)
        for suffix, t in ql["tensors"].items():
            tensors[f"{name}.{suffix}"] = t
        meta[f"xn_mm.{name}"] = json.dumps(ql["meta"], separators=(",", ":"))
    for name, t in (extra or {}).items():
        tensors[name] = t
    write_safetensors(path, tensors, meta)


def load_quantized(path: str):
    """-> (linears: name -> {"scheme", "n", "k", tensors...}, others: name -> array)."""
    tensors, meta = read_safetensors(path)
    ver = meta.get("xn_mm.format_version")
    if ver != FORMAT_VERSION:
        raise ValueError(f"{path}: quantized-checkpoint format version {ver!r}, this reader handles {FORMAT_VERSION!r}")
    linears, used = {}, set()
    for key, val in meta.items():
        if not key.startswith("xn_mm.") or key == "xn_mm.format_version":
            continue
        name = key[len("xn_mm."):]
        info = json.loads(val)
        need = {"q4": ["q4"], "q8": ["q8"], "fp8": ["fp8", "fp8_scale"]}[info["scheme"]]
        entry = dict(info)
        for suffix in need:
            full = f"{name}.{suffix}"
            if full not in tensors:
                raise ValueError(f"{path}: {full} is missing")
            entry[suffix] = tensors[full]
            used.add(full)
        n, k = info["n"], info["k"]
        if info["scheme"] == "q4" and entry["q4"].size != lib().xn_mm_q4_packed_bytes(n, k):
            raise ValueError(f"{path}: {name}.q4 has {entry['q4'].size} bytes, expected {lib().xn_mm_q4_packed_bytes(n, k)}")
        if info["scheme"] == "q8" and entry["q8"].size != lib().xn_mm_q8_packed_bytes(n, k):
            raise ValueError(f"{path}: {name}.q8 has the wrong size")
        if info["scheme"] == "fp8" and (entry["fp8"].shape != (n, k) or entry["fp8_scale"].shape != (n,)):
            raise ValueError(f"{path}: {name}.fp8 tensors do not match n={n}, k={k}")
        linears[name] = entry
    others = {k: v for k, v in tensors.items() if k not in used}
    return linears, others


def linear_from_entry(entry: dict, device, variant: int = 0):
    """One entry of load_quantized() -> the matching device-side linear (LinearQ4 or LinearFp8 of xn_b200.ops).
    The stored bytes go to the GPU as they are: no re-quantization, no re-packing."""
    import torch

    from . import ops

    if entry["scheme"] == "q4":
        return ops.LinearQ4(torch.from_numpy(np.array(entry["q4"])).to(device), entry["n"], entry["k"])
    if entry["scheme"] == "fp8":
        return ops.LinearFp8(torch.from_numpy(np.array(entry["fp8"])).to(device),
                             torch.from_numpy(np.array(entry["fp8_scale"])).to(device), variant)
    raise ValueError(f"no device-side linear class for scheme {entry['scheme']!r}")
