"""Reader and validator for GLQ checkpoints: the on-disk side of the boundary.

A GLQ checkpoint is a Hugging Face model folder whose ``quantize_config.json`` (or the ``quantization_config`` of
``config.json``) names the codebook and rates (glq_vllm/config.py:60-73) and whose ``*.safetensors`` files hold,
per quantized linear, the buffers of the reference's ``E8RHTLinear`` (glq/quantized_linear.py:235-247, 351-361):

* E8 shell: ``Qidxs (m_pad, n_pad / 8) int16`` [+ ``Qidxs2..4`` and scalar ``inv_resid_scale{,2,3}``],
* trellis 3INST: ``trellis_packed ((m / 16)(n / 16), 16 K) int16`` [+ ``trellis_packed2`` and ``inv_resid_scale2``],
* both: ``SU (m_pad,) fp16``, ``SV (n_pad,) fp16``, ``Wscale () fp32``.

This module parses safetensors files itself (an 8-byte little-endian header length, a JSON header, raw
little-endian tensors: the published format), so reading a checkpoint needs nothing beyond torch and numpy.
No file is downloaded or expected here; the tests write small checkpoints with :func:`write_safetensors`.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, Iterable, Iterator, List, Mapping, Optional, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class CheckpointError(ValueError):
    """A file or a layer of the checkpoint does not have the form the kernels serve."""


# ---------------------------------------------------------------------------------------------------------
# safetensors
# ---------------------------------------------------------------------------------------------------------
class SafetensorsFile:
    """Read-only view of one ``.safetensors`` file: the header is parsed once, a tensor is copied out of the
    memory map when it is asked for."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise CheckpointError(f"{path}: shorter than a safetensors header")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8 or hlen > (100 << 20):
            raise CheckpointError(f"{path}: header length {hlen} does not fit the file")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        data_len = size - self._base
        for name, e in header.items():
            if e.get("dtype") not in _DTYPES:
                raise CheckpointError(f"{path}: tensor {name!r} has unsupported dtype {e.get('dtype')!r}")
            dt, width = _DTYPES[e["dtype"]]
            shape = tuple(int(d) for d in e["shape"])
            b0, b1 = (int(v) for v in e["data_offsets"])
            n = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if b0 < 0 or b1 < b0 or b1 > data_len or b1 - b0 != n * width:
                raise CheckpointError(f"{path}: tensor {name!r} {shape} {e['dtype']} does not match its byte range {b0}:{b1}")
            self._entries[name] = (dt, shape, b0, b1)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def keys(self) -> List[str]:
        return list(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b0, b1 = self._entries[name]
        if b1 == b0:
            return torch.empty(shape, dtype=dt)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=b1 - b0, offset=self._base + b0)
        return torch.from_numpy(raw.copy()).view(dt).reshape(shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._f.close()


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    f = SafetensorsFile(path)
    out = {k: f.tensor(k) for k in f.keys()}
    f.close()
    return out


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors in the safetensors layout (header padded to 8 bytes, tensors in name order)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    blobs, off = [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise CheckpointError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


# ---------------------------------------------------------------------------------------------------------
# quantize_config.json
# ---------------------------------------------------------------------------------------------------------
_MERGED = {".qkv_proj": (".q_proj", ".k_proj", ".v_proj"), ".gate_up_proj": (".gate_proj", ".up_proj")}


@dataclass
class QuantizeConfig:
    """The keys the reference's serving config reads (glq_vllm/config.py:60-73), with the same defaults and the
    same refusals (:30-47), plus this library's own: HYB trellis layers and E8P layers have no kernel here."""
    bpw: int = 2
    layer_bpw: Dict[str, int] = field(default_factory=dict)
    codebook: str = "e8_shell"
    block_diagonal: bool = True
    variant: str = "hyb"
    trellis_layout: Optional[str] = None

    def __post_init__(self):
        if self.codebook not in ("e8_shell", "trellis", "e8p"):
            raise CheckpointError(f"unknown GLQ codebook {self.codebook!r}")
        if self.codebook == "e8p":
            raise CheckpointError("E8P checkpoints are not served by glq_b200 (codebook 'e8_shell' or 'trellis')")
        if self.codebook == "trellis":
            if self.variant not in ("hyb", "3inst"):
                raise CheckpointError(f"GLQ trellis variant {self.variant!r} has no kernel (only 'hyb' and '3inst' exist)")
            if self.variant == "hyb":
                raise CheckpointError("HYB (tlut) trellis checkpoints are not served by glq_b200; re-quantize with variant 3inst")
            if self.trellis_layout != "kernel":
                raise CheckpointError("this 3inst trellis checkpoint is stored in the natural tile layout "
                                      "(no trellis_layout: \"kernel\"); the kernels would decode it to the wrong weights")

    @classmethod
    def from_dict(cls, d: Mapping[str, object]) -> "QuantizeConfig":
        return cls(bpw=int(d.get("bpw", 2)), layer_bpw=dict(d.get("layer_bpw") or {}), codebook=str(d.get("codebook", "e8_shell")),
                   block_diagonal=bool(d.get("block_diagonal", True)), variant=str(d.get("variant", "hyb")),
                   trellis_layout=d.get("trellis_layout"))

    @classmethod
    def from_folder(cls, folder: str) -> "QuantizeConfig":
        qc = os.path.join(folder, "quantize_config.json")
        if os.path.exists(qc):
            with open(qc) as f:
                return cls.from_dict(json.load(f))
        cfg = os.path.join(folder, "config.json")
        if os.path.exists(cfg):
            with open(cfg) as f:
                q = json.load(f).get("quantization_config")
            if q:
                return cls.from_dict(q)
        raise CheckpointError(f"{folder}: neither quantize_config.json nor a quantization_config in config.json")

    def bpw_of(self, prefix: str) -> Optional[int]:
        """Rate of the layer a serving framework calls ``prefix``; None = not quantized.  Frameworks rename layers
        on the way (``model.language_model.`` folded into ``model.`` or moved to ``language_model.model.``) and merge
        q/k/v and gate/up; the per-layer table lists the checkpoint's own, unmerged names
        (behaviour of glq_vllm/config.py:75-121; a merged layer takes the largest rate of its parts)."""
        if not self.layer_bpw:
            return self.bpw
        forms = [prefix]
        if prefix.startswith("language_model.model."):
            forms.append("model.language_model." + prefix[len("language_model.model."):])
        elif prefix.startswith("model.") and ".language_model." not in prefix:
            forms.append("model.language_model." + prefix[len("model."):])
        best: Optional[int] = None
        for f in forms:
            if f in self.layer_bpw:
                best = max(best or 0, int(self.layer_bpw[f]))
            for merged, parts in _MERGED.items():
                if f.endswith(merged):
                    for p in parts:
                        b = self.layer_bpw.get(f[:-len(merged)] + p)
                        if b is not None:
                            best = max(best or 0, int(b))
        return best


# ---------------------------------------------------------------------------------------------------------
# layers
# ---------------------------------------------------------------------------------------------------------
E8_BUFFERS = ("Qidxs", "Qidxs2", "Qidxs3", "Qidxs4", "inv_resid_scale", "inv_resid_scale2", "inv_resid_scale3")
TRELLIS_BUFFERS = ("trellis_packed", "trellis_packed2", "inv_resid_scale2", "tlut")
COMMON_BUFFERS = ("SU", "SV", "Wscale", "bias")


def trellis_rates(bpw: int) -> Tuple[int, int]:
    """(K1, K2) of a trellis layer of nominal rate bpw: one stage up to 4 bpw, 4 + (bpw - 4) above
    (glq/trellis.py:788-808)."""
    if not 1 <= bpw <= 8:
        raise CheckpointError(f"trellis rate {bpw} bpw is outside 1..8")
    return (bpw, 0) if bpw <= 4 else (4, bpw - 4)


def split_trellis_packed(packed: torch.Tensor, gate_rows: int, up_rows: int, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Cut a jointly quantized [gate; up] bit-stream into its two layers (glq/quantize_model.py:654-677).
    The storage unit is a 32 x 32 group of four tiles, groups run row-major, so a cut is exact only between
    groups of rows: both parts must be multiples of 32 rows (a cut inside a pair of 16-row tile rows would
    interleave the two layers' bytes, and still decode — to the wrong weights)."""
    if gate_rows % 32 or up_rows % 32:
        raise CheckpointError(f"trellis [gate; up] split at rows ({gate_rows}, {up_rows}): both must be multiples of 32")
    if n % 16:
        raise CheckpointError(f"trellis layer width {n} is not a multiple of 16")
    g, u = (gate_rows // 16) * (n // 16), (up_rows // 16) * (n // 16)
    if g + u != packed.shape[0]:
        raise CheckpointError(f"trellis [gate; up] split: {g} + {u} tiles expected, the buffer holds {packed.shape[0]}")
    return packed[:g].clone(), packed[g:].clone()


@dataclass
class LayerInfo:
    """What :func:`validate_layer` derives from a layer's buffers."""
    codebook: str
    m_pad: int
    n_pad: int
    n_stages: int
    bits: Tuple[int, ...]            # trellis: K per stage; E8: 2 bits per weight and stage
    block_diagonal: bool
    code_bytes: int


def _is_pow2(v: int) -> bool:
    return v > 0 and v & (v - 1) == 0


def validate_layer(buffers: Mapping[str, torch.Tensor], codebook: str, name: str = "layer") -> LayerInfo:
    """Check one layer's buffers against the storage rules of its format and return its dimensions.  Raises
    :class:`CheckpointError` with the offending buffer named; nothing is modified."""
    def need(key, dtype, ndim):
        t = buffers.get(key)
        if t is None:
            raise CheckpointError(f"{name}: buffer {key} is missing")
        if t.dtype != dtype:
            raise CheckpointError(f"{name}: {key} is {t.dtype}, expected {dtype}")
        if t.dim() != ndim:
            raise CheckpointError(f"{name}: {key} has {t.dim()} dimensions, expected {ndim}")
        return t

    su, sv = need("SU", torch.float16, 1), need("SV", torch.float16, 1)
    ws = buffers.get("Wscale")
    if ws is None or ws.numel() != 1 or ws.dtype != torch.float32:
        raise CheckpointError(f"{name}: Wscale must be one fp32 value")
    for key, t in (("SU", su), ("SV", sv)):
        if t.numel() and not bool(((t == 1) | (t == -1)).all()):
            raise CheckpointError(f"{name}: {key} holds values other than +1 / -1")
    m_pad, n_pad = su.numel(), sv.numel()
    if codebook == "trellis":
        tl = buffers.get("tlut")
        if tl is not None and tl.numel():
            raise CheckpointError(f"{name}: carries a tlut (HYB variant); only the 3INST variant is served")
        p1 = need("trellis_packed", torch.int16, 2)
        if m_pad % 32 or n_pad % 32:
            raise CheckpointError(f"{name}: trellis layers are stored in 32 x 32 groups; {m_pad} x {n_pad} is not a multiple")
        tiles = (m_pad // 16) * (n_pad // 16)
        if p1.shape[0] != tiles or p1.shape[1] % 16 or not 1 <= p1.shape[1] // 16 <= 4:
            raise CheckpointError(f"{name}: trellis_packed {tuple(p1.shape)} does not describe {m_pad} x {n_pad} at 1..4 bits")
        bits = [p1.shape[1] // 16]
        p2 = buffers.get("trellis_packed2")
        if p2 is not None and p2.numel():
            if p2.dtype != torch.int16 or p2.dim() != 2 or p2.shape[0] != tiles or p2.shape[1] % 16 or not 1 <= p2.shape[1] // 16 <= 4:
                raise CheckpointError(f"{name}: trellis_packed2 {tuple(p2.shape)} does not match the first stage")
            s2 = buffers.get("inv_resid_scale2")
            if s2 is None or s2.numel() != 1 or float(s2) == 0.0:
                raise CheckpointError(f"{name}: a second trellis stage needs a non-zero inv_resid_scale2")
            bits.append(p2.shape[1] // 16)
        code_bytes = sum(tiles * 32 * k for k in bits)
        return LayerInfo("trellis", m_pad, n_pad, len(bits), tuple(bits), True, code_bytes)
    if codebook != "e8_shell":
        raise CheckpointError(f"{name}: codebook {codebook!r} is not served")
    q1 = need("Qidxs", torch.int16, 2)
    if n_pad % 8 or tuple(q1.shape) != (m_pad, n_pad // 8):
        raise CheckpointError(f"{name}: Qidxs {tuple(q1.shape)} does not match SU ({m_pad}) and SV ({n_pad})")
    n_stages = 1
    for k, (qname, sname) in enumerate((("Qidxs2", "inv_resid_scale"), ("Qidxs3", "inv_resid_scale2"), ("Qidxs4", "inv_resid_scale3"))):
        s = buffers.get(sname)
        if s is None or s.numel() != 1 or float(s) == 0.0:
            break                                    # stages are counted by leading non-zero scales (glq/quantized_linear.py:434-451)
        q = buffers.get(qname)
        if q is None or q.dtype != torch.int16 or tuple(q.shape) != tuple(q1.shape):
            raise CheckpointError(f"{name}: {sname} is set but {qname} does not match Qidxs")
        n_stages = k + 2
    block_diagonal = not (_is_pow2(m_pad) and _is_pow2(n_pad))          # glq_vllm/linear_method.py:172-184
    return LayerInfo("e8_shell", m_pad, n_pad, n_stages, (2,) * n_stages, block_diagonal, 2 * n_stages * q1.numel())


_ALL_BUFFERS = set(E8_BUFFERS) | set(TRELLIS_BUFFERS) | set(COMMON_BUFFERS)


def group_layers(keys: Iterable[str]) -> Dict[str, List[str]]:
    """Quantized layers among tensor names: prefix -> buffer names, for every prefix that carries SU and SV."""
    layers: Dict[str, List[str]] = {}
    for k in keys:
        prefix, _, leaf = k.rpartition(".")
        if leaf in _ALL_BUFFERS:
            layers.setdefault(prefix, []).append(leaf)
    return {p: sorted(b) for p, b in layers.items() if "SU" in b and "SV" in b}


class Checkpoint:
    """A checkpoint folder: its config and a lazy index of all ``*.safetensors`` files."""

    def __init__(self, folder: str):
        self.folder = folder
        self.config = QuantizeConfig.from_folder(folder)
        self.files = [SafetensorsFile(os.path.join(folder, f)) for f in sorted(os.listdir(folder)) if f.endswith(".safetensors")]
        if not self.files:
            raise CheckpointError(f"{folder}: no .safetensors files")
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for k in f.keys():
                if k in self._where:
                    raise CheckpointError(f"{folder}: tensor {k!r} appears in two files")
                self._where[k] = f
        self.layers = group_layers(self._where)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def layer_buffers(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {b: self.tensor(f"{prefix}.{b}") for b in self.layers[prefix]}

    def validate(self) -> Dict[str, LayerInfo]:
        """Validate every quantized layer; returns prefix -> LayerInfo (raises on the first bad one)."""
        out = {}
        for prefix in self.layers:
            info = validate_layer(self.layer_buffers(prefix), self.config.codebook, prefix)
            rate = self.config.bpw_of(prefix)
            if self.config.codebook == "trellis" and rate is not None and trellis_rates(int(rate)) != (info.bits + (0,))[:2]:
                raise CheckpointError(f"{prefix}: stored at {info.bits} bits per stage, the config says {rate} bpw")
            out[prefix] = info
        return out

    def iter_layers(self) -> Iterator[Tuple[str, Dict[str, torch.Tensor]]]:
        for prefix in self.layers:
            yield prefix, self.layer_buffers(prefix)

    def load_linear(self, prefix: str, device=None, codebook=None, codebook2=None):
        """Build the ``GLQLinear`` of one layer (dimensions from the buffers, unpadded sizes = padded sizes unless the
        caller slices afterwards) and load its buffers."""
        from .linear import GLQLinear
        bufs = self.layer_buffers(prefix)
        info = validate_layer(bufs, self.config.codebook, prefix)
        lin = GLQLinear(info.n_pad, info.m_pad, bias="bias" in bufs, block_diagonal=info.block_diagonal,
                        codebook_type=info.codebook)
        lin.load_state_dict({k: v for k, v in bufs.items() if k != "tlut" or v.numel()}, strict=False)
        if codebook is not None:
            lin.set_codebook(codebook, codebook2)
        return lin.to(device) if device is not None else lin

    def close(self) -> None:
        for f in self.files:
            f.close()
