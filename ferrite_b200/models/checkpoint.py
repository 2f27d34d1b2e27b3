"""HF safetensors checkpoints: header index, zero-copy views, name mapping, fp8 block
dequant and tensor-parallel slicing.

The byte work (mmap, row/column range copies, e4m3 block dequant) is done by the C++
``SafetensorsFile``; this module resolves names and shapes.  Checkpoint-side names follow
``glm_weights.checkpoint_sources`` (reference ``crates/ferrite-model/src/checkpoint.rs:43-90``):
``qkv_proj`` / ``qkv_conv1d`` are assembled from q/k/v tensors, fp8 e4m3 weights carry a
``<name>_scale_inv`` sibling of shape [rows/128, cols/128] (``checkpoint.rs:281-292``), and the
fused aliases of ``apply_fused_aliases`` are accepted.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..config import GlmConfig
from .glm_weights import FUSED_CONV, FUSED_QKV, checkpoint_sources, weight_layout

_DT = {"F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
       "F8_E4M3": (torch.float8_e4m3fn, 1), "I32": (torch.int32, 4), "I64": (torch.int64, 8), "U8": (torch.uint8, 1)}
_DT_NAME = {v[0]: k for k, v in _DT.items()}


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None) -> None:
    """Minimal writer (tests, converted checkpoints)."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _DT_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


class TensorInfo:
    __slots__ = ("file", "dtype", "shape", "begin", "end")

    def __init__(self, file, dtype, shape, begin, end):
        self.file, self.dtype, self.shape, self.begin, self.end = file, dtype, tuple(shape), begin, end


class CheckpointIndex:
    """All tensors of a model directory (single file or sharded with an index json)."""

    def __init__(self, model_dir: str):
        from .. import build
        build.build_runtime()
        from .. import _runtime as rt
        self.rt = rt
        self.dir = model_dir
        self.files: Dict[str, object] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        names = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
        if not names:
            raise FileNotFoundError(f"no .safetensors file in {model_dir}")
        for fn in names:
            f = rt.SafetensorsFile(os.path.join(model_dir, fn))
            self.files[fn] = f
            try:
                hdr = json.loads(f.header())
            except Exception as e:
                raise ValueError(f"corrupt safetensors header in {fn}: {e}") from e
            for name, meta in hdr.items():
                if name == "__metadata__":
                    continue
                b, e = meta["data_offsets"]
                if meta["dtype"] not in _DT or e > f.data_size or b > e:
                    raise ValueError(f"bad entry {name} in {fn}")
                want = _DT[meta["dtype"]][1]
                for d in meta["shape"]:
                    want *= int(d)
                if e - b != want:   # a row copy would otherwise read the neighbouring tensor's bytes
                    raise ValueError(f"bad entry {name} in {fn}: {e - b} bytes for shape {meta['shape']} {meta['dtype']}")
                self.tensors[name] = TensorInfo(f, meta["dtype"], meta["shape"], b, e)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def view(self, name: str) -> torch.Tensor:
        """Zero-copy tensor over the mapped file (read-only memory: clone before writing)."""
        ti = self.tensors[name]
        dt, _ = _DT[ti.dtype]
        raw = ti.file.view(ti.begin, ti.end)
        if raw.size == 0:
            return torch.empty(ti.shape, dtype=dt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # non-writable buffer
            return torch.frombuffer(raw, dtype=torch.uint8).view(dt).view(ti.shape)

    def rows(self, name: str, r0: int, r1: int, c0: int = 0, c1: Optional[int] = None) -> torch.Tensor:
        """Copy of rows [r0, r1) x columns [c0, c1) of a 2-D tensor, read by byte ranges."""
        ti = self.tensors[name]
        dt, esz = _DT[ti.dtype]
        rows, cols = ti.shape
        c1 = cols if c1 is None else c1
        out = np.empty((r1 - r0) * (c1 - c0) * esz, dtype=np.uint8)
        ti.file.copy_rows(ti.begin, cols * esz, r0, r1, c0 * esz, c1 * esz, out)
        return torch.from_numpy(out).view(dt).view(r1 - r0, c1 - c0)

    def dequant_fp8(self, name: str, scale_name: str, r0: int = 0, r1: Optional[int] = None, block: int = 128) -> torch.Tensor:
        ti, si = self.tensors[name], self.tensors[scale_name]
        if ti.dtype != "F8_E4M3" or len(ti.shape) != 2:
            raise ValueError(f"{name}: not a 2-D e4m3 tensor")
        rows, cols = ti.shape
        want = [(rows + block - 1) // block, (cols + block - 1) // block]
        if list(si.shape) != want:
            raise ValueError(f"{scale_name}: scale shape {list(si.shape)} != {want} for a {rows}x{cols} weight")
        r1 = rows if r1 is None else r1
        if ti.file is si.file and si.dtype == "F32":   # the C++ path reads f32 scales; others go through torch
            return torch.from_numpy(ti.file.dequant_e4m3_block(ti.begin, si.begin, rows, cols, block, r0, r1))
        w = self.view(name)[r0:r1].float()
        s = self.view(scale_name).float().repeat_interleave(block, 0)[r0:r1].repeat_interleave(block, 1)[:, :cols]
        return w * s


def _scale_name(src: str) -> str:
    return src + "_scale_inv" if src.endswith(".weight") else src + ".weight_scale_inv"


class CheckpointSource:
    """``get(name)`` over a checkpoint directory for :class:`GlmDeviceModel` and the reference
    engine: resolves internal names to checkpoint tensors, assembles fused q/k/v, accepts the
    fused aliases and dequantises fp8 block-scaled weights."""

    def __init__(self, model_dir: str, cfg: GlmConfig, device="cpu"):
        self.idx = CheckpointIndex(model_dir)
        self.cfg, self.device = cfg, device
        self.layout = weight_layout(cfg)

    def _load_src(self, src: str) -> torch.Tensor:
        sn = _scale_name(src)
        if self.idx.tensors[src].dtype == "F8_E4M3" and sn in self.idx:
            return self.idx.dequant_fp8(src, sn)
        return self.idx.view(src)

    def _alias(self, name: str) -> Optional[torch.Tensor]:
        """Serve a canonical name out of a fused checkpoint tensor."""
        la, ds = self.cfg.linear_attn, self.cfg.dsa
        pre = "model.language_model." + name[len("model."):] if name.startswith("model.") else name
        head, _, leaf = pre.rpartition(".self_attn.")
        if leaf in ("qkv_proj.weight", "b_proj.weight", "f_a_proj.weight", "g_a_proj.weight"):
            f = f"{head}.self_attn.fused_qkvbfg_a_proj.weight"
            if f in self.idx:
                parts = dict(zip(("qkv_proj.weight", "b_proj.weight", "f_a_proj.weight", "g_a_proj.weight"),
                                 self._load_src(f).split([3 * la.proj, la.num_heads, la.low_rank, la.low_rank], 0)))
                return parts[leaf]
        if leaf in ("f_b_proj.weight", "g_b_proj.weight"):
            f = f"{head}.self_attn.fused_fg_b_proj.weight"
            if f in self.idx:
                t = self._load_src(f)
                if t.dim() == 2:     # flat [2 * proj, low_rank]: f rows first, then g (reference weights.rs:374-387)
                    t = t.view(2, t.shape[0] // 2, t.shape[1])
                return t[0 if leaf.startswith("f_") else 1]
        if leaf in ("q_a_proj.weight", "kv_a_proj_with_mqa.weight"):
            f = f"{head}.self_attn.fused_qkv_a_proj_with_mqa.weight"
            if f in self.idx:
                t = self._load_src(f)
                return t[:ds.q_lora_rank] if leaf.startswith("q_a") else t[ds.q_lora_rank:]
        for nm in ("gate_proj.weight", "up_proj.weight"):
            if pre.endswith(nm):
                f = pre[: -len(nm)].replace(".shared_expert.", ".shared_experts.") + "gate_up_proj.weight"
                if f in self.idx:
                    t = self._load_src(f)
                    half = t.shape[0] // 2
                    return t[:half] if nm.startswith("gate") else t[half:]
        return None

    def get(self, name: str) -> torch.Tensor:
        marker, srcs = checkpoint_sources(name)
        if all(s in self.idx for s in srcs):
            parts = [self._load_src(s) for s in srcs]
            t = parts[0] if marker is None else torch.cat(parts, 0)
        else:
            t = self._alias(name)
            if t is None and name in self.idx:  # already in the internal layout
                t = self._load_src(name)
            if t is None:
                raise KeyError(f"{name}: none of {srcs} (nor a fused alias) is in the checkpoint")
        want = self.layout.get(name)
        if want is not None and tuple(t.shape) != tuple(want):
            if marker == FUSED_CONV and t.dim() == 3:  # conv weights stored [ch, 1, k]
                t = t.reshape(want)
            else:
                raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != expected {tuple(want)}")
        return t.to(self.device)

    def get_fp8(self, name: str) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        """(e4m3 weight, f32 block scales) when the checkpoint stores the tensor in fp8."""
        marker, srcs = checkpoint_sources(name)
        if marker is not None or srcs[0] not in self.idx:
            return None
        sn = _scale_name(srcs[0])
        if self.idx.tensors[srcs[0]].dtype != "F8_E4M3" or sn not in self.idx:
            return None
        return self.idx.view(srcs[0]).to(self.device), self.idx.view(sn).float().to(self.device)


def save_internal_checkpoint(path: str, weights: Dict[str, torch.Tensor], hf_names: bool = True,
                             fp8_names: Tuple[str, ...] = ()) -> None:
    """Write weights under checkpoint-side names (q/k/v split, plural shared_experts); tensors
    whose name contains one of ``fp8_names`` are stored e4m3 with a ``_scale_inv`` sibling."""
    from ..ops.reference import quant_fp8_block
    out: Dict[str, torch.Tensor] = {}
    for name, t in weights.items():
        marker, srcs = checkpoint_sources(name) if hf_names else (None, [name])
        pieces = list(t.chunk(3, 0)) if marker is not None else [t]
        for src, piece in zip(srcs, pieces):
            if any(k in name for k in fp8_names) and piece.dim() == 2:
                q, s = quant_fp8_block(piece.float())
                out[src], out[_scale_name(src)] = q, s
            else:
                out[src] = piece.to(torch.bfloat16) if piece.dim() > 1 else piece.float()
    write_safetensors(path, out)
