"""DSV41 vision tower: ViT with 2-D RoPE, the 3x3 aligner and the image-span token plan.

Golden model (f32 PyTorch) and the device twin.  Semantics of ``ref_inference/vision.py:9-120``
(patch embedding, bidirectional attention with rotary halves driven by the patch's (row, column),
SwiGLU MLP, final RMSNorm; aligner = zero-padded r x r unfold -> linear -> GELU -> linear) and of
``ref_inference/image_processor.py:23,133-173`` (span layout); reference device kernels
``kernels/cuda/dsv41_vision.cu``.  On the device every linear layer is the tcgen05 + TMA GEMM
(``csrc/kernels/gemm_tc.cu``); attention, rotary, bias/GELU and the aligner pack are the kernels of
``csrc/kernels/vision.cu``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

IMAGE_START, IMAGE, IMAGE_NEW_LINE, IMAGE_END = range(4)
TEXT = -1


def vision_specs(cfg) -> Dict[str, "Spec"]:
    from .dsv41_weights import Spec
    v, d = cfg.vision, cfg.dim
    out: Dict[str, Spec] = {}
    pin = 3 * v.patch_size ** 2
    out["vision.patch_embed.proj.weight"] = Spec((v.dim, pin), "bf16")
    out["vision.patch_embed.proj.bias"] = Spec((v.dim,), "f32", None, "small")
    for i in range(v.n_layers):
        p = f"vision.blocks.{i}."
        out[p + "norm1.weight"] = Spec((v.dim,), "f32", None, "ones")
        out[p + "attn.wqkv.weight"] = Spec((3 * v.dim, v.dim), "bf16")
        out[p + "attn.wqkv.bias"] = Spec((3 * v.dim,), "f32", None, "small")
        out[p + "attn.wo.weight"] = Spec((v.dim, v.dim), "bf16")
        out[p + "attn.wo.bias"] = Spec((v.dim,), "f32", None, "small")
        out[p + "norm2.weight"] = Spec((v.dim,), "f32", None, "ones")
        out[p + "mlp.w1.weight"] = Spec((2 * v.inter_dim, v.dim), "bf16")
        out[p + "mlp.w2.weight"] = Spec((v.dim, v.inter_dim), "bf16")
    out["vision.norm.weight"] = Spec((v.dim,), "f32", None, "ones")
    r2 = v.downsample_ratio ** 2
    out["aligner.w1.weight"] = Spec((d, v.dim * r2), "bf16")
    out["aligner.w1.bias"] = Spec((d,), "f32", None, "small")
    out["aligner.w2.weight"] = Spec((d, d), "bf16")
    out["aligner.w2.bias"] = Spec((d,), "f32", None, "small")
    for n in ("image_start", "image_end", "image_newline"):
        out[n] = Spec((d,), "bf16", None, "small")
    return out


def image_token_types(n_llm_h: int, n_llm_w: int) -> List[int]:
    """Span layout: START, then each aligner row followed by NEW_LINE, then END."""
    return [IMAGE_START] + ([IMAGE] * n_llm_w + [IMAGE_NEW_LINE]) * n_llm_h + [IMAGE_END]


def llm_grid(n_vit_h: int, n_vit_w: int, ratio: int):
    return (n_vit_h + ratio - 1) // ratio, (n_vit_w + ratio - 1) // ratio


@dataclass
class ImageSpan:
    start: int                 # first position of the span in the prompt
    types: List[int]
    n_vit_h: int
    n_vit_w: int


def expand_image_tokens(tokens: List[int], image_token_id: int, grids: List[tuple], ratio: int):
    """Replace every image placeholder by its span.  Returns (tokens, token_types, spans)."""
    out, types, spans = [], [], []
    it = iter(grids)
    for t in tokens:
        if t != image_token_id:
            out.append(t)
            types.append(TEXT)
            continue
        n_h, n_w = next(it)
        lh, lw = llm_grid(n_h, n_w, ratio)
        ty = image_token_types(lh, lw)
        spans.append(ImageSpan(len(out), ty, n_h, n_w))
        out += [image_token_id] * len(ty)
        types += ty
    return out, types, spans


def vision_angles(n_h: int, n_w: int, rope_dim: int, theta: float) -> torch.Tensor:
    """[n_h * n_w, rope_dim]: first half of the angles follows the row index, second half the column."""
    inv = 1.0 / (theta ** (torch.arange(0, rope_dim, 2, dtype=torch.float32) / rope_dim))
    hpos = torch.arange(n_h).unsqueeze(1).expand(n_h, n_w)
    wpos = torch.arange(n_w).unsqueeze(0).expand(n_h, n_w)
    fr = torch.stack([hpos, wpos], -1).reshape(-1, 2, 1).float() * inv
    return fr.flatten(1)


def _rms(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * w.float()


class VisionReference:
    def __init__(self, cfg, weights: Dict[str, torch.Tensor]):
        self.cfg, self.v, self.w = cfg, cfg.vision, weights

    def lin(self, x, name, bias=True):
        y = x.float() @ self.w[name + ".weight"].float().t()
        return y + self.w[name + ".bias"].float() if bias else y

    def vit(self, patches: torch.Tensor, n_h: int, n_w: int) -> torch.Tensor:
        """patches [n_h * n_w, 3 * patch^2] -> [n, vision_dim]."""
        v = self.v
        H, hd = v.n_heads, v.head_dim
        ang = vision_angles(n_h, n_w, hd // 2, v.rope_theta)
        cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
        x = self.lin(patches.flatten(1), "vision.patch_embed.proj")
        n = x.shape[0]
        for i in range(v.n_layers):
            p = f"vision.blocks.{i}."
            h = _rms(x, self.w[p + "norm1.weight"], v.norm_eps)
            q, k, val = (t.view(n, H, hd) for t in self.lin(h, p + "attn.wqkv").chunk(3, -1))

            def rot(t):
                a, b = t.chunk(2, -1)
                return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
            q, k = rot(q), rot(k)
            s = torch.einsum("nhd,mhd->hnm", q, k) * hd ** -0.5
            o = torch.einsum("hnm,mhd->nhd", s.softmax(-1), val).reshape(n, -1)
            x = x + self.lin(o, p + "attn.wo")
            h = _rms(x, self.w[p + "norm2.weight"], v.norm_eps)
            g, u = self.lin(h, p + "mlp.w1", bias=False).chunk(2, -1)
            x = x + self.lin(F.silu(g) * u, p + "mlp.w2", bias=False)
        return _rms(x, self.w["vision.norm.weight"], v.norm_eps)

    def aligner(self, x: torch.Tensor, n_h: int, n_w: int) -> torch.Tensor:
        r = self.v.downsample_ratio
        t = x.float().view(n_h, n_w, -1).permute(2, 0, 1)
        t = F.pad(t, (0, -n_w % r, 0, -n_h % r))
        t = F.unfold(t.unsqueeze(0), r, stride=r).squeeze(0).transpose(0, 1)
        return self.lin(F.gelu(self.lin(t, "aligner.w1")), "aligner.w2")

    def encode_image(self, patches, n_h, n_w) -> torch.Tensor:
        return self.aligner(self.vit(patches, n_h, n_w), n_h, n_w)

    def span_embeddings(self, span: ImageSpan, patches: torch.Tensor) -> torch.Tensor:
        """[len(span.types), dim]: aligner rows for IMAGE slots, learned vectors for the delimiters."""
        emb = self.encode_image(patches, span.n_vit_h, span.n_vit_w)
        ty = torch.tensor(span.types)
        out = torch.zeros(len(span.types), self.cfg.dim)
        out[ty == IMAGE_START] = self.w["image_start"].float()
        out[ty == IMAGE_END] = self.w["image_end"].float()
        out[ty == IMAGE_NEW_LINE] = self.w["image_newline"].float()
        out[ty == IMAGE] = emb
        return out


class VisionDevice:
    """Device twin: tcgen05 GEMMs for every linear layer, custom kernels for the rest."""

    def __init__(self, cfg, src, device="cuda"):
        from .. import _lib
        self.cfg, self.v = cfg, cfg.vision
        self.K = _lib.lib()
        self.dev = torch.device(device)
        bf = lambda n: src.get(n).to(self.dev, torch.bfloat16).contiguous()
        f32 = lambda n: src.get(n).to(self.dev, torch.float32).contiguous()
        self.w = {}
        for name, spec in vision_specs(cfg).items():
            self.w[name] = bf(name) if (spec.kind == "bf16" and name.endswith("weight")) else f32(name)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.dev)

    def _gemm(self, x_bf16, name, M, N, Kd):
        out = torch.empty(M, N, device=self.dev)
        self.K.call("fb_gemm_tc_bf16", self.w[name], x_bf16, Kd, out, N, M, N, Kd, 0, self.status)
        return out

    def _bf16(self, x_f32, M, Kd):
        out = torch.empty(M, Kd, dtype=torch.bfloat16, device=self.dev)
        self.K.call("fb_vit_to_bf16", x_f32, out, M * Kd)
        return out

    def vit(self, patches: torch.Tensor, n_h: int, n_w: int) -> torch.Tensor:
        v, K = self.v, self.K
        n, D, H, hd, I = n_h * n_w, v.dim, v.n_heads, v.head_dim, v.inter_dim
        pin = patches.shape[1] if patches.dim() == 2 else patches[0].numel()
        pk = (pin + 7) // 8 * 8
        xp = torch.zeros(n, pk, dtype=torch.bfloat16, device=self.dev)
        xp[:, :pin] = patches.reshape(n, -1).to(self.dev)
        wname = "vision.patch_embed.proj.weight"
        if pk != pin and self.w[wname].shape[1] != pk:   # pad K to the 16-byte rule of the tensor map
            wp = torch.zeros(D, pk, dtype=torch.bfloat16, device=self.dev)
            wp[:, :pin] = self.w[wname]
            self.w[wname] = wp
        x = self._gemm(xp, wname, n, D, pk)
        K.call("fb_vit_bias_act", x, self.w["vision.patch_embed.proj.bias"], None, x, n, D, 0)
        ang = vision_angles(n_h, n_w, hd // 2, v.rope_theta).to(self.dev).contiguous()
        h = torch.empty(n, D, device=self.dev)
        o = torch.empty(n, D, device=self.dev)
        act = torch.empty(n, I, device=self.dev)
        for i in range(v.n_layers):
            p = f"vision.blocks.{i}."
            K.call("fb_rmsnorm", x, None, None, self.w[p + "norm1.weight"], h, n, D, D, D, float(v.norm_eps), None, 0, 0, 0)
            qkv = self._gemm(self._bf16(h, n, D), p + "attn.wqkv.weight", n, 3 * D, D)
            K.call("fb_vit_bias_act", qkv, self.w[p + "attn.wqkv.bias"], None, qkv, n, 3 * D, 0)
            K.call("fb_vit_attention", qkv, ang, o, n, H, hd, float(hd ** -0.5))
            y = self._gemm(self._bf16(o, n, D), p + "attn.wo.weight", n, D, D)
            K.call("fb_vit_bias_act", y, self.w[p + "attn.wo.bias"], x, x, n, D, 0)          # x += y + bias
            K.call("fb_rmsnorm", x, None, None, self.w[p + "norm2.weight"], h, n, D, D, D, float(v.norm_eps), None, 0, 0, 0)
            gu = self._gemm(self._bf16(h, n, D), p + "mlp.w1.weight", n, 2 * I, D)
            K.call("fb_d4_swiglu_clamp", gu, 2 * I, act, I, n, I, 0.0)
            y = self._gemm(self._bf16(act, n, I), p + "mlp.w2.weight", n, D, I)
            K.call("fb_vit_bias_act", y, None, x, x, n, D, 0)
        K.call("fb_rmsnorm", x, None, None, self.w["vision.norm.weight"], h, n, D, D, D, float(v.norm_eps), None, 0, 0, 0)
        return h

    def aligner(self, x: torch.Tensor, n_h: int, n_w: int) -> torch.Tensor:
        v, K, d = self.v, self.K, self.cfg.dim
        r = v.downsample_ratio
        lh, lw = llm_grid(n_h, n_w, r)
        m, kin = lh * lw, v.dim * r * r
        packed = torch.empty(m, kin, dtype=torch.bfloat16, device=self.dev)
        K.call("fb_vit_unfold", x, packed, n_h, n_w, v.dim, r)
        y = self._gemm(packed, "aligner.w1.weight", m, d, kin)
        K.call("fb_vit_bias_act", y, self.w["aligner.w1.bias"], None, y, m, d, 1)            # GELU(y + bias)
        z = self._gemm(self._bf16(y, m, d), "aligner.w2.weight", m, d, d)
        K.call("fb_vit_bias_act", z, self.w["aligner.w2.bias"], None, z, m, d, 0)
        return z

    def encode_image(self, patches, n_h, n_w) -> torch.Tensor:
        return self.aligner(self.vit(patches, n_h, n_w), n_h, n_w)
