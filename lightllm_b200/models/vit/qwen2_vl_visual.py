"""Qwen2-VL vision tower: patch embedding (a 2 x 14 x 14 convolution with stride = kernel, i.e. one GEMM over
flattened patches), pre-norm transformer blocks with 2-D rotary position embedding over the patch grid and
full (non-causal) attention inside each image, and the 2 x 2 patch merger that projects to the language model's
hidden size.  Image preprocessing (`smart_resize`, normalisation, patch layout) lives here too.

The tower runs in the visual server process, once per new image, on plain torch ops (its GEMMs are library
GEMMs; the language model's hot path does not pass through here).
Reference: lightllm/models/qwen2_vl/qwen2_visual.py, vision_process.py.
"""
from __future__ import annotations

import math
from io import BytesIO
from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    """Closest size with both sides multiples of `factor` and an area inside [min_pixels, max_pixels]."""
    if max(height, width) / max(min(height, width), 1) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt((height * width) / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def image_token_num(width: int, height: int, patch: int = 14, merge: int = 2, **kw) -> Tuple[int, Tuple[int, int, int]]:
    h, w = smart_resize(height, width, patch * merge, **kw)
    gh, gw = h // patch, w // patch
    return (gh * gw) // (merge * merge), (1, gh, gw)


def patchify(pixels: torch.Tensor, patch: int = 14, merge: int = 2, temporal: int = 2):
    """pixels [frames, 3, H, W] (H, W multiples of patch * merge) -> ([t*gh*gw, 3*temporal*patch*patch], (t, gh, gw)).
    Patches of one merge window are adjacent rows, which is what the merger's reshape relies on."""
    f, c, H, W = pixels.shape
    if f % temporal:
        pixels = torch.cat([pixels, pixels[-1:].expand(temporal - f % temporal, -1, -1, -1)], dim=0)
        f = pixels.shape[0]
    t, gh, gw = f // temporal, H // patch, W // patch
    x = pixels.view(t, temporal, c, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return x.reshape(t * gh * gw, c * temporal * patch * patch), (t, gh, gw)


def preprocess_image(data: bytes, patch: int = 14, merge: int = 2, temporal: int = 2, **resize_kw):
    from PIL import Image

    with Image.open(BytesIO(data)) as im:
        im = im.convert("RGB")
        h, w = smart_resize(im.height, im.width, patch * merge, **resize_kw)
        im = im.resize((w, h), Image.BICUBIC)
        arr = np.asarray(im, dtype=np.float32) / 255.0
    x = torch.from_numpy(arr).permute(2, 0, 1)
    x = (x - torch.tensor(CLIP_MEAN).view(3, 1, 1)) / torch.tensor(CLIP_STD).view(3, 1, 1)
    return patchify(x.unsqueeze(0), patch, merge, temporal)


def grid_rotary(grids: Sequence[Tuple[int, int, int]], head_dim: int, merge: int, theta: float = 10000.0):
    """cos/sin [N, head_dim] of the 2-D rotary embedding: the first quarter of the frequency slots rotates
    with the patch row, the second with the patch column (repeated for the rotate-half partner)."""
    rows, cols = [], []
    for t, h, w in grids:
        r = torch.arange(h).unsqueeze(1).expand(h, w)
        c = torch.arange(w).unsqueeze(0).expand(h, w)
        order = lambda x: x.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten()  # noqa: E731
        rows.append(order(r).repeat(t))
        cols.append(order(c).repeat(t))
    rows, cols = torch.cat(rows), torch.cat(cols)
    dim = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    fr = torch.cat([rows.float()[:, None] * inv[None], cols.float()[:, None] * inv[None]], dim=1)  # [N, head_dim/2]
    emb = torch.cat([fr, fr], dim=1)
    return emb.cos(), emb.sin()


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


class Qwen2VLVisionTower:
    def __init__(self, vcfg: dict, source, device, dtype=torch.bfloat16, prefix: str = None):
        self.cfg = vcfg
        self.embed = vcfg["embed_dim"]
        self.depth = vcfg["depth"]
        self.heads = vcfg["num_heads"]
        self.head_dim = self.embed // self.heads
        self.patch = vcfg.get("patch_size", 14)
        self.merge = vcfg.get("spatial_merge_size", 2)
        self.temporal = vcfg.get("temporal_patch_size", 2)
        self.out_hidden = vcfg.get("hidden_size")
        self.act = vcfg.get("hidden_act", "quick_gelu")
        self.device, self.dtype = device, dtype
        if prefix is None:
            prefix = next(p for p in ("visual.", "model.visual.") if source.has(p + "patch_embed.proj.weight"))
        g = lambda n: source.get(prefix + n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        self.patch_w = g("patch_embed.proj.weight").reshape(self.embed, -1)
        self.blocks = []
        for i in range(self.depth):
            b = f"blocks.{i}."
            self.blocks.append({k: g(b + k) for k in (
                "norm1.weight", "norm1.bias", "attn.qkv.weight", "attn.qkv.bias", "attn.proj.weight", "attn.proj.bias",
                "norm2.weight", "norm2.bias", "mlp.fc1.weight", "mlp.fc1.bias", "mlp.fc2.weight", "mlp.fc2.bias")})
        self.merger = {k: g("merger." + k) for k in ("ln_q.weight", "ln_q.bias", "mlp.0.weight", "mlp.0.bias",
                                                     "mlp.2.weight", "mlp.2.bias")}

    @staticmethod
    def weight_shapes(vcfg: dict, prefix: str = "visual.") -> dict:
        E, Hd = vcfg["embed_dim"], int(vcfg["embed_dim"] * vcfg.get("mlp_ratio", 4))
        p, t, m = vcfg.get("patch_size", 14), vcfg.get("temporal_patch_size", 2), vcfg.get("spatial_merge_size", 2)
        s = {prefix + "patch_embed.proj.weight": (E, 3, t, p, p)}
        for i in range(vcfg["depth"]):
            b = f"{prefix}blocks.{i}."
            s.update({b + "norm1.weight": (E,), b + "norm1.bias": (E,), b + "norm2.weight": (E,), b + "norm2.bias": (E,),
                      b + "attn.qkv.weight": (3 * E, E), b + "attn.qkv.bias": (3 * E,), b + "attn.proj.weight": (E, E),
                      b + "attn.proj.bias": (E,), b + "mlp.fc1.weight": (Hd, E), b + "mlp.fc1.bias": (Hd,),
                      b + "mlp.fc2.weight": (E, Hd), b + "mlp.fc2.bias": (E,)})
        M = E * m * m
        s.update({prefix + "merger.ln_q.weight": (E,), prefix + "merger.ln_q.bias": (E,),
                  prefix + "merger.mlp.0.weight": (M, M), prefix + "merger.mlp.0.bias": (M,),
                  prefix + "merger.mlp.2.weight": (vcfg["hidden_size"], M), prefix + "merger.mlp.2.bias": (vcfg["hidden_size"],)})
        return s

    def _act(self, x):
        if self.act == "quick_gelu":
            return x * torch.sigmoid(1.702 * x)
        if self.act in ("gelu_pytorch_tanh", "gelu_tanh"):
            return F.gelu(x, approximate="tanh")
        if self.act == "silu":
            return F.silu(x)
        return F.gelu(x)

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grids: List[Tuple[int, int, int]]) -> torch.Tensor:
        """patches [N, 3*temporal*patch*patch] of all images; returns [N / merge^2, out_hidden]."""
        x = F.linear(patches.to(self.device, self.dtype), self.patch_w)
        cos, sin = grid_rotary(grids, self.head_dim, self.merge)
        cos, sin = cos.to(self.device)[:, None, :], sin.to(self.device)[:, None, :]
        lens = [h * w for t, h, w in grids for _ in range(t)]
        N = x.shape[0]
        for b in self.blocks:
            h = F.layer_norm(x, (self.embed,), b["norm1.weight"], b["norm1.bias"], 1e-6)
            qkv = F.linear(h, b["attn.qkv.weight"], b["attn.qkv.bias"]).view(N, 3, self.heads, self.head_dim)
            q, k, v = qkv.unbind(1)
            q = (q.float() * cos + _rotate_half(q.float()) * sin).to(self.dtype)
            k = (k.float() * cos + _rotate_half(k.float()) * sin).to(self.dtype)
            outs, s0 = [], 0
            for n in lens:  # full attention inside each frame
                qs, ks, vs = (z[s0:s0 + n].transpose(0, 1).unsqueeze(0) for z in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qs, ks, vs).squeeze(0).transpose(0, 1))
                s0 += n
            a = torch.cat(outs, dim=0).reshape(N, self.embed)
            x = x + F.linear(a, b["attn.proj.weight"], b["attn.proj.bias"])
            h = F.layer_norm(x, (self.embed,), b["norm2.weight"], b["norm2.bias"], 1e-6)
            x = x + F.linear(self._act(F.linear(h, b["mlp.fc1.weight"], b["mlp.fc1.bias"])), b["mlp.fc2.weight"],
                             b["mlp.fc2.bias"])
        m = self.merger
        x = F.layer_norm(x, (self.embed,), m["ln_q.weight"], m["ln_q.bias"], 1e-6).view(-1, self.embed * self.merge ** 2)
        x = F.gelu(F.linear(x, m["mlp.0.weight"], m["mlp.0.bias"]))
        return F.linear(x, m["mlp.2.weight"], m["mlp.2.bias"])

    def encode_images(self, payloads: List[bytes], items=None) -> List[torch.Tensor]:
        items = [preprocess_image(p, self.patch, self.merge, self.temporal) for p in payloads]
        out = self.forward(torch.cat([x for x, _ in items], dim=0), [g for _, g in items])
        res, s0 = [], 0
        for _, (t, gh, gw) in items:
            n = t * gh * gw // (self.merge ** 2)
            res.append(out[s0:s0 + n])
            s0 += n
        return res
