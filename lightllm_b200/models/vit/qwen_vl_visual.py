"""Qwen-VL (first generation) vision tower: an OpenCLIP-style ViT over a fixed 448 x 448 picture (patch 14, learned
position table interpolated bicubically to the patch grid, pre-norm blocks whose fused qkv projection is packed per
head as [q | k | v]), followed by a one-layer cross-attention resampler: 256 learned queries with a 2-D sin-cos
position code attend to the patch features (keys carry the same code interpolated to the patch grid), then
LayerNorm and a square projection.  Every picture gives `n_queries` embeddings of the language model's width.
Tensors live under `transformer.visual.` in the checkpoint.  Runs in the visual server on torch ops.

Reference: lightllm/models/qwen_vl/qwen_visual.py.
"""
from __future__ import annotations

import math
from io import BytesIO
from typing import List

import numpy as np
import torch
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def sincos_2d(dim: int, grid: int) -> torch.Tensor:
    """[grid * grid, dim]: the first half of the channels encodes one grid axis, the second half the other; each
    half is [sin | cos] over dim / 4 frequencies 10000^(-i / (dim / 4))."""
    def axis(pos):
        omega = 1.0 / 10000 ** (np.arange(dim // 4, dtype=np.float32) / (dim / 4.0))
        out = np.einsum("m,d->md", pos.reshape(-1), omega)
        return np.concatenate([np.sin(out), np.cos(out)], axis=1)

    gw, gh = np.meshgrid(np.arange(grid, dtype=np.float32), np.arange(grid, dtype=np.float32))
    return torch.from_numpy(np.concatenate([axis(gw), axis(gh)], axis=1)).float()


def resize_positions(table: torch.Tensor, n: int) -> torch.Tensor:
    """A [s * s, C] position table resampled (bicubic) to n = t * t positions."""
    s, t = int(math.sqrt(table.shape[0])), int(math.sqrt(n))
    if s == t:
        return table
    x = table.float().reshape(1, s, s, -1).permute(0, 3, 1, 2)
    x = F.interpolate(x, size=(t, t), mode="bicubic", align_corners=False)
    return x.permute(0, 2, 3, 1).flatten(0, 2).to(table.dtype)


class QwenVLVisionTower:
    def __init__(self, vcfg: dict, source, device, dtype=torch.bfloat16, prefix: str = "transformer.visual."):
        self.image_size = int(vcfg.get("image_size", 448))
        self.patch = int(vcfg.get("patch_size", 14))
        self.width = int(vcfg["width"])
        self.layers = int(vcfg["layers"])
        self.heads = int(vcfg["heads"])
        self.out_dim = int(vcfg.get("output_dim", 4096))
        self.n_queries = int(vcfg.get("n_queries", 256))
        self.pool_heads = max(self.out_dim // 128, 1)
        self.out_hidden = self.out_dim
        self.device, self.dtype = device, dtype
        g = lambda n: source.get(prefix + n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        self.conv_w = g("conv1.weight").reshape(self.width, -1)
        self.pos = g("positional_embedding")
        self.ln_pre = (g("ln_pre.weight"), g("ln_pre.bias"))
        self.blocks = []
        for i in range(self.layers):
            b = f"transformer.resblocks.{i}."
            self.blocks.append({k: g(b + k) for k in self._block_names()})
        p = "attn_pool."
        self.pool = {k: g(p + k) for k in ("pos_embed", "query", "attn.in_proj_weight", "attn.in_proj_bias",
                                           "attn.out_proj.weight", "attn.out_proj.bias", "ln_q.weight", "ln_q.bias",
                                           "ln_kv.weight", "ln_kv.bias")}
        self.pool_kv_w = g(p + "kv_proj.weight") if source.has(prefix + p + "kv_proj.weight") else None
        self.ln_post = (g("ln_post.weight"), g("ln_post.bias"))
        self.proj = g("proj")

    @staticmethod
    def _block_names():
        return ("ln_1.weight", "ln_1.bias", "ln_2.weight", "ln_2.bias", "attn.in_proj.weight", "attn.in_proj.bias",
                "attn.out_proj.weight", "attn.out_proj.bias", "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight",
                "mlp.c_proj.bias")

    @staticmethod
    def weight_shapes(vcfg: dict, prefix: str = "transformer.visual.") -> dict:
        W, L, E = int(vcfg["width"]), int(vcfg["layers"]), int(vcfg.get("output_dim", 4096))
        p, Q = int(vcfg.get("patch_size", 14)), int(vcfg.get("n_queries", 256))
        M = int(W * float(vcfg.get("mlp_ratio", 4.9231)))
        s = {prefix + "conv1.weight": (W, 3, p, p), prefix + "positional_embedding": (256, W),
             prefix + "ln_pre.weight": (W,), prefix + "ln_pre.bias": (W,), prefix + "ln_post.weight": (E,),
             prefix + "ln_post.bias": (E,), prefix + "proj": (E, E)}
        for i in range(L):
            b = f"{prefix}transformer.resblocks.{i}."
            s.update({b + "ln_1.weight": (W,), b + "ln_1.bias": (W,), b + "ln_2.weight": (W,), b + "ln_2.bias": (W,),
                      b + "attn.in_proj.weight": (3 * W, W), b + "attn.in_proj.bias": (3 * W,),
                      b + "attn.out_proj.weight": (W, W), b + "attn.out_proj.bias": (W,),
                      b + "mlp.c_fc.weight": (M, W), b + "mlp.c_fc.bias": (M,), b + "mlp.c_proj.weight": (W, M),
                      b + "mlp.c_proj.bias": (W,)})
        a = prefix + "attn_pool."
        s.update({a + "pos_embed": (Q, E), a + "query": (Q, E), a + "kv_proj.weight": (E, W),
                  a + "attn.in_proj_weight": (3 * E, E), a + "attn.in_proj_bias": (3 * E,),
                  a + "attn.out_proj.weight": (E, E), a + "attn.out_proj.bias": (E,), a + "ln_q.weight": (E,),
                  a + "ln_q.bias": (E,), a + "ln_kv.weight": (E,), a + "ln_kv.bias": (E,)})
        return s

    def preprocess(self, data: bytes) -> torch.Tensor:
        from PIL import Image

        with Image.open(BytesIO(data)) as im:
            im = im.convert("RGB").resize((self.image_size, self.image_size), Image.BICUBIC)
            arr = np.asarray(im, dtype=np.float32) / 255.0
        x = torch.from_numpy(arr).permute(2, 0, 1)
        return (x - torch.tensor(CLIP_MEAN).view(3, 1, 1)) / torch.tensor(CLIP_STD).view(3, 1, 1)

    def _resample(self, x: torch.Tensor) -> torch.Tensor:
        """x [B, N, width] patch features -> [B, n_queries, out_dim]."""
        m, E, H = self.pool, self.out_dim, self.pool_heads
        B, N, _ = x.shape
        if self.pool_kv_w is not None:
            x = F.linear(x, self.pool_kv_w)
        kv = F.layer_norm(x, (E,), m["ln_kv.weight"], m["ln_kv.bias"], 1e-6)
        q = F.layer_norm(m["query"], (E,), m["ln_q.weight"], m["ln_q.bias"], 1e-6) + m["pos_embed"]
        k_in = kv + resize_positions(m["pos_embed"], N)
        wq, wk, wv = m["attn.in_proj_weight"].split(E, dim=0)
        bq, bk, bv = m["attn.in_proj_bias"].split(E, dim=0)
        D = E // H
        qh = F.linear(q, wq, bq).view(1, -1, H, D).transpose(1, 2).expand(B, -1, -1, -1)
        kh = F.linear(k_in, wk, bk).view(B, N, H, D).transpose(1, 2)
        vh = F.linear(kv, wv, bv).view(B, N, H, D).transpose(1, 2)
        a = F.scaled_dot_product_attention(qh, kh, vh).transpose(1, 2).reshape(B, -1, E)
        return F.linear(a, m["attn.out_proj.weight"], m["attn.out_proj.bias"])

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [B, 3, S, S] -> [B, n_queries, out_dim]."""
        B, p, W, H = pixels.shape[0], self.patch, self.width, self.heads
        x = pixels.to(self.device, self.dtype)
        g = x.shape[-1] // p
        x = x.view(B, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B, g * g, 3 * p * p)
        x = F.linear(x, self.conv_w) + resize_positions(self.pos, g * g)
        x = F.layer_norm(x, (W,), *self.ln_pre, 1e-6)
        D = W // H
        N = x.shape[1]
        for b in self.blocks:
            h = F.layer_norm(x, (W,), b["ln_1.weight"], b["ln_1.bias"], 1e-6)
            qkv = F.linear(h, b["attn.in_proj.weight"], b["attn.in_proj.bias"]).view(B, N, H, 3 * D)   # per head [q|k|v]
            q, k, v = (t.transpose(1, 2) for t in qkv.split(D, dim=-1))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, W)
            x = x + F.linear(a, b["attn.out_proj.weight"], b["attn.out_proj.bias"])
            h = F.layer_norm(x, (W,), b["ln_2.weight"], b["ln_2.bias"], 1e-6)
            x = x + F.linear(F.gelu(F.linear(h, b["mlp.c_fc.weight"], b["mlp.c_fc.bias"])), b["mlp.c_proj.weight"],
                             b["mlp.c_proj.bias"])
        x = self._resample(x)
        x = F.layer_norm(x, (self.out_dim,), *self.ln_post, 1e-6)
        return x @ self.proj

    def encode_images(self, payloads: List[bytes], items=None) -> List[torch.Tensor]:
        out = self.forward(torch.stack([self.preprocess(p) for p in payloads]))
        return [out[i] for i in range(out.shape[0])]
