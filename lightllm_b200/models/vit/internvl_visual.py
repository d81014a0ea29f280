"""InternViT vision tower + InternVL projector (`internvl_chat` checkpoints: `vision_model.*`, `mlp1.*`).

Every image is cut into 448 x 448 tiles on the aspect-ratio grid closest to the picture (at most `max_num` tiles,
plus a thumbnail of the whole picture when there is more than one tile); a tile goes through the ViT (class token +
patch embedding + learned positions, pre-norm blocks with layer scale, LayerNorm or RMSNorm, optional q/k
RMSNorm), the class token is dropped, the 32 x 32 patch grid is folded 2 x 2 into the channel dimension ("pixel
shuffle", 256 tokens per tile) and mapped to the language model's width by LayerNorm -> Linear -> GELU -> Linear.
Runs in the visual server on torch ops.

Reference: lightllm/models/internvl/internvl_visual.py, lightllm/models/internvl/img_process.py (tile grid),
lightllm/models/vit/model.py (the tensor-parallel InternViT).
"""
from __future__ import annotations

import math
from io import BytesIO
from typing import List

import numpy as np
import torch
import torch.nn.functional as F

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


def closest_grid(width: int, height: int, max_num: int = 6, image_size: int = 448):
    """(columns, rows) of the tile grid: about ceil(area / tile area) tiles (one fewer / one more also tried, never
    above `max_num`), aspect ratio closest to the picture's in log space."""
    log_ratio = math.log(width / height)
    multiple = min(math.ceil(width * height / (image_size * image_size)), max_num)
    if multiple <= 1:
        return 1, 1
    best, best_err = (1, 1), float("inf")
    for n in (multiple - 1, multiple, multiple + 1):
        if n > max_num or n < 1:
            continue
        for m in range(1, n + 1):
            if n % m == 0:
                err = abs(log_ratio - math.log(m / (n // m)))
                if err < best_err:
                    best, best_err = (m, n // m), err
    return best


def num_tiles(width: int, height: int, max_num: int = 6, image_size: int = 448, use_thumbnail: bool = True) -> int:
    c, r = closest_grid(width, height, max_num, image_size)
    n = c * r
    return n + 1 if (use_thumbnail and n != 1) else n


def tile_image(data: bytes, max_num: int = 6, image_size: int = 448, use_thumbnail: bool = True) -> torch.Tensor:
    """Image bytes -> [tiles, 3, S, S], ImageNet-normalised (bicubic resize to the grid, row-major tiles, thumbnail
    last)."""
    from PIL import Image

    with Image.open(BytesIO(data)) as im:
        im = im.convert("RGB")
        c, r = closest_grid(im.size[0], im.size[1], max_num, image_size)
        big = im.resize((c * image_size, r * image_size), Image.BICUBIC)
        tiles = [big.crop((i % c * image_size, i // c * image_size, (i % c + 1) * image_size, (i // c + 1) * image_size))
                 for i in range(c * r)]
        if use_thumbnail and len(tiles) != 1:
            tiles.append(im.resize((image_size, image_size), Image.BICUBIC))
        arr = np.stack([np.asarray(t, dtype=np.float32) / 255.0 for t in tiles])
    x = torch.from_numpy(arr).permute(0, 3, 1, 2)
    return (x - torch.tensor(IMAGENET_MEAN).view(1, 3, 1, 1)) / torch.tensor(IMAGENET_STD).view(1, 3, 1, 1)


def pixel_shuffle(x: torch.Tensor, scale: float = 0.5) -> torch.Tensor:
    """[N, W, H, C] -> [N, W*s, H*s, C/s^2] (the v2 ordering of the released checkpoints)."""
    n, w, h, c = x.shape
    x = x.reshape(n, w, int(h * scale), int(c / scale))
    x = x.permute(0, 2, 1, 3).contiguous()
    x = x.reshape(n, int(h * scale), int(w * scale), int(c / (scale * scale)))
    return x.permute(0, 2, 1, 3).contiguous()


class InternVLVisionTower:
    def __init__(self, cfg: dict, source, device, dtype=torch.bfloat16):
        vc = cfg["vision_config"]
        self.hidden = vc["hidden_size"]
        self.heads = vc["num_attention_heads"]
        self.layers = vc["num_hidden_layers"]
        self.patch = vc.get("patch_size", 14)
        self.image_size = vc.get("image_size", cfg.get("force_image_size") or 448)
        self.eps = vc.get("layer_norm_eps", 1e-6)
        self.norm_type = vc.get("norm_type", "layer_norm")
        self.qk_norm = bool(vc.get("qk_normalization", False))
        self.act = vc.get("hidden_act", "gelu")
        self.scale = float(cfg.get("downsample_ratio", 0.5))
        self.select_layer = int(cfg.get("select_layer", -1))
        self.max_num = int(cfg.get("max_dynamic_patch", 12))
        self.use_thumbnail = bool(cfg.get("use_thumbnail", True))
        self.device, self.dtype = device, dtype
        g = lambda n: source.get(n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        v = "vision_model."
        self.cls = g(v + "embeddings.class_embedding").reshape(1, 1, -1)
        self.patch_w = g(v + "embeddings.patch_embedding.weight").reshape(self.hidden, -1)
        self.patch_b = g(v + "embeddings.patch_embedding.bias")
        self.pos = g(v + "embeddings.position_embedding").reshape(-1, self.hidden)
        n_run = self.layers + 1 + self.select_layer if self.select_layer < 0 else self.select_layer
        self.blocks = []
        for i in range(n_run):
            b = f"{v}encoder.layers.{i}."
            names = ["attn.qkv.weight", "attn.proj.weight", "attn.proj.bias", "ls1", "ls2", "norm1.weight",
                     "norm2.weight", "mlp.fc1.weight", "mlp.fc1.bias", "mlp.fc2.weight", "mlp.fc2.bias"]
            if source.has(b + "attn.qkv.bias"):
                names.append("attn.qkv.bias")
            if self.norm_type == "layer_norm":
                names += ["norm1.bias", "norm2.bias"]
            if self.qk_norm:
                names += ["attn.q_norm.weight", "attn.k_norm.weight"]
            self.blocks.append({k: g(b + k) for k in names})
        self.mlp1 = {k: g("mlp1." + k) for k in ("0.weight", "0.bias", "1.weight", "1.bias", "3.weight", "3.bias")}
        self.tokens_per_tile = int((self.image_size // self.patch) ** 2 * self.scale * self.scale)

    @staticmethod
    def weight_shapes(cfg: dict) -> dict:
        vc = cfg["vision_config"]
        H, I, L = vc["hidden_size"], vc["intermediate_size"], vc["num_hidden_layers"]
        p = vc.get("patch_size", 14)
        size = vc.get("image_size", 448)
        out = (cfg.get("llm_config") or cfg)["hidden_size"]
        s = {"vision_model.embeddings.class_embedding": (1, 1, H),
             "vision_model.embeddings.patch_embedding.weight": (H, 3, p, p),
             "vision_model.embeddings.patch_embedding.bias": (H,),
             "vision_model.embeddings.position_embedding": (1, (size // p) ** 2 + 1, H)}
        ln = vc.get("norm_type", "layer_norm") == "layer_norm"
        for i in range(L):
            b = f"vision_model.encoder.layers.{i}."
            s.update({b + "attn.qkv.weight": (3 * H, H), b + "attn.proj.weight": (H, H), b + "attn.proj.bias": (H,),
                      b + "ls1": (H,), b + "ls2": (H,), b + "norm1.weight": (H,), b + "norm2.weight": (H,),
                      b + "mlp.fc1.weight": (I, H), b + "mlp.fc1.bias": (I,), b + "mlp.fc2.weight": (H, I),
                      b + "mlp.fc2.bias": (H,)})
            if vc.get("qkv_bias", True):
                s[b + "attn.qkv.bias"] = (3 * H,)
            if ln:
                s[b + "norm1.bias"] = (H,)
                s[b + "norm2.bias"] = (H,)
            if vc.get("qk_normalization", False):
                s[b + "attn.q_norm.weight"] = (H,)
                s[b + "attn.k_norm.weight"] = (H,)
        c4 = int(H / (float(cfg.get("downsample_ratio", 0.5)) ** 2))
        s.update({"mlp1.0.weight": (c4,), "mlp1.0.bias": (c4,), "mlp1.1.weight": (out, c4), "mlp1.1.bias": (out,),
                  "mlp1.3.weight": (out, out), "mlp1.3.bias": (out,)})
        return s

    def _norm(self, x, w, b):
        if self.norm_type == "layer_norm":
            return F.layer_norm(x, (x.shape[-1],), w, b, self.eps)
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * w

    def _rms(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * w

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [tiles, 3, S, S] -> [tiles, tokens_per_tile, llm hidden]."""
        B = pixels.shape[0]
        p = self.patch
        x = pixels.to(self.device, self.dtype)
        g = x.shape[-1] // p
        x = x.view(B, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B, g * g, 3 * p * p)
        x = F.linear(x, self.patch_w, self.patch_b)
        x = torch.cat([self.cls.expand(B, 1, -1), x], dim=1) + self.pos[: g * g + 1]
        D = self.hidden // self.heads
        for b in self.blocks:
            h = self._norm(x, b["norm1.weight"], b.get("norm1.bias"))
            qkv = F.linear(h, b["attn.qkv.weight"], b.get("attn.qkv.bias"))
            q, k, v = qkv.split(self.hidden, dim=-1)
            if self.qk_norm:  # RMSNorm over the whole hidden width, before the split into heads
                q, k = self._rms(q, b["attn.q_norm.weight"]), self._rms(k, b["attn.k_norm.weight"])
            q, k, v = (t.view(B, -1, self.heads, D).transpose(1, 2) for t in (q, k, v))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, -1, self.hidden)
            x = x + F.linear(a, b["attn.proj.weight"], b["attn.proj.bias"]) * b["ls1"]
            h = self._norm(x, b["norm2.weight"], b.get("norm2.bias"))
            h = F.linear(F.gelu(F.linear(h, b["mlp.fc1.weight"], b["mlp.fc1.bias"])), b["mlp.fc2.weight"], b["mlp.fc2.bias"])
            x = x + h * b["ls2"]
        x = x[:, 1:]
        x = pixel_shuffle(x.reshape(B, g, g, self.hidden), self.scale).reshape(B, -1, int(self.hidden / self.scale ** 2))
        m = self.mlp1
        x = F.layer_norm(x, (x.shape[-1],), m["0.weight"], m["0.bias"], 1e-5)
        x = F.gelu(F.linear(x, m["1.weight"], m["1.bias"]))
        return F.linear(x, m["3.weight"], m["3.bias"])

    def encode_images(self, payloads: List[bytes], items=None) -> List[torch.Tensor]:
        """One [tiles * tokens_per_tile, hidden] tensor per image; an item's `image_patch_max_num` caps its grid."""
        def cap(i):
            ep = (items[i].get("extra_params") or {}) if items else {}
            return int(ep.get("image_patch_max_num", self.max_num)) or 1

        tiles = [tile_image(p, cap(i), self.image_size, self.use_thumbnail) for i, p in enumerate(payloads)]
        out = self.forward(torch.cat(tiles, dim=0))
        res, k = [], 0
        for t in tiles:
            res.append(out[k:k + t.shape[0]].reshape(-1, out.shape[-1]))
            k += t.shape[0]
        return res
