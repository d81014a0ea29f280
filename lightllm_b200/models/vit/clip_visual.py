"""CLIP ViT vision tower + LLaVA projector: class token + patch embedding + learned positions, pre-LayerNorm,
pre-norm transformer blocks (LayerNorm, biased multi-head attention, QuickGELU MLP); LLaVA takes the hidden
states of the second-to-last layer without the class token and maps them to the language model's width with
Linear -> GELU -> Linear.  Every image gives (image_size / patch)^2 tokens.  Runs in the visual server on torch ops.
Reference: lightllm/models/llava/llava_visual.py.
"""
from __future__ import annotations

from io import BytesIO
from typing import List

import numpy as np
import torch
import torch.nn.functional as F

from .qwen2_vl_visual import CLIP_MEAN, CLIP_STD


def clip_preprocess(data: bytes, size: int) -> torch.Tensor:
    """Shortest side to `size` (bicubic), centre crop, CLIP normalisation -> [3, size, size]."""
    from PIL import Image

    with Image.open(BytesIO(data)) as im:
        im = im.convert("RGB")
        w, h = im.size
        s = size / min(w, h)
        im = im.resize((max(size, round(w * s)), max(size, round(h * s))), Image.BICUBIC)
        w, h = im.size
        l, t = (w - size) // 2, (h - size) // 2
        im = im.crop((l, t, l + size, t + size))
        arr = np.asarray(im, dtype=np.float32) / 255.0
    x = torch.from_numpy(arr).permute(2, 0, 1)
    return (x - torch.tensor(CLIP_MEAN).view(3, 1, 1)) / torch.tensor(CLIP_STD).view(3, 1, 1)


class ClipLlavaTower:
    def __init__(self, cfg: dict, source, device, dtype=torch.bfloat16):
        vc = cfg["vision_config"]
        self.hidden = vc["hidden_size"]
        self.heads = vc["num_attention_heads"]
        self.layers = vc["num_hidden_layers"]
        self.patch = vc.get("patch_size", 14)
        self.image_size = vc.get("image_size", 336)
        self.eps = vc.get("layer_norm_eps", 1e-5)
        self.act = vc.get("hidden_act", "quick_gelu")
        self.feature_layer = cfg.get("vision_feature_layer", -2)
        self.drop_cls = cfg.get("vision_feature_select_strategy", "default") == "default"
        self.out_hidden = (cfg.get("text_config") or cfg)["hidden_size"]
        self.device, self.dtype = device, dtype
        vp = next(p for p in ("model.vision_tower.vision_model.", "vision_tower.vision_model.")
                  if source.has(p + "embeddings.class_embedding"))
        pp = next(p for p in ("model.multi_modal_projector.", "multi_modal_projector.") if source.has(p + "linear_1.weight"))
        g = lambda n: source.get(n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        self.cls = g(vp + "embeddings.class_embedding")
        self.patch_w = g(vp + "embeddings.patch_embedding.weight").reshape(self.hidden, -1)
        self.pos = g(vp + "embeddings.position_embedding.weight")
        self.pre_ln = (g(vp + "pre_layrnorm.weight"), g(vp + "pre_layrnorm.bias"))
        n_run = self.layers + 1 + self.feature_layer if self.feature_layer < 0 else self.feature_layer
        self.blocks = []
        for i in range(n_run):  # layers after the feature layer are never needed
            b = f"{vp}encoder.layers.{i}."
            self.blocks.append({k: g(b + k) for k in (
                "layer_norm1.weight", "layer_norm1.bias", "self_attn.q_proj.weight", "self_attn.q_proj.bias",
                "self_attn.k_proj.weight", "self_attn.k_proj.bias", "self_attn.v_proj.weight", "self_attn.v_proj.bias",
                "self_attn.out_proj.weight", "self_attn.out_proj.bias", "layer_norm2.weight", "layer_norm2.bias",
                "mlp.fc1.weight", "mlp.fc1.bias", "mlp.fc2.weight", "mlp.fc2.bias")})
        self.proj = {k: g(pp + k) for k in ("linear_1.weight", "linear_1.bias", "linear_2.weight", "linear_2.bias")}

    @property
    def tokens_per_image(self) -> int:
        n = (self.image_size // self.patch) ** 2
        return n if self.drop_cls else n + 1

    def _act(self, x):
        return x * torch.sigmoid(1.702 * x) if self.act == "quick_gelu" else F.gelu(x)

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [B, 3, S, S] -> [B, tokens_per_image, out_hidden]."""
        B = pixels.shape[0]
        p = self.patch
        x = pixels.to(self.device, self.dtype)
        g = x.shape[-1] // p
        x = x.view(B, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B, g * g, 3 * p * p)
        x = F.linear(x, self.patch_w)
        x = torch.cat([self.cls.view(1, 1, -1).expand(B, 1, -1), x], dim=1) + self.pos[: g * g + 1]
        x = F.layer_norm(x, (self.hidden,), *self.pre_ln, self.eps)
        D = self.hidden // self.heads
        for b in self.blocks:
            h = F.layer_norm(x, (self.hidden,), b["layer_norm1.weight"], b["layer_norm1.bias"], self.eps)
            q, k, v = (F.linear(h, b[f"self_attn.{n}_proj.weight"], b[f"self_attn.{n}_proj.bias"])
                       .view(B, -1, self.heads, D).transpose(1, 2) for n in "qkv")
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, -1, self.hidden)
            x = x + F.linear(a, b["self_attn.out_proj.weight"], b["self_attn.out_proj.bias"])
            h = F.layer_norm(x, (self.hidden,), b["layer_norm2.weight"], b["layer_norm2.bias"], self.eps)
            x = x + F.linear(self._act(F.linear(h, b["mlp.fc1.weight"], b["mlp.fc1.bias"])), b["mlp.fc2.weight"],
                             b["mlp.fc2.bias"])
        if self.drop_cls:
            x = x[:, 1:]
        x = F.gelu(F.linear(x, self.proj["linear_1.weight"], self.proj["linear_1.bias"]))
        return F.linear(x, self.proj["linear_2.weight"], self.proj["linear_2.bias"])

    def encode_images(self, payloads: List[bytes], items=None) -> List[torch.Tensor]:
        px = torch.stack([clip_preprocess(p, self.image_size) for p in payloads])
        return list(self.forward(px))
