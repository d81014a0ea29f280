"""SigLIP vision tower + Gemma-3 projector.  A picture is resized to the tower's square input (896 x 896 for the
released models), cut into 14 x 14 patches, embedded with learned positions (no class token) and run through
pre-norm transformer blocks (LayerNorm, biased attention, GELU-tanh MLP) and a final LayerNorm; the projector
average-pools the patch grid down to mm_tokens_per_image (256) positions, applies a zero-centred RMSNorm and
multiplies by the projection matrix.  Runs in the visual server on torch ops.
Reference: lightllm/models/gemma3/gemma3_visual.py.
"""
from __future__ import annotations

from io import BytesIO
from typing import List

import numpy as np
import torch
import torch.nn.functional as F


class SiglipGemma3Tower:
    def __init__(self, cfg: dict, source, device, dtype=torch.bfloat16):
        vc = cfg["vision_config"]
        self.hidden = vc["hidden_size"]
        self.heads = vc["num_attention_heads"]
        self.layers = vc["num_hidden_layers"]
        self.patch = vc.get("patch_size", 14)
        self.image_size = vc.get("image_size", 896)
        self.eps = vc.get("layer_norm_eps", 1e-6)
        self.tokens = int(cfg.get("mm_tokens_per_image", 256))
        self.out_hidden = (cfg.get("text_config") or cfg)["hidden_size"]
        self.device, self.dtype = device, dtype
        vp = next(p for p in ("model.vision_tower.vision_model.", "vision_tower.vision_model.")
                  if source.has(p + "embeddings.patch_embedding.weight"))
        pp = next(p for p in ("model.multi_modal_projector.", "multi_modal_projector.")
                  if source.has(p + "mm_input_projection_weight"))
        g = lambda n: source.get(n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        self.patch_w = g(vp + "embeddings.patch_embedding.weight").reshape(self.hidden, -1)
        self.patch_b = g(vp + "embeddings.patch_embedding.bias")
        self.pos = g(vp + "embeddings.position_embedding.weight")
        self.blocks = []
        for i in range(self.layers):
            b = f"{vp}encoder.layers.{i}."
            self.blocks.append({k: g(b + k) for k in (
                "layer_norm1.weight", "layer_norm1.bias", "self_attn.q_proj.weight", "self_attn.q_proj.bias",
                "self_attn.k_proj.weight", "self_attn.k_proj.bias", "self_attn.v_proj.weight", "self_attn.v_proj.bias",
                "self_attn.out_proj.weight", "self_attn.out_proj.bias", "layer_norm2.weight", "layer_norm2.bias",
                "mlp.fc1.weight", "mlp.fc1.bias", "mlp.fc2.weight", "mlp.fc2.bias")})
        self.post_ln = (g(vp + "post_layernorm.weight"), g(vp + "post_layernorm.bias"))
        self.proj_w = g(pp + "mm_input_projection_weight")
        self.soft_norm_w = g(pp + "mm_soft_emb_norm.weight")

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [B, 3, S, S] -> [B, mm_tokens_per_image, llm hidden]."""
        B = pixels.shape[0]
        p = self.patch
        x = pixels.to(self.device, self.dtype)
        g = x.shape[-1] // p
        x = x.view(B, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B, g * g, 3 * p * p)
        x = F.linear(x, self.patch_w, self.patch_b) + self.pos[: g * g]
        D = self.hidden // self.heads
        for b in self.blocks:
            h = F.layer_norm(x, (self.hidden,), b["layer_norm1.weight"], b["layer_norm1.bias"], self.eps)
            q, k, v = (F.linear(h, b[f"self_attn.{n}_proj.weight"], b[f"self_attn.{n}_proj.bias"])
                       .view(B, -1, self.heads, D).transpose(1, 2) for n in "qkv")
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, -1, self.hidden)
            x = x + F.linear(a, b["self_attn.out_proj.weight"], b["self_attn.out_proj.bias"])
            h = F.layer_norm(x, (self.hidden,), b["layer_norm2.weight"], b["layer_norm2.bias"], self.eps)
            h = F.gelu(F.linear(h, b["mlp.fc1.weight"], b["mlp.fc1.bias"]), approximate="tanh")
            x = x + F.linear(h, b["mlp.fc2.weight"], b["mlp.fc2.bias"])
        x = F.layer_norm(x, (self.hidden,), *self.post_ln, self.eps)
        side = int(round(self.tokens ** 0.5))
        kernel = g // side
        x = F.avg_pool2d(x.transpose(1, 2).reshape(B, self.hidden, g, g), kernel, stride=kernel)
        x = x.flatten(2).transpose(1, 2)
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * (1.0 + self.soft_norm_w.float())
        return torch.matmul(xf.to(self.dtype), self.proj_w)

    def preprocess(self, data: bytes) -> torch.Tensor:
        from PIL import Image

        with Image.open(BytesIO(data)) as im:
            im = im.convert("RGB").resize((self.image_size, self.image_size), Image.BILINEAR)
            arr = np.asarray(im, dtype=np.float32) / 255.0
        return (torch.from_numpy(arr).permute(2, 0, 1) - 0.5) / 0.5

    def encode_images(self, payloads: List[bytes], items=None) -> List[torch.Tensor]:
        return list(self.forward(torch.stack([self.preprocess(p) for p in payloads])))
