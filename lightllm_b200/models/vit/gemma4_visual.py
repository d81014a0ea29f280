"""Gemma-4 vision tower and its projection into the language model.

A picture is resized (aspect ratio kept) to the largest size whose 16 x 16 patches number at most
`max_soft_tokens * pooling_kernel_size^2` with both sides multiples of `pooling_kernel_size * patch_size`; pixels
are scaled to [-1, 1]; every patch is a row, with its (x, y) grid position.  Patch rows go through a linear
embedding plus two learned position tables (one per axis, added), pre / post-norm encoder blocks (q, k RMS-normed
with scale, v without, attention scale 1, rotary embedding with the first half of a head turning with x and the
second half with y, optional clipping of linear inputs / outputs), are averaged over k x k neighbourhoods by grid
position and multiplied by sqrt(width); then an unscaled RMSNorm and a projection to the language model's width.
Runs in the visual server on torch ops, one picture at a time (no padding patches are needed then).

Reference: lightllm/models/gemma4/gemma4_visual.py.
"""
from __future__ import annotations

import math
from io import BytesIO
from typing import List, Tuple

import numpy as np
import torch
import torch.nn.functional as F


def target_size(height: int, width: int, patch: int, max_patches: int, k: int) -> Tuple[int, int]:
    factor = math.sqrt(max_patches * patch * patch / (height * width))
    side = k * patch
    th = int(math.floor(factor * height / side)) * side
    tw = int(math.floor(factor * width / side)) * side
    longest = (max_patches // (k * k)) * side
    if th == 0 and tw == 0:
        raise ValueError("the picture cannot be resized to a whole number of pooled patches")
    if th == 0:
        th, tw = side, min(int(math.floor(width / height)) * side, longest)
    elif tw == 0:
        tw, th = side, min(int(math.floor(height / width)) * side, longest)
    return th, tw


def soft_token_num(width: int, height: int, patch: int = 16, max_soft_tokens: int = 280, k: int = 3) -> int:
    th, tw = target_size(height, width, patch, max_soft_tokens * k * k, k)
    return (th // patch) * (tw // patch) // (k * k)


def _rms(x, w, eps):
    xf = x.float()
    y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    return (y * w.float() if w is not None else y).to(x.dtype)


def _rot(x, cos, sin):
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos[..., :h] - x2 * sin[..., :h], x2 * cos[..., h:] + x1 * sin[..., h:]], dim=-1)


class Gemma4VisionTower:
    def __init__(self, cfg: dict, source, device, dtype=torch.bfloat16):
        vc = cfg["vision_config"]
        self.hidden = vc["hidden_size"]
        self.layers_n = vc["num_hidden_layers"]
        self.heads = vc["num_attention_heads"]
        self.kv_heads = vc.get("num_key_value_heads", self.heads)
        self.head_dim = vc.get("head_dim", self.hidden // self.heads)
        self.patch = vc.get("patch_size", 16)
        self.k = vc.get("pooling_kernel_size", 3)
        self.eps = vc.get("rms_norm_eps", 1e-6)
        self.clip = bool(vc.get("use_clipped_linears", False))
        self.standardize = bool(vc.get("standardize", False))
        self.theta = float((vc.get("rope_parameters") or {}).get("rope_theta", 100.0))
        self.max_soft_tokens = int(cfg.get("max_soft_tokens", 280))
        self.device, self.dtype = device, dtype
        pre = next(p for p in ("model.vision_tower.", "vision_tower.") if source.has(p + "patch_embedder.input_proj.weight"))
        emb = pre.replace("vision_tower.", "embed_vision.")
        g = lambda n: source.get(n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        self.in_w = g(pre + "patch_embedder.input_proj.weight")
        self.pos_table = g(pre + "patch_embedder.position_embedding_table")          # [2, P, hidden]
        self.blocks = []
        for i in range(self.layers_n):
            b = f"{pre}encoder.layers.{i}."
            blk = {}
            for name in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
                         "mlp.up_proj", "mlp.down_proj"):
                blk[name] = g(b + name + ".linear.weight")
                if self.clip:
                    blk[name + ".clip"] = tuple(float(source.get(b + name + "." + c)) for c in
                                                ("input_min", "input_max", "output_min", "output_max"))
            for name in ("self_attn.q_norm", "self_attn.k_norm", "input_layernorm", "post_attention_layernorm",
                         "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                blk[name] = g(b + name + ".weight")
            self.blocks.append(blk)
        if self.standardize:
            self.std_bias, self.std_scale = g(pre + "std_bias"), g(pre + "std_scale")
        self.proj_w = g(emb + "embedding_projection.weight")
        self.out_hidden = self.proj_w.shape[0]
        d = self.head_dim // 2
        self.inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d)).to(device)

    def _lin(self, blk, name, x):
        if self.clip:
            lo, hi, olo, ohi = blk[name + ".clip"]
            return F.linear(x.clamp(lo, hi), blk[name]).clamp(olo, ohi)
        return F.linear(x, blk[name])

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """One picture: patches [N, 3 * patch^2] in [0, 1], pos [N, 2] (x, y) -> [N / k^2, language-model width]."""
        N, H, D = patches.shape[0], self.heads, self.head_dim
        pos = pos.to(self.device).long()
        x = F.linear((2 * (patches.to(self.device, torch.float32) - 0.5)).to(self.dtype), self.in_w)
        x = x + self.pos_table[0][pos[:, 0]] + self.pos_table[1][pos[:, 1]]
        ang = [pos[:, a].float()[:, None] * self.inv_freq[None, :] for a in (0, 1)]
        emb = torch.cat([torch.cat([a, a], dim=-1) for a in ang], dim=-1)             # [N, D]: x half, then y half
        cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
        half = D // 2

        def rope(t):   # each half of a head is rotated on its own with that axis' angles
            tf = t.float()
            a = _rot(tf[..., :half], cos[..., :half], sin[..., :half])
            b = _rot(tf[..., half:], cos[..., half:], sin[..., half:])
            return torch.cat([a, b], dim=-1).to(t.dtype)

        for blk in self.blocks:
            h = _rms(x, blk["input_layernorm"], self.eps)
            q = _rms(self._lin(blk, "self_attn.q_proj", h).view(N, H, D), blk["self_attn.q_norm"], self.eps)
            k = _rms(self._lin(blk, "self_attn.k_proj", h).view(N, self.kv_heads, D), blk["self_attn.k_norm"], self.eps)
            v = _rms(self._lin(blk, "self_attn.v_proj", h).view(N, self.kv_heads, D), None, self.eps)
            q, k = rope(q), rope(k)
            if self.kv_heads != H:
                k = k.repeat_interleave(H // self.kv_heads, dim=1)
                v = v.repeat_interleave(H // self.kv_heads, dim=1)
            a = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                               v.transpose(0, 1).unsqueeze(0), scale=1.0)
            a = a.squeeze(0).transpose(0, 1).reshape(N, H * D)
            x = x + _rms(self._lin(blk, "self_attn.o_proj", a), blk["post_attention_layernorm"], self.eps)
            h = _rms(x, blk["pre_feedforward_layernorm"], self.eps)
            m = F.gelu(self._lin(blk, "mlp.gate_proj", h), approximate="tanh") * self._lin(blk, "mlp.up_proj", h)
            x = x + _rms(self._lin(blk, "mlp.down_proj", m), blk["post_feedforward_layernorm"], self.eps)
        k2 = self.k * self.k
        if k2 > 1:   # average over k x k neighbourhoods, in row-major order of the pooled grid
            gw = int(pos[:, 0].max().item()) + 1
            cell = (pos[:, 0] // self.k) + (gw // self.k) * (pos[:, 1] // self.k)
            pooled = torch.zeros((N // k2, x.shape[1]), dtype=torch.float32, device=self.device)
            pooled.index_add_(0, cell, x.float() / k2)
            x = pooled.to(self.dtype)
        x = x * self.hidden ** 0.5
        if self.standardize:
            x = (x - self.std_bias) * self.std_scale
        return F.linear(_rms(x, None, self.eps), self.proj_w)

    def preprocess(self, data: bytes):
        from PIL import Image

        with Image.open(BytesIO(data)) as im:
            im = im.convert("RGB")
            th, tw = target_size(im.height, im.width, self.patch, self.max_soft_tokens * self.k * self.k, self.k)
            if (th, tw) != (im.height, im.width):
                im = im.resize((tw, th), Image.BICUBIC)
            arr = np.asarray(im, dtype=np.float32) / 255.0                          # [H, W, 3]
        return self.patchify(torch.from_numpy(arr).permute(2, 0, 1))

    def patchify(self, img: torch.Tensor):
        """img [3, H, W] -> (patches [N, patch * patch * 3] with channels innermost, positions [N, 2] as (x, y))."""
        p = self.patch
        c, Hh, Ww = img.shape
        gh, gw = Hh // p, Ww // p
        x = img.reshape(c, gh, p, gw, p).permute(1, 3, 2, 4, 0).reshape(gh * gw, p * p * c)
        ys, xs = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
        return x, torch.stack([xs.reshape(-1), ys.reshape(-1)], dim=-1)

    def encode_images(self, payloads: List[bytes], items=None) -> List[torch.Tensor]:
        return [self.forward(*self.preprocess(p)) for p in payloads]
