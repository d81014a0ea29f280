"""Qwen3-VL vision tower.  Differences from the Qwen2-VL tower (`qwen2_vl_visual.py`): the patch embedding has a bias
and 16 x 16 patches, a learned position table (a square grid, bilinearly interpolated to the image's patch grid) is
added before the blocks, the MLP is plain fc1 -> GELU(tanh) -> fc2, the merger normalises before the 2 x 2 fold,
and the hidden states after a few chosen blocks go through mergers of their own ("deep-stack" features) that the
language model adds to the image positions after its first decoder layers.  One output row per merged patch:
[merged embedding | deep-stack feature 0 | deep-stack feature 1 | ...].

Reference: lightllm/models/qwen3_vl/qwen3_visual.py.
"""
from __future__ import annotations

from io import BytesIO
from typing import List, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .qwen2_vl_visual import _rotate_half, grid_rotary, patchify, smart_resize


def interpolate_positions(table: torch.Tensor, grids, merge: int) -> torch.Tensor:
    """Rows of the learned position table for every patch of every image: bilinear interpolation of the square
    table to the (h, w) patch grid, repeated over frames, in merge-window order (the order `patchify` emits)."""
    side = int(round(table.shape[0] ** 0.5))
    out = []
    for t, h, w in grids:
        hi, wi = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
        h0, w0 = hi.long(), wi.long()
        h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
        dh, dw = (hi - h0).to(table.dtype).to(table.device), (wi - w0).to(table.dtype).to(table.device)
        idx = lambda a, b: (a[:, None] * side + b[None, :]).reshape(-1).to(table.device)  # noqa: E731
        wgt = lambda a, b: (a[:, None] * b[None, :]).reshape(-1, 1)  # noqa: E731
        pe = (table[idx(h0, w0)] * wgt(1 - dh, 1 - dw) + table[idx(h0, w1)] * wgt(1 - dh, dw)
              + table[idx(h1, w0)] * wgt(dh, 1 - dw) + table[idx(h1, w1)] * wgt(dh, dw))
        pe = pe.repeat(t, 1).view(t, h // merge, merge, w // merge, merge, -1).permute(0, 1, 3, 2, 4, 5)
        out.append(pe.reshape(t * h * w, -1))
    return torch.cat(out, dim=0)


class Qwen3VLVisionTower:
    image_mean = (0.5, 0.5, 0.5)
    image_std = (0.5, 0.5, 0.5)
    merger_keys: dict = {}                          # canonical merger tensor name -> name in the checkpoint
    deepstack_prefix = "deepstack_merger_list."

    def __init__(self, vcfg: dict, source, device, dtype=torch.bfloat16, prefix: str = None):
        self.cfg = vcfg
        self.embed = vcfg["hidden_size"]
        self.depth = vcfg["depth"]
        self.heads = vcfg["num_heads"]
        self.head_dim = self.embed // self.heads
        self.patch = vcfg.get("patch_size", 16)
        self.merge = vcfg.get("spatial_merge_size", 2)
        self.temporal = vcfg.get("temporal_patch_size", 2)
        self.llm_hidden = vcfg["out_hidden_size"]
        self.deepstack = list(vcfg.get("deepstack_visual_indexes") or [])
        self.out_hidden = self.llm_hidden * (1 + len(self.deepstack))  # row width in the embedding arena
        self.act = vcfg.get("hidden_act", "gelu_pytorch_tanh")
        self.device, self.dtype = device, dtype
        if prefix is None:
            prefix = next(p for p in ("model.visual.", "visual.") if source.has(p + "patch_embed.proj.weight"))
        g = lambda n: source.get(prefix + n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        self.patch_w = g("patch_embed.proj.weight").reshape(self.embed, -1)
        self.patch_b = g("patch_embed.proj.bias")
        self.pos_table = g("pos_embed.weight")
        self.blocks = []
        for i in range(self.depth):
            b = f"blocks.{i}."
            self.blocks.append({k: g(b + k) for k in (
                "norm1.weight", "norm1.bias", "attn.qkv.weight", "attn.qkv.bias", "attn.proj.weight", "attn.proj.bias",
                "norm2.weight", "norm2.bias", "mlp.linear_fc1.weight", "mlp.linear_fc1.bias", "mlp.linear_fc2.weight",
                "mlp.linear_fc2.bias")})
        names = ("norm.weight", "norm.bias", "linear_fc1.weight", "linear_fc1.bias", "linear_fc2.weight", "linear_fc2.bias")
        ck = self.merger_keys
        self.merger = {k: g("merger." + ck.get(k, k)) for k in names}
        self.ds_mergers = [{k: g(f"{self.deepstack_prefix}{j}." + ck.get(k, k)) for k in names}
                           for j in range(len(self.deepstack))]

    @staticmethod
    def weight_shapes(vcfg: dict, prefix: str = "model.visual.") -> dict:
        E, I = vcfg["hidden_size"], vcfg["intermediate_size"]
        p, t, m = vcfg.get("patch_size", 16), vcfg.get("temporal_patch_size", 2), vcfg.get("spatial_merge_size", 2)
        s = {prefix + "patch_embed.proj.weight": (E, 3, t, p, p), prefix + "patch_embed.proj.bias": (E,),
             prefix + "pos_embed.weight": (vcfg.get("num_position_embeddings", 2304), E)}
        for i in range(vcfg["depth"]):
            b = f"{prefix}blocks.{i}."
            s.update({b + "norm1.weight": (E,), b + "norm1.bias": (E,), b + "norm2.weight": (E,), b + "norm2.bias": (E,),
                      b + "attn.qkv.weight": (3 * E, E), b + "attn.qkv.bias": (3 * E,), b + "attn.proj.weight": (E, E),
                      b + "attn.proj.bias": (E,), b + "mlp.linear_fc1.weight": (I, E), b + "mlp.linear_fc1.bias": (I,),
                      b + "mlp.linear_fc2.weight": (E, I), b + "mlp.linear_fc2.bias": (E,)})
        M = E * m * m

        def merger(pre, post_norm):
            n = M if post_norm else E
            return {pre + "norm.weight": (n,), pre + "norm.bias": (n,), pre + "linear_fc1.weight": (M, M),
                    pre + "linear_fc1.bias": (M,), pre + "linear_fc2.weight": (vcfg["out_hidden_size"], M),
                    pre + "linear_fc2.bias": (vcfg["out_hidden_size"],)}

        s.update(merger(prefix + "merger.", False))
        for j in range(len(vcfg.get("deepstack_visual_indexes") or [])):
            s.update(merger(f"{prefix}deepstack_merger_list.{j}.", True))
        return s

    def _merge(self, x, m, post_norm: bool):
        M = self.embed * self.merge ** 2
        if post_norm:
            x = F.layer_norm(x.view(-1, M), (M,), m["norm.weight"], m["norm.bias"], 1e-6)
        else:
            x = F.layer_norm(x, (self.embed,), m["norm.weight"], m["norm.bias"], 1e-6).view(-1, M)
        x = F.gelu(F.linear(x, m["linear_fc1.weight"], m["linear_fc1.bias"]))
        return F.linear(x, m["linear_fc2.weight"], m["linear_fc2.bias"])

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grids: List[Tuple[int, int, int]]) -> torch.Tensor:
        """patches [N, 3*temporal*patch*patch] of all images -> [N / merge^2, llm hidden * (1 + deep-stack sets)]."""
        x = F.linear(patches.to(self.device, self.dtype), self.patch_w, self.patch_b)
        x = x + interpolate_positions(self.pos_table, grids, self.merge)
        cos, sin = grid_rotary(grids, self.head_dim, self.merge)
        cos, sin = cos.to(self.device)[:, None, :], sin.to(self.device)[:, None, :]
        lens = [h * w for t, h, w in grids for _ in range(t)]
        N = x.shape[0]
        feats = []
        for li, b in enumerate(self.blocks):
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
            h = F.linear(h, b["mlp.linear_fc1.weight"], b["mlp.linear_fc1.bias"])
            h = F.gelu(h, approximate="tanh") if self.act in ("gelu_pytorch_tanh", "gelu_tanh") else F.gelu(h)
            x = x + F.linear(h, b["mlp.linear_fc2.weight"], b["mlp.linear_fc2.bias"])
            if li in self.deepstack:
                feats.append(self._merge(x, self.ds_mergers[self.deepstack.index(li)], True))
        return torch.cat([self._merge(x, self.merger, False)] + feats, dim=1)

    def preprocess(self, data: bytes, **resize_kw):
        from PIL import Image

        with Image.open(BytesIO(data)) as im:
            im = im.convert("RGB")
            h, w = smart_resize(im.height, im.width, self.patch * self.merge, **resize_kw)
            im = im.resize((w, h), Image.BICUBIC)
            arr = np.asarray(im, dtype=np.float32) / 255.0
        x = torch.from_numpy(arr).permute(2, 0, 1)
        x = (x - torch.tensor(self.image_mean).view(3, 1, 1)) / torch.tensor(self.image_std).view(3, 1, 1)
        return patchify(x.unsqueeze(0), self.patch, self.merge, self.temporal)

    def encode_images(self, payloads: List[bytes], items=None) -> List[torch.Tensor]:
        pre = [self.preprocess(p) for p in payloads]
        out = self.forward(torch.cat([x for x, _ in pre], dim=0), [g for _, g in pre])
        res, k = [], 0
        for _, (t, gh, gw) in pre:
            n = t * gh * gw // (self.merge ** 2)
            res.append(out[k:k + n])
            k += n
        return res
