"""Qwen3-Omni "thinker": the Qwen3-VL-MoE language path (interleaved M-RoPE, deep-stack image features) with an
audio tower next to the vision tower.  The checkpoint nests everything under `thinker.` and the configuration under
`thinker_config`; the talker / code2wav speech synthesis parts are not loaded (text output only).

Audio tower: 128-bin log-mel frames are cut into windows of `2 * n_window` frames; every window goes through three
stride-2 3 x 3 convolutions (8 x fewer frames, 13 per 100), a linear map of the (channel, frequency) plane to
d_model and sinusoidal positions that restart in every window; the frames of a clip are then concatenated and run
through pre-norm transformer blocks whose attention is confined to blocks of `n_window_infer` input frames;
LayerNorm, Linear, GELU, Linear give embeddings of the language model's width.  Audio tokens take consecutive
rotary positions like text.

Reference: lightllm/models/qwen3_omni_moe_thinker/{model.py,qwen3_omni_audio.py,qwen3_omni_visual.py,
audio_process.py}.
"""
from __future__ import annotations

import math
import os
from typing import List

import numpy as np
import torch
import torch.nn.functional as F

from .qwen2_vl import Qwen3VLMoeLM, Qwen3VLTokenizer
from .registry import register_model
from .remap import RemapSource
from .vit.qwen3_vl_visual import Qwen3VLVisionTower

SAMPLE_RATE = 16000
HOP = 160
MIN_AUDIO_LEN = 480
MAX_AUDIO_SECONDS = int(os.environ.get("LIGHTLLM_MAX_AUDIO_DURATION_SECONDS", "3600"))   # longer clips are cut


def _after_conv(n: int) -> int:
    """Frames left of n after the three stride-2 convolutions (kernel 3, padding 1)."""
    for _ in range(3):
        n = (n - 1) // 2 + 1
    return n


def audio_token_num(num_samples: int, window: int = 100) -> int:
    """Embeddings of a clip of `num_samples` 16 kHz samples: 13 per full window of 100 mel frames plus the tail's."""
    frames = max(int(num_samples), MIN_AUDIO_LEN) // HOP
    full, tail = divmod(frames, window)
    return full * _after_conv(window) + (_after_conv(tail) if tail else 0)


@register_model("qwen3_omni_moe", is_multimodal=True)
class Qwen3OmniThinkerLM(Qwen3VLMoeLM):
    model_type = "qwen3_omni_moe"

    def _wrap_source(self, src):
        if any(n.startswith("thinker.") for n in src.names()):
            t = {n[len("thinker."):]: n for n in src.names() if n.startswith("thinker.model.") or
                 n.startswith("thinker.lm_head.")}
            src = RemapSource(src, t, passthrough=False)
        return super()._wrap_source(src)


class Qwen3OmniVisionTower(Qwen3VLVisionTower):
    """The Qwen3-VL tower under the thinker's tensor names (`merger.ln_q`, `merger.mlp.0/2`, `merger_list.j`)."""

    merger_keys = {"norm.weight": "ln_q.weight", "norm.bias": "ln_q.bias", "linear_fc1.weight": "mlp.0.weight",
                   "linear_fc1.bias": "mlp.0.bias", "linear_fc2.weight": "mlp.2.weight", "linear_fc2.bias": "mlp.2.bias"}
    deepstack_prefix = "merger_list."

    def __init__(self, vcfg, source, device, dtype=torch.bfloat16, prefix: str = None):
        if prefix is None:
            prefix = next((p for p in ("thinker.visual.", "visual.") if source.has(p + "patch_embed.proj.weight")),
                          "thinker.visual.")
        super().__init__(vcfg, source, device, dtype, prefix=prefix)

    @staticmethod
    def weight_shapes(vcfg: dict, prefix: str = "thinker.visual.") -> dict:
        out = {}
        for n, shp in Qwen3VLVisionTower.weight_shapes(vcfg, prefix).items():
            n = n.replace("deepstack_merger_list.", "merger_list.")
            if ".merger." in n or ".merger_list." in n:
                head, tail = n.rsplit(".", 2)[0], ".".join(n.rsplit(".", 2)[1:])
                n = head + "." + Qwen3OmniVisionTower.merger_keys.get(tail, tail)
            out[n] = shp
        return out


class Qwen3OmniAudioTower:
    def __init__(self, cfg: dict, source, device, dtype=torch.bfloat16, prefix: str = None):
        ac = cfg["audio_config"]
        self.d = ac["d_model"]
        self.heads = ac["encoder_attention_heads"]
        self.n_layers = ac.get("encoder_layers", ac.get("num_hidden_layers"))
        self.n_mels = ac.get("num_mel_bins", 128)
        self.window = 2 * int(ac.get("n_window", 50))
        self.infer_window = int(ac.get("n_window_infer", 800))
        self.max_pos = int(ac.get("max_source_positions", 1500))
        self.act = ac.get("activation_function", "gelu")
        self.device, self.dtype = device, dtype
        self._fe = None
        from .base import embed_row_width

        self.out_hidden = embed_row_width(cfg)   # row width of the shared arena (deep-stack columns included)
        if prefix is None:
            prefix = next((p for p in ("thinker.audio_tower.", "audio_tower.") if source.has(p + "conv2d1.weight")),
                          "thinker.audio_tower.")
        g = lambda n: source.get(prefix + n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        self.convs = [(g(f"conv2d{i}.weight"), g(f"conv2d{i}.bias")) for i in (1, 2, 3)]
        self.conv_out = g("conv_out.weight")
        self.blocks = []
        for i in range(self.n_layers):
            b = f"layers.{i}."
            self.blocks.append({k: g(b + k) for k in self._layer_names()})
        self.ln_post = (g("ln_post.weight"), g("ln_post.bias"))
        self.proj1 = (g("proj1.weight"), g("proj1.bias"))
        self.proj2 = (g("proj2.weight"), g("proj2.bias"))
        half = self.d // 2
        inc = math.log(10000.0) / (half - 1)
        inv = torch.exp(-inc * torch.arange(half).float())
        ang = torch.arange(self.max_pos).float()[:, None] * inv[None]
        self.pos = torch.cat([ang.sin(), ang.cos()], dim=1).to(device=device, dtype=dtype)

    @staticmethod
    def _layer_names():
        names = []
        for p in ("q_proj", "k_proj", "v_proj", "out_proj"):
            names += [f"self_attn.{p}.weight", f"self_attn.{p}.bias"]
        for p in ("self_attn_layer_norm", "final_layer_norm", "fc1", "fc2"):
            names += [f"{p}.weight", f"{p}.bias"]
        return names

    @staticmethod
    def weight_shapes(cfg: dict, prefix: str = "thinker.audio_tower.") -> dict:
        ac = cfg["audio_config"]
        d, f, c, mel = ac["d_model"], ac["encoder_ffn_dim"], ac["downsample_hidden_size"], ac.get("num_mel_bins", 128)
        fr = mel
        for _ in range(3):
            fr = (fr + 1) // 2
        s = {prefix + "conv2d1.weight": (c, 1, 3, 3), prefix + "conv2d1.bias": (c,),
             prefix + "conv2d2.weight": (c, c, 3, 3), prefix + "conv2d2.bias": (c,),
             prefix + "conv2d3.weight": (c, c, 3, 3), prefix + "conv2d3.bias": (c,),
             prefix + "conv_out.weight": (d, c * fr), prefix + "ln_post.weight": (d,), prefix + "ln_post.bias": (d,),
             prefix + "proj1.weight": (d, d), prefix + "proj1.bias": (d,),
             prefix + "proj2.weight": (ac["output_dim"], d), prefix + "proj2.bias": (ac["output_dim"],)}
        for i in range(ac.get("encoder_layers", ac.get("num_hidden_layers"))):
            b = f"{prefix}layers.{i}."
            for p in ("q_proj", "k_proj", "v_proj", "out_proj"):
                s[b + f"self_attn.{p}.weight"], s[b + f"self_attn.{p}.bias"] = (d, d), (d,)
            for p in ("self_attn_layer_norm", "final_layer_norm"):
                s[b + p + ".weight"], s[b + p + ".bias"] = (d,), (d,)
            s.update({b + "fc1.weight": (f, d), b + "fc1.bias": (f,), b + "fc2.weight": (d, f), b + "fc2.bias": (d,)})
        return s

    def log_mel(self, audio: np.ndarray) -> torch.Tensor:
        """[n_mels, len // 160] log-mel features of the clip itself (no padding to 30 s)."""
        if self._fe is None:
            from transformers import WhisperFeatureExtractor

            self._fe = WhisperFeatureExtractor(feature_size=self.n_mels)
        out = self._fe(audio, sampling_rate=SAMPLE_RATE, return_tensors="pt", padding="do_not_pad", truncation=False)
        return out.input_features[0][:, : audio.shape[0] // HOP]

    def token_num(self, num_samples: int) -> int:
        return audio_token_num(num_samples, self.window)

    @torch.no_grad()
    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [n_mels, frames] of one clip -> [tokens, output_dim]."""
        W = self.window
        chunks = list(mel.t().to(self.device, self.dtype).split(W, dim=0))
        lens = [c.shape[0] for c in chunks]
        x = torch.nn.utils.rnn.pad_sequence(chunks, batch_first=True).transpose(1, 2).unsqueeze(1)   # [n, 1, mel, W']
        for w, b in self.convs:
            x = F.gelu(F.conv2d(x, w, b, stride=2, padding=1))
        n, c, f, t = x.shape
        x = F.linear(x.permute(0, 3, 1, 2).reshape(n, t, c * f), self.conv_out) + self.pos[:t]
        after = [_after_conv(l) for l in lens]
        x = torch.cat([x[i, :a] for i, a in enumerate(after)], dim=0)                                # [tokens, d]
        total = x.shape[0]
        block = max(after) * max(self.infer_window // W, 1)
        D = self.d // self.heads
        for blk in self.blocks:
            h = F.layer_norm(x, (self.d,), blk["self_attn_layer_norm.weight"], blk["self_attn_layer_norm.bias"])
            q, k, v = (F.linear(h, blk[f"self_attn.{p}.weight"], blk[f"self_attn.{p}.bias"]).view(total, self.heads, D)
                       for p in ("q_proj", "k_proj", "v_proj"))
            outs = []
            for s0 in range(0, total, block):
                qs, ks, vs = (z[s0:s0 + block].transpose(0, 1).unsqueeze(0) for z in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qs, ks, vs).squeeze(0).transpose(0, 1))
            a = torch.cat(outs, dim=0).reshape(total, self.d)
            x = x + F.linear(a, blk["self_attn.out_proj.weight"], blk["self_attn.out_proj.bias"])
            h = F.layer_norm(x, (self.d,), blk["final_layer_norm.weight"], blk["final_layer_norm.bias"])
            x = x + F.linear(F.gelu(F.linear(h, blk["fc1.weight"], blk["fc1.bias"])), blk["fc2.weight"], blk["fc2.bias"])
        x = F.layer_norm(x, (self.d,), *self.ln_post)
        return F.linear(F.gelu(F.linear(x, *self.proj1)), *self.proj2)

    def encode_audio(self, audio: np.ndarray) -> torch.Tensor:
        audio = np.asarray(audio, dtype=np.float32)[: MAX_AUDIO_SECONDS * SAMPLE_RATE]
        if audio.shape[0] < MIN_AUDIO_LEN:
            audio = np.pad(audio, (0, MIN_AUDIO_LEN - audio.shape[0]))
        return self.forward(self.log_mel(audio))

    def encode_audios(self, clips: List[np.ndarray], items=None) -> List[torch.Tensor]:
        return [self.encode_audio(c) for c in clips]


class Qwen3OmniTokenizer(Qwen3VLTokenizer):
    """Image placeholders as Qwen3-VL; every `<|audio_pad|>` becomes the id run of the corresponding clip."""

    def __init__(self, tokenizer, model_cfg: dict):
        super().__init__(tokenizer, model_cfg)
        self.audio_pad_id = model_cfg.get("audio_token_id", 151675)
        self.audio_window = 2 * int((model_cfg.get("audio_config") or {}).get("n_window", 50))

    def init_audioitem_extral_params(self, audio, multi_params=None, sampling_params=None):
        pass

    def get_audio_token_length(self, audio) -> int:
        n = min(int(audio.audio_length), MAX_AUDIO_SECONDS * SAMPLE_RATE)
        return audio_token_num(n, self.audio_window)

    def encode(self, prompt, multimodal_params=None, add_special_tokens: bool = False, **kw):
        ids = super().encode(prompt, multimodal_params, add_special_tokens=add_special_tokens, **kw)
        audios = list(getattr(multimodal_params, "audios", None) or []) if multimodal_params is not None else []
        if not audios:
            return ids
        out, k = [], 0
        for t in ids:
            if t == self.audio_pad_id and k < len(audios):
                a = audios[k]
                out.extend(range(a.token_id, a.token_id + a.token_num))
                k += 1
            else:
                out.append(t)
        if k != len(audios):
            raise ValueError(f"the prompt has {k} audio placeholders for {len(audios)} clips")
        return out
