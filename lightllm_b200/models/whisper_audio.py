"""Whisper audio encoder + projector for speech-capable chat models (`audio_model.encoder.*`, `mlp2.*` in the
checkpoint).  A clip is 16 kHz mono; clips longer than 30 s are cut into 30 s chunks, shorter than 480 samples are
zero padded.  Per chunk: log-mel features of the 30 s window truncated to the chunk's own frames -> two GELU
convolutions (the second with stride 2) -> learned positions -> pre-norm transformer blocks -> average pooling of
neighbouring frames -> LayerNorm -> projector (LayerNorm, Linear, GELU, Linear).  One embedding per 40 ms.
Runs in the audio server on torch ops.

Reference: lightllm/models/whisper/whisper_audio.py, lightllm/models/whisper/modeling_whisper.py (WhisperEncoder
with its average pooler), token count in lightllm/models/internvl/model.py (get_audio_token_length).
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch
import torch.nn.functional as F

SAMPLE_RATE = 16000
MAX_SAMPLES = 30 * SAMPLE_RATE
MIN_AUDIO_LEN = 480
HOP = 160


def frames_after_cnn(mel_frames: int) -> int:
    """Length after the two convolutions (kernel 3, padding 1, strides 1 and 2)."""
    n = mel_frames  # stride 1 keeps the length
    return 1 + (n + 2 - 2 - 1) // 2


def chunk_lengths(num_samples: int) -> List[int]:
    """Sample counts of the 30 s chunks of a clip (each at least MIN_AUDIO_LEN)."""
    if num_samples <= MAX_SAMPLES:
        return [max(num_samples, MIN_AUDIO_LEN)]
    out, start = [], 0
    while start < num_samples:
        end = min(start + MAX_SAMPLES, num_samples)
        out.append(max(end - start, MIN_AUDIO_LEN))
        start = end
    return out


def audio_token_num(num_samples: int) -> int:
    """Embeddings a clip of `num_samples` samples produces (what the prompt must reserve)."""
    total = 0
    for n in chunk_lengths(num_samples):
        total += (frames_after_cnn(n // HOP) - 2) // 2 + 1
    return int(total)


class WhisperAudioTower:
    def __init__(self, cfg: dict, source, device, dtype=torch.bfloat16):
        ac = cfg["audio_config"]
        self.d = ac["d_model"]
        self.heads = ac["encoder_attention_heads"]
        self.layers = ac["encoder_layers"]
        self.n_mels = ac.get("num_mel_bins", 80)
        self.max_pos = ac.get("max_source_positions", 1500)
        self.scale_embedding = bool(ac.get("scale_embedding", False))
        self.device, self.dtype = device, dtype
        g = lambda n: source.get(n).to(device=device, dtype=dtype).contiguous()  # noqa: E731
        a = "audio_model.encoder."
        self.conv1 = (g(a + "conv1.weight"), g(a + "conv1.bias"))
        self.conv2 = (g(a + "conv2.weight"), g(a + "conv2.bias"))
        self.pos = g(a + "embed_positions.weight")
        self.blocks = []
        for i in range(self.layers):
            b = f"{a}layers.{i}."
            self.blocks.append({k: g(b + k) for k in (
                "self_attn_layer_norm.weight", "self_attn_layer_norm.bias", "self_attn.q_proj.weight",
                "self_attn.q_proj.bias", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.v_proj.bias",
                "self_attn.out_proj.weight", "self_attn.out_proj.bias", "final_layer_norm.weight",
                "final_layer_norm.bias", "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias")})
        self.ln = (g(a + "layer_norm.weight"), g(a + "layer_norm.bias"))
        self.mlp2 = {k: g("mlp2." + k) for k in ("0.weight", "0.bias", "1.weight", "1.bias", "3.weight", "3.bias")}
        self.out_hidden = self.mlp2["3.weight"].shape[0]
        self._fe = None

    @staticmethod
    def weight_shapes(cfg: dict) -> dict:
        ac = cfg["audio_config"]
        d, f, L = ac["d_model"], ac["encoder_ffn_dim"], ac["encoder_layers"]
        out = (cfg.get("llm_config") or cfg)["hidden_size"]
        a = "audio_model.encoder."
        s = {a + "conv1.weight": (d, ac.get("num_mel_bins", 80), 3), a + "conv1.bias": (d,),
             a + "conv2.weight": (d, d, 3), a + "conv2.bias": (d,),
             a + "embed_positions.weight": (ac.get("max_source_positions", 1500), d),
             a + "layer_norm.weight": (d,), a + "layer_norm.bias": (d,)}
        for i in range(L):
            b = f"{a}layers.{i}."
            for n in ("self_attn_layer_norm", "final_layer_norm"):
                s[b + n + ".weight"], s[b + n + ".bias"] = (d,), (d,)
            for n in ("q_proj", "v_proj", "out_proj"):
                s[b + f"self_attn.{n}.weight"], s[b + f"self_attn.{n}.bias"] = (d, d), (d,)
            s[b + "self_attn.k_proj.weight"] = (d, d)
            s.update({b + "fc1.weight": (f, d), b + "fc1.bias": (f,), b + "fc2.weight": (d, f), b + "fc2.bias": (d,)})
        s.update({"mlp2.0.weight": (d,), "mlp2.0.bias": (d,), "mlp2.1.weight": (out, d), "mlp2.1.bias": (out,),
                  "mlp2.3.weight": (out, out), "mlp2.3.bias": (out,)})
        return s

    def log_mel(self, audio: np.ndarray) -> torch.Tensor:
        """[n_mels, 3000] log-mel features of the clip padded to 30 s (Whisper's feature extractor)."""
        if self._fe is None:
            from transformers import WhisperFeatureExtractor

            self._fe = WhisperFeatureExtractor(feature_size=self.n_mels)
        return self._fe(audio, sampling_rate=SAMPLE_RATE, return_tensors="pt").input_features[0]

    @torch.no_grad()
    def encode_features(self, mel: torch.Tensor, pool: bool = True) -> torch.Tensor:
        """mel [n_mels, frames] -> encoder output [frames / 2 (/ 2 when pooled), d_model] after the final norm."""
        x = mel.to(self.device, self.dtype).unsqueeze(0)
        x = F.gelu(F.conv1d(x, *self.conv1, padding=1))
        x = F.gelu(F.conv1d(x, *self.conv2, stride=2, padding=1))
        x = x.permute(0, 2, 1)
        n = x.shape[1]
        x = x * (self.d ** 0.5 if self.scale_embedding else 1.0) + self.pos[:n]
        D = self.d // self.heads
        for b in self.blocks:
            h = F.layer_norm(x, (self.d,), b["self_attn_layer_norm.weight"], b["self_attn_layer_norm.bias"])
            q = F.linear(h, b["self_attn.q_proj.weight"], b["self_attn.q_proj.bias"])
            k = F.linear(h, b["self_attn.k_proj.weight"])
            v = F.linear(h, b["self_attn.v_proj.weight"], b["self_attn.v_proj.bias"])
            q, k, v = (t.view(1, n, self.heads, D).transpose(1, 2) for t in (q, k, v))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(1, n, self.d)
            x = x + F.linear(a, b["self_attn.out_proj.weight"], b["self_attn.out_proj.bias"])
            h = F.layer_norm(x, (self.d,), b["final_layer_norm.weight"], b["final_layer_norm.bias"])
            x = x + F.linear(F.gelu(F.linear(h, b["fc1.weight"], b["fc1.bias"])), b["fc2.weight"], b["fc2.bias"])
        if pool:
            x = F.avg_pool1d(x.permute(0, 2, 1), 2, stride=2).permute(0, 2, 1)
        return F.layer_norm(x, (self.d,), *self.ln)[0]

    @torch.no_grad()
    def project(self, x: torch.Tensor) -> torch.Tensor:
        m = self.mlp2
        x = F.layer_norm(x, (x.shape[-1],), m["0.weight"], m["0.bias"])
        x = F.gelu(F.linear(x, m["1.weight"], m["1.bias"]))
        return F.linear(x, m["3.weight"], m["3.bias"])

    def encode_audio(self, audio: np.ndarray) -> torch.Tensor:
        """16 kHz mono float32 samples -> [audio_token_num(len), llm hidden]."""
        audio = np.asarray(audio, dtype=np.float32)
        if audio.shape[0] < MIN_AUDIO_LEN:
            audio = np.pad(audio, (0, MIN_AUDIO_LEN - audio.shape[0]))
        outs, start = [], 0
        while start < audio.shape[0]:
            chunk = audio[start:start + MAX_SAMPLES]
            if chunk.shape[0] < MIN_AUDIO_LEN:
                chunk = np.pad(chunk, (0, MIN_AUDIO_LEN - chunk.shape[0]))
            after = frames_after_cnn(chunk.shape[0] // HOP)
            mel = self.log_mel(chunk)[:, : 2 * after]
            tokens = (after - 2) // 2 + 1
            if tokens > 0:
                outs.append(self.project(self.encode_features(mel))[:tokens])
            start += MAX_SAMPLES
        return torch.cat(outs, dim=0)

    def encode_audios(self, clips: List[np.ndarray], items=None) -> List[torch.Tensor]:
        return [self.encode_audio(c) for c in clips]
