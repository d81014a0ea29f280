"""Multi-token-prediction draft modules (speculative decoding).

A draft module is one extra transformer layer of the target model's family that predicts the token after next:
its input at position i is `eh_proj([RMSNorm_e(embed(token i+1)) ; RMSNorm_h(target hidden i)])`, it runs one
decoder layer over its own KV layer (appended to the target model's pool, same slots and request table), and
`shared_head` (norm + the target's lm_head unless the checkpoint carries its own) gives the logits of token i+2.
Checkpoints keep the module under `model.layers.{num_hidden_layers + j}.`.

Qwen3.5 keeps its module under `mtp.` (`mtp.fc`, `mtp.pre_fc_norm_embedding`, `mtp.pre_fc_norm_hidden`,
`mtp.norm`, `mtp.layers.{j}.`): one full-attention layer of the hybrid stack, fed with the target's hidden state
after the target's final norm.

Reference: lightllm/models/deepseek_mtp, qwen3_moe_mtp, mistral_mtp, glm4_moe_lite_mtp, qwen3_5_mtp,
qwen3_5_moe_mtp (pre_layer_infer.py: the enorm / hnorm / eh_proj fusion; model.py: sharing of the memory and
request managers).
"""
from __future__ import annotations

import torch

from .. import ops
from .deepseek2 import DeepseekV2LM
from .deepseek_v32 import DeepseekV32LM
from .llama import LlamaLM
from .qwen3_moe import Qwen3MoeLM
from .qwen3_next import Qwen3_5LM, Qwen3_5MoeLM, Qwen3NextLM
from .remap import RemapSource


class MTPMixin:
    """Mixed into a family class; construct with share_with=<target model>, mtp_index=j."""

    def _read_config(self, c):
        super()._read_config(c)
        self.mtp_index = int(self.extra.get("mtp_index", 0))
        self.target_layers = self.num_layers
        self.num_layers = 1
        self.kv_layer_offset = self.target_layers + self.mtp_index

    def _module_prefix(self):
        return f"model.layers.{self.target_layers + self.mtp_index}."

    def weight_shapes(self):
        s = super().weight_shapes()
        H = self.hidden
        s.update({"model.layers.0.enorm.weight": (H,), "model.layers.0.hnorm.weight": (H,),
                  "model.layers.0.eh_proj.weight": (H, 2 * H), "model.layers.0.shared_head.norm.weight": (H,)})
        return s

    def _wrap_source(self, src):
        pre = self._module_prefix()
        t = {}
        for n in src.names():
            if n.startswith(pre):
                t["model.layers.0." + n[len(pre):]] = n
        t["model.norm.weight"] = pre + "shared_head.norm.weight"
        if src.has(pre + "embed_tokens.weight"):
            t["model.embed_tokens.weight"] = pre + "embed_tokens.weight"
        if src.has(pre + "shared_head.head.weight"):
            t["lm_head.weight"] = pre + "shared_head.head.weight"
        return RemapSource(src, t)

    def _load_weights(self, src):
        if not src.has("model.norm.weight"):      # random-init source: canonical names
            src = RemapSource(src, {"model.norm.weight": "model.layers.0.shared_head.norm.weight"})
        super()._load_weights(src)
        main = self.share_with
        if main is not None:                      # one copy of the big tables
            if self.embed_w.shape == main.embed_w.shape:
                self.embed_w, self.embed_range = main.embed_w, main.embed_range
            if self.lm_head_w.shape == main.lm_head_w.shape:
                self.lm_head_w = main.lm_head_w
        p = "model.layers.0."
        self.enorm_w = self._dev(src.get(p + "enorm.weight"))
        self.hnorm_w = self._dev(src.get(p + "hnorm.weight"))
        self.eh_proj_w = self._dev(src.get(p + "eh_proj.weight"))

    def _target_hidden(self, prev):
        return prev

    def _embed(self, ids, st):
        e = super()._embed(ids, st)
        prev = st.extra.get("draft_input_hidden")
        assert prev is not None and prev.shape[0] == e.shape[0], "a draft module needs the target's hidden states"
        prev = self._target_hidden(prev.to(e.dtype))
        off = self.norm_w_offset
        cat = torch.cat([ops.rmsnorm(e, self.enorm_w, self.eps, off), ops.rmsnorm(prev, self.hnorm_w, self.eps, off)],
                        dim=-1)
        return ops.gemm(cat, self.eh_proj_w)


class DeepseekV3MTP(MTPMixin, DeepseekV2LM):
    def _is_moe_layer(self, i):
        return self.moe is not None   # the module's layer follows the target's last (MoE) layer


class DeepseekV32MTP(MTPMixin, DeepseekV32LM):
    def _is_moe_layer(self, i):
        return self.moe is not None


class Qwen3MoeMTP(MTPMixin, Qwen3MoeLM):
    pass


class LlamaMTP(MTPMixin, LlamaLM):
    pass


class _Qwen3_5MTPMixin(MTPMixin):
    """The draft layer is a full-attention layer whatever the target's layer pattern; its KV layer follows the
    target's full-attention layers in the pool."""

    def _read_config(self, c):
        c = dict(c)
        n = c["num_hidden_layers"]
        interval = int(c.get("full_attention_interval", 4))
        types = c.get("layer_types") or ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
                                         for i in range(n)]
        n_full = sum(t == "full_attention" for t in types)
        c["layer_types"] = ["full_attention"] * n
        super()._read_config(c)
        self.layer_types, self.full_layers, self.lin_layers = ["full_attention"], [0], []
        self._kv_slot, self._lin_slot = {0: 0}, {}
        self.kv_layer_offset = n_full + self.mtp_index

    def _wrap_source(self, src):
        names = list(src.names())
        t = {}
        pre = f"mtp.layers.{self.mtp_index}."
        for n in names:
            if n.startswith(pre):
                t["model.layers.0." + n[len(pre):]] = n
        t.update({"model.layers.0.eh_proj.weight": "mtp.fc.weight",
                  "model.layers.0.enorm.weight": "mtp.pre_fc_norm_embedding.weight",
                  "model.layers.0.hnorm.weight": "mtp.pre_fc_norm_hidden.weight",
                  "model.norm.weight": "mtp.norm.weight"})
        for canon, tails in (("model.embed_tokens.weight", ("model.language_model.embed_tokens.weight",
                                                            "language_model.model.embed_tokens.weight",
                                                            "model.embed_tokens.weight")),
                             ("lm_head.weight", ("lm_head.weight", "language_model.lm_head.weight"))):
            for n in tails:
                if src.has(n):
                    t[canon] = n
                    break
        return Qwen3NextLM._wrap_source(self, RemapSource(src, t))

    def _target_hidden(self, prev):
        main = self.share_with
        return ops.rmsnorm(prev, main.final_norm_w, main.eps, main.norm_w_offset)


class Qwen3_5MTP(_Qwen3_5MTPMixin, Qwen3_5LM):
    pass


class Qwen3_5MoeMTP(_Qwen3_5MTPMixin, Qwen3_5MoeLM):
    pass


MTP_CLASSES = {"deepseek_v3": DeepseekV3MTP, "deepseek_v2": DeepseekV3MTP, "glm4_moe_lite": DeepseekV3MTP,
               "kimi_k2": DeepseekV3MTP, "deepseek_v32": DeepseekV32MTP, "qwen3_moe": Qwen3MoeMTP, "mistral": LlamaMTP, "llama": LlamaMTP,
               "qwen3_5": Qwen3_5MTP, "qwen3_5_text": Qwen3_5MTP, "qwen3_5_moe": Qwen3_5MoeMTP,
               "qwen3_5_moe_text": Qwen3_5MoeMTP}


def build_mtp_modules(main, n_modules: int, model_dir=None, weight_source=None, **kw):
    """Draft modules 0..n-1 of `main` (which must have been built with extra_kv_layers >= n)."""
    cls = MTP_CLASSES.get(main.config.get("model_type"))
    if cls is None:
        raise ValueError(f"no multi-token-prediction module for model_type {main.config.get('model_type')!r}")
    assert main.extra_kv_layers >= n_modules, "build the target model with extra_kv_layers = number of draft modules"
    extra = {k: v for k, v in main.extra.items() if k != "mtp_index"}
    return [cls(main.config, model_dir=model_dir, weight_source=weight_source, pstate=main.ps,
                data_type=str(main.dtype).replace("torch.", ""), max_req_num=main.max_req_num,
                max_seq_length=main.max_seq_length, batch_max_tokens=main.batch_max_tokens, disable_cudagraph=True,
                share_with=main, mtp_index=j, random_seed=1000 + j, **{**extra, **kw}) for j in range(n_modules)]
