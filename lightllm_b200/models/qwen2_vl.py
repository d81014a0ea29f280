"""Qwen2-VL / Qwen2.5-VL language model: Qwen2 decoder with multimodal rotary embedding (M-RoPE).  The rotary
frequency slots are split in three sections (temporal, height, width); text tokens advance all three together,
the tokens of an image take the (t, row, column) of their merged patch, and the text after an image continues
from the largest index used so far.  Image embeddings come from the shared arena (the vision tower runs in the
visual server).
Reference: lightllm/models/qwen2_vl/{model.py,infer_struct.py,triton_kernel/mrope.py,get_mrope_position_ids.py}.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch

from .llama import LlamaLM, Qwen2LM, Qwen3LM
from .registry import register_model
from .remap import RemapSource


def mrope_positions(ids: np.ndarray, items: List[dict], merge: int = 2) -> Tuple[np.ndarray, int]:
    """[3, len(ids)] rotary positions and the offset (next position - len(ids)) for the decode steps.
    `items`: image dicts with token_id / token_num / grid_thwd = (t, gh, gw, merge) in prompt order."""
    n = len(ids)
    pos = np.zeros((3, n), dtype=np.int64)
    spans = []
    for it in items:
        t0, cnt = it.get("token_id"), it.get("token_num")
        if t0 is None:
            continue
        hit = np.nonzero((ids >= t0) & (ids < t0 + cnt))[0]
        if hit.size:
            spans.append((int(hit[0]), int(hit[-1]) + 1, it))
    spans.sort(key=lambda s: s[0])
    cur, nxt = 0, 0  # token cursor, next free position
    for s, e, it in spans:
        if s > cur:  # text run
            pos[:, cur:s] = nxt + np.arange(s - cur)
            nxt += s - cur
        g = it.get("grid_thwd") or (1, 1, e - s, 1)
        t, gh, gw = int(g[0]), int(g[1]) // merge, int(g[2]) // merge
        if t * gh * gw != e - s:  # a chunk boundary cut the image: positions of the part present
            t, gh, gw = 1, 1, e - s
        tt = np.repeat(np.arange(t), gh * gw)
        hh = np.tile(np.repeat(np.arange(gh), gw), t)
        ww = np.tile(np.arange(gw), t * gh)
        pos[0, s:e], pos[1, s:e], pos[2, s:e] = nxt + tt, nxt + hh, nxt + ww
        nxt += max(t, gh, gw)
        cur = e
    if cur < n:
        pos[:, cur:] = nxt + np.arange(n - cur)
        nxt += n - cur
    return pos, nxt - n


class MRopeMixin:
    """Multimodal rotary embedding on top of a decoder class: per-token (t, row, column) positions, one of which
    drives every rotary frequency slot."""

    needs_prompt_ids = True  # the backend hands every prefill pass the request's whole prompt (M-RoPE is global)
    mrope_interleaved = False  # False: slots in three contiguous sections; True: t / h / w slots alternate

    def _read_config(self, c):
        super()._read_config(c)
        rs = c.get("rope_scaling") or c.get("rope_parameters") or {}
        sec = rs.get("mrope_section") or [16, 24, 24]
        self.mrope_section = [int(x) for x in sec]
        assert sum(self.mrope_section) == self.rot_dim // 2, "mrope_section must cover the rotary half"
        self.mrope_interleaved = bool(rs.get("mrope_interleaved", self.mrope_interleaved))
        self.rope_scaling = None  # "mrope" is not a frequency scaling
        vc = c.get("vision_config") or {}
        self.merge = int(vc.get("spatial_merge_size", 2))

    def _wrap_source(self, src):
        if src.has("model.embed_tokens.weight"):
            return src
        t = {}
        for pre in ("model.language_model.", "language_model.model."):
            if src.has(pre + "embed_tokens.weight"):
                for n in src.names():
                    if n.startswith(pre):
                        t["model." + n[len(pre):]] = n
        return RemapSource(src, t) if t else src

    def _init_rope(self):
        super()._init_rope()
        half = self.rot_dim // 2
        if self.mrope_interleaved:  # slot i belongs to h (i % 3 == 1) or w (i % 3 == 2) while that axis has slots left
            i = torch.arange(half)
            sec = torch.zeros(half, dtype=torch.long)
            sec[(i % 3 == 1) & (i < 3 * self.mrope_section[1])] = 1
            sec[(i % 3 == 2) & (i < 3 * self.mrope_section[2])] = 2
        else:
            sec = torch.repeat_interleave(torch.arange(3), torch.tensor(self.mrope_section))
        self._section_of_slot = sec.to(self.device)          # [half] -> 0 / 1 / 2
        self._slot = torch.arange(half, device=self.device)

    def _prepare_prefill_state(self, st):
        mm = st.extra.get("multimodal_params") or []
        q_len, ready, req_idx = st.extra["q_len_cpu"], st.extra["ready_cpu"], st.extra["req_idx_cpu"]
        ids = st.extra["input_ids_cpu"].numpy()
        B = st.batch_size
        cols, off = [], 0
        deltas = np.zeros(B, dtype=np.int32)
        for b in range(B):
            n, r = int(q_len[b]), int(ready[b])
            params = mm[b] if b < len(mm) and mm[b] else {}
            images = params.get("images", [])
            if images:
                full = params.get("_prompt_ids")
                if full is None:
                    assert r == 0, "chunked prefill of a multimodal request needs the whole prompt (_prompt_ids)"
                    full = ids[off:off + n]
                p3, delta = mrope_positions(np.asarray(full), images, self.merge)
                cols.append(p3[:, r:r + n])
                deltas[b] = delta
            else:
                cols.append(np.broadcast_to(np.arange(r, r + n), (3, n)))
            off += n
        pos3 = torch.from_numpy(np.ascontiguousarray(np.concatenate(cols, axis=1))).to(self.device)
        self.req_manager.req_to_position_delta[req_idx.long().to(self.device)] = torch.from_numpy(deltas).to(self.device)
        p = pos3[self._section_of_slot].t()                   # [T, half]: the position each frequency slot uses
        st.extra["rope"] = (self.cos[p, self._slot].contiguous(), self.sin[p, self._slot].contiguous(),
                            torch.arange(pos3.shape[1], dtype=torch.int32, device=self.device))

    def _prepare_decode_state(self, st):
        st.position_ids = st.position_ids + self.req_manager.req_to_position_delta[st.b_req_idx.long()]
        st.extra.pop("rope", None)

    def _rope_inputs(self, st, layer):
        r = st.extra.get("rope")
        return r if r is not None else (self.cos, self.sin, st.position_ids)


@register_model("qwen2_vl", "qwen2_5_vl", is_multimodal=True)
class Qwen2VLLM(MRopeMixin, Qwen2LM):
    model_type = "qwen2_vl"


class Qwen2VLTokenizer:
    """Wraps the text tokenizer: every `<|image_pad|>` of the prompt becomes the run of virtual token ids of the
    corresponding image (the embed cache assigned them), so that equal images give equal prompt ids.
    Reference: lightllm/server/tokenizer.py (QWen2VLTokenizer), models/qwen2_vl/vision_process.py."""

    def __init__(self, tokenizer, model_cfg: dict):
        self.tokenizer = tokenizer
        vc = model_cfg.get("vision_config") or {}
        self.patch = int(vc.get("patch_size", 14))
        self.merge = int(vc.get("spatial_merge_size", 2))
        tc = model_cfg.get("text_config") or {}
        self.image_pad_id = model_cfg.get("image_token_id", tc.get("image_token_id",
                                                                   model_cfg.get("image_token_index", 151655)))
        self.min_pixels = int(model_cfg.get("min_pixels", 56 * 56))
        self.max_pixels = int(model_cfg.get("max_pixels", 14 * 14 * 4 * 1280))

    def __getattr__(self, name):
        return getattr(self.tokenizer, name)

    def init_imageitem_extral_params(self, img, multi_params=None, sampling_params=None):
        pass

    def get_image_token_length(self, img) -> int:
        from .vit.qwen2_vl_visual import image_token_num

        n, (t, gh, gw) = image_token_num(img.image_w, img.image_h, self.patch, self.merge, min_pixels=self.min_pixels,
                                         max_pixels=self.max_pixels)
        img.grid_thwd = (t, gh, gw, self.merge)
        return n

    def encode(self, prompt, multimodal_params=None, add_special_tokens: bool = False, **kw):
        ids = list(prompt) if isinstance(prompt, (list, tuple)) else \
            list(self.tokenizer.encode(prompt, add_special_tokens=add_special_tokens))
        images = list(multimodal_params.images) if multimodal_params is not None else []
        if not images:
            return ids
        out, k = [], 0
        for t in ids:
            if t == self.image_pad_id and k < len(images):
                im = images[k]
                out.extend(range(im.token_id, im.token_id + im.token_num))
                k += 1
            else:
                out.append(t)
        if k != len(images):
            raise ValueError(f"the prompt has {k} image placeholders for {len(images)} images")
        return out


@register_model("qwen3_vl", is_multimodal=True)
class Qwen3VLLM(MRopeMixin, Qwen3LM):
    """Qwen3-VL language model: Qwen3 decoder (q/k RMSNorm), M-RoPE with interleaved t / h / w frequency slots, and
    deep-stack: the vision tower's extra feature sets are added to the image positions of the residual stream after
    the first decoder layers.  Reference: lightllm/models/qwen3_vl/."""

    model_type = "qwen3_vl"
    mrope_interleaved = True

    def _read_config(self, c):
        super()._read_config(c)
        vc = c.get("vision_config") or {}
        self.n_deepstack = len(vc.get("deepstack_visual_indexes") or [])
        self.embed_row_width = self.hidden * (1 + self.n_deepstack)

    def _merge_multimodal(self, h, st):
        """Arena rows are [embedding | deep-stack sets]: the embedding replaces the placeholder rows, the rest is
        kept for `_after_layer`."""
        st.extra.pop("deepstack", None)
        mm = st.extra.get("multimodal_params")
        if not st.is_prefill or not mm or self.embed_arena is None or self.n_deepstack == 0:
            return super()._merge_multimodal(h, st)
        ids = st.extra["input_ids_cpu"]
        pos_all, rows_all, seen = [], [], set()
        for params in mm:
            # audio rows carry zeros in the deep-stack columns
            for it in list((params or {}).get("images", [])) + list((params or {}).get("audios", [])):
                t0, n = it.get("token_id"), it.get("token_num")
                if t0 is None or (t0, n) in seen:
                    continue
                seen.add((t0, n))
                hit = ((ids >= t0) & (ids < t0 + n)).nonzero(as_tuple=True)[0]
                if hit.numel():
                    pos_all.append(hit)
                    rows_all.append(ids[hit] - t0 + it["start_index_in_embed_cache"])
        if not pos_all:
            return h
        pos, rows = torch.cat(pos_all).to(h.device), torch.cat(rows_all)
        emb = self.embed_arena.read_rows(rows).to(device=h.device, dtype=h.dtype)
        h[pos] = emb[:, : self.hidden]
        st.extra["deepstack"] = (pos, emb[:, self.hidden:])
        return h

    def _after_layer(self, i, residual, h, st):
        ds = st.extra.get("deepstack")
        if ds is None or i >= self.n_deepstack:
            return h
        pos, feats = ds
        residual[pos] += feats[:, i * self.hidden:(i + 1) * self.hidden]
        if i + 1 < self.num_layers:
            from .. import ops

            return ops.rmsnorm(residual, self.layers[i + 1].in_norm, self.eps, self.norm_w_offset)
        return h


class Qwen3VLTokenizer(Qwen2VLTokenizer):
    """Same placeholder expansion as Qwen2-VL with 16 x 16 patches (factor 32) and Qwen3-VL's pixel budget."""

    def __init__(self, tokenizer, model_cfg: dict):
        super().__init__(tokenizer, model_cfg)
        vc = model_cfg.get("vision_config") or {}
        self.patch = int(vc.get("patch_size", 16))
        self.min_pixels = int(model_cfg.get("min_pixels", 64 * 32 * 32 // 16))
        self.max_pixels = int(model_cfg.get("max_pixels", 16384 * 32 * 32 // 16))


def _qwen3_vl_moe_class():
    from .qwen3_moe import Qwen3MoeLM
    from .remap import FusedExperts

    class Qwen3VLMoeLM(Qwen3VLLM, Qwen3MoeLM):
        """Qwen3-VL-MoE: the Qwen3-VL language path on the Qwen3-MoE decoder; the checkpoint stores every layer's
        experts as two 3-D tensors (`experts.gate_up_proj`, `experts.down_proj`).  Reference: lightllm/models/
        qwen3_vl_moe/."""

        model_type = "qwen3_vl_moe"

        def _wrap_source(self, src):
            src = super()._wrap_source(src)
            if not src.has("model.layers.0.mlp.experts.gate_up_proj") and not any(
                    n.endswith("mlp.experts.gate_up_proj") for n in src.names()):
                return src
            t = {n: n for n in src.names()}
            E, I, H = self.moe.num_experts, self.moe.inter, self.hidden
            cache = FusedExperts()
            for n in list(src.names()):
                if n.endswith("mlp.experts.gate_up_proj"):
                    p = n[: -len("gate_up_proj")]
                    for e in range(E):
                        t[f"{p}{e}.gate_proj.weight"] = cache.entry(n, e, 2 * I, 0, I)
                        t[f"{p}{e}.up_proj.weight"] = cache.entry(n, e, 2 * I, I, 2 * I)
                    t.pop(n)
                elif n.endswith("mlp.experts.down_proj"):
                    p = n[: -len("down_proj")]
                    for e in range(E):
                        t[f"{p}{e}.down_proj.weight"] = cache.entry(n, e, H)
                    t.pop(n)
            return RemapSource(src, t)

    return Qwen3VLMoeLM


Qwen3VLMoeLM = register_model("qwen3_vl_moe", is_multimodal=True)(_qwen3_vl_moe_class())


def _has_vision(cfg: dict) -> bool:
    return bool(cfg.get("vision_config"))


def _qwen3_5_vl_classes():
    from .qwen3_next import Qwen3_5LM, Qwen3_5MoeLM

    class Qwen3_5VLLM(MRopeMixin, Qwen3_5LM):
        """Qwen3.5 with its vision tower: the hybrid decoder with interleaved M-RoPE over the rotary quarter of the
        full-attention heads; the tower is Qwen3-VL's without deep-stack outputs.  Reference: lightllm/models/
        qwen3_5/model.py."""

        model_type = "qwen3_5"
        mrope_interleaved = True

        def _wrap_source(self, src):
            return Qwen3_5LM._wrap_source(self, src)

    class Qwen3_5MoeVLLM(MRopeMixin, Qwen3_5MoeLM):
        """Qwen3.5-MoE with its vision tower.  Reference: lightllm/models/qwen3_5_moe/model.py."""

        model_type = "qwen3_5_moe"
        mrope_interleaved = True

        def _wrap_source(self, src):
            return Qwen3_5MoeLM._wrap_source(self, src)

    return Qwen3_5VLLM, Qwen3_5MoeVLLM


Qwen3_5VLLM, Qwen3_5MoeVLLM = _qwen3_5_vl_classes()
register_model("qwen3_5", condition=_has_vision, is_multimodal=True)(Qwen3_5VLLM)
register_model("qwen3_5_moe", condition=_has_vision, is_multimodal=True)(Qwen3_5MoeVLLM)


def is_tarsier2(cfg: dict) -> bool:
    """A `llava` wrapper config around the Qwen2-VL vision tower (Tarsier2), whatever its decoder."""
    if cfg.get("model_type") != "llava":
        return False
    vc = cfg.get("vision_config") or {}
    return (cfg.get("text_config") or {}).get("model_type") == "qwen2_vl" or vc.get("model_type") == "qwen2_vl" or \
        ("spatial_merge_size" in vc and "embed_dim" in vc)


def _text_type_is(kind: str, tarsier: bool = False):
    return lambda cfg: (cfg.get("text_config") or {}).get("model_type") == kind and (not tarsier or is_tarsier2(cfg))


@register_model("llava", condition=_text_type_is("qwen2_vl"), is_multimodal=True)
class Tarsier2Qwen2VLLM(Qwen2VLLM):
    """Tarsier2: a `llava` wrapper config whose `text_config` is a Qwen2-VL decoder and whose `vision_tower.*`
    tensors are the Qwen2-VL tower; the language model sits under `language_model.`.
    Reference: lightllm/models/tarsier2/model.py (Tarsier2Qwen2VLTpPartModel), tarsier2_visual.py."""

    model_type = "llava"

    def _wrap_source(self, src):
        if src.has("model.embed_tokens.weight"):
            return src
        t = {}
        for n in src.names():
            if n.startswith("language_model.model."):
                t["model." + n[len("language_model.model."):]] = n
            elif n.startswith("language_model.lm_head."):
                t["lm_head." + n[len("language_model.lm_head."):]] = n
        return RemapSource(src, t) if t else src


def _language_model_tensors(src):
    from .llava import LlavaLM

    return LlavaLM._wrap_source(None, src)


@register_model("llava", condition=_text_type_is("qwen2", tarsier=True), is_multimodal=True)
class Tarsier2Qwen2LM(Qwen2LM):
    """Tarsier2 over a plain Qwen2 decoder (sequential positions): the Qwen2-VL tower's embeddings stand in for the
    picture's run of token ids.  Reference: lightllm/models/tarsier2/model.py (Tarsier2Qwen2TpPartModel)."""

    model_type = "llava"

    def _wrap_source(self, src):
        return _language_model_tensors(src)


@register_model("llava", condition=_text_type_is("llama", tarsier=True), is_multimodal=True)
class Tarsier2LlamaLM(LlamaLM):
    """Tarsier2 over a Llama decoder.  Reference: lightllm/models/tarsier2/model.py (Tarsier2LlamaTpPartModel)."""

    model_type = "llava"

    def _wrap_source(self, src):
        return _language_model_tensors(src)
