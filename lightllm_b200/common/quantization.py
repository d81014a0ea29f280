"""Quantisation method registry: resolves `--quant_type`, a `--quant_cfg` YAML and the checkpoint's own
`quantization_config` to the method each weight of each layer uses.

Reference behaviour: lightllm/common/quantization/__init__.py:21-130 (`Quantcfg`: HF fp8 with
`weight_block_size [128, 128]` selects the block-scaled fp8 method, `--quant_cfg` may override single layers /
weights, `--expert_dtype` the routed experts) and lightllm/common/quantization/registry.py (`QUANTMETHODS`).

Methods here:
  none                    bf16 tcgen05 GEMM
  fp8w8a8-b128            e4m3 weights with 128 x 128 block scales, activations per token and 128-wide group,
                          `csrc/gemm_fp8.cu` (tcgen05 kind::f8f6f4).  The reference's -deepgemm / -vllm / -triton
                          spellings of this scheme are aliases: there is one kernel.
  fp8w8a8, fp8w8a8-pt,    per-channel / per-tensor / per-group fp8 schemes of the reference: run on the same block-scaled
  fp8w8a8g128, ...        kernel (weights are re-quantised at load with block scales, which are at least as fine)
  w8a8                    s8 weights with per-channel scales, s8 activations with per-token scales, s32 accumulation
                          (tcgen05 kind::i8, `csrc/gemm_fp8.cu`); dense matrices only, experts stay bf16
Methods that need a kernel that does not exist here (`awq`, `awq_marlin`, `fp4fp8-b32`) raise at start-up instead
of silently running in another precision.
"""
from __future__ import annotations

from typing import Dict, Optional

FP8_BLOCK = "fp8w8a8-b128"
INT8 = "w8a8"
NONE = "none"

_ALIASES = {
    "none": NONE, "": NONE, None: NONE,
    "fp8w8a8-b128": FP8_BLOCK, "fp8w8a8-b128-deepgemm": FP8_BLOCK, "fp8w8a8-b128-vllm": FP8_BLOCK,
    "fp8w8a8-b128-triton": FP8_BLOCK, "deepgemm-fp8w8a8-b128": FP8_BLOCK, "vllm-fp8w8a8-b128": FP8_BLOCK,
    "fp8w8a8": FP8_BLOCK, "fp8w8a8-vllm": FP8_BLOCK, "vllm-fp8w8a8": FP8_BLOCK, "fp8w8a8-pt-vllm": FP8_BLOCK,
    "fp8w8a8-pt-sgl": FP8_BLOCK, "fp8w8a8-pt-triton": FP8_BLOCK, "fp8w8a8g128": FP8_BLOCK, "fp8w8a8g64": FP8_BLOCK,
    "fp8w8a8g128-triton": FP8_BLOCK, "triton-fp8w8a8g128": FP8_BLOCK, "fp8": FP8_BLOCK,
    "w8a8": INT8, "vllm-w8a8": INT8, "w8a8-vllm": INT8,
}
_UNBUILT = ("awq", "awq_marlin", "fp4fp8-b32-deepgemm", "fp4fp8-b32", "fp4")

QUANTMETHODS = (NONE, FP8_BLOCK, INT8)


def canonical(name: Optional[str]) -> str:
    if name in _ALIASES:
        return _ALIASES[name]
    if name in _UNBUILT:
        raise NotImplementedError(f"quantisation method {name!r} has no kernel in this build "
                                  f"(available: {', '.join(QUANTMETHODS)} and the fp8w8a8* aliases)")
    raise ValueError(f"unknown quantisation method {name!r}")


class QuantConfig:
    """method_for(layer, weight_name) -> canonical method.  Precedence: per-layer entries of the YAML
    (`mix_bits`), the YAML / command-line default, the checkpoint's quantization_config."""

    def __init__(self, model_config: dict, quant_type: Optional[str] = None, quant_cfg_path: Optional[str] = None,
                 expert_dtype: Optional[str] = None):
        hf = (model_config or {}).get("quantization_config") or {}
        self.from_checkpoint = NONE
        if hf.get("quant_method") == "fp8" and list(hf.get("weight_block_size") or []) == [128, 128]:
            self.from_checkpoint = FP8_BLOCK
        elif hf.get("quant_method") in ("gptq", "compressed-tensors"):
            raise NotImplementedError(f"checkpoints quantised with {hf.get('quant_method')} are not supported")
        # quant_method "awq": the loader expands the 4-bit weights to bf16 (models/quant.py), method stays "none"
        self.default = canonical(quant_type)
        self.per_layer: Dict[int, Dict[str, str]] = {}
        if quant_cfg_path:
            import yaml

            with open(quant_cfg_path) as f:
                data = yaml.safe_load(f) or {}
            if data.get("quant_type") is not None:
                self.default = canonical(data["quant_type"])
            for item in data.get("mix_bits") or []:
                method = canonical(item.get("quant_type"))
                names = item.get("name") or item.get("names") or ["*"]
                names = [names] if isinstance(names, str) else list(names)
                for layer in item.get("layer_nums") or item.get("layers") or []:
                    for n in names:
                        self.per_layer.setdefault(int(layer), {})[n] = method
        if self.default == NONE and self.from_checkpoint != NONE:
            self.default = self.from_checkpoint
        self.expert_method = canonical(expert_dtype) if expert_dtype not in (None, "", "default") else None

    def method_for(self, layer: int, weight_name: str = "*") -> str:
        over = self.per_layer.get(layer)
        if over:
            if weight_name in over:
                return over[weight_name]
            if "*" in over:
                return over["*"]
        if self.expert_method is not None and weight_name in ("experts", "w13", "w2"):
            return self.expert_method
        return self.default

    @property
    def any_fp8(self) -> bool:
        """True if some weight asks for online quantisation (fp8 or int8)."""
        q = (FP8_BLOCK, INT8)
        return self.default in q or self.expert_method in q or any(
            m in q for d in self.per_layer.values() for m in d.values())
