"""How many KV-cache tokens fit: an estimate from the checkpoint alone, before anything is loaded.

    python -m lightllm_b200.utils.profile_max_tokens --model_dir /path --tp 8 --mem_fraction 0.9 [--gpu_gib 180]

Weights: the tensor sizes in the safetensors headers (no tensor is read), rescaled when `--data_type` differs from
the stored type, divided by tp.  KV cache: bytes per token from config.json (MLA latent rows, GQA heads per rank,
full-attention layers only for hybrid models).  The serving processes measure the same at start-up with the
weights resident (`models/base.py`); this tool answers the question for a machine one does not have at hand.

Reference: lightllm/utils/profile_max_tokens.py.
"""
from __future__ import annotations

import glob
import json
import os
import struct
from typing import Dict, Tuple

ELEM = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1,
        "F8_E4M3": 1, "F8_E5M2": 1}
DTYPE_BYTES = {"bf16": 2, "bfloat16": 2, "fp16": 2, "float16": 2, "fp32": 4, "float32": 4}


def safetensors_bytes(model_dir: str) -> Tuple[int, Dict[str, int]]:
    """(total bytes, bytes per stored dtype) over every *.safetensors file of the directory."""
    total, by = 0, {}
    for f in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
        with open(f, "rb") as fh:
            (n,) = struct.unpack("<Q", fh.read(8))
            header = json.loads(fh.read(n))
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            b0, b1 = meta["data_offsets"]
            total += b1 - b0
            by[meta["dtype"]] = by.get(meta["dtype"], 0) + (b1 - b0)
    return total, by


def weight_bytes_per_rank(model_dir: str, tp: int, data_type: str = None) -> int:
    total, by = safetensors_bytes(model_dir)
    if data_type:
        want = DTYPE_BYTES[data_type]
        total = 0
        for dt, b in by.items():
            e = ELEM.get(dt, 2)
            # 16/32-bit float payloads are converted at load; quantised payloads stay as stored
            total += b * want // e if dt in ("F32", "F16", "BF16") else b
    return total // max(tp, 1)


def kv_bytes_per_token(cfg: dict, tp: int, kv_elem_bytes: int = 2) -> int:
    c = dict(cfg)
    for k in ("text_config", "llm_config"):
        if isinstance(c.get(k), dict):
            c = {**c, **c[k]}
    L = int(c.get("num_hidden_layers") or c.get("n_layer"))
    if c.get("layer_types"):
        L = sum(1 for t in c["layer_types"][:L] if t != "linear_attention")
    elif c.get("full_attention_interval") and c.get("linear_num_key_heads"):
        L = L // int(c["full_attention_interval"])
    if c.get("kv_lora_rank"):  # MLA: one latent row per token and layer, replicated on every rank
        return L * (int(c["kv_lora_rank"]) + int(c.get("qk_rope_head_dim", 64))) * kv_elem_bytes
    hq = int(c.get("num_attention_heads") or c.get("n_head"))
    hkv = int(c.get("num_key_value_heads") or hq)
    D = int(c.get("head_dim") or int(c["hidden_size"]) // hq)
    per_rank = max(hkv // tp, 1)  # fewer kv heads than ranks: heads are replicated
    return L * 2 * per_rank * D * kv_elem_bytes


def max_total_tokens(model_dir: str, tp: int = 1, mem_fraction: float = 0.9, gpu_gib: float = None,
                     data_type: str = None, kv_elem_bytes: int = 2) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    if gpu_gib is None:
        import torch

        if not torch.cuda.is_available():
            raise SystemExit("no GPU here: pass --gpu_gib")
        gpu_gib = torch.cuda.get_device_properties(0).total_memory / 2 ** 30
    w = weight_bytes_per_rank(model_dir, tp, data_type)
    kv = kv_bytes_per_token(cfg, tp, kv_elem_bytes)
    budget = gpu_gib * 2 ** 30 * mem_fraction - w
    return {"weight_gib_per_rank": round(w / 2 ** 30, 3), "kv_bytes_per_token_per_rank": kv,
            "max_total_token_num": max(int(budget // kv), 0), "gpu_gib": gpu_gib, "mem_fraction": mem_fraction}


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--model_dir", required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--mem_fraction", type=float, default=0.9)
    ap.add_argument("--gpu_gib", type=float, default=None)
    ap.add_argument("--data_type", default=None, choices=sorted(DTYPE_BYTES))
    ap.add_argument("--kv_elem_bytes", type=int, default=2)
    a = ap.parse_args()
    print(json.dumps(max_total_tokens(a.model_dir, a.tp, a.mem_fraction, a.gpu_gib, a.data_type, a.kv_elem_bytes)))


if __name__ == "__main__":
    main()
