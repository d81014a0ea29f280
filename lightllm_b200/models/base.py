"""Per-rank causal LM runtime: weights, KV pool, request table, prefill / decode forward,
decode CUDA graphs.

One `TransformerLM` lives in each model-rank process (one process per GPU).  The forward pass
is a flat sequence of this package's kernels on a [tokens, hidden] activation:

    embedding -> N x [ rmsnorm -> qkv GEMM -> rope + KV scatter -> paged attention
                       -> o_proj GEMM (+residual / +TP reduce) -> rmsnorm
                       -> gate_up GEMM with gated-activation epilogue -> down GEMM (+residual / +TP reduce) ]
              -> final rmsnorm -> lm_head GEMM (fp32 logits)

Decode runs as one CUDA graph per batch-size bucket (1..split, then every `grow_step` up to the
maximum, the reference's bucket rule: lightllm/common/basemodel/cuda_graph.py:24-51); prefill is
launched eagerly (it is GPU-bound).  Subclasses override `_attention_block` / `_ffn_block` and the
weight loaders (MoE, MLA).

Reference: lightllm/common/basemodel/basemodel.py (TpPartBaseModel), layer_infer/template/
transformer_layer_infer_template.py, models/llama/*.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

from .. import ops
from ..common.infer_state import ShardedLogits, InferState, ModelInput, ModelOutput
from ..common.mem_manager import MemoryManager, profile_max_tokens
from ..common.req_manager import ReqManager
from ..ops import reference as ref
from ..parallel import dist as pdist
from ..parallel.tp import TPContext
from .weights import RandomSource, SafetensorsSource, WeightSource, kv_head_range, tp_range


def normalize_config(cfg: dict) -> dict:
    """One spelling for keys that differ between config generations: `rope_parameters` (new) is unfolded into
    `rope_theta` / `rope_scaling`, `num_local_experts` doubles as `num_experts`, multimodal wrappers expose
    their `text_config` at the top level."""
    cfg = dict(cfg)
    if isinstance(cfg.get("thinker_config"), dict) and "text_config" not in cfg:  # Qwen3-Omni: thinker / talker parts
        cfg = {**cfg, **cfg["thinker_config"], "model_type": cfg.get("model_type")}
    if "text_config" in cfg and "hidden_size" not in cfg:  # multimodal wrappers
        base = dict(cfg["text_config"])
        outer = cfg.get("model_type") or base.get("model_type")
        keep = {k: cfg[k] for k in ("tie_word_embeddings",) if k in cfg}  # the wrapper decides about its own head
        cfg = {**cfg, **base, **keep, "model_type": outer}
    rp = cfg.get("rope_parameters")
    if isinstance(rp, dict):
        if "rope_theta" in rp:
            cfg.setdefault("rope_theta", rp["rope_theta"])
        kind = rp.get("rope_type", rp.get("type", "default"))
        if kind not in (None, "default") and not cfg.get("rope_scaling"):
            cfg["rope_scaling"] = {k: v for k, v in rp.items() if k != "rope_theta"}
        if "partial_rotary_factor" in rp:
            cfg.setdefault("partial_rotary_factor", rp["partial_rotary_factor"])
    if "num_local_experts" in cfg:
        cfg.setdefault("num_experts", cfg["num_local_experts"])
    return cfg


def embed_row_width(cfg: dict) -> int:
    """Elements per row of the shared multimodal embedding arena: the language model's width, times (1 + number
    of deep-stack feature sets) for towers that also feed early decoder layers (Qwen3-VL)."""
    cfg = normalize_config(cfg)
    k = len((cfg.get("vision_config") or {}).get("deepstack_visual_indexes") or [])
    return int(cfg["hidden_size"]) * (1 + k)


def load_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return normalize_config(json.load(f))


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
           "float32": torch.float32, "fp32": torch.float32}


class LayerWeights:
    """Plain attribute bag for one transformer layer (tensors already fused / sliced / on device)."""

    def __init__(self):
        self.__dict__["_t"] = {}

    def __getattr__(self, k):
        try:
            return self.__dict__["_t"][k]
        except KeyError:
            return None

    def __setattr__(self, k, v):
        self.__dict__["_t"][k] = v

    def tensors(self):
        return self.__dict__["_t"]


class TransformerLM:
    model_type = "llama"

    # ------------------------------------------------------------------ init
    def __init__(self, config: dict, *, weight_source: Optional[WeightSource] = None, model_dir: Optional[str] = None,
                 pstate: Optional[pdist.ParallelState] = None, data_type: Optional[str] = None,
                 max_total_token_num: Optional[int] = None, mem_fraction: float = 0.9, max_req_num: int = 256,
                 max_seq_length: int = 8192, batch_max_tokens: int = 16384, graph_max_batch_size: int = 256,
                 graph_split_batch_size: int = 32, graph_grow_step_size: int = 16, disable_cudagraph: bool = False,
                 graph_max_len_in_batch: Optional[int] = None, tp_fused=None, random_seed: int = 0,
                 vocab_parallel_embedding: bool = False, num_layers_override: Optional[int] = None,
                 share_with: Optional["TransformerLM"] = None, extra_kv_layers: int = 0, **extra):
        config = normalize_config(config)
        self.config = config
        self.model_dir = model_dir
        self.ps = pstate or pdist.state()
        self.device = self.ps.device
        self.tp = TPContext(self.ps, fused=tp_fused)
        dt = data_type or config.get("torch_dtype") or config.get("dtype") or "bfloat16"
        self.dtype = _DTYPES[str(dt).replace("torch.", "")]
        if self.device.type == "cuda" and self.dtype != torch.bfloat16:
            self.dtype = torch.bfloat16  # the sm_100a kernels are bf16
        self.extra = extra
        self.tpsp_mix_mode = bool(extra.get("tpsp_mix_mode", False))  # token-sharded residual stream between layers
        from ..common.quantization import QuantConfig

        self.quant_cfg = QuantConfig(config, extra.get("quant_type"), extra.get("quant_cfg"), extra.get("expert_dtype"))
        self.share_with = share_with          # draft module: lives on the target model's KV pool / request table
        self.extra_kv_layers = extra_kv_layers  # pool layers appended for draft modules
        self.kv_layer_offset = 0
        self._read_config(config)
        if num_layers_override:
            self.num_layers = num_layers_override
        self.max_req_num = max_req_num
        self.max_seq_length = max_seq_length
        self.batch_max_tokens = batch_max_tokens
        self.vocab_parallel_embedding = vocab_parallel_embedding
        self.disable_cudagraph = disable_cudagraph or self.device.type != "cuda"
        self.graph_max_batch_size = graph_max_batch_size
        self.graph_split_batch_size = graph_split_batch_size
        self.graph_grow_step_size = graph_grow_step_size
        self.graph_max_len_in_batch = graph_max_len_in_batch or max_seq_length

        if weight_source is None:
            weight_source = self._wrap_source(self._open_checkpoint(model_dir)) \
                if model_dir and self._has_weights(model_dir) else RandomSource(self.weight_shapes(), dtype=self.dtype, seed=random_seed,
                             device=str(self.device) if self.device.type == "cuda" else "cpu",
                             fp8_names=self.fp8_weight_names())
        self.weight_source = weight_source
        from ..engine.redundancy import RedundancyConfig

        self.redundancy_cfg = RedundancyConfig.load(extra.get("ep_redundancy_expert_config_path"))
        self._load_weights(weight_source)
        self._init_rope()
        if share_with is not None:
            self.mem_manager, self.req_manager = share_with.mem_manager, share_with.req_manager
            self.max_total_token_num = share_with.max_total_token_num
        else:
            self._init_mem(max_total_token_num, mem_fraction)
            self.req_manager = ReqManager(max_req_num, max_seq_length, self.mem_manager, self.device)
        if getattr(self.mem_manager, "no_cuda_graph", False):    # a pool whose attention route syncs with the host
            self.disable_cudagraph = True
        self.route_capture = None
        if extra.get("enable_return_routed_experts") and share_with is None:
            from ..common.route_capture import RouteCapture

            self.route_capture = RouteCapture(config, self.mem_manager.size + 1, self.device)
        self._graphs: Dict[int, dict] = {}
        self._graph_pool = None
        self.weight_version = "default"
        self.debug_status = None
        if self.device.type == "cuda":
            from ..ops._native import debug_bounds_enabled, set_debug_bounds

            if debug_bounds_enabled():   # LLB_DEBUG_BOUNDS=1: the kernels check slot / request / expert indices
                self.debug_status = torch.zeros(1, dtype=torch.int32, device=self.device)
                set_debug_bounds(pool_slots=self.mem_manager.size + 1, req_rows=self.max_req_num + 1,
                                 r2t_cols=self.max_seq_length,
                                 num_experts=int(config.get("num_experts") or config.get("n_routed_experts") or
                                                 config.get("num_local_experts") or 0) +
                                 self.ps.world_size * self.redundancy_cfg.num +
                                 (int(config.get("n_shared_experts") or 0)
                                  if extra.get("enable_fused_shared_experts") else 0), status=self.debug_status)

    def _open_checkpoint(self, model_dir):
        """The checkpoint as a WeightSource; AWQ checkpoints are presented de-quantised (no int4 GEMM here)."""
        src = SafetensorsSource(model_dir)
        q = self.config.get("quantization_config") or {}
        if q.get("quant_method") == "awq":
            from .quant import AwqDequantSource

            src = AwqDequantSource(src, self.dtype)
        return src

    def _wrap_source(self, src: WeightSource) -> WeightSource:
        """Hook for families whose checkpoints use other tensor names or fused tensors: return a view of `src`
        under this package's canonical (Llama-style) names."""
        return src

    @staticmethod
    def _has_weights(model_dir):
        import glob

        return bool(glob.glob(os.path.join(model_dir, "*.safetensors")) or glob.glob(os.path.join(model_dir, "*.bin")))

    def _read_config(self, c: dict):
        self.hidden = c["hidden_size"]
        self.num_layers = c["num_hidden_layers"]
        self.num_q_heads = c["num_attention_heads"]
        self.num_kv_heads = c.get("num_key_value_heads", self.num_q_heads)
        self.head_dim = c.get("head_dim") or self.hidden // self.num_q_heads
        self.inter = c.get("intermediate_size")
        self.vocab = c["vocab_size"]
        self.eps = c.get("rms_norm_eps", c.get("layer_norm_epsilon", 1e-6))
        self.rope_theta = c.get("rope_theta", 10000.0)
        self.rope_scaling = c.get("rope_scaling")
        self.partial_rotary = c.get("partial_rotary_factor", 1.0)
        self.tie_embeddings = c.get("tie_word_embeddings", False)
        self.attn_bias = c.get("attention_bias", False)
        self.act = "gelu" if "gelu" in str(c.get("hidden_act", c.get("hidden_activation", "silu"))) else "silu"
        self.norm_w_offset = 0.0
        self.qk_norm = False
        self.embed_scale = 1.0
        tp = self.tp.size
        assert self.num_q_heads % tp == 0, "q heads must divide by tp"
        self.hq = self.num_q_heads // tp
        k0, k1 = kv_head_range(self.num_kv_heads, self.tp.rank, tp)
        self.hkv = k1 - k0
        self._kv_range = (k0, k1)
        self.rot_dim = int(self.head_dim * self.partial_rotary)
        self.sm_scale = 1.0 / math.sqrt(self.head_dim)

    # ------------------------------------------------------------------ weights
    def fp8_weight_names(self):
        return set()

    def weight_shapes(self) -> Dict[str, tuple]:
        """HF names -> full (unsharded) shapes; drives RandomSource and documents the checkpoint format."""
        H, D = self.hidden, self.head_dim
        s = {"model.embed_tokens.weight": (self.vocab, H), "model.norm.weight": (H,)}
        if not self.tie_embeddings:
            s["lm_head.weight"] = (self.vocab, H)
        for i in range(self.num_layers):
            p = f"model.layers.{i}."
            s[p + "input_layernorm.weight"] = (H,)
            s[p + "post_attention_layernorm.weight"] = (H,)
            s.update(self._attn_weight_shapes(p))
            s.update(self._ffn_weight_shapes(p, i))
        return s

    def _attn_weight_shapes(self, p):
        H, D = self.hidden, self.head_dim
        s = {p + "self_attn.q_proj.weight": (self.num_q_heads * D, H),
             p + "self_attn.k_proj.weight": (self.num_kv_heads * D, H),
             p + "self_attn.v_proj.weight": (self.num_kv_heads * D, H),
             p + "self_attn.o_proj.weight": (H, self.num_q_heads * D)}
        if self.attn_bias:
            s[p + "self_attn.q_proj.bias"] = (self.num_q_heads * D,)
            s[p + "self_attn.k_proj.bias"] = (self.num_kv_heads * D,)
            s[p + "self_attn.v_proj.bias"] = (self.num_kv_heads * D,)
        if self.qk_norm:
            s[p + "self_attn.q_norm.weight"] = (D,)
            s[p + "self_attn.k_norm.weight"] = (D,)
        return s

    def _ffn_weight_shapes(self, p, layer):
        H, I = self.hidden, self.inter
        return {p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H),
                p + "mlp.down_proj.weight": (H, I)}

    def _dev(self, t: torch.Tensor, dtype=None) -> torch.Tensor:
        return t.to(device=self.device, dtype=dtype or self.dtype).contiguous()

    def _load_weights(self, src: WeightSource):
        tp, r = self.tp.size, self.tp.rank
        emb = src.get("model.embed_tokens.weight")
        if self.vocab_parallel_embedding and tp > 1:
            v0, v1 = tp_range(self.vocab, r, tp)
            self.embed_w = self._dev(emb[v0:v1])
            self.embed_range = (v0, v1)
        else:
            self.embed_w = self._dev(emb)
            self.embed_range = (0, self.vocab)
        self.final_norm_w = self._dev(src.get("model.norm.weight"))
        v0, v1 = tp_range(self.vocab, r, tp)
        if src.has("lm_head.weight") and not self.tie_embeddings:
            self.lm_head_w = self._dev(src.get("lm_head.weight", 0, v0, v1))
        else:
            self.lm_head_w = self._dev(emb[v0:v1]) if tp > 1 or self.vocab_parallel_embedding else self.embed_w
        self.layers: List[LayerWeights] = []
        for i in range(self.num_layers):
            lw = LayerWeights()
            p = f"model.layers.{i}."
            lw.in_norm = self._dev(src.get(p + "input_layernorm.weight"))
            lw.post_norm = self._dev(src.get(p + "post_attention_layernorm.weight"))
            self._load_attn(lw, src, p, i)
            self._load_ffn(lw, src, p, i)
            if self.quant_cfg.any_fp8 and not self.extra.get("dequant_fp8", False):
                self._quantize_layer_online(lw, i)
            self.layers.append(lw)

    def _quantize_layer_online(self, lw, layer: int):
        """`--quant_type fp8w8a8*` (or a `--quant_cfg` entry for this layer) on weights that are still bf16 after
        loading: quantise them to e4m3 with block scales so the layer runs on the fp8 GEMM.  Weights a model
        already loaded as fp8 (block-quantised checkpoints) are left alone."""
        from ..common.quantization import FP8_BLOCK, INT8
        from ..ops.fp8 import Fp8Experts, Fp8Weight, stack_experts
        from ..ops.int8 import Int8Weight

        t = lw.tensors()
        silu = getattr(self, "act", "silu") == "silu"

        def want(name):
            return self.quant_cfg.method_for(layer, name) == FP8_BLOCK

        def q2(name, rows=128):
            w = t.get(name)
            if not (isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 16 == 0 and w.is_floating_point()):
                return
            method = self.quant_cfg.method_for(layer, name)
            if method == FP8_BLOCK:
                t[name] = Fp8Weight.from_float(w, rows)
            elif method == INT8:
                t[name] = Int8Weight.from_float(w)

        for name in ("qkv_w", "o_w", "down_w", "shared_down_w", "q_b_w"):
            q2(name)
        for name, flag in (("gate_up_w", "gate_up_fused"), ("shared_gate_up_w", "shared_fused")):
            if not t.get(flag):
                q2(name)            # plain GEMM followed by a standalone gated activation
            elif silu:
                q2(name, 32)        # interleaved in 32-row blocks: one scale row per block
        w13, w2 = t.get("w13"), t.get("w2")
        if (isinstance(w13, torch.Tensor) and w13.dim() == 3 and silu and t.get("b13") is None and want("experts")
                and w13.shape[2] % 16 == 0 and w2.shape[2] % 16 == 0 and w13.shape[1] % 128 == 0
                and w2.shape[1] % 128 == 0):
            E = w13.shape[0]
            t["w13"] = Fp8Experts(stack_experts([Fp8Weight.from_float(w13[e], 32) for e in range(E)]), E)
            t["w2"] = Fp8Experts(stack_experts([Fp8Weight.from_float(w2[e], 128) for e in range(E)]), E)

    def _load_attn(self, lw, src, p, layer):
        D = self.head_dim
        tp, r = self.tp.size, self.tp.rank
        q0, q1 = tp_range(self.num_q_heads, r, tp)
        k0, k1 = self._kv_range
        q = src.get(p + "self_attn.q_proj.weight", 0, q0 * D, q1 * D)
        k = src.get(p + "self_attn.k_proj.weight", 0, k0 * D, k1 * D)
        v = src.get(p + "self_attn.v_proj.weight", 0, k0 * D, k1 * D)
        lw.qkv_w = self._dev(torch.cat([q, k, v], dim=0))
        if self.attn_bias and src.has(p + "self_attn.q_proj.bias"):
            lw.qkv_b = self._dev(torch.cat([src.get(p + "self_attn.q_proj.bias", 0, q0 * D, q1 * D),
                                            src.get(p + "self_attn.k_proj.bias", 0, k0 * D, k1 * D),
                                            src.get(p + "self_attn.v_proj.bias", 0, k0 * D, k1 * D)], dim=0))
        lw.o_w = self._dev(src.get(p + "self_attn.o_proj.weight", 1, q0 * D, q1 * D))
        if src.has(p + "self_attn.o_proj.bias"):
            ob = src.get(p + "self_attn.o_proj.bias")
            lw.o_b = self._dev(ob / tp)  # every rank adds its share (reference: ColSliceMixin._slice_bias)
        if self.qk_norm:
            lw.q_norm = self._dev(src.get(p + "self_attn.q_norm.weight"))
            lw.k_norm = self._dev(src.get(p + "self_attn.k_norm.weight"))

    def _load_dense_ffn(self, lw, src, prefix, inter, tp=None, r=None):
        tp = self.tp.size if tp is None else tp
        r = self.tp.rank if r is None else r
        i0, i1 = tp_range(inter, r, tp)
        g = src.get(prefix + "gate_proj.weight", 0, i0, i1)
        u = src.get(prefix + "up_proj.weight", 0, i0, i1)
        il = i1 - i0
        if il % ref.GATE_UP_BLOCK == 0:
            lw.gate_up_w = self._dev(ref.interleave_gate_up(g, u))
            lw.gate_up_fused = True
        else:  # odd shard size: plain [gate; up] rows and a standalone gated activation
            lw.gate_up_w = self._dev(torch.cat([g, u], dim=0))
            lw.gate_up_fused = False
        lw.down_w = self._dev(src.get(prefix + "down_proj.weight", 1, i0, i1))

    def _load_ffn(self, lw, src, p, layer):
        self._load_dense_ffn(lw, src, p + "mlp.", self.inter)

    def _init_rope(self):
        n = max(self.max_seq_length + 8, 16)
        theta = self.rope_theta
        # LIGHTLLM_NTK_ALPHA > 1: NTK-aware context extension without fine-tuning, by raising the rotary base
        # (reference: lightllm/models/llama/model.py:117-126)
        try:
            alpha = float(os.environ.get("LLB_NTK_ALPHA", os.environ.get("LIGHTLLM_NTK_ALPHA", "1")))
        except ValueError:
            alpha = 1.0
        if alpha > 1.0 and self.rot_dim > 2 and not self.rope_scaling:
            theta = theta * alpha ** (self.rot_dim / (self.rot_dim - 2))
        self.cos, self.sin = ref.build_rope_cache(n, self.rot_dim, theta, self.rope_scaling,
                                                  device=self.device)

    # ------------------------------------------------------------------ memory
    def _kv_manager_class(self):
        from ..common.mem_manager import select_mem_manager_class

        return select_mem_manager_class(self.extra.get("kv_type"))

    def kv_bytes_per_token(self) -> int:
        kw = {"group_size": self._kv_group_size()} if self._is_int4_kv() else {}
        return self._kv_manager_class().bytes_per_token(self.dtype, self.hkv, self.head_dim,
                                                        self.num_layers + self.extra_kv_layers, **kw)

    def _is_int4_kv(self) -> bool:
        return str(self.extra.get("kv_type") or "").lower() == "int4kv"

    def _kv_group_size(self) -> int:
        return int(self.extra.get("kv_quant_group_size") or 8)

    def _kv_manager_kwargs(self) -> dict:
        kw = {}
        if str(self.extra.get("kv_type") or "").startswith("fp8kv"):
            kw["calibration"] = self.extra.get("kv_quant_calibration_config_path")
            kw["head_range"] = getattr(self, "_kv_range", None)
        if self._is_int4_kv():
            kw["group_size"] = self._kv_group_size()
        return kw

    def _make_mem_manager(self, size):
        return self._kv_manager_class()(size, self.dtype, self.hkv, self.head_dim,
                                        self.num_layers + self.extra_kv_layers, self.device,
                                        **self._kv_manager_kwargs())

    def _kv_layer(self, i: int):
        return self.mem_manager.layer(self.kv_layer_offset + i)

    def _init_mem(self, max_total_token_num, mem_fraction):
        if max_total_token_num is None:
            max_total_token_num = profile_max_tokens(self.device, self.kv_bytes_per_token(), mem_fraction)
            if self.ps.world_size > 1:
                import torch.distributed as dist

                t = torch.tensor([max_total_token_num], dtype=torch.int64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
                max_total_token_num = int(t.item())
        self.max_total_token_num = int(max_total_token_num)
        self.mem_manager = self._make_mem_manager(self.max_total_token_num)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, mi: ModelInput) -> ModelOutput:
        if mi.max_kv_len > self.max_seq_length:
            # the request table's rows and the rotary tables end there: a longer sequence would read past them
            raise ValueError(f"sequence of {mi.max_kv_len} tokens exceeds the model's max_seq_length "
                             f"{self.max_seq_length} (max_req_total_len + 8)")
        # expert-parallel exchanges size their launches by the largest token count any rank can bring to this pass:
        # a decode step is bounded by the largest graph batch (the same on all ranks), a prompt pass by what the
        # data-parallel backend learnt from the other replicas (`ep_prefill_tokens_bound`) or the chunk limit
        if mi.is_prefill:
            self._ep_tokens_bound = int(getattr(self, "ep_prefill_tokens_bound", 0) or self.batch_max_tokens)
            return self._prefill(mi)
        self._ep_tokens_bound = max(self.graph_max_batch_size, self.max_req_num)
        return self._decode(mi)

    # ---- prefill ----
    def _build_prefill_state(self, mi: ModelInput):
        """Stages a prompt pass' index tensors and runs the step prologue: (state, input ids on the device)."""
        dev = self.device
        B = mi.batch_size
        b_req_idx = mi.b_req_idx.to(dev, non_blocking=True)
        b_seq_len = mi.b_seq_len.to(dev, non_blocking=True)
        ready = mi.b_ready_cache_len.to(dev, non_blocking=True)
        mem_index = mi.mem_indexes.to(dev, non_blocking=True)
        input_ids = mi.input_ids.to(dev, non_blocking=True)
        T = input_ids.shape[0]
        q_len = mi.b_q_len if mi.b_q_len is not None else (mi.b_seq_len - mi.b_ready_cache_len)
        cu_host = torch.zeros(B + 1, dtype=torch.int32)
        cu_host[1:] = torch.cumsum(q_len.to(torch.int32), 0)
        cu_q = cu_host.to(dev, non_blocking=True)
        pos, batch_of = ops.prefill_prologue(self.req_manager.req_to_token_indexs, b_req_idx, ready, cu_q, mem_index, T)
        st = InferState(is_prefill=True, batch_size=B, num_tokens=T, max_kv_len=mi.max_kv_len, max_q_len=mi.max_q_len,
                        b_req_idx=b_req_idx, b_seq_len=b_seq_len, mem_index=mem_index, position_ids=pos, cu_q=cu_q,
                        b_ready_cache_len=ready, batch_of_token=batch_of)
        st.seq_pos = pos
        st.extra["multimodal_params"] = mi.multimodal_params
        st.extra["input_ids_cpu"] = mi.input_ids
        st.extra["q_len_cpu"] = q_len
        st.extra["ready_cpu"] = mi.b_ready_cache_len
        st.extra["req_idx_cpu"] = mi.b_req_idx
        st.extra["draft_input_hidden"] = mi.draft_input_hidden
        st.extra["verify_pass"] = bool(getattr(mi, "verify_pass", False))
        st.extra["want_hidden"] = bool(mi.return_hidden)
        self._prepare_prefill_state(st)
        return st, input_ids

    def _last_rows(self, h, st: InferState, all_rows: bool):
        if all_rows:
            return h
        B = st.batch_size
        last_idx = (st.cu_q[1:] - 1).to(torch.int32)
        last = torch.empty((B, self.hidden), dtype=h.dtype, device=self.device)
        ops.copy_rows(last, h, None, last_idx, B)
        return last

    def _prefill(self, mi: ModelInput) -> ModelOutput:
        balance_on = self._dp_balance_on()      # a static property: every replica takes the same path
        halves = None if balance_on else self._split_for_pipeline(mi)
        if halves is not None:
            return self._prefill_pipelined(mi, halves)
        st, input_ids = self._build_prefill_state(mi)
        h = self._embed(input_ids, st)
        bal = self._prepare_dp_balance(st) if balance_on else None
        if bal is not None:       # token-wise work on an even split of all replicas' tokens
            h = bal.to_balanced(h)
        h = self._layers_forward(h, st)
        if bal is not None:
            h = bal.to_origin(h)
        hidden = h if mi.return_hidden else None
        last = self._last_rows(h, st, mi.return_all_logits)
        logits = self._lm_head(last, normed=True) if st.extra.get("normed") else self._lm_head(last)
        return ModelOutput(logits=logits, hidden=hidden)

    def _dp_balance_on(self) -> bool:
        """`--enable_dp_prefill_balance` applies to this model: data parallel, a plain decoder stack (families that
        edit the stream between layers keep their own token layout) and no draft modules riding on the passes."""
        if not self.extra.get("enable_dp_prefill_balance") or self.ps.dp_size <= 1 or self.extra_kv_layers or \
                self.share_with is not None:
            return False
        cls, base = type(self), TransformerLM
        return cls._after_layer is base._after_layer and cls._layers_forward is base._layers_forward

    def _prepare_dp_balance(self, st: InferState):
        """The token exchange of this prompt pass (common/dp_balance.py), or None when the replicas are balanced
        already.  Collective: every replica runs a prompt pass on the same step (the data-parallel backend's
        lock-step)."""
        from ..common.dp_balance import DPBalance

        bal = DPBalance.prepare(self.ps, st.num_tokens)
        st.extra["balance"] = bal
        return bal

    # ---- prompt passes as two micro-batches whose reductions run under each other's GEMMs ----
    PIPELINE_MIN_TOKENS = 2048   # below this the pass is latency-bound and the fused kernels are faster

    def _split_for_pipeline(self, mi: ModelInput):
        """Two ModelInputs (a split of the requests with balanced token counts) when this pass qualifies for the
        pipelined schedule: tensor parallelism on GPUs with a copy-engine reducer attached, a plain decoder stack
        (no family hook between the layers, no multimodal rows, no hidden states wanted back), at least two
        requests and enough tokens for the transfers to matter."""
        ce = getattr(self.tp, "ce", None)
        if ce is None or self.tp.size == 1 or mi.batch_size < 2 or mi.multimodal_params or mi.return_hidden \
                or mi.draft_input_hidden is not None or getattr(mi, "verify_pass", False) or ce.hidden != self.hidden:
            return None
        cls = type(self)
        base = TransformerLM
        if any(getattr(cls, f) is not getattr(base, f) for f in
               ("_layers_forward", "_after_layer", "_prepare_prefill_state", "_embed", "_attention_block",
                "_row_parallel", "_reduce_partial")):
            return None
        q_len = (mi.b_q_len if mi.b_q_len is not None else (mi.b_seq_len - mi.b_ready_cache_len)).to(torch.int64)
        T = int(q_len.sum())
        if T < self.PIPELINE_MIN_TOKENS or T != mi.input_ids.shape[0]:
            return None
        cum = torch.cumsum(q_len, 0)
        b0 = int(torch.searchsorted(cum, torch.tensor(T // 2), right=False)) + 1
        b0 = max(1, min(mi.batch_size - 1, b0))
        t0 = int(cum[b0 - 1])
        if max(t0, T - t0) > ce.max_tokens:
            return None
        out = []
        for lo, hi, tlo, thi in ((0, b0, 0, t0), (b0, mi.batch_size, t0, T)):
            seq, rdy = mi.b_seq_len[lo:hi], mi.b_ready_cache_len[lo:hi]
            ql = mi.b_q_len[lo:hi] if mi.b_q_len is not None else None
            qn = (ql if ql is not None else (seq - rdy))
            out.append(ModelInput(batch_size=hi - lo, total_token_num=int(seq.sum()), max_kv_len=int(seq.max()),
                                  is_prefill=True, b_req_idx=mi.b_req_idx[lo:hi], b_seq_len=seq,
                                  mem_indexes=mi.mem_indexes[tlo:thi], input_ids=mi.input_ids[tlo:thi],
                                  b_ready_cache_len=rdy, b_q_len=ql, max_q_len=int(qn.max()),
                                  return_all_logits=mi.return_all_logits))
        return out

    def _prefill_pipelined(self, mi: ModelInput, halves) -> ModelOutput:
        """The layer stack over two micro-batches A and B.  Compute (attention, GEMMs) runs on the current stream
        in the order A, B, A, B ...; every row-parallel GEMM is followed by a copy-engine reduction
        (`parallel.ce.CopyEngineTP`: reduce-scatter, residual + RMSNorm on the owned rows, all-gather) queued on a
        side stream, so the reduction of one micro-batch moves its bytes while the other micro-batch computes.
        The residual stream is token-sharded inside the pass (each rank keeps its rows up to date) and the last
        reduction applies the final norm.  Reference: the two-micro-batch overlap of
        lightllm/common/basemodel/basemodel.py:757-945 (there for the expert-parallel path)."""
        ce = self.tp.ce
        dev = self.device
        comp = torch.cuda.current_stream(dev)
        if getattr(self, "_ce_stream", None) is None:
            self._ce_stream = torch.cuda.Stream(device=dev)
        comm = self._ce_stream
        comm.wait_stream(comp)
        sts, res, h = [], [], []
        for m in halves:
            st, ids = self._build_prefill_state(m)
            x = self._embed(ids, st)
            sts.append(st)
            res.append(x)
            h.append(ops.rmsnorm(x, self.layers[0].in_norm, self.eps, self.norm_w_offset))
        ready = [None, None]          # event after which h[m] may be read on the compute stream
        n = self.num_layers

        def reduce_on_side_stream(m, partial, norm_w):
            ev = torch.cuda.Event()
            ev.record(comp)
            with torch.cuda.stream(comm):
                comm.wait_event(ev)
                out = ce.reduce(partial, res[m], norm_w, self.eps, self.norm_w_offset)
                done = torch.cuda.Event()
                done.record(comm)
            h[m], ready[m] = out, done

        for i, lw in enumerate(self.layers):
            for m in (0, 1):
                if ready[m] is not None:
                    comp.wait_event(ready[m])
                a = self._attention_block(i, lw, h[m], sts[m])
                partial = ops.gemm(a, lw.o_w, epi="store", bias=lw.o_b, out=ce.partial_out(a.shape[0]))
                reduce_on_side_stream(m, partial, lw.post_norm)
            nxt = self.layers[i + 1].in_norm if i + 1 < n else self.final_norm_w
            for m in (0, 1):
                comp.wait_event(ready[m])
                f = self._ffn_block(i, lw, h[m], sts[m])
                T = h[m].shape[0]
                if f[0] == "rowpar":
                    partial = ops.gemm(f[1], f[2], epi="store", out=ce.partial_out(T))
                else:
                    partial = ce.partial_out(T)
                    partial.copy_(f[1])
                reduce_on_side_stream(m, partial, nxt)
        logits = []
        for m in (0, 1):
            comp.wait_event(ready[m])
            last = self._last_rows(h[m], sts[m], mi.return_all_logits)
            logits.append(self._lm_head(last, normed=True))
        if isinstance(logits[0], ShardedLogits):
            out = ShardedLogits(torch.cat([logits[0].local, logits[1].local], 0), self.tp, logits[0].v0, self.vocab)
        else:
            out = torch.cat(logits, 0)
        return ModelOutput(logits=out)

    # ---- decode ----
    def graph_batch_sizes(self) -> List[int]:
        sizes = list(range(1, min(self.graph_split_batch_size, self.graph_max_batch_size) + 1))
        b = self.graph_split_batch_size + self.graph_grow_step_size
        while b <= self.graph_max_batch_size:
            sizes.append(b)
            b += self.graph_grow_step_size
        if sizes[-1] != self.graph_max_batch_size:
            sizes.append(self.graph_max_batch_size)
        return sizes

    def _bucket(self, B: int) -> Optional[int]:
        for s in self.graph_batch_sizes():
            if s >= B:
                return s
        return None

    def _decode(self, mi: ModelInput) -> ModelOutput:
        B = mi.batch_size
        use_graph = (not self.disable_cudagraph and B <= self.graph_max_batch_size
                     and mi.max_kv_len <= self.graph_max_len_in_batch)
        if not use_graph:
            dev = self.device
            st = self._make_decode_state(B, mi.b_req_idx.to(dev, non_blocking=True),
                                         mi.b_seq_len.to(dev, non_blocking=True),
                                         mi.mem_indexes.to(dev, non_blocking=True), mi.max_kv_len)
            return ModelOutput(logits=self._decode_body(st))
        bucket = self._bucket(B)
        g = self._graphs.get(bucket)
        if g is None:
            g = self._capture_decode_graph(bucket)
        # stage inputs (rows beyond B keep the HOLD request / HOLD slot)
        g["b_req_idx"][:B].copy_(mi.b_req_idx, non_blocking=True)
        g["b_seq_len"][:B].copy_(mi.b_seq_len, non_blocking=True)
        g["mem_index"][:B].copy_(mi.mem_indexes, non_blocking=True)
        if bucket > B:
            g["b_req_idx"][B:].fill_(self.req_manager.HOLD_REQUEST_ID)
            g["b_seq_len"][B:].fill_(1)
            g["mem_index"][B:].fill_(self.mem_manager.HOLD_TOKEN_MEMINDEX)
        g["graph"].replay()
        ops._count(g["launches"])
        return ModelOutput(logits=g["logits"][:B])

    def _make_decode_state(self, B, b_req_idx, b_seq_len, mem_index, max_kv_len, num_splits=None) -> InferState:
        st = InferState(is_prefill=False, batch_size=B, num_tokens=B, max_kv_len=max_kv_len, max_q_len=1,
                        b_req_idx=b_req_idx, b_seq_len=b_seq_len, mem_index=mem_index)
        if self.device.type == "cuda":
            st.decode_num_splits = num_splits or ops.gqa_decode_num_splits(B, self.hq, max(self.hkv, 1), max_kv_len)
        return st

    def _decode_body(self, st: InferState) -> torch.Tensor:
        ids, pos = ops.decode_prologue(self.req_manager.req_to_token_indexs, self.req_manager.req_to_next_token_ids,
                                       st.b_req_idx, st.b_seq_len, st.mem_index)
        st.position_ids = pos
        st.seq_pos = pos
        self._prepare_decode_state(st)
        h = self._embed(ids, st)
        h = self._layers_forward(h, st)
        return self._lm_head(h, normed=True) if st.extra.get("normed") else self._lm_head(h)

    def _capture_decode_graph(self, bucket: int) -> dict:
        dev = self.device
        # the launch shapes of the expert-parallel exchange are frozen into the graph: use the decode bound, also
        # when graphs are captured ahead of the first forward call (warmup_graphs)
        self._ep_tokens_bound = max(self.graph_max_batch_size, self.max_req_num)
        g = {
            "b_req_idx": torch.full((bucket,), self.req_manager.HOLD_REQUEST_ID, dtype=torch.int32, device=dev),
            "b_seq_len": torch.ones(bucket, dtype=torch.int32, device=dev),
            "mem_index": torch.full((bucket,), self.mem_manager.HOLD_TOKEN_MEMINDEX, dtype=torch.int32, device=dev),
        }
        splits = ops.gqa_decode_num_splits(bucket, self.hq, max(self.hkv, 1), self.graph_max_len_in_batch)
        st = self._make_decode_state(bucket, g["b_req_idx"], g["b_seq_len"], g["mem_index"],
                                     self.graph_max_len_in_batch, num_splits=splits)
        if splits > 1:
            st.decode_scratch = (torch.empty(bucket * self.hq * splits * self.head_dim, dtype=torch.float32, device=dev),
                                 torch.empty(bucket * self.hq * splits, dtype=torch.float32, device=dev))
        # warm-up on a side stream (allocations, lazy kernel attribute set-up), then capture
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._decode_body(st)
        torch.cuda.current_stream(dev).wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        n0 = ops.launch_count()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self._decode_body(st)
        g["launches"] = ops.launch_count() - n0
        g["graph"] = graph
        g["logits"] = logits
        g["state"] = st
        self._graphs[bucket] = g
        return g

    def warmup_graphs(self, sizes: Optional[List[int]] = None):
        """Capture decode graphs up front, largest first (shares the memory pool)."""
        if self.disable_cudagraph:
            return
        for b in sorted(sizes or self.graph_batch_sizes(), reverse=True):
            if b not in self._graphs:
                self._capture_decode_graph(b)

    # ---- pieces ----
    def _prepare_prefill_state(self, st: InferState):
        """Hook: per-pass inputs a family derives on the host (multimodal rotary positions)."""

    def _prepare_decode_state(self, st: InferState):
        """Hook: runs inside the decode graph after the positions are known."""

    def _rope_inputs(self, st: InferState, layer: int):
        """(cos table, sin table, row index per token) for the rotary kernel."""
        return self.cos, self.sin, st.position_ids

    embed_arena = None  # shared embedding arena of the visual / audio servers (set by the rank process)

    def _merge_multimodal(self, h, st: InferState):
        """Rows of `h` whose token id lies in an image / audio item's virtual id range are replaced by the item's
        embeddings from the shared arena (reference: lightllm/common/basemodel/triton_kernel/multimodal_emb.py)."""
        mm = st.extra.get("multimodal_params")
        if not st.is_prefill or not mm or self.embed_arena is None:
            return h
        ids = st.extra["input_ids_cpu"]
        pos_all, rows_all = [], []
        seen = set()
        for params in mm:
            for kind in ("images", "audios"):
                for it in (params or {}).get(kind, []):
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
        pos, rows = torch.cat(pos_all), torch.cat(rows_all)
        emb = self.embed_arena.read_rows(rows).to(device=h.device, dtype=h.dtype)
        if self.embed_scale != 1.0 and getattr(self, "scale_multimodal_embeds", False):
            emb = emb * self.embed_scale
        ops.copy_rows(h, emb, pos.to(h.device, torch.int32), None, pos.numel())
        return h

    def _embed(self, ids, st):
        h = ops.embedding(ids, self.embed_w, self.embed_range[0], self.embed_range[1])
        if self.vocab_parallel_embedding and self.tp.size > 1:
            self.tp.all_reduce_(h)
        if self.embed_scale != 1.0:
            h = h * self.embed_scale
        return self._merge_multimodal(h, st)

    def _lm_head(self, h, normed: bool = False):
        hn = h if normed else ops.rmsnorm(h, self.final_norm_w, self.eps, self.norm_w_offset)
        logits = ops.gemm(hn, self.lm_head_w, epi="f32")
        scale = getattr(self, "logit_scale", 1.0)
        if scale != 1.0:
            logits = logits * scale
        if self.tp.size == 1:
            return logits
        # vocabulary-parallel: the consumer decides whether it needs the gathered matrix (ModelOutput.logits)
        return ShardedLogits(logits, self.tp, self.tp.rank * logits.shape[1], self.vocab)

    def _layers_forward(self, x, st: InferState):
        """x: embeddings [T, H]; returns the final residual stream (pre final-norm).  In the token-sharded mode
        the residual stream is only complete on its owner ranks, so the last reduction applies the final norm and
        the normalised activations are returned instead (st.extra["normed"] tells the caller)."""
        residual = x
        h = ops.rmsnorm(residual, self.layers[0].in_norm, self.eps, self.norm_w_offset)
        n = self.num_layers
        self._tpsp_now = self._tpsp_active(x.shape[0], st)
        bal = st.extra.get("balance")   # data-parallel token balance: attention on the owners, the rest balanced
        for i, lw in enumerate(self.layers):
            if bal is None:
                a = self._attention_block(i, lw, h, st)                  # [T, hq*D] (pre o_proj)
            else:
                a = bal.to_balanced(self._attention_block(i, lw, bal.to_origin(h), st))
            h = self._row_parallel(a, lw.o_w, lw.o_b, residual, lw.post_norm)
            nxt = self.layers[i + 1].in_norm if i + 1 < n else (self.final_norm_w if self._tpsp_now else None)
            f = self._ffn_block(i, lw, h, st)
            if f[0] == "rowpar":    # (activation, down weight): dense row-parallel tail
                h = self._row_parallel(f[1], f[2], None, residual, nxt)
            else:                   # ("partial", tensor): per-rank partial sum of the FFN output (MoE)
                h = self._reduce_partial(f[1], residual, nxt)
            h = self._after_layer(i, residual, h, st)
        if self._tpsp_now:
            self._tpsp_now = False
            st.extra["normed"] = True
            return h
        return residual

    def _after_layer(self, i: int, residual, h, st):
        """Hook run after decoder layer `i`: `residual` is the layer's output stream, `h` the normalised input of the
        next layer (None after the last).  A family that edits the stream here returns the recomputed `h`."""
        return h

    def _tpsp_active(self, T: int, st) -> bool:
        """Token-sharded residual stream (--enable_tpsp_mix_mode) for this pass: needs the fused peer-memory
        kernel, and is skipped when the caller wants the un-normalised hidden states back (draft models)."""
        fused = self.tp.fused
        return bool(getattr(self, "tpsp_mix_mode", False) and fused is not None and self.tp.size > 1
                    and T <= fused.max_tokens and self.hidden == fused.hidden and self.device.type == "cuda"
                    and not st.extra.get("want_hidden"))

    def _partial_out(self, T: int):
        """Buffer a layer should write a to-be-reduced [T, hidden] partial sum into (the symmetric
        buffer of the fused reduction when it is active, else a fresh tensor)."""
        fused = self.tp.fused
        if fused is not None and self.tp.size > 1 and T <= fused.max_tokens and self.hidden == fused.hidden \
                and fused.prefers(T, self.hidden):
            return fused.partial_out(T, self.hidden)
        return torch.empty((T, self.hidden), dtype=self.dtype, device=self.device)

    def _reduce_partial(self, partial, residual, next_norm_w):
        """residual += sum over TP ranks of `partial`; returns rmsnorm(residual) * next_norm_w (or None)."""
        if self.tp.size == 1:
            if next_norm_w is None:
                residual.add_(partial)
                return None
            return ops.add_rmsnorm_(residual, partial, next_norm_w, self.eps, self.norm_w_offset)
        if getattr(self, "_tpsp_now", False):
            fused = self.tp.fused
            if not fused.owns(partial):
                buf = fused.partial_out(partial.shape[0], partial.shape[1])
                buf.copy_(partial)
                partial = buf
            return fused.tpsp_reduce(partial, residual, next_norm_w, self.eps, self.norm_w_offset)
        if next_norm_w is None:
            if self.tp.fused is not None:
                self.tp.fused.skip()
            self.tp.all_reduce_(partial)
            residual.add_(partial)
            return None
        return self.tp.reduce_residual_norm(partial, residual, next_norm_w, self.eps, self.norm_w_offset)

    def _row_parallel(self, a, w, bias, residual, next_norm_w):
        """residual += a . w^T (summed over TP ranks); returns rmsnorm(residual) * next_norm_w (or None)."""
        if self.tp.size == 1:
            ops.gemm(a, w, epi="residual", residual=residual, bias=bias, out=residual)
            if next_norm_w is None:
                return None
            return ops.rmsnorm(residual, next_norm_w, self.eps, self.norm_w_offset)
        fused = self.tp.fused
        if getattr(self, "_tpsp_now", False):
            partial = ops.gemm(a, w, epi="store", bias=bias, out=fused.partial_out(a.shape[0], w.shape[0]))
            return fused.tpsp_reduce(partial, residual, next_norm_w, self.eps, self.norm_w_offset)
        if (fused is not None and next_norm_w is not None and a.is_cuda and isinstance(w, torch.Tensor)
                and fused.can_push(a.shape[0], w.shape[0])):
            # GEMM epilogue pushes the partial tiles to every rank; the reduction + residual + norm reads locally
            T, H = fused.gemm_push(a, w, bias)
            return fused.reduce_pushed(T, H, residual, next_norm_w, self.eps, self.norm_w_offset)
        use_fused = (fused is not None and next_norm_w is not None and a.is_cuda
                     and a.shape[0] <= fused.max_tokens and w.shape[0] == fused.hidden
                     and fused.prefers(a.shape[0], w.shape[0]))
        partial = ops.gemm(a, w, epi="store", bias=bias,
                           out=fused.partial_out(a.shape[0], w.shape[0]) if use_fused else None)
        if next_norm_w is None:
            if fused is not None:
                fused.skip()
            self.tp.all_reduce_(partial)
            residual.add_(partial)
            return None
        return self.tp.reduce_residual_norm(partial, residual, next_norm_w, self.eps, self.norm_w_offset)

    def _attention_block(self, i, lw, h, st: InferState):
        D, hq, hkv = self.head_dim, self.hq, self.hkv
        qkv = ops.gemm(h, lw.qkv_w, bias=lw.qkv_b)
        kv_layer = self._kv_layer(i)
        cos, sin, rope_rows = self._rope_inputs(st, i)
        ops.rope_kv_scatter_(qkv, kv_layer, cos, sin, rope_rows, st.mem_index, hq, hkv, D,
                             self.rot_dim, lw.q_norm, lw.k_norm, self.eps, self.norm_w_offset)
        q = qkv[:, : hq * D]
        r2t = self.req_manager.req_to_token_indexs
        if D not in (64, 128):  # no tensor-core attention kernel for this head size
            o = ops.attention_generic(q, kv_layer, r2t, st.b_req_idx, st.seq_pos,
                                      st.batch_of_token if st.is_prefill else None, hq, hkv, D, self.sm_scale)
        elif st.is_prefill:
            o = ops.gqa_prefill(q, kv_layer, r2t, st.b_req_idx, st.cu_q, st.b_ready_cache_len, hq, hkv, D,
                                st.max_q_len, self.sm_scale)
        else:
            o = ops.gqa_decode(q, kv_layer, r2t, st.b_req_idx, st.b_seq_len, hq, hkv, D, st.max_kv_len,
                               self.sm_scale, num_splits=st.decode_num_splits, scratch=st.decode_scratch)
        return o.view(-1, hq * D)

    def _dense_ffn(self, lw, h):
        if lw.gate_up_fused:
            act = ops.gemm(h, lw.gate_up_w, epi="gated_" + self.act)
        else:
            act = ops.gated_act(ops.gemm(h, lw.gate_up_w), self.act)
        return "rowpar", act, lw.down_w

    def _ffn_block(self, i, lw, h, st):
        return self._dense_ffn(lw, h)

    # ------------------------------------------------------------------ misc
    def check_debug_bounds(self):
        """Raises if the checked build (LLB_DEBUG_BOUNDS=1) saw an index outside its table."""
        if self.debug_status is not None:
            code = int(self.debug_status.item())
            if code:
                what = {901: "KV pool slot", 902: "request row", 903: "request-table column", 904: "expert id"}
                raise RuntimeError(f"index check failed on the device: {what.get(code, code)} out of range")

    def flush_graphs(self):
        self._graphs.clear()

    def param_bytes(self) -> int:
        seen, n = set(), 0
        tensors = [self.embed_w, self.lm_head_w, self.final_norm_w]
        for lw in self.layers:
            vals = list(lw.tensors().values())
            tensors += [t for t in vals if isinstance(t, torch.Tensor)]
            n += sum(t.nbytes() for t in vals if type(t).__name__ in ("Fp8Weight", "Fp8Experts", "Int8Weight"))
        for t in tensors:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        return n
