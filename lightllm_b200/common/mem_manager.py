"""Token-level KV pool ("TokenAttention"): page size = one token.

``kv_buffer[layer, slot, 2*kv_heads_per_rank, head_dim]`` with K heads first, V heads second;
slot ``size`` is the HOLD slot that padded (inactive) batch rows write to.  A stack allocator
hands out slot indices; a request's slots need not be contiguous.  Sized for HBM3e: by default
the pool takes ``mem_fraction`` of the memory left after weights (180 GB parts hold >1M tokens
of an 8B model).

Behavioural counterpart: lightllm/common/kv_cache_mem_manager/mem_manager.py:61-161 and
allocator.py:11-80.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch


class SlotAllocator:
    """LIFO stack of free slot ids kept by the C++ runtime (host side, int32).  `alloc` returns a pinned
    int32 tensor taken from a small ring so an async H2D copy of the previous step's result stays valid."""

    RING = 4

    def __init__(self, size: int, pin: bool = False):
        import ctypes

        from ..ops._native import runtime

        self.size = size
        self._lib = runtime()
        self._lib.llb_slots_create.restype = ctypes.c_void_p
        self._lib.llb_slots_free_count.restype = ctypes.c_int64
        self._ct = ctypes
        self._h = ctypes.c_void_p(self._lib.llb_slots_create(ctypes.c_int64(size)))
        self._pin = pin and torch.cuda.is_available()
        self._ring = [None] * self.RING
        self._ring_i = 0
        self._on_change = None

    def __del__(self):
        try:
            self._lib.llb_slots_destroy(self._h)
        except Exception:
            pass

    @property
    def can_use_mem_size(self) -> int:
        return int(self._lib.llb_slots_free_count(self._h))

    def set_listener(self, fn):
        self._on_change = fn

    def _buf(self, n: int) -> torch.Tensor:
        i = self._ring_i
        self._ring_i = (i + 1) % self.RING
        b = self._ring[i]
        if b is None or b.numel() < n:
            cap = max(n, 4096)
            b = torch.empty(cap, dtype=torch.int32, pin_memory=self._pin)
            self._ring[i] = b
        return b[:n]

    def alloc(self, n: int) -> torch.Tensor:
        """`n` free slot numbers as an int32 host tensor.  The tensor is a view of one of RING reusable (pinned)
        buffers: it is valid until RING - 1 further alloc() calls have been made; keep a copy (`.clone()`) of
        anything needed longer."""
        out = self._buf(n)
        rc = self._lib.llb_slots_alloc(self._h, self._ct.c_int64(n), self._ct.c_void_p(out.data_ptr()))
        if rc != 0:
            raise MemoryError(f"KV pool exhausted: need {n}, free {self.can_use_mem_size}")
        if self._on_change:
            self._on_change(self.can_use_mem_size)
        return out

    def free(self, idx) -> None:
        if isinstance(idx, torch.Tensor):
            idx = idx.detach().cpu().numpy()
        idx = np.ascontiguousarray(idx, dtype=np.int32).reshape(-1)
        n = idx.shape[0]
        if n == 0:
            return
        rc = self._lib.llb_slots_free(self._h, self._ct.c_void_p(idx.ctypes.data), self._ct.c_int64(n))
        assert rc == 0, "double free of KV slots"
        if self._on_change:
            self._on_change(self.can_use_mem_size)

    def free_all(self) -> None:
        self._lib.llb_slots_reset(self._h)
        if self._on_change:
            self._on_change(self.can_use_mem_size)


class MemoryManager:
    """GQA/MHA pool.  `head_num` is the number of KV heads held by this rank."""

    def __init__(self, size: int, dtype: torch.dtype, head_num: int, head_dim: int, layer_num: int,
                 device: torch.device, always_copy: bool = False):
        self.size = int(size)
        self.dtype = dtype
        self.head_num = head_num
        self.head_dim = head_dim
        self.layer_num = layer_num
        self.device = device
        self.HOLD_TOKEN_MEMINDEX = self.size
        self.allocator = SlotAllocator(self.size, pin=device.type == "cuda")
        self._init_buffers()

    # subclasses (MLA, quantised KV) override the next two
    def kv_row_shape(self):
        return (2 * self.head_num, self.head_dim)

    def _init_buffers(self):
        self.kv_buffer = torch.zeros((self.layer_num, self.size + 1, *self.kv_row_shape()), dtype=self.dtype,
                                     device=self.device)

    @staticmethod
    def bytes_per_token(dtype, head_num, head_dim, layer_num) -> int:
        return layer_num * 2 * head_num * head_dim * torch.empty((), dtype=dtype).element_size()

    @property
    def can_use_mem_size(self) -> int:
        return self.allocator.can_use_mem_size

    def alloc(self, n: int) -> torch.Tensor:
        return self.allocator.alloc(n)

    def free(self, idx) -> None:
        self.allocator.free(idx)

    def free_all(self) -> None:
        self.allocator.free_all()

    def layer(self, i: int) -> torch.Tensor:
        return self.kv_buffer[i]

    # ---- KV movement (prefix copies, PD staging pages, host offload) ----
    def gather_pages(self, slots: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """[L, n, ...] staging copy of the given slots (device or pinned-host destination)."""
        from .. import ops

        n = slots.shape[0]
        if out is None:
            out = torch.empty((self.layer_num, n, *self.kv_row_shape()), dtype=self.dtype, device=self.device)
        idx = slots.to(self.device, torch.int32)
        for l in range(self.layer_num):
            ops.copy_rows(out[l], self.kv_buffer[l], None, idx, n)
        return out

    def scatter_pages(self, slots: torch.Tensor, pages: torch.Tensor) -> None:
        from .. import ops

        n = slots.shape[0]
        idx = slots.to(self.device, torch.int32)
        for l in range(self.layer_num):
            ops.copy_rows(self.kv_buffer[l], pages[l], idx, None, n)


class Int8KVMemoryManager(MemoryManager):
    """GQA/MHA pool with int8 rows: every (slot, head) row is `head_dim` int8 values, an fp32 scale and padding to
    a multiple of 16 bytes (`ops/kv_quant.py`).  `layer(i)` returns an `Int8KVLayer`, which the attention ops accept
    in place of a bf16 slice; everything that moves rows (prefix copies, staging pages, host offload) sees opaque
    int8 rows.  Reference: lightllm/common/kv_cache_mem_manager/ppl_int8kv_mem_manager.py (`--llm_kv_type int8kv`)."""

    def __init__(self, size: int, dtype: torch.dtype, head_num: int, head_dim: int, layer_num: int,
                 device: torch.device, always_copy: bool = False):
        self.compute_dtype = dtype
        super().__init__(size, torch.int8, head_num, head_dim, layer_num, device)

    def kv_row_shape(self):
        from ..ops.kv_quant import PAD

        return (2 * self.head_num, self.head_dim + PAD)

    @staticmethod
    def bytes_per_token(dtype, head_num, head_dim, layer_num) -> int:
        from ..ops.kv_quant import PAD

        return layer_num * 2 * head_num * (head_dim + PAD)

    def layer(self, i: int):
        from ..ops.kv_quant import Int8KVLayer

        return Int8KVLayer(self.kv_buffer[i], self.head_dim)


class Fp8KVMemoryManager(MemoryManager):
    """GQA/MHA pool with e4m3 rows and static scales per (layer, head) (`fp8kv_sph`) or per layer for K and for V
    (`fp8kv_spt`), read from a calibration file: JSON with qmin / qmax (the e4m3 limits), num_layers, num_head (KV
    heads of the whole model), quant_type ("per_head" | "per_tensor"), scales (flat list) and scales_shape
    ([layers, 2 * num_head] or [layers, 2]; K first, then V).  Without a file every scale is 1.
    Reference: lightllm/common/kv_cache_mem_manager/fp8_static_per_head_quant_mem_manager.py,
    fp8_static_per_tensor_quant_mem_manager.py."""

    per_tensor = False

    def __init__(self, size: int, dtype: torch.dtype, head_num: int, head_dim: int, layer_num: int,
                 device: torch.device, always_copy: bool = False, calibration: Optional[str] = None,
                 head_range: Optional[tuple] = None):
        self.compute_dtype = dtype
        super().__init__(size, torch.uint8, head_num, head_dim, layer_num, device)
        self.scales = torch.ones((layer_num, 2 * head_num), dtype=torch.float32, device=device)
        if calibration:
            self.load_calibration(calibration, head_range)

    def load_calibration(self, path: str, head_range: Optional[tuple] = None):
        import json

        with open(path) as f:
            cfg = json.load(f)
        lim = float(torch.finfo(torch.float8_e4m3fn).max)
        if abs(float(cfg.get("qmax", lim)) - lim) > 1e-3 or abs(float(cfg.get("qmin", -lim)) + lim) > 1e-3:
            raise ValueError("the calibration file was made for another number format than e4m3")
        want = "per_tensor" if self.per_tensor else "per_head"
        if cfg.get("quant_type", want) != want:
            raise ValueError(f"calibration quant_type {cfg.get('quant_type')!r}, the pool wants {want!r}")
        sc = torch.tensor(cfg["scales"], dtype=torch.float32).view(*cfg["scales_shape"])
        if sc.shape[0] < self.layer_num:     # extra cache layers (draft modules) keep scale 1
            sc = torch.cat([sc, torch.ones(self.layer_num - sc.shape[0], sc.shape[1])])
        sc = sc[: self.layer_num]
        if self.per_tensor:
            k, v = sc[:, :1].expand(-1, self.head_num), sc[:, 1:2].expand(-1, self.head_num)
        else:
            all_heads = sc.shape[1] // 2
            h0, h1 = head_range if head_range is not None else (0, self.head_num)
            if h1 - h0 != self.head_num:      # fewer KV heads than ranks: this rank holds copies of one head
                h1 = h0 + 1
            k, v = sc[:, h0:h1], sc[:, all_heads + h0:all_heads + h1]
            if k.shape[1] != self.head_num:
                k, v = k.expand(-1, self.head_num), v.expand(-1, self.head_num)
        self.scales = torch.cat([k, v], dim=1).contiguous().to(self.device)

    @staticmethod
    def bytes_per_token(dtype, head_num, head_dim, layer_num) -> int:
        return layer_num * 2 * head_num * head_dim

    def layer(self, i: int):
        from ..ops.kv_quant import Fp8KVLayer

        return Fp8KVLayer(self.kv_buffer[i], self.head_dim, self.scales[i])


class Int4KVMemoryManager(MemoryManager):
    """GQA/MHA pool with 4-bit rows and one fp16 scale per group of `group_size` values (`ops/kv_quant.py`:
    Int4KVLayer): a quarter of the bf16 pool's payload plus the scales.  There is no attention kernel over the packed
    rows: every pass attends over a widened copy of the rows its requests refer to, so this pool trades decode speed
    for capacity and decode steps run outside CUDA graphs.
    Reference: lightllm/common/kv_cache_mem_manager/ppl_int4kv_mem_manager.py (`--llm_kv_type int4kv`)."""

    no_cuda_graph = True

    def __init__(self, size: int, dtype: torch.dtype, head_num: int, head_dim: int, layer_num: int,
                 device: torch.device, always_copy: bool = False, group_size: int = 8):
        self.compute_dtype = dtype
        self.group_size = int(group_size or 8)
        if head_dim % self.group_size or self.group_size % 2:
            raise ValueError(f"int4 KV cache: group size {self.group_size} must be even and divide the head size")
        super().__init__(size, torch.uint8, head_num, head_dim, layer_num, device)

    def kv_row_shape(self):
        from ..ops.kv_quant import Int4KVLayer

        return (2 * self.head_num, Int4KVLayer.row_bytes(self.head_dim, self.group_size))

    @staticmethod
    def bytes_per_token(dtype, head_num, head_dim, layer_num, group_size: int = 8) -> int:
        from ..ops.kv_quant import Int4KVLayer

        return layer_num * 2 * head_num * Int4KVLayer.row_bytes(head_dim, group_size)

    def layer(self, i: int):
        from ..ops.kv_quant import Int4KVLayer

        return Int4KVLayer(self.kv_buffer[i], self.head_dim, self.group_size)


class Fp8PerTensorKVMemoryManager(Fp8KVMemoryManager):
    per_tensor = True


class CalibrationKVMemoryManager(MemoryManager):
    """The plain pool that also records, per layer and head, the largest |K| and |V| value written: run
    representative prompts, then `export(path)` writes the scale file the fp8 pools read (scale = amax / 448, per
    head, K heads first).  Selected with kv_type "calibrate" (offline API); every rank of a tensor-parallel run
    exports the heads it holds, `merge_exports` joins them."""

    def __init__(self, size, dtype, head_num, head_dim, layer_num, device, always_copy: bool = False, **_):
        super().__init__(size, dtype, head_num, head_dim, layer_num, device)
        self.amax = torch.zeros((layer_num, 2 * head_num), dtype=torch.float32, device=device)

    def layer(self, i: int):
        from ..ops.kv_quant import CalibratingKVLayer

        return CalibratingKVLayer(self.kv_buffer[i], self.head_dim, self.amax[i])

    def export(self, path: str, architectures=None, per_tensor: bool = False, num_layers: Optional[int] = None):
        import json

        lim = float(torch.finfo(torch.float8_e4m3fn).max)
        L = num_layers or self.layer_num
        amax = self.amax[:L].float().cpu().clamp_min(1e-6)
        if per_tensor:
            H = self.head_num
            amax = torch.stack([amax[:, :H].amax(1), amax[:, H:].amax(1)], dim=1)
        scales = amax / lim
        cfg = {"qmin": -lim, "qmax": lim, "num_layers": L, "num_head": self.head_num,
               "quant_type": "per_tensor" if per_tensor else "per_head", "architectures": architectures,
               "scales": scales.flatten().tolist(), "scales_shape": list(scales.shape)}
        with open(path, "w") as f:
            json.dump(cfg, f)
        return cfg

    @staticmethod
    def merge_exports(paths, out_path: str):
        """Joins per-rank per-head files (rank order) into one file for the whole model."""
        import json

        parts = [json.load(open(p)) for p in paths]
        L = parts[0]["num_layers"]
        ks, vs = [], []
        for c in parts:
            sc = torch.tensor(c["scales"]).view(*c["scales_shape"])
            h = sc.shape[1] // 2
            ks.append(sc[:, :h])
            vs.append(sc[:, h:])
        sc = torch.cat(ks + vs, dim=1)
        cfg = dict(parts[0], num_head=sc.shape[1] // 2, scales=sc.flatten().tolist(), scales_shape=[L, sc.shape[1]])
        with open(out_path, "w") as f:
            json.dump(cfg, f)
        return cfg


KV_MANAGERS = {"none": MemoryManager, "calibrate": CalibrationKVMemoryManager, "int8kv": Int8KVMemoryManager, "fp8kv_sph": Fp8KVMemoryManager,
               "fp8kv_spt": Fp8PerTensorKVMemoryManager, "int4kv": Int4KVMemoryManager}


def select_mem_manager_class(kv_type: Optional[str]):
    """Pool class for `--llm_kv_type` (reference: kv_cache_mem_manager/mem_utils.py select_mem_manager_class)."""
    k = (kv_type or "none").lower()
    if k not in KV_MANAGERS:
        raise ValueError(f"--llm_kv_type {kv_type!r} is not available (have: {sorted(KV_MANAGERS)})")
    return KV_MANAGERS[k]


class MLAMemoryManager(MemoryManager):
    """DeepSeek MLA latent cache: one row [kv_lora_rank + qk_rope_head_dim] per token and layer
    (lightllm/common/kv_cache_mem_manager/deepseek2_mem_manager.py)."""

    def __init__(self, size, dtype, kv_lora_rank, rope_dim, layer_num, device):
        self.kv_lora_rank = kv_lora_rank
        self.rope_dim = rope_dim
        super().__init__(size, dtype, 1, kv_lora_rank + rope_dim, layer_num, device)

    def kv_row_shape(self):
        return (1, self.kv_lora_rank + self.rope_dim)

    @staticmethod
    def bytes_per_token(dtype, kv_lora_rank, rope_dim, layer_num) -> int:
        return layer_num * (kv_lora_rank + rope_dim) * torch.empty((), dtype=dtype).element_size()


def profile_max_tokens(device: torch.device, bytes_per_token: int, mem_fraction: float = 0.9,
                       reserve_bytes: int = 6 << 30) -> int:
    """Tokens that fit in `mem_fraction` of the currently free device memory, leaving `reserve_bytes`
    for activations and CUDA graphs."""
    if device.type != "cuda":
        return 16384
    free, total = torch.cuda.mem_get_info(device)
    usable = int(free * mem_fraction) - reserve_bytes
    return max(usable // bytes_per_token, 1024)
