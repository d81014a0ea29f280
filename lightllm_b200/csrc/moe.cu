// Mixture-of-experts routing and data movement kernels.
//
//   topk_softmax     softmax over E expert logits, top-k, optional renormalisation  (Qwen3-MoE, Mixtral)
//   grouped_topk     sigmoid (or softmax) scores + correction bias, experts arranged in groups, the
//                    topk_group best groups (by the sum of their two best biased scores) stay, top-k
//                    inside them, weights from the unbiased scores, renormalised and scaled (DeepSeek-V3)
//   moe_align        counting sort of the T*k (token, slot) pairs by expert: per-expert row ranges padded
//                    to 128 rows, the source pair of every sorted row, and the expert of every 128-row block
//   moe_gather       A_sorted[row] = x[token of row]   (zero rows for padding)
//   moe_combine      out[t] = sum_k w[t,k] * y[row of (t,k)]   (+ optional shared-expert output)
//
// One warp per token for the routers (E <= 512); one CTA does the sort (T*k up to a few 100k pairs).
// Reference behaviour: lightllm/common/basemodel/triton_kernel/fused_moe/{topk_select,grouped_topk,
// softmax_topk,grouped_fused_moe (moe_align*), moe_sum_reduce}.py.
#include "common.cuh"

using namespace llb;
LLB_DEBUG_BOUNDS_STORAGE(moe)


namespace {

constexpr int MAX_E_PER_LANE = 16;  // E <= 512

// Picks the top-k of per-lane candidate arrays (value v[j] belongs to expert lane + 32*j) by k rounds of
// warp arg-max; ties go to the lower expert id.  `sel` (optional) receives a copy of the selected scores.
template <typename F>
__device__ __forceinline__ void warp_topk(float* v, int n_per_lane, int k, F emit) {
  const int lane = threadIdx.x & 31;
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = 0; j < n_per_lane; ++j) {
      if (v[j] > best) {
        best = v[j];
        bi = lane + 32 * j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    emit(r, bi, best);
    if ((bi & 31) == lane && bi != 0x7fffffff) v[bi >> 5] = -INFINITY;
  }
}

template <typename T>
__device__ __forceinline__ float ld_f(const T* p, int64_t i);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p, int64_t i) {
  return p[i];
}
template <>
__device__ __forceinline__ float ld_f<bf16>(const bf16* p, int64_t i) {
  return __bfloat162float(p[i]);
}

template <typename T>
__global__ void __launch_bounds__(128) topk_softmax_kernel(const T* __restrict__ logits, int64_t stride, int Tn, int E,
                                                           int k, int renorm, float scale, int* __restrict__ ids,
                                                           float* __restrict__ weights) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const int lane = threadIdx.x & 31;
  const int npl = (E + 31) >> 5;
  float v[MAX_E_PER_LANE];
  float mx = -INFINITY;
  for (int j = 0; j < npl; ++j) {
    int e = lane + 32 * j;
    v[j] = e < E ? ld_f(logits, (int64_t)t * stride + e) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float z = 0.f;
  for (int j = 0; j < npl; ++j) {
    v[j] = (lane + 32 * j) < E ? __expf(v[j] - mx) : -INFINITY;
    if (lane + 32 * j < E) z += v[j];
  }
  z = warp_sum(z);
  float sel_sum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  warp_topk(v, npl, k, [&](int r, int e, float val) {
    sel_sum += val;
    if (r == lane) {
      my_w = val;
      my_id = e;
    }
  });
  // k <= 32: lane r holds the r-th choice
  if (lane < k) {
    float w = my_w / (renorm ? sel_sum : z);
    ids[(int64_t)t * k + lane] = my_id;
    weights[(int64_t)t * k + lane] = w * scale;
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
grouped_topk_kernel(const T* __restrict__ logits, int64_t stride, const float* __restrict__ bias, int Tn, int E, int k,
                    int n_group, int topk_group, int use_sigmoid, int renorm, float scale, int* __restrict__ ids,
                    float* __restrict__ weights) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const int lane = threadIdx.x & 31;
  const int npl = (E + 31) >> 5;
  const int gsz = E / n_group;
  __shared__ float s_score[4][512];   // unbiased scores
  __shared__ float s_biased[4][512];  // scores + correction bias (selection only)
  __shared__ float s_group[4][32];
  float* sc = s_score[threadIdx.x >> 5];
  float* sb = s_biased[threadIdx.x >> 5];
  float* sg = s_group[threadIdx.x >> 5];
  float mx = -INFINITY;
  for (int j = 0; j < npl; ++j) {
    int e = lane + 32 * j;
    if (e < E) mx = fmaxf(mx, ld_f(logits, (int64_t)t * stride + e));
  }
  mx = warp_max(mx);
  float z = 0.f;
  for (int j = 0; j < npl; ++j) {
    int e = lane + 32 * j;
    if (e < E) {
      float x = ld_f(logits, (int64_t)t * stride + e);
      float s = use_sigmoid ? 1.f / (1.f + __expf(-x)) : __expf(x - mx);
      sc[e] = s;
      z += s;
    }
  }
  z = warp_sum(z);
  for (int j = 0; j < npl; ++j) {
    int e = lane + 32 * j;
    if (e < E) {
      if (!use_sigmoid) sc[e] /= z;
      sb[e] = sc[e] + (bias ? bias[e] : 0.f);
    }
  }
  __syncwarp();
  // group score: sum of the two best biased scores of the group (with a bias) or the best one (without)
  if (lane < n_group) {
    float b1 = -INFINITY, b2 = -INFINITY;
    for (int i = 0; i < gsz; ++i) {
      float x = sb[lane * gsz + i];
      if (x > b1) {
        b2 = b1;
        b1 = x;
      } else if (x > b2) {
        b2 = x;
      }
    }
    sg[lane] = bias ? (b1 + b2) : b1;
  }
  __syncwarp();
  // keep the topk_group best groups
  float gv[1] = {lane < n_group ? sg[lane] : -INFINITY};
  unsigned keep_mask = 0;
  warp_topk(gv, 1, topk_group, [&](int r, int g, float val) { keep_mask |= 1u << g; });
  float v[MAX_E_PER_LANE];
  for (int j = 0; j < npl; ++j) {
    int e = lane + 32 * j;
    v[j] = (e < E && ((keep_mask >> (e / gsz)) & 1u)) ? sb[e] : -INFINITY;
  }
  float sel_sum = 0.f, my_w = 0.f;
  int my_id = 0;
  warp_topk(v, npl, k, [&](int r, int e, float val) {
    float w = (e != 0x7fffffff) ? sc[e] : 0.f;
    sel_sum += w;
    if (r == lane) {
      my_w = w;
      my_id = e == 0x7fffffff ? 0 : e;
    }
  });
  if (lane < k) {
    float w = renorm ? my_w / (sel_sum + 1e-20f) : my_w;
    ids[(int64_t)t * k + lane] = my_id;
    weights[(int64_t)t * k + lane] = w * scale;
  }
}

// ---- alignment (counting sort by expert) ----
// pairs: p = t*k + slot, expert ids[p] (ids outside [e0, e0+E_local) are dropped: expert parallel ranks)
// outputs: sorted_pair[M_pad] (pair index of each sorted row, -1 for padding), pair_row[T*k] (row of each pair,
// -1 if dropped), mblock_expert[M_pad/128] (local expert id or -1), expert_rows[E_local+1] (padded offsets),
// total_rows[1]
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int n_pairs, int e0, int E_local, int m_pad, int* __restrict__ sorted_pair,
                 int* __restrict__ pair_row, int* __restrict__ mblock_expert, int* __restrict__ expert_off,
                 int* __restrict__ total_rows) {
  extern __shared__ int sm[];
  int* cnt = sm;                 // [E_local]
  int* off = sm + E_local;       // [E_local + 1]
  int* cur = sm + 2 * E_local + 1;  // [E_local]
  for (int i = threadIdx.x; i < E_local; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    int e = (ids[p] < 0 ? ids[p] : LLB_CHECK_EXPERT(ids[p])) - e0;
    if (e >= 0 && e < E_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E_local; ++e) {
      off[e] = acc;
      acc += ((cnt[e] + 127) / 128) * 128;
    }
    off[E_local] = acc;
    total_rows[0] = acc;
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= E_local; i += blockDim.x) expert_off[i] = off[i];
  for (int i = threadIdx.x; i < E_local; i += blockDim.x) cur[i] = 0;
  for (int r = threadIdx.x; r < m_pad; r += blockDim.x) sorted_pair[r] = -1;
  for (int b = threadIdx.x; b < m_pad / 128; b += blockDim.x) {
    // expert of block b: the one whose padded range contains row b*128
    int row = b * 128, e = -1;
    if (row < off[E_local]) {
      int lo = 0, hi = E_local - 1;
      while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (off[mid] <= row) lo = mid; else hi = mid - 1;
      }
      e = lo;
      // skip experts with zero rows that share the same offset
      while (e + 1 < E_local && off[e + 1] <= row) ++e;
    }
    mblock_expert[b] = e;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    int e = ids[p] - e0;
    if (e >= 0 && e < E_local) {
      int r = off[e] + atomicAdd(&cur[e], 1);
      sorted_pair[r] = p;
      pair_row[p] = r;
    } else {
      pair_row[p] = -1;
    }
  }
}

// A_sorted[row] = x[sorted_pair[row] / k]  (zeros for padding rows)
__global__ void __launch_bounds__(256)
moe_gather_kernel(bf16* __restrict__ a_sorted, const bf16* __restrict__ x, const int* __restrict__ sorted_pair,
                  const int* __restrict__ total_rows, int k, int H_vec, int64_t x_stride_vec) {
  const int rows = total_rows[0];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const int p = sorted_pair[r];
    uint4* dst = reinterpret_cast<uint4*>(a_sorted) + (int64_t)r * H_vec;
    if (p < 0) {
      for (int v = threadIdx.x; v < H_vec; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(x) + (int64_t)(p / k) * x_stride_vec;
      for (int v = threadIdx.x; v < H_vec; v += blockDim.x) dst[v] = src[v];
    }
  }
}

// out[t] = (accumulate ? out[t] : 0) + sum_k w[t,k] * y[pair_row[t*k + s]]
__global__ void __launch_bounds__(256)
moe_combine_kernel(bf16* __restrict__ out, const bf16* __restrict__ y, const int* __restrict__ pair_row,
                   const float* __restrict__ weights, int k, int H_vec, int accumulate) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < H_vec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (accumulate) unpack8(reinterpret_cast<const bf16x8*>(out)[(int64_t)t * H_vec + v], acc);
    for (int s = 0; s < k; ++s) {
      const int r = pair_row[t * k + s];
      if (r < 0) continue;
      const float w = weights[t * k + s];
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(y)[(int64_t)r * H_vec + v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += w * f[i];
    }
    reinterpret_cast<bf16x8*>(out)[(int64_t)t * H_vec + v] = pack8(acc);
  }
}

}  // namespace

// dtype: 0 = fp32 logits, 1 = bf16 logits
LLB_EXPORT int llb_topk_softmax(const void* logits, int dtype, int64_t stride, int T, int E, int k, int renorm,
                                float scale, int* ids, float* weights, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (E > 512 || k > 32 || k > E) return LLB_ERR_UNSUPPORTED;
  if (dtype == 0)
    topk_softmax_kernel<float><<<cdiv(T, 4), 128, 0, st>>>((const float*)logits, stride, T, E, k, renorm, scale, ids, weights);
  else
    topk_softmax_kernel<bf16><<<cdiv(T, 4), 128, 0, st>>>((const bf16*)logits, stride, T, E, k, renorm, scale, ids, weights);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_grouped_topk(const void* logits, int dtype, int64_t stride, const float* bias, int T, int E, int k,
                                int n_group, int topk_group, int use_sigmoid, int renorm, float scale, int* ids,
                                float* weights, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (E > 512 || k > 32 || n_group > 32 || E % n_group != 0 || topk_group > n_group) return LLB_ERR_UNSUPPORTED;
  if (dtype == 0)
    grouped_topk_kernel<float><<<cdiv(T, 4), 128, 0, st>>>((const float*)logits, stride, bias, T, E, k, n_group,
                                                            topk_group, use_sigmoid, renorm, scale, ids, weights);
  else
    grouped_topk_kernel<bf16><<<cdiv(T, 4), 128, 0, st>>>((const bf16*)logits, stride, bias, T, E, k, n_group,
                                                           topk_group, use_sigmoid, renorm, scale, ids, weights);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// Redundant experts under expert parallelism: counts how often every expert is chosen (the statistic the placement
// of redundant experts is taken from) and rewrites the router's expert ids into the "physical" id space
// rank x (experts per rank + redundant per rank) through this rank's table, in which an expert this rank holds a
// copy of points at the copy.
__global__ void moe_count_remap_kernel(const int* __restrict__ ids, int n_pairs, const int* __restrict__ table, int E,
                                       int* __restrict__ counter, int* __restrict__ out) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    int e = ids[i];
    if (e < 0 || e >= E) {
      out[i] = -1;
      continue;
    }
    if (counter != nullptr) atomicAdd(counter + e, 1);
    out[i] = table[e];
  }
}

// Routed-expert capture: buf[slot[t], layer, :] = ids[t, :] as 8- or 16-bit integers (buf is [slots, layers, k]).
template <typename OUT>
__global__ void route_capture_kernel(const int* __restrict__ ids, const int* __restrict__ slot, int n_pairs, int k,
                                     OUT* __restrict__ buf, int n_slots, int n_layers, int layer) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    int t = i / k, j = i - t * k;
    int s = slot[t];
    if (s < 0 || s >= n_slots) continue;
    buf[((int64_t)s * n_layers + layer) * k + j] = (OUT)ids[i];
  }
}

LLB_EXPORT int llb_route_capture(const int* ids, const int* slot, int T, int k, void* buf, int n_slots, int n_layers,
                                 int layer, int elem_bytes, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (elem_bytes != 1 && elem_bytes != 2) return LLB_ERR_UNSUPPORTED;
  int n = T * k, blocks = cdiv(n, 256);
  if (blocks > 296) blocks = 296;
  if (elem_bytes == 1)
    route_capture_kernel<uint8_t><<<blocks, 256, 0, st>>>(ids, slot, n, k, (uint8_t*)buf, n_slots, n_layers, layer);
  else
    route_capture_kernel<int16_t><<<blocks, 256, 0, st>>>(ids, slot, n, k, (int16_t*)buf, n_slots, n_layers, layer);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_moe_count_remap(const int* ids, int n_pairs, const int* table, int E, int* counter, int* out,
                                   cudaStream_t st) {
  if (n_pairs <= 0) return LLB_OK;
  int blocks = cdiv(n_pairs, 256);
  moe_count_remap_kernel<<<blocks < 296 ? blocks : 296, 256, 0, st>>>(ids, n_pairs, table, E, counter, out);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_moe_align(const int* ids, int n_pairs, int e0, int E_local, int m_pad, int* sorted_pair,
                             int* pair_row, int* mblock_expert, int* expert_off, int* total_rows, cudaStream_t st) {
  if (E_local > 2048 || m_pad % 128 != 0) return LLB_ERR_UNSUPPORTED;
  int smem = (3 * E_local + 1) * sizeof(int);
  moe_align_kernel<<<1, 1024, smem, st>>>(ids, n_pairs, e0, E_local, m_pad, sorted_pair, pair_row, mblock_expert,
                                          expert_off, total_rows);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_moe_gather(void* a_sorted, const void* x, const int* sorted_pair, const int* total_rows, int k,
                              int H, int64_t x_stride, int max_rows, cudaStream_t st) {
  if (max_rows <= 0) return LLB_OK;
  if (H % 8 || x_stride % 8) return LLB_ERR_UNSUPPORTED;
  int blocks = max_rows < 148 * 8 ? max_rows : 148 * 8;
  moe_gather_kernel<<<blocks, 256, 0, st>>>((bf16*)a_sorted, (const bf16*)x, sorted_pair, total_rows, k, H / 8,
                                            x_stride / 8);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_moe_combine(void* out, const void* y, const int* pair_row, const float* weights, int T, int k, int H,
                               int accumulate, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (H % 8) return LLB_ERR_UNSUPPORTED;
  moe_combine_kernel<<<T, 256, 0, st>>>((bf16*)out, (const bf16*)y, pair_row, weights, k, H / 8, accumulate);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// ---------------------------------------------------------------------------------------
// Experts with biases (GPT-OSS): the grouped GEMMs run with the plain store epilogue and these two kernels add
// the per-expert bias rows.  Rows live in 128-row blocks of one expert each (mblock_expert, -1 = padding block).
//   moe_bias_act: h [M_pad, 2I] with gate / up interleaved in 32-column blocks -> out [M_pad, I]
//     kind 0 / 1: SiLU / GELU(tanh) gate;  kind 2: clamped "swiglu_oai":
//       g = min(g, limit); u = clamp(u, -limit, limit); out = (u + 1) * g * sigmoid(alpha * g)
//   moe_add_bias: y [M_pad, H] += b2[expert of the row's block]
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_bias_act_kernel(const bf16* __restrict__ h, const bf16* __restrict__ b13,
                                                           const int* __restrict__ mblock_expert,
                                                           bf16* __restrict__ out, int I, int kind, float alpha,
                                                           float limit) {
  const int row = blockIdx.x;
  const int e = mblock_expert[row >> 7];
  if (e < 0) return;
  const bf16* hr = h + (int64_t)row * 2 * I;
  const bf16* br = b13 ? b13 + (int64_t)e * 2 * I : nullptr;
  for (int i = threadIdx.x; i < I; i += blockDim.x) {
    const int blk = i >> 5, j = i & 31;
    const int gi = blk * 64 + j, ui = gi + 32;
    float g = __bfloat162float(hr[gi]), u = __bfloat162float(hr[ui]);
    if (br) {
      g += __bfloat162float(br[gi]);
      u += __bfloat162float(br[ui]);
    }
    float o;
    if (kind == 2) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      o = (u + 1.f) * g / (1.f + __expf(-alpha * g));
    } else if (kind == 1) {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      o = 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g))) * u;
    } else {
      o = g / (1.f + __expf(-g)) * u;
    }
    out[(int64_t)row * I + i] = __float2bfloat16(o);
  }
}

__global__ void __launch_bounds__(256) moe_add_bias_kernel(bf16* __restrict__ y, const bf16* __restrict__ b2,
                                                           const int* __restrict__ mblock_expert, int H) {
  const int row = blockIdx.x;
  const int e = mblock_expert[row >> 7];
  if (e < 0) return;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    y[(int64_t)row * H + i] = __float2bfloat16(__bfloat162float(y[(int64_t)row * H + i]) +
                                                __bfloat162float(b2[(int64_t)e * H + i]));
}

LLB_EXPORT int llb_moe_bias_act(const void* h, const void* b13, const int* mblock_expert, void* out, int M_pad, int I,
                                int kind, float alpha, float limit, cudaStream_t st) {
  if (M_pad <= 0) return LLB_OK;
  if ((I % 32) || kind < 0 || kind > 2) return LLB_ERR_UNSUPPORTED;
  moe_bias_act_kernel<<<M_pad, 256, 0, st>>>((const bf16*)h, (const bf16*)b13, mblock_expert, (bf16*)out, I, kind, alpha,
                                             limit);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_moe_add_bias(void* y, const void* b2, const int* mblock_expert, int M_pad, int H, cudaStream_t st) {
  if (M_pad <= 0) return LLB_OK;
  moe_add_bias_kernel<<<M_pad, 256, 0, st>>>((bf16*)y, (const bf16*)b2, mblock_expert, H);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
