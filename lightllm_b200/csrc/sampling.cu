// Token sampling over fp32 logits [B, V]: penalties, temperature, softmax, top-k / top-p
// filtering and the draw itself, one CTA per request, no sort.
//
//   * the top-k / top-p cut is found by bisection on the logit value: the kept set is
//     S(tau) = {i : x_i >= tau}; the largest tau with |S| >= k or mass(S) >= p is the
//     tighter of the two filters (each pass is one sweep over the row, served by L2);
//   * the draw is an exponential race: argmax_i p_i / E_i with E_i ~ Exp(1) from a
//     counter-based generator keyed by (seed, step, i), so a request with a fixed seed
//     reproduces its stream whatever batch it lands in;
//   * greedy rows (top_k == 1) take the argmax of the penalised logits in the first sweep.
//
// Behavioural counterpart in the reference: lightllm/server/router/model_infer/mode_backend/
// generic_post_process.py (sample) and common/basemodel/triton_kernel/apply_penalty.py.
#include "common.cuh"

using namespace llb;

namespace {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t step, uint32_t i) {
  uint64_t h = splitmix64(seed ^ splitmix64(step * 0x100000001B3ull + i));
  return ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* sh) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax t;
    t.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    t.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, t);
  }
  __syncthreads();
  if (lane == 0) sh[w] = a;
  __syncthreads();
  if (w == 0) {
    ArgMax t = lane < nw ? sh[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax u;
      u.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      u.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, u);
    }
    if (lane == 0) sh[32] = t;
  }
  __syncthreads();
  return sh[32];
}

// ---- penalties (in place) ----
// CSR per request: ids/counts of tokens generated so far (and prompt tokens when input_penalty).
__global__ void __launch_bounds__(256)
apply_penalty_kernel(float* __restrict__ logits, int64_t stride, const float* __restrict__ presence,
                     const float* __restrict__ frequency, const float* __restrict__ repetition,
                     const int* __restrict__ cu, const int* __restrict__ tok_ids, const int* __restrict__ tok_cnt,
                     const int* __restrict__ mask_cu, const int* __restrict__ mask_ids, int V) {
  int b = blockIdx.x;
  float* row = logits + (int64_t)b * stride;
  if (cu != nullptr) {
    float pp = presence[b], fp = frequency[b], rp = repetition[b];
    for (int j = cu[b] + threadIdx.x; j < cu[b + 1]; j += blockDim.x) {
      int id = tok_ids[j];
      if (id < 0 || id >= V) continue;
      float c = (float)tok_cnt[j];
      float x = row[id];
      x = x > 0.f ? x / rp : x * rp;
      x -= fp * c + pp;
      row[id] = x;
    }
  }
  if (mask_cu != nullptr) {
    __syncthreads();
    for (int j = mask_cu[b] + threadIdx.x; j < mask_cu[b + 1]; j += blockDim.x) {
      int id = mask_ids[j];
      if (id >= 0 && id < V) row[id] = -INFINITY;
    }
  }
}

// ---- the sampler ----
template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, int i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, int i) {
  return p[i];
}
template <>
__device__ __forceinline__ float ld_logit<bf16>(const bf16* p, int i) {
  return __bfloat162float(p[i]);
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, int64_t stride, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const int* __restrict__ top_k, const uint64_t* __restrict__ seeds,
              const int64_t* __restrict__ steps, int64_t* __restrict__ out_ids, float* __restrict__ out_logprob) {
  __shared__ float red[33];
  __shared__ ArgMax am[33];
  const int b = blockIdx.x;
  const T* row = logits + (int64_t)b * stride;
  const int k = top_k ? top_k[b] : 1;
  const bool greedy = (k == 1);
  float temp = temperature ? temperature[b] : 1.f;
  if (greedy || temp < 1e-5f) temp = 1.f;
  const float inv_t = 1.f / temp;

  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float x = ld_logit(row, i) * inv_t;
    best = better(best, ArgMax{x, i});
  }
  best = block_argmax(best, am);
  const float xmax = best.v;
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += __expf(ld_logit(row, i) * inv_t - xmax);
  z = block_sum(z, red);
  const float logz = __logf(z);

  if (greedy || (temperature && temperature[b] < 1e-5f)) {
    if (threadIdx.x == 0) {
      out_ids[b] = best.i;
      if (out_logprob) out_logprob[b] = -logz;
    }
    return;
  }

  const float p_lim = top_p ? top_p[b] : 1.f;
  const bool use_p = p_lim < 1.f;
  const bool use_k = k > 0 && k < V;
  float tau = -INFINITY;  // keep everything
  if (use_p || use_k) {
    float lo = xmax - 30.f, hi = xmax;  // predicate true at lo (or the tail below it is < 1e-13 of the mass)
    const float need_mass = p_lim * z;
    for (int it = 0; it < 24; ++it) {
      float mid = 0.5f * (lo + hi);
      float cnt = 0.f, mass = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float x = ld_logit(row, i) * inv_t;
        if (x >= mid) {
          cnt += 1.f;
          mass += __expf(x - xmax);
        }
      }
      cnt = block_sum(cnt, red);
      mass = block_sum(mass, red);
      bool ok = (use_k && cnt >= (float)k) || (use_p && mass >= need_mass);
      if (ok)
        lo = mid;
      else
        hi = mid;
    }
    tau = lo;
  }

  const uint64_t seed = seeds ? seeds[b] : 0x1234ull + b;
  const uint64_t step = steps ? (uint64_t)steps[b] : 0ull;
  ArgMax pick{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float x = ld_logit(row, i) * inv_t;
    if (x >= tau) {
      float u = uniform01(seed, step, (uint32_t)i);
      float key = x - __logf(-__logf(u));
      pick = better(pick, ArgMax{key, i});
    }
  }
  pick = block_argmax(pick, am);
  if (threadIdx.x == 0) {
    int id = pick.i == 0x7fffffff ? best.i : pick.i;
    out_ids[b] = id;
    if (out_logprob) out_logprob[b] = ld_logit(row, id) * inv_t - xmax - logz;
  }
}

// log-softmax value of given token ids (prompt_logprobs / chosen-token logprob): out[b] = log p(ids[b])
template <typename T>
__global__ void __launch_bounds__(1024)
token_logprob_kernel(const T* __restrict__ logits, int64_t stride, int V, const int64_t* __restrict__ ids,
                     float* __restrict__ out) {
  __shared__ float red[33];
  const int b = blockIdx.x;
  const T* row = logits + (int64_t)b * stride;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, ld_logit(row, i));
  mx = block_max(mx, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += __expf(ld_logit(row, i) - mx);
  z = block_sum(z, red);
  if (threadIdx.x == 0) {
    int64_t id = ids[b];
    out[b] = (id >= 0 && id < V) ? ld_logit(row, (int)id) - mx - __logf(z) : -INFINITY;
  }
}

}  // namespace

LLB_EXPORT int llb_apply_penalty(float* logits, int64_t stride, const float* presence, const float* frequency,
                                 const float* repetition, const int* cu, const int* tok_ids, const int* tok_cnt,
                                 const int* mask_cu, const int* mask_ids, int B, int V, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  apply_penalty_kernel<<<B, 256, 0, st>>>(logits, stride, presence, frequency, repetition, cu, tok_ids, tok_cnt,
                                          mask_cu, mask_ids, V);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// dtype: 0 = fp32 logits, 1 = bf16 logits
LLB_EXPORT int llb_sample(const void* logits, int dtype, int64_t stride, int B, int V, const float* temperature,
                          const float* top_p, const int* top_k, const uint64_t* seeds, const int64_t* steps,
                          int64_t* out_ids, float* out_logprob, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (dtype == 0)
    sample_kernel<float><<<B, 1024, 0, st>>>((const float*)logits, stride, V, temperature, top_p, top_k, seeds, steps,
                                             out_ids, out_logprob);
  else if (dtype == 1)
    sample_kernel<bf16><<<B, 1024, 0, st>>>((const bf16*)logits, stride, V, temperature, top_p, top_k, seeds, steps,
                                            out_ids, out_logprob);
  else
    return LLB_ERR_UNSUPPORTED;
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// ---- all-greedy batches: arg-max + log-probability in two small passes over many CTAs ----
// pass 1: CTA (b, s) scans slice s of row b (coalesced loads) and keeps (max, arg-max, sum exp(x - max));
// pass 2: one warp per row merges the S partials.  part: [B, S, 3] floats (max, index bits, sum).
// `idx_off` is added to the stored arg-max index: a tensor-parallel rank that holds columns [idx_off, idx_off + V)
// of the full vocabulary writes global token ids, so the partials of all ranks can be merged as they are.
template <typename T>
__global__ void __launch_bounds__(256) greedy_partial_kernel(const T* __restrict__ logits, int64_t stride, int V,
                                                             int per, float* __restrict__ part, int idx_off) {
  __shared__ float red[33];
  __shared__ ArgMax am[33];
  const int b = blockIdx.x, s = blockIdx.y, S = gridDim.y;
  const T* row = logits + (int64_t)b * stride;
  const int i0 = s * per, i1 = min(V, i0 + per);
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) best = better(best, ArgMax{ld_logit(row, i), i});
  best = block_argmax(best, am);
  float z = 0.f;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) z += __expf(ld_logit(row, i) - best.v);
  z = block_sum(z, red);
  if (threadIdx.x == 0) {
    float* o = part + ((int64_t)b * S + s) * 3;
    o[0] = best.v;
    o[1] = __int_as_float(i1 > i0 ? best.i + idx_off : 0x7fffffff);
    o[2] = i1 > i0 ? z : 0.f;
  }
}

// part: [R, B, S, 3]; R > 1 when the partials of R vocabulary shards (tensor-parallel ranks) were gathered.
__global__ void greedy_final_kernel(const float* __restrict__ part, int S, int R, int64_t* __restrict__ out_ids,
                                    float* __restrict__ out_logprob) {
  const int b = blockIdx.x, lane = threadIdx.x, B = gridDim.x;
  const int n = S * R;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int j = lane; j < n; j += 32) {
    const float* o = part + (((int64_t)(j / S) * B + b) * S + (j % S)) * 3;
    best = better(best, ArgMax{o[0], __float_as_int(o[1])});
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) {
    ArgMax t;
    t.v = __shfl_xor_sync(0xffffffffu, best.v, k);
    t.i = __shfl_xor_sync(0xffffffffu, best.i, k);
    best = better(best, t);
  }
  float z = 0.f;
  for (int j = lane; j < n; j += 32) {
    const float* o = part + (((int64_t)(j / S) * B + b) * S + (j % S)) * 3;
    if (o[2] > 0.f) z += o[2] * __expf(o[0] - best.v);
  }
  z = warp_sum(z);
  if (lane == 0) {
    out_ids[b] = best.i;
    if (out_logprob) out_logprob[b] = -__logf(z);
  }
}

// scratch: B * splits * 3 floats.
LLB_EXPORT int llb_sample_greedy(const void* logits, int dtype, int64_t stride, int B, int V, float* scratch, int splits,
                                 int64_t* out_ids, float* out_logprob, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (splits < 1 || splits > 1024 || scratch == nullptr) return LLB_ERR_BAD_ARG;
  const int per = ((V + splits - 1) / splits + 3) & ~3;
  dim3 grid(B, splits);
  if (dtype == 0)
    greedy_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)logits, stride, V, per, scratch, 0);
  else if (dtype == 1)
    greedy_partial_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)logits, stride, V, per, scratch, 0);
  else
    return LLB_ERR_UNSUPPORTED;
  LLB_LAUNCH_CHECK();
  greedy_final_kernel<<<B, 32, 0, st>>>(scratch, splits, 1, out_ids, out_logprob);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// The two passes on their own, for vocabulary-parallel logits: every rank runs the first pass over its shard
// (`idx_off` = first token id of the shard), the [B, splits, 3] partials of all ranks are exchanged (a few KB
// instead of the logits), and the second pass merges `ranks` of them: part [ranks, B, splits, 3].
LLB_EXPORT int llb_greedy_partial(const void* logits, int dtype, int64_t stride, int B, int V, int idx_off, float* part,
                                  int splits, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (splits < 1 || splits > 1024 || part == nullptr) return LLB_ERR_BAD_ARG;
  const int per = ((V + splits - 1) / splits + 3) & ~3;
  dim3 grid(B, splits);
  if (dtype == 0)
    greedy_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)logits, stride, V, per, part, idx_off);
  else if (dtype == 1)
    greedy_partial_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)logits, stride, V, per, part, idx_off);
  else
    return LLB_ERR_UNSUPPORTED;
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_greedy_merge(const float* part, int B, int splits, int ranks, int64_t* out_ids, float* out_logprob,
                                cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (splits < 1 || ranks < 1 || part == nullptr) return LLB_ERR_BAD_ARG;
  greedy_final_kernel<<<B, 32, 0, st>>>(part, splits, ranks, out_ids, out_logprob);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_token_logprob(const void* logits, int dtype, int64_t stride, int B, int V, const int64_t* ids,
                                 float* out, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (dtype == 0)
    token_logprob_kernel<float><<<B, 1024, 0, st>>>((const float*)logits, stride, V, ids, out);
  else if (dtype == 1)
    token_logprob_kernel<bf16><<<B, 1024, 0, st>>>((const bf16*)logits, stride, V, ids, out);
  else
    return LLB_ERR_UNSUPPORTED;
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
