// Paged causal attention for the layer shapes the tensor-core kernels do not cover: any head size up to
// 256 (Gemma 256, Phi-3 96, StableLM 80 ...), sliding windows, ALiBi slopes, logit soft-capping and
// attention sinks.  One CTA per (query token, query head); its four warps stride over the keys, each
// keeps an online-softmax state with the head vector spread over the lanes, and the states are merged
// in shared memory.  Prefill and decode use the same kernel: a query is described by its position and
// the request row it belongs to.
//
// KV pool row layout (one layer): [slot][2 * Hkv][D], K heads first, then V heads.
#include "common.cuh"

using namespace llb;

constexpr int GEN_WARPS = 4;
constexpr int GEN_MAX_EPL = 8;  // elements per lane: D <= 256

__global__ void __launch_bounds__(GEN_WARPS * 32)
attn_generic_kernel(const bf16* __restrict__ q, int64_t q_stride, const bf16* __restrict__ kv,
                    const int* __restrict__ req_to_token, int64_t r2t_stride, const int* __restrict__ b_req_idx,
                    const int* __restrict__ pos, const int* __restrict__ batch_of, bf16* __restrict__ out,
                    int64_t out_stride, int Hq, int Hkv, int D, float sm_scale, int window, float softcap,
                    const float* __restrict__ alibi, const float* __restrict__ sinks) {
  const int t = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = batch_of ? batch_of[t] : t;
  const int qpos = pos[t];
  const int kvh = h / (Hq / Hkv);
  const int* slots = req_to_token + (int64_t)b_req_idx[b] * r2t_stride;
  const int64_t row = (int64_t)2 * Hkv * D;

  float qv[GEN_MAX_EPL], acc[GEN_MAX_EPL];
#pragma unroll
  for (int e = 0; e < GEN_MAX_EPL; ++e) {
    int d = lane + e * 32;
    qv[e] = d < D ? __bfloat162float(q[(int64_t)t * q_stride + (int64_t)h * D + d]) * sm_scale : 0.f;
    acc[e] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int j0 = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
  const float slope = alibi ? alibi[h] : 0.f;
  for (int j = j0 + warp; j <= qpos; j += GEN_WARPS) {
    const bf16* kr = kv + (int64_t)slots[j] * row + (int64_t)kvh * D;
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < GEN_MAX_EPL; ++e) {
      int d = lane + e * 32;
      if (d < D) s += qv[e] * __bfloat162float(kr[d]);
    }
    s = warp_sum(s);
    if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    s += slope * (float)(j - qpos);
    const float mn = fmaxf(m, s);
    const float corr = __expf(m - mn), p = __expf(s - mn);
    l = l * corr + p;
    const bf16* vr = kr + (int64_t)Hkv * D;
#pragma unroll
    for (int e = 0; e < GEN_MAX_EPL; ++e) {
      int d = lane + e * 32;
      if (d < D) acc[e] = acc[e] * corr + p * __bfloat162float(vr[d]);
    }
    m = mn;
  }
  __shared__ float s_m[GEN_WARPS], s_l[GEN_WARPS];
  __shared__ float s_acc[GEN_WARPS][GEN_MAX_EPL * 32];
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
#pragma unroll
  for (int e = 0; e < GEN_MAX_EPL; ++e) s_acc[warp][lane + e * 32] = acc[e];
  __syncthreads();
  if (warp == 0) {
    float M = sinks ? sinks[h] : -INFINITY;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; ++w) M = fmaxf(M, s_m[w]);
    float L = sinks ? __expf(sinks[h] - M) : 0.f;
    float o[GEN_MAX_EPL];
#pragma unroll
    for (int e = 0; e < GEN_MAX_EPL; ++e) o[e] = 0.f;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; ++w) {
      if (s_m[w] == -INFINITY) continue;
      const float c = __expf(s_m[w] - M);
      L += s_l[w] * c;
#pragma unroll
      for (int e = 0; e < GEN_MAX_EPL; ++e) o[e] += s_acc[w][lane + e * 32] * c;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int e = 0; e < GEN_MAX_EPL; ++e) {
      int d = lane + e * 32;
      if (d < D) out[(int64_t)t * out_stride + (int64_t)h * D + d] = __float2bfloat16(o[e] * inv);
    }
  }
}

LLB_EXPORT int llb_attn_generic(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                                int64_t r2t_stride, const int* b_req_idx, const int* pos, const int* batch_of, void* out,
                                int64_t out_stride, int T, int Hq, int Hkv, int D, float sm_scale, int window,
                                float softcap, const float* alibi_slopes, const float* sinks, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (D <= 0 || D > 32 * GEN_MAX_EPL || Hkv <= 0 || Hq % Hkv != 0) return LLB_ERR_UNSUPPORTED;
  dim3 grid(T, Hq);
  attn_generic_kernel<<<grid, GEN_WARPS * 32, 0, st>>>((const bf16*)q, q_stride, (const bf16*)kv_layer, req_to_token,
                                                       r2t_stride, b_req_idx, pos, batch_of, (bf16*)out, out_stride,
                                                       Hq, Hkv, D, sm_scale, window, softcap, alibi_slopes, sinks);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// RoPE + KV scatter for head sizes / rotary widths the vectorised kernel does not take (head size not 64, 128
// or 256, rotary width not a multiple of 16).  One CTA per token: the token's qkv row is staged in shared
// memory so that rotation partners are read before anything is overwritten.  Same contract as
// llb_rope_kv_scatter (half-split rotary layout, q rotated in place, K and V written to kv_layer[slot]).
__global__ void __launch_bounds__(256) rope_kv_scatter_generic_kernel(bf16* __restrict__ qkv, bf16* __restrict__ kv_layer,
                                                                      const float* __restrict__ cos_t,
                                                                      const float* __restrict__ sin_t,
                                                                      const int* __restrict__ pos,
                                                                      const int* __restrict__ slot, int Hq, int Hkv,
                                                                      int D, int rot_dim, int64_t qkv_stride) {
  extern __shared__ float srow[];
  const int t = blockIdx.x;
  const int n = (Hq + 2 * Hkv) * D;
  bf16* row = qkv + (int64_t)t * qkv_stride;
  for (int i = threadIdx.x; i < n; i += blockDim.x) srow[i] = __bfloat162float(row[i]);
  __syncthreads();
  const int half = rot_dim >> 1;
  const int p = pos[t], s = slot[t];
  const float* cr = cos_t + (int64_t)p * half;
  const float* sr = sin_t + (int64_t)p * half;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int head = i / D, d = i - head * D;
    const int kind = head < Hq ? 0 : (head < Hq + Hkv ? 1 : 2);
    float x = srow[i];
    if (kind != 2 && d < rot_dim) {
      if (d < half)
        x = x * cr[d] - srow[i + half] * sr[d];
      else
        x = x * cr[d - half] + srow[i - half] * sr[d - half];
    }
    const bf16 o = __float2bfloat16(x);
    if (kind == 0)
      row[i] = o;
    else
      kv_layer[((int64_t)s * (2 * Hkv) + (head - Hq)) * D + d] = o;
  }
}

LLB_EXPORT int llb_rope_kv_scatter_generic(void* qkv, void* kv_layer, const float* cos_t, const float* sin_t,
                                           const int* pos, const int* slot, int T, int Hq, int Hkv, int D, int rot_dim,
                                           int64_t qkv_stride, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  const size_t smem = (size_t)(Hq + 2 * Hkv) * D * sizeof(float);
  if ((rot_dim & 1) || rot_dim > D || smem > 200 * 1024) return LLB_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(rope_kv_scatter_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  rope_kv_scatter_generic_kernel<<<T, 256, smem, st>>>((bf16*)qkv, (bf16*)kv_layer, cos_t, sin_t, pos, slot, Hq, Hkv, D,
                                                      rot_dim, qkv_stride);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
