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
