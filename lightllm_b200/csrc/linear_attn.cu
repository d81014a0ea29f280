// Gated DeltaNet decode step (Qwen3-Next / Qwen3.5 linear-attention layers): one new token of every request.
//
//   conv step      y[b, c]   = silu( sum_t full[c, t] * w[c, t] ),  full = [conv_state[req[b], c, :], x[b, c]];
//                  conv_state[req[b], c, :] <- full[c, 1:]
//   recurrent step per (request b, value head h), state S [dk, dv] of the request's slot:
//                  q <- l2norm(q) / sqrt(dk),  k <- l2norm(k)
//                  S <- exp(g) S ;  d = beta (v - S^T k) ;  S <- S + k d^T ;  o = S^T q
//
// The recurrent step is bound by streaming the state (dk x dv numbers per head in and out): a CTA owns one (b, h),
// every thread keeps a strip of one state column in registers, so the state is read once and written once.
#include "common.cuh"

using namespace llb;

namespace {

__device__ __forceinline__ float ld_state(const float* p) { return *p; }
__device__ __forceinline__ float ld_state(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_state(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_state(bf16* p, float v) { *p = __float2bfloat16(v); }

template <typename ST>
__global__ void gdn_conv_step_kernel(const float* __restrict__ x, ST* __restrict__ state, const float* __restrict__ w,
                                     const int* __restrict__ req, float* __restrict__ y, int B, int C, int K) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)B * C) return;
  int b = (int)(i / C), c = (int)(i - (int64_t)b * C);
  ST* s = state + ((int64_t)req[b] * C + c) * (K - 1);
  const float* wc = w + (int64_t)c * K;
  float xv = x[i];
  float acc = xv * wc[K - 1];
  float prev = 0.f;
  for (int t = 0; t < K - 1; ++t) {
    float v = ld_state(s + t);
    acc += v * wc[t];
    if (t > 0) st_state(s + t - 1, v);   // shift left; element t-1 was read in the previous iteration
    prev = v;
  }
  (void)prev;
  if (K > 1) st_state(s + K - 2, xv);
  y[i] = acc / (1.f + __expf(-acc));
}

constexpr int GDN_MAX_RPT = 64;   // state rows a thread keeps in registers

template <typename ST>
__global__ void __launch_bounds__(256) gdn_recurrent_step_kernel(
    const float* __restrict__ y, const float* __restrict__ g, const float* __restrict__ beta, ST* __restrict__ state,
    const int* __restrict__ req, float* __restrict__ out, int nk, int nv, int dk, int dv, int C, int rpt) {
  extern __shared__ float sm[];          // q[dk], k[dk], red[groups * dv]
  __shared__ float red33[33];
  float* qs = sm;
  float* ks = sm + dk;
  float* red = sm + 2 * dk;
  const int b = blockIdx.x / nv, h = blockIdx.x - b * nv;
  const int hk = h / (nv / nk);
  const int kd = nk * dk;
  const float* yb = y + (int64_t)b * C;
  const int tid = threadIdx.x, col = tid % dv, grp = tid / dv, groups = blockDim.x / dv;
  // q, k of the key head: l2-normalise (eps inside the root, as x * rsqrt(sum x^2 + 1e-6)); q also scaled by dk^-1/2
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < dk; i += blockDim.x) {
    float qv = yb[hk * dk + i], kv = yb[kd + hk * dk + i];
    qs[i] = qv;
    ks[i] = kv;
    sq += qv * qv;
    sk += kv * kv;
  }
  sq = block_sum(sq, red33);
  sk = block_sum(sk, red33);
  const float qscale = rsqrtf(sq + 1e-6f) * rsqrtf((float)dk), kscale = rsqrtf(sk + 1e-6f);
  for (int i = tid; i < dk; i += blockDim.x) {
    qs[i] *= qscale;
    ks[i] *= kscale;
  }
  __syncthreads();
  const float vj = yb[2 * kd + h * dv + col];
  const float decay = __expf(g[(int64_t)b * nv + h]), bt = beta[(int64_t)b * nv + h];
  ST* S = state + (((int64_t)req[b] * nv + h) * dk) * dv + col;
  const int r0 = grp * rpt;
  float s[GDN_MAX_RPT];
  float acc = 0.f;
#pragma unroll
  for (int t = 0; t < GDN_MAX_RPT; ++t) {
    int r = r0 + t;
    if (t < rpt && r < dk) {
      s[t] = decay * ld_state(S + (int64_t)r * dv);
      acc += s[t] * ks[r];
    } else {
      s[t] = 0.f;
    }
  }
  red[grp * dv + col] = acc;
  __syncthreads();
  float kv_mem = 0.f;
  for (int gi = 0; gi < groups; ++gi) kv_mem += red[gi * dv + col];
  const float d = bt * (vj - kv_mem);
  __syncthreads();
  float o = 0.f;
#pragma unroll
  for (int t = 0; t < GDN_MAX_RPT; ++t) {
    int r = r0 + t;
    if (t < rpt && r < dk) {
      float v = s[t] + ks[r] * d;
      st_state(S + (int64_t)r * dv, v);
      o += v * qs[r];
    }
  }
  red[grp * dv + col] = o;
  __syncthreads();
  if (grp == 0) {
    float t = 0.f;
    for (int gi = 0; gi < groups; ++gi) t += red[gi * dv + col];
    out[((int64_t)b * nv + h) * dv + col] = t;
  }
}

// The serving shape (head sizes known at compile time): a warp owns DK / 8 state rows, a lane four neighbouring
// columns of them, so a thread's strip is DK / 8 vector loads that do not depend on anything and are all in
// flight before the first product; the same registers are written back after the update.
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
  float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
__device__ __forceinline__ void ld4(const bf16* p, float (&v)[4]) {
  uint2 t = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&t.x), b = *reinterpret_cast<__nv_bfloat162*>(&t.y);
  v[0] = __low2float(a), v[1] = __high2float(a), v[2] = __low2float(b), v[3] = __high2float(b);
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(bf16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<unsigned*>(&a);
  t.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

template <typename ST, int DK, int DV>
__global__ void __launch_bounds__(256, 2) gdn_recurrent_step_vec_kernel(
    const float* __restrict__ y, const float* __restrict__ g, const float* __restrict__ beta, ST* __restrict__ state,
    const int* __restrict__ req, float* __restrict__ out, int nk, int nv, int C) {
  constexpr int NW = 8, RPW = DK / NW;
  static_assert(DV == 128 && DK % NW == 0, "a lane owns four columns of a 128-wide value head");
  __shared__ float qs[DK], ks[DK];
  __shared__ __align__(16) float red[NW][DV];
  __shared__ float red33[33];
  const int b = blockIdx.x / nv, h = blockIdx.x - b * nv;
  const int hk = h / (nv / nk), kd = nk * DK;
  const float* yb = y + (int64_t)b * C;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, col0 = lane * 4;
  // the state strip first: nothing below depends on it until the products
  ST* S = state + (((int64_t)req[b] * nv + h) * DK + warp * RPW) * DV + col0;
  float s[RPW][4];
#pragma unroll
  for (int t = 0; t < RPW; ++t) ld4(S + t * DV, s[t]);
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < DK; i += 256) {
    float qv = yb[hk * DK + i], kv = yb[kd + hk * DK + i];
    qs[i] = qv;
    ks[i] = kv;
    sq += qv * qv;
    sk += kv * kv;
  }
  sq = block_sum(sq, red33);
  sk = block_sum(sk, red33);
  const float qscale = rsqrtf(sq + 1e-6f) * rsqrtf((float)DK), kscale = rsqrtf(sk + 1e-6f);
  float v[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) v[c] = yb[2 * kd + h * DV + col0 + c];
  const float decay = __expf(g[(int64_t)b * nv + h]), bt = beta[(int64_t)b * nv + h];
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int t = 0; t < RPW; ++t) {
    const float kr = ks[warp * RPW + t] * kscale;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      s[t][c] *= decay;
      acc[c] += s[t][c] * kr;
    }
  }
  st4(&red[warp][col0], acc);
  __syncthreads();
  float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    float t4[4];
    ld4(&red[w][col0], t4);
#pragma unroll
    for (int c = 0; c < 4; ++c) d[c] += t4[c];
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) d[c] = bt * (v[c] - d[c]);
  __syncthreads();
  float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int t = 0; t < RPW; ++t) {
    const float kr = ks[warp * RPW + t] * kscale, qr = qs[warp * RPW + t] * qscale;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      s[t][c] += kr * d[c];
      o[c] += s[t][c] * qr;
    }
    st4(S + t * DV, s[t]);
  }
  st4(&red[warp][col0], o);
  __syncthreads();
  if (tid < DV) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) t += red[w][tid];
    out[((int64_t)b * nv + h) * DV + tid] = t;
  }
}

}  // namespace

// x, y [B, C] fp32; state [slots, C, K-1] (fp32: state_bf16 = 0, bf16: 1); w [C, K] fp32; req [B] slot of every row
LLB_EXPORT int llb_gdn_conv_step(const float* x, void* state, int state_bf16, const float* w, const int* req, float* y,
                                 int B, int C, int K, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (K < 1 || K > 16) return LLB_ERR_UNSUPPORTED;
  int64_t n = (int64_t)B * C;
  int blocks = (int)((n + 255) / 256);
  if (state_bf16)
    gdn_conv_step_kernel<bf16><<<blocks, 256, 0, st>>>(x, (bf16*)state, w, req, y, B, C, K);
  else
    gdn_conv_step_kernel<float><<<blocks, 256, 0, st>>>(x, (float*)state, w, req, y, B, C, K);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// y [B, C] fp32 (C = 2 nk dk + nv dv: q heads, k heads, v heads after the convolution); g, beta [B, nv] fp32;
// state [slots, nv, dk, dv]; out [B, nv, dv] fp32
LLB_EXPORT int llb_gdn_recurrent_step(const float* y, const float* g, const float* beta, void* state, int state_bf16,
                                      const int* req, float* out, int B, int nk, int nv, int dk, int dv,
                                      cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (nk < 1 || nv % nk != 0 || dv < 32 || dv > 256 || dv % 32 != 0 || dk < 1) return LLB_ERR_UNSUPPORTED;
  if (dk == 128 && dv == 128) {                // the serving shape: vector loads, two CTAs per SM
    int C = 2 * nk * dk + nv * dv;
    if (state_bf16)
      gdn_recurrent_step_vec_kernel<bf16, 128, 128><<<B * nv, 256, 0, st>>>(y, g, beta, (bf16*)state, req, out, nk, nv,
                                                                            C);
    else
      gdn_recurrent_step_vec_kernel<float, 128, 128><<<B * nv, 256, 0, st>>>(y, g, beta, (float*)state, req, out, nk,
                                                                             nv, C);
    LLB_LAUNCH_CHECK();
    return LLB_OK;
  }
  int groups = 256 / dv;                       // threads = dv * groups <= 256
  if (groups > dk) groups = dk;
  int rpt = (dk + groups - 1) / groups;
  if (rpt > GDN_MAX_RPT) return LLB_ERR_UNSUPPORTED;      // dk <= 64 * groups
  // fewer groups when the strips would be very short (keeps small heads from spreading over idle threads)
  while (groups > 1 && (dk + groups - 2) / (groups - 1) <= 16) --groups, rpt = (dk + groups - 1) / groups;
  int threads = dv * groups;
  int C = 2 * nk * dk + nv * dv;
  size_t smem = (size_t)(2 * dk + groups * dv) * sizeof(float);
  if (state_bf16)
    gdn_recurrent_step_kernel<bf16><<<B * nv, threads, smem, st>>>(y, g, beta, (bf16*)state, req, out, nk, nv, dk, dv,
                                                                  C, rpt);
  else
    gdn_recurrent_step_kernel<float><<<B * nv, threads, smem, st>>>(y, g, beta, (float*)state, req, out, nk, nv, dk,
                                                                   dv, C, rpt);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
