// Elementwise / normalisation / indexing kernels (bf16 activations, fp32 math).
//
// These are the bandwidth-bound "small" ops of a decoder layer.  Each one is a
// single pass over its operands with 16-byte accesses; the ones that follow a
// GEMM also exist as GEMM epilogues (see gemm_tcgen05.cu), the standalone forms
// here serve the first/last layer and the non-fused paths.
#include "common.cuh"

using namespace llb;
LLB_DEBUG_BOUNDS_STORAGE(ops_basic)


// ---------------------------------------------------------------------------------------
// RMSNorm:  y = x * rsqrt(mean(x^2) + eps) * (w + w_offset)
// add_rmsnorm: residual += x ; y = rmsnorm(residual)
// One CTA per row, the row stays in registers between the two passes.
// ---------------------------------------------------------------------------------------
template <int MAX_VEC, bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_kernel(bf16* __restrict__ out, bf16* __restrict__ residual,
                                                      const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                      int H, float eps, float w_offset, int64_t x_stride,
                                                      int64_t out_stride, int64_t res_stride) {
  __shared__ float red[33];
  const int row = blockIdx.x;
  const int nvec = H >> 3;
  pdl_wait();
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (int64_t)row * x_stride);
  bf16x8* rr = ADD ? reinterpret_cast<bf16x8*>(residual + (int64_t)row * res_stride) : nullptr;
  float vals[MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    int v = threadIdx.x + i * 256;
    if (v < nvec) {
      bf16x8 p = xr[v];
      unpack8(p, vals[i]);
      if (ADD) {
        float r[8];
        bf16x8 q = rr[v];
        unpack8(q, r);
#pragma unroll
        for (int k = 0; k < 8; ++k) vals[i][k] += r[k];
        // the residual stream is stored in bf16: normalise what is stored
        bf16x8 s = pack8(vals[i]);
        rr[v] = s;
        unpack8(s, vals[i]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += vals[i][k] * vals[i][k];
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* orow = reinterpret_cast<bf16x8*>(out + (int64_t)row * out_stride);
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    int v = threadIdx.x + i * 256;
    if (v < nvec) {
      float wf[8];
      unpack8(wr[v], wf);
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = vals[i][k] * inv * (wf[k] + w_offset);
      orow[v] = pack8(o);
    }
  }
}

template <bool ADD>
static int launch_rmsnorm(bf16* out, bf16* residual, const bf16* x, const bf16* w, int T, int H, float eps,
                          float w_offset, int64_t xs, int64_t os, int64_t rs, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (H % 8 != 0 || H > 8 * 256 * 8) return LLB_ERR_UNSUPPORTED;
  int nvec = H / 8;
  int per = cdiv(nvec, 256);
  if (per <= 1)
    launch_pdl(rmsnorm_kernel<1, ADD>, dim3(T), dim3(256), 0, st, out, residual, x, w, H, eps, w_offset, xs, os, rs);
  else if (per <= 2)
    launch_pdl(rmsnorm_kernel<2, ADD>, dim3(T), dim3(256), 0, st, out, residual, x, w, H, eps, w_offset, xs, os, rs);
  else if (per <= 4)
    launch_pdl(rmsnorm_kernel<4, ADD>, dim3(T), dim3(256), 0, st, out, residual, x, w, H, eps, w_offset, xs, os, rs);
  else
    launch_pdl(rmsnorm_kernel<8, ADD>, dim3(T), dim3(256), 0, st, out, residual, x, w, H, eps, w_offset, xs, os, rs);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_rmsnorm(void* out, const void* x, const void* w, int T, int H, float eps, float w_offset,
                           int64_t x_stride, int64_t out_stride, cudaStream_t st) {
  return launch_rmsnorm<false>((bf16*)out, nullptr, (const bf16*)x, (const bf16*)w, T, H, eps, w_offset, x_stride,
                               out_stride, 0, st);
}
LLB_EXPORT int llb_add_rmsnorm(void* out, void* residual, const void* x, const void* w, int T, int H, float eps,
                               float w_offset, cudaStream_t st) {
  return launch_rmsnorm<true>((bf16*)out, (bf16*)residual, (const bf16*)x, (const bf16*)w, T, H, eps, w_offset, H, H,
                              H, st);
}

// ---------------------------------------------------------------------------------------
// Gated activations:  out[t, i] = act(x[t, i]) * x[t, I + i]      (x is [T, 2I])
// act: 0 = SiLU, 1 = GELU(tanh)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float act_silu(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float act_gelu_tanh(float v) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * v * (1.f + tanhf(k0 * (v + k1 * v * v * v)));
}

template <int ACT>
__global__ void __launch_bounds__(256) gated_act_kernel(bf16* __restrict__ out, const bf16* __restrict__ x,
                                                        int64_t n_vec_total, int I_vec) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_vec_total) return;
  int64_t t = idx / I_vec;
  int c = (int)(idx - t * I_vec);
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x) + t * (2 * (int64_t)I_vec);
  float g[8], u[8], o[8];
  unpack8(xr[c], g);
  unpack8(xr[c + I_vec], u);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = (ACT == 0 ? act_silu(g[k]) : act_gelu_tanh(g[k])) * u[k];
  reinterpret_cast<bf16x8*>(out)[idx] = pack8(o);
}

LLB_EXPORT int llb_gated_act(void* out, const void* x, int T, int I, int act, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (I % 8 != 0) return LLB_ERR_UNSUPPORTED;
  int64_t n = (int64_t)T * (I / 8);
  int blocks = (int)cdiv64(n, 256);
  if (act == 0)
    gated_act_kernel<0><<<blocks, 256, 0, st>>>((bf16*)out, (const bf16*)x, n, I / 8);
  else
    gated_act_kernel<1><<<blocks, 256, 0, st>>>((bf16*)out, (const bf16*)x, n, I / 8);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// ---------------------------------------------------------------------------------------
// Fused: optional per-head q/k RMSNorm -> RoPE (half-split "neox" layout, partial rotary)
//        -> scatter of K and V rows into the token-level KV pool.
//
//   qkv        [T, (Hq + 2*Hkv) * D]  output of the fused qkv GEMM; q is rotated in place
//   kv_layer   [slots, 2*Hkv, D]      pool slice of this layer; K heads first, then V heads
//   cos/sin    [max_pos, rot_dim/2]   fp32 tables
//   pos        [T] int32, slot [T] int32 (destination slot of each new token)
// A group of D/8 consecutive lanes owns one head (each lane one 16-byte vector); the
// rotation partner's values come by warp shuffle, so every lane writes only its own vector.
// ---------------------------------------------------------------------------------------
template <int LANES_PER_HEAD>
__global__ void __launch_bounds__(256) rope_kv_scatter_kernel(bf16* __restrict__ qkv, bf16* __restrict__ kv_layer,
                                                              const float* __restrict__ cos_t,
                                                              const float* __restrict__ sin_t,
                                                              const int* __restrict__ pos, const int* __restrict__ slot,
                                                              const bf16* __restrict__ q_norm_w,
                                                              const bf16* __restrict__ k_norm_w, float norm_eps,
                                                              float norm_w_offset, int Hq, int Hkv, int rot_dim,
                                                              int64_t qkv_stride) {
  constexpr int D = LANES_PER_HEAD * 8;
  const int t = blockIdx.x;
  pdl_wait();
  const int total = (Hq + 2 * Hkv) * LANES_PER_HEAD;
  const int half = rot_dim >> 1;
  const int half_lanes = half >> 3;
  const int p = pos[t];
  const int s = LLB_CHECK_SLOT(slot[t]);
  bf16* row = qkv + (int64_t)t * qkv_stride;
  const float* cr = cos_t + (int64_t)p * half;
  const float* sr = sin_t + (int64_t)p * half;
  const int iters = cdiv(total, (int)blockDim.x);
  for (int it = 0; it < iters; ++it) {
    int item = threadIdx.x + it * blockDim.x;
    bool valid = item < total;
    int head = valid ? item / LANES_PER_HEAD : 0;
    int v = item % LANES_PER_HEAD;
    int kind = head < Hq ? 0 : (head < Hq + Hkv ? 1 : 2);  // q, k, v
    float x[8];
    bf16x8 raw = reinterpret_cast<const bf16x8*>(row + (int64_t)head * D)[v];
    unpack8(raw, x);
    const bf16* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
    // the whole warp runs the shuffles (heads of different kinds share a warp)
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += x[k] * x[k];
#pragma unroll
    for (int o = LANES_PER_HEAD / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (nw != nullptr) {
      float inv = rsqrtf(ss / (float)D + norm_eps);
      float wf[8];
      unpack8(reinterpret_cast<const bf16x8*>(nw)[v], wf);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        x[k] = x[k] * inv * (wf[k] + norm_w_offset);
        x[k] = __bfloat162float(__float2bfloat16(x[k]));  // the norm output is a bf16 tensor in the unfused form
      }
    }
    // rotation partner: lane +- half_lanes inside the head group
    bool lower = v < half_lanes;
    bool rotary = (kind != 2) && (v < 2 * half_lanes);
    int lane = threadIdx.x & 31;
    int partner = lower ? lane + half_lanes : lane - half_lanes;
    partner = rotary ? partner : lane;
    float y[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) y[k] = __shfl_sync(0xffffffffu, x[k], partner & 31);
    if (rotary) {
      int base = (lower ? v : v - half_lanes) * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float c = cr[base + k], sn = sr[base + k];
        x[k] = lower ? (x[k] * c - y[k] * sn) : (x[k] * c + y[k] * sn);
      }
    }
    if (!valid) continue;
    bf16x8 o = pack8(x);
    if (kind == 0) {
      reinterpret_cast<bf16x8*>(row + (int64_t)head * D)[v] = o;
    } else {
      int h = head - Hq;  // 0..2*Hkv-1 : K heads then V heads, the pool's order
      reinterpret_cast<bf16x8*>(kv_layer + ((int64_t)s * (2 * Hkv) + h) * D)[v] = o;
    }
  }
}

LLB_EXPORT int llb_rope_kv_scatter(void* qkv, void* kv_layer, const float* cos_t, const float* sin_t, const int* pos,
                                   const int* slot, const void* q_norm_w, const void* k_norm_w, float norm_eps,
                                   float norm_w_offset, int T, int Hq, int Hkv, int D, int rot_dim, int64_t qkv_stride,
                                   cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (rot_dim % 16 != 0 || rot_dim > D) return LLB_ERR_UNSUPPORTED;
#define LAUNCH_ROPE(L)                                                                                              \
  launch_pdl(rope_kv_scatter_kernel<L>, dim3(T), dim3(256), 0, st, (bf16*)qkv, (bf16*)kv_layer, cos_t, sin_t, pos,  \
             slot, (const bf16*)q_norm_w, (const bf16*)k_norm_w, norm_eps, norm_w_offset, Hq, Hkv, rot_dim, qkv_stride)
  if (D == 128)
    LAUNCH_ROPE(16);
  else if (D == 64)
    LAUNCH_ROPE(8);
  else if (D == 256)
    LAUNCH_ROPE(32);
  else
    return LLB_ERR_UNSUPPORTED;
#undef LAUNCH_ROPE
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// ---------------------------------------------------------------------------------------
// Vocab-parallel embedding gather: out[t] = table[id - vocab_start] or 0 when out of shard.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embedding_kernel(bf16* __restrict__ out, const int64_t* __restrict__ ids,
                                                        const bf16* __restrict__ table, int H_vec, int vocab_start,
                                                        int vocab_end) {
  int t = blockIdx.x;
  int64_t id = ids[t];
  bool in = id >= vocab_start && id < vocab_end;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(table) + (in ? (id - vocab_start) * (int64_t)H_vec : 0);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out) + (int64_t)t * H_vec;
  bf16x8 z;
#pragma unroll
  for (int i = 0; i < 4; ++i) z.w[i] = 0u;
  for (int v = threadIdx.x; v < H_vec; v += blockDim.x) dst[v] = in ? src[v] : z;
}

LLB_EXPORT int llb_embedding(void* out, const int64_t* ids, const void* table, int T, int H, int vocab_start,
                             int vocab_end, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (H % 8 != 0) return LLB_ERR_UNSUPPORTED;
  embedding_kernel<<<T, 256, 0, st>>>((bf16*)out, ids, (const bf16*)table, H / 8, vocab_start, vocab_end);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// ---------------------------------------------------------------------------------------
// Step prologues (all the index math of a forward pass in one launch each).
//
// decode:  for request b: ids[b] = next_token[req]; pos[b] = seq_len[b]-1;
//          req_to_token[req, seq_len-1] = new_slot[b]
// prefill: for new token i of request b (cu_q[b] <= j < cu_q[b+1]):
//          pos[j] = ready_len[b] + (j - cu_q[b]); batch_of[j] = b;
//          req_to_token[req, pos[j]] = new_slot[j]
// ---------------------------------------------------------------------------------------
__global__ void decode_prologue_kernel(int64_t* __restrict__ ids, int* __restrict__ pos,
                                       int* __restrict__ req_to_token, const int64_t* __restrict__ next_token,
                                       const int* __restrict__ b_req_idx, const int* __restrict__ b_seq_len,
                                       const int* __restrict__ new_slot, int B, int64_t r2t_stride,
                                       int next_token_stride) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int req = LLB_CHECK_REQ(b_req_idx[b]);
  int L = b_seq_len[b];
  if (ids != nullptr) ids[b] = next_token[(int64_t)req * next_token_stride];
  pos[b] = L - 1;
  req_to_token[(int64_t)req * r2t_stride + LLB_CHECK_POS(L - 1)] = LLB_CHECK_SLOT(new_slot[b]);
}

LLB_EXPORT int llb_decode_prologue(int64_t* ids, int* pos, int* req_to_token, const int64_t* next_token,
                                   const int* b_req_idx, const int* b_seq_len, const int* new_slot, int B,
                                   int64_t r2t_stride, int next_token_stride, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  decode_prologue_kernel<<<cdiv(B, 128), 128, 0, st>>>(ids, pos, req_to_token, next_token, b_req_idx, b_seq_len,
                                                       new_slot, B, r2t_stride, next_token_stride);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

__global__ void prefill_prologue_kernel(int* __restrict__ pos, int* __restrict__ batch_of,
                                        int* __restrict__ req_to_token, const int* __restrict__ b_req_idx,
                                        const int* __restrict__ b_ready_len, const int* __restrict__ cu_q,
                                        const int* __restrict__ new_slot, int64_t r2t_stride) {
  int b = blockIdx.x;
  int req = LLB_CHECK_REQ(b_req_idx[b]);
  int ready = b_ready_len[b];
  int s = cu_q[b], e = cu_q[b + 1];
  for (int j = s + threadIdx.x; j < e; j += blockDim.x) {
    int p = ready + (j - s);
    pos[j] = p;
    batch_of[j] = b;
    req_to_token[(int64_t)req * r2t_stride + LLB_CHECK_POS(p)] = LLB_CHECK_SLOT(new_slot[j]);
  }
}

LLB_EXPORT int llb_prefill_prologue(int* pos, int* batch_of, int* req_to_token, const int* b_req_idx,
                                    const int* b_ready_len, const int* cu_q, const int* new_slot, int B,
                                    int64_t r2t_stride, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  prefill_prologue_kernel<<<B, 256, 0, st>>>(pos, batch_of, req_to_token, b_req_idx, b_ready_len, cu_q, new_slot,
                                             r2t_stride);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// next_token[req] = sampled[b] for the requests that produced a token this step
__global__ void scatter_next_token_kernel(int64_t* __restrict__ next_token, const int64_t* __restrict__ sampled,
                                          const int* __restrict__ b_req_idx, const uint8_t* __restrict__ has_out,
                                          int B, int next_token_stride) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (has_out != nullptr && !has_out[b]) return;
  next_token[(int64_t)LLB_CHECK_REQ(b_req_idx[b]) * next_token_stride] = sampled[b];
}
LLB_EXPORT int llb_scatter_next_token(int64_t* next_token, const int64_t* sampled, const int* b_req_idx,
                                      const uint8_t* has_out, int B, int next_token_stride, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  scatter_next_token_kernel<<<cdiv(B, 128), 128, 0, st>>>(next_token, sampled, b_req_idx, has_out, B,
                                                          next_token_stride);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// ---------------------------------------------------------------------------------------
// Row gather / scatter of KV pool rows (prefix copies, PD staging pages, host offload).
//   dst[dst_idx[i]] = src[src_idx[i]]   rows of `row_bytes` bytes (multiple of 16)
// Either index array may be null (= identity).  Works on pinned host pointers too.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) copy_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                        const int* __restrict__ dst_idx,
                                                        const int* __restrict__ src_idx, int n_rows, int row_vec,
                                                        int64_t dst_row_stride_vec, int64_t src_row_stride_vec) {
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
    int64_t d = dst_idx ? dst_idx[r] : r;
    int64_t s = src_idx ? src_idx[r] : r;
    const uint4* sp = src + s * src_row_stride_vec;
    uint4* dp = dst + d * dst_row_stride_vec;
    for (int v = threadIdx.x; v < row_vec; v += blockDim.x) dp[v] = sp[v];
  }
}
LLB_EXPORT int llb_copy_rows(void* dst, const void* src, const int* dst_idx, const int* src_idx, int n_rows,
                             int64_t row_bytes, int64_t dst_row_stride_bytes, int64_t src_row_stride_bytes,
                             cudaStream_t st) {
  if (n_rows <= 0) return LLB_OK;
  if (row_bytes % 16 || dst_row_stride_bytes % 16 || src_row_stride_bytes % 16) return LLB_ERR_UNSUPPORTED;
  int blocks = n_rows < 148 * 8 ? n_rows : 148 * 8;
  copy_rows_kernel<<<blocks, 256, 0, st>>>((uint4*)dst, (const uint4*)src, dst_idx, src_idx, n_rows,
                                           (int)(row_bytes / 16), dst_row_stride_bytes / 16,
                                           src_row_stride_bytes / 16);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
