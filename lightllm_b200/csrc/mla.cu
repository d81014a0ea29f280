// Multi-head latent attention (DeepSeek-V2/V3) kernels over the latent KV pool.
//
// Pool row of a token: [c_kv (512, RMS-normalised) | k_pe (64, rotated)], one "head" shared by all
// query heads.  Attention is absorbed: scores = q_lat . c_kv + q_pe . k_pe, output = P . c_kv.
//
//   mla_rope_kv_scatter  RoPE on the rope part of every q head (in place), RMSNorm of the new kv latent,
//                        RoPE of k_pe, scatter of the 576-wide row into the pool -- one launch
//   mla_attention        one CTA per (query token, group of 16 heads), 8 warps.  A 64-token KV tile
//                        (64 x 576 bf16) is gathered once through the slot table and used for both
//                        products: Q.K^T has its 36 k-steps split over the warps (partials reduced through
//                        shared memory), P.V has the 512 value columns split over the warps (64 each), so
//                        the 16 x 512 fp32 output lives in 32 registers per thread.  Causal masking by the
//                        query's position makes the same kernel serve decode (one row per request) and
//                        prefill (cached-prefix aware).
//
// Reference behaviour: lightllm/models/deepseek2/triton_kernel/* (rotary_emb, destindex_copy_kv, gqa flash
// decoding stage 1/2, context attention with v) and the FlashInfer MLA wrappers.
#include "common.cuh"

using namespace llb;
LLB_DEBUG_BOUNDS_STORAGE(mla)


namespace {

constexpr int KVL = 512, ROPE = 64, DQK = KVL + ROPE;  // 576
constexpr int CH = DQK / 8;                            // 72 chunks of 16 bytes per row
constexpr int TILE = 64;                               // tokens per KV tile
constexpr int ROW_BYTES = DQK * 2;
constexpr int Q_BYTES = 16 * ROW_BYTES;                // 18432
constexpr int KV_BYTES = TILE * ROW_BYTES;             // 73728
constexpr int SP_BYTES = 8 * 16 * TILE * 4;            // per-warp partial scores
constexpr int S_BYTES = 16 * TILE * 4;
constexpr int MLA_SMEM = Q_BYTES + 2 * KV_BYTES + SP_BYTES + S_BYTES;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t swz576(int row, int chunk) {
  return (uint32_t)(row * ROW_BYTES + ((chunk ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(256)
mla_attention_kernel(const bf16* __restrict__ q_lat, const bf16* __restrict__ q_pe, int64_t qpe_st, int64_t qpe_sh,
                     const bf16* __restrict__ kv_layer, const int* __restrict__ req_to_token, int64_t r2t_stride,
                     const int* __restrict__ b_req_idx, const int* __restrict__ cu_q,
                     const int* __restrict__ b_ready_len, const int* __restrict__ batch_of, bf16* __restrict__ out,
                     int hq, float scale_log2) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + Q_BYTES;
  float* sp = reinterpret_cast<float*>(smem + Q_BYTES + 2 * KV_BYTES);  // [8][16][TILE]
  float* s_red = sp + 8 * 16 * TILE;                                    // [16][TILE]

  const int t = blockIdx.y;
  const int head0 = blockIdx.x * 16;
  const int nrows = min(16, hq - head0);
  const int b = batch_of ? batch_of[t] : t;
  const int req = LLB_CHECK_REQ(b_req_idx[b]);
  const int kv_len = b_ready_len[b] + (t - cu_q[b]) + 1;  // causal: positions 0 .. own position
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int64_t r2t_base = (int64_t)req * r2t_stride;

  // ---- Q tile: [16 heads][512 latent | 64 rope] ----
  for (int c = threadIdx.x; c < 16 * CH; c += blockDim.x) {
    int r = c / CH, ch = c % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows) {
      if (ch < KVL / 8)
        v = *reinterpret_cast<const uint4*>(q_lat + ((int64_t)t * hq + head0 + r) * KVL + ch * 8);
      else
        v = *reinterpret_cast<const uint4*>(q_pe + (int64_t)t * qpe_st + (int64_t)(head0 + r) * qpe_sh +
                                            (ch - KVL / 8) * 8);
    }
    *reinterpret_cast<uint4*>(q_s + swz576(r, ch)) = v;
  }

  auto issue = [&](int tile, int stage) {
    const uint32_t sb = smem_u32(kv_s) + stage * KV_BYTES;
    const int p0 = tile * TILE;
    for (int c = threadIdx.x; c < TILE * CH; c += blockDim.x) {
      int tok = c / CH, ch = c % CH;
      int pos = p0 + tok;
      bool ok = pos < kv_len;
      int sl = ok ? LLB_CHECK_SLOT(req_to_token[r2t_base + pos]) : 0;
      cp_async16(sb + swz576(tok, ch), kv_layer + (int64_t)sl * DQK + ch * 8, ok);
    }
    cp_async_commit();
  };

  const int n_tiles = (kv_len + TILE - 1) / TILE;
  issue(0, 0);

  float o[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const uint32_t qb = smem_u32(q_s);

  for (int tile = 0; tile < n_tiles; ++tile) {
    if (tile + 1 < n_tiles) {
      issue(tile + 1, (tile + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kb = smem_u32(kv_s) + (tile & 1) * KV_BYTES;

    // ---- partial S = Q K^T over this warp's k-steps (ks = warp, warp + 8, ...) ----
    float ps[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) ps[j][0] = ps[j][1] = ps[j][2] = ps[j][3] = 0.f;
    for (int ks = warp; ks < DQK / 16; ks += 8) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(a0, a1, a2, a3, qb + swz576((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
#pragma unroll
      for (int n2 = 0; n2 < TILE / 16; ++n2) {
        uint32_t b0, b1, b2, b3;
        const int tok = n2 * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(b0, b1, b2, b3, kb + swz576(tok, ks * 2 + ((lane >> 3) & 1)));
        mma_bf16_16816(ps[2 * n2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(ps[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    float* my_sp = sp + warp * 16 * TILE;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      *reinterpret_cast<float2*>(my_sp + g * TILE + j * 8 + tig * 2) = make_float2(ps[j][0], ps[j][1]);
      *reinterpret_cast<float2*>(my_sp + (g + 8) * TILE + j * 8 + tig * 2) = make_float2(ps[j][2], ps[j][3]);
    }
    __syncthreads();
    // ---- reduce the 8 partials: 1024 scores, 4 per thread ----
    {
      const int e0 = threadIdx.x * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        float4 v = *reinterpret_cast<const float4*>(sp + w * 16 * TILE + e0);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      *reinterpret_cast<float4*>(s_red + e0) = acc;
    }
    __syncthreads();
    // ---- every warp: softmax bookkeeping on the full 16 x 64 score tile (identical in all warps) ----
    float s[8][4];
    float mx[2] = {-INFINITY, -INFINITY};
    const int p0 = tile * TILE;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2 lo = *reinterpret_cast<const float2*>(s_red + g * TILE + j * 8 + tig * 2);
      float2 hi = *reinterpret_cast<const float2*>(s_red + (g + 8) * TILE + j * 8 + tig * 2);
      const int pos = p0 + j * 8 + tig * 2;
      s[j][0] = pos < kv_len ? lo.x * scale_log2 : -INFINITY;
      s[j][1] = pos + 1 < kv_len ? lo.y * scale_log2 : -INFINITY;
      s[j][2] = pos < kv_len ? hi.x * scale_log2 : -INFINITY;
      s[j][3] = pos + 1 < kv_len ? hi.y * scale_log2 : -INFINITY;
      mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      float m_new = fmaxf(m_run[r], mx[r]);
      float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[r] = exp2f(m_run[r] - m_use);
      m_run[r] = m_new;
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j][2 * r] = exp2f(s[j][2 * r] - m_use);
        s[j][2 * r + 1] = exp2f(s[j][2 * r + 1] - m_use);
        rs += s[j][2 * r] + s[j][2 * r + 1];
      }
      l_run[r] = l_run[r] * alpha[r] + rs;
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      o[nt][0] *= alpha[0];
      o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1];
      o[nt][3] *= alpha[1];
    }
    // ---- O[:, warp*64 .. +64] += P . V  (V = first 512 dims of the same tile) ----
#pragma unroll
    for (int kk = 0; kk < TILE / 16; ++kk) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                     a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const int tok = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, kb + swz576(tok, warp * 8 + n2 * 2 + (lane >> 4)));
        mma_bf16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();  // tile (and the score buffers) free for the next iteration
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + r * 8;
    if (row < nrows) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      bf16* orow = out + ((int64_t)t * hq + head0 + row) * KVL + warp * 64;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
        *reinterpret_cast<bf162*>(orow + nt * 8 + tig * 2) =
            __floats2bfloat162_rn(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
    }
  }
}

// One CTA per token: q rope parts, latent norm, k_pe rope, pool write.
__global__ void __launch_bounds__(256)
mla_rope_kv_scatter_kernel(bf16* __restrict__ q3, int64_t q_st, int64_t q_sh, const bf16* __restrict__ kv_a,
                           int64_t kva_st, bf16* __restrict__ kv_layer, const bf16* __restrict__ norm_w,
                           const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                           const int* __restrict__ pos, const int* __restrict__ slot, int hq, int nope, int rope,
                           int kv_lora, float eps) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int half = rope >> 1;
  const float* cr = cos_t + (int64_t)pos[t] * half;
  const float* sr = sin_t + (int64_t)pos[t] * half;
  // q: pairs (i, i + half) of every head
  for (int idx = threadIdx.x; idx < hq * half; idx += blockDim.x) {
    int h = idx / half, i = idx % half;
    bf16* p = q3 + (int64_t)t * q_st + (int64_t)h * q_sh + nope;
    float x1 = __bfloat162float(p[i]), x2 = __bfloat162float(p[i + half]);
    float c = cr[i], s = sr[i];
    p[i] = __float2bfloat16(x1 * c - x2 * s);
    p[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
  // kv latent: RMSNorm
  const bf16* src = kv_a + (int64_t)t * kva_st;
  bf16* dst = kv_layer + (int64_t)slot[t] * (kv_lora + rope);
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_lora; i += blockDim.x) {
    float x = __bfloat162float(src[i]);
    ss += x * x;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)kv_lora + eps);
  for (int i = threadIdx.x; i < kv_lora; i += blockDim.x)
    dst[i] = __float2bfloat16(__bfloat162float(src[i]) * inv * __bfloat162float(norm_w[i]));
  // k_pe: RoPE
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float x1 = __bfloat162float(src[kv_lora + i]), x2 = __bfloat162float(src[kv_lora + i + half]);
    float c = cr[i], s = sr[i];
    dst[kv_lora + i] = __float2bfloat16(x1 * c - x2 * s);
    dst[kv_lora + i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
}

}  // namespace

// q_lat [T, hq, 512] contiguous, q_pe [T, hq, 64] (strides given), out [T, hq, 512] contiguous.
// batch_of: request index of every query token (null: token i belongs to request i, i.e. decode).
LLB_EXPORT int llb_mla_attention(const void* q_lat, const void* q_pe, int64_t qpe_st, int64_t qpe_sh,
                                 const void* kv_layer, const int* req_to_token, int64_t r2t_stride,
                                 const int* b_req_idx, const int* cu_q, const int* b_ready_len, const int* batch_of,
                                 void* out, int B, int T, int hq, int max_q_len, float sm_scale, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  static DeviceOnce configured;     
  if (!configured.done()) {
    cudaError_t e =
        cudaFuncSetAttribute(mla_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MLA_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured.set();  
  }
  dim3 grid((hq + 15) / 16, T);
  mla_attention_kernel<<<grid, 256, MLA_SMEM, st>>>((const bf16*)q_lat, (const bf16*)q_pe, qpe_st, qpe_sh,
                                                    (const bf16*)kv_layer, req_to_token, r2t_stride, b_req_idx, cu_q,
                                                    b_ready_len, batch_of, (bf16*)out, hq, sm_scale * kLog2e);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_mla_rope_kv_scatter(void* q3, int64_t q_st, int64_t q_sh, const void* kv_a, int64_t kva_st,
                                       void* kv_layer, const void* norm_w, const float* cos_t, const float* sin_t,
                                       const int* pos, const int* slot, int T, int hq, int nope, int rope, int kv_lora,
                                       float eps, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  mla_rope_kv_scatter_kernel<<<T, 256, 0, st>>>((bf16*)q3, q_st, q_sh, (const bf16*)kv_a, kva_st, (bf16*)kv_layer,
                                                (const bf16*)norm_w, cos_t, sin_t, pos, slot, hq, nope, rope, kv_lora,
                                                eps);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
