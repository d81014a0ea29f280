// Paged (page size = 1 token) GQA attention over the token-level KV pool.
//
//   pool slice of a layer : kv_layer[slot, 2*Hkv, D]   (K heads first, then V heads)
//   request -> slots      : req_to_token[req, pos]
//
// Decode is HBM-bound (every cached K/V row is read once per step), so the kernel is
// organised around memory-level parallelism: every warp runs a private cp.async ring
// (no CTA barriers in the main loop) that gathers 16 tokens per stage, and the math for
// the G = Hq/Hkv query heads that share a KV head runs on tensor cores as one 16-row
// tile so a K/V row is fetched once for all of them.  Long sequences at small batch
// are split along KV; the partial (o, lse) pairs are merged by a second small kernel.
//
// Prefill is compute-bound but is ~2% of a prefill step's FLOPs for the model sizes
// served here; it is a 64x64-tile online-softmax kernel reading K/V through the same
// slot indirection, aware of an already-cached prefix (chunked prefill / radix hits).
//
// Behavioural counterpart in the reference: token attention over req_to_token_indexs
// (lightllm/common/basemodel/triton_kernel/att/decode_att/gqa/flash_decoding/*,
//  .../att/prefill_att/context_flashattention_nopad.py).
#include "common.cuh"

using namespace llb;
LLB_DEBUG_BOUNDS_STORAGE(attention)


namespace {

template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  // 16-byte chunk index XOR-swizzled by the row so ldmatrix rows hit distinct banks
  return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------
template <int D, int STAGES>
__global__ void __launch_bounds__(128)
gqa_decode_kernel(const bf16* __restrict__ q, int64_t q_stride, const bf16* __restrict__ kv_layer,
                  const int* __restrict__ req_to_token, int64_t r2t_stride, const int* __restrict__ b_req_idx,
                  const int* __restrict__ b_seq_len, bf16* __restrict__ out, int64_t out_stride,
                  float* __restrict__ part_o, float* __restrict__ part_lse, int Hq, int Hkv, int num_splits,
                  float scale_log2) {
  pdl_wait();
  constexpr int CH = D / 8;            // 16-byte chunks per row
  constexpr int ROW_BYTES = D * 2;
  constexpr int TILE_BYTES = 16 * ROW_BYTES;           // 16 tokens
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;          // K + V
  constexpr int WARP_BYTES = STAGES * STAGE_BYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_smem = smem;                                // 16 x D bf16
  uint8_t* warp_smem = smem + TILE_BYTES + (threadIdx.x >> 5) * WARP_BYTES;

  const int split = blockIdx.x;
  const int G = Hq / Hkv;
  const int gc = (G + 15) >> 4;
  const int kvh = blockIdx.y / gc;
  const int chunk_id = blockIdx.y % gc;
  const int head0 = kvh * G + chunk_id * 16;
  const int nrows = min(16, G - chunk_id * 16);
  const int b = blockIdx.z;
  const int req = LLB_CHECK_REQ(b_req_idx[b]);
  const int L = b_seq_len[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;

  const int tiles_total = (L + 15) >> 4;
  const int tiles_per_split = (tiles_total + num_splits - 1) / num_splits;
  const int s0 = split * tiles_per_split * 16;
  const int e0 = min(L, s0 + tiles_per_split * 16);

  if (s0 >= e0) {  // empty split: tell the merge kernel to ignore it
    if (num_splits > 1) {
      for (int r = threadIdx.x; r < nrows; r += blockDim.x)
        part_lse[((int64_t)b * Hq + head0 + r) * num_splits + split] = -INFINITY;
    } else {
      for (int i = threadIdx.x; i < nrows * D; i += blockDim.x)
        out[(int64_t)b * out_stride + (int64_t)(head0 + i / D) * D + (i % D)] = __float2bfloat16(0.f);
    }
    return;
  }

  // ---- Q tile (rows >= nrows are zero) ----
  for (int c = threadIdx.x; c < 16 * CH; c += blockDim.x) {
    int r = c / CH, ch = c % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (int64_t)b * q_stride + (int64_t)(head0 + r) * D + ch * 8);
    *reinterpret_cast<uint4*>(q_smem + swz<D>(r, ch)) = v;
  }
  __syncthreads();
  uint32_t qa[D / 16][4];
  {
    const uint32_t qb = smem_u32(q_smem);
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], qb + swz<D>(row, ks * 2 + (lane >> 4)));
  }

  const int ntiles = (e0 - s0 + 15) >> 4;
  const int my_count = ntiles > warp ? (ntiles - warp + 3) / 4 : 0;
  const int64_t r2t_base = (int64_t)req * r2t_stride;
  const uint32_t wbase = smem_u32(warp_smem);

  // slot numbers of the tile that will be issued next: fetched one call ahead, so that the dependent load (slot
  // number, then the row) does not sit between two issues
  auto load_slots = [&](int i) {
    int slot = -1;
    if (i < my_count) {
      const int p0 = s0 + (warp + 4 * i) * 16;
      if (lane < 16 && p0 + lane < e0) slot = LLB_CHECK_SLOT(req_to_token[r2t_base + p0 + lane]);
    }
    return slot;
  };
  int slot_ahead = load_slots(0);

  auto issue = [&](int i) {  // i-th tile of this warp
    const int slot = slot_ahead;
    slot_ahead = load_slots(i + 1);
    if (i < my_count) {
      const uint32_t sb = wbase + (i % STAGES) * STAGE_BYTES;
#pragma unroll
      for (int j = 0; j < (16 * CH) / 32; ++j) {
        int c = lane + 32 * j;
        int tok = c / CH, ch = c % CH;
        int sl = __shfl_sync(0xffffffffu, slot, tok);
        bool ok = sl >= 0;
        const bf16* src = kv_layer + ((int64_t)(ok ? sl : 0) * (2 * Hkv) + kvh) * D + ch * 8;
        cp_async16(sb + swz<D>(tok, ch), src, ok);
        cp_async16(sb + TILE_BYTES + swz<D>(tok, ch), src + (int64_t)Hkv * D, ok);
      }
    }
    cp_async_commit();
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) issue(i);

  for (int i = 0; i < my_count; ++i) {
    issue(i + STAGES - 1);
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const uint32_t kb = wbase + (i % STAGES) * STAGE_BYTES;
    const uint32_t vb = kb + TILE_BYTES;
    const int p0 = s0 + (warp + 4 * i) * 16;

    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    {
      const int tok = (lane & 7) + (lane >> 4) * 8;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kb + swz<D>(tok, ks * 2 + ((lane >> 3) & 1)));
        mma_bf16_16816(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16_16816(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
    }
    // scale + tail mask
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int pos = p0 + j * 8 + tig * 2 + (e & 1);
        float v = pos < e0 ? s[j][e] * scale_log2 : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
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
      for (int j = 0; j < 2; ++j) {
        s[j][2 * r] = exp2f(s[j][2 * r] - m_use);
        s[j][2 * r + 1] = exp2f(s[j][2 * r + 1] - m_use);
        rs += s[j][2 * r] + s[j][2 * r + 1];
      }
      l_run[r] = l_run[r] * alpha[r] + rs;
    }
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      o[nt][0] *= alpha[0];
      o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1];
      o[nt][3] *= alpha[1];
    }
    const uint32_t a0 = pack_bf16x2(s[0][0], s[0][1]), a1 = pack_bf16x2(s[0][2], s[0][3]);
    const uint32_t a2 = pack_bf16x2(s[1][0], s[1][1]), a3 = pack_bf16x2(s[1][2], s[1][3]);
    {
      const int tok = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int n2 = 0; n2 < D / 16; ++n2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vb + swz<D>(tok, n2 * 2 + (lane >> 4)));
        mma_bf16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncwarp();

  // ---- cross-warp merge through this warp's own ring memory ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  static_assert(WARP_BYTES >= 16 * D * 4 + 128, "ring too small for the merge buffer");
  float* wo = reinterpret_cast<float*>(warp_smem);          // [16][D]
  float* wml = reinterpret_cast<float*>(warp_smem + 16 * D * 4);  // m[16], l[16]
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    int d = nt * 8 + tig * 2;
    *reinterpret_cast<float2*>(wo + g * D + d) = make_float2(o[nt][0], o[nt][1]);
    *reinterpret_cast<float2*>(wo + (g + 8) * D + d) = make_float2(o[nt][2], o[nt][3]);
  }
  if (tig == 0) {
    wml[g] = m_run[0];
    wml[g + 8] = m_run[1];
    wml[16 + g] = l_run[0];
    wml[16 + g + 8] = l_run[1];
  }
  __syncthreads();
  const uint8_t* ring0 = smem + TILE_BYTES;
  for (int idx = threadIdx.x; idx < nrows * D; idx += blockDim.x) {
    int r = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, reinterpret_cast<const float*>(ring0 + w * WARP_BYTES + 16 * D * 4)[r]);
    float num = 0.f, den = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* po = reinterpret_cast<const float*>(ring0 + w * WARP_BYTES);
        const float* pml = reinterpret_cast<const float*>(ring0 + w * WARP_BYTES + 16 * D * 4);
        float sc = exp2f(pml[r] - M);
        num += sc * po[r * D + d];
        den += sc * pml[16 + r];
      }
    }
    float val = den > 0.f ? num / den : 0.f;
    int head = head0 + r;
    if (num_splits == 1) {
      out[(int64_t)b * out_stride + (int64_t)head * D + d] = __float2bfloat16(val);
    } else {
      int64_t pi = ((int64_t)b * Hq + head) * num_splits + split;
      part_o[pi * D + d] = val;
      if (d == 0) part_lse[pi] = den > 0.f ? (M + log2f(den)) * kLn2 : -INFINITY;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(D)
decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, bf16* __restrict__ out,
                    int64_t out_stride, int Hq, int num_splits) {
  pdl_wait();
  const int bh = blockIdx.x;
  const int b = bh / Hq, h = bh % Hq;
  const int d = threadIdx.x;
  const float* lse = part_lse + (int64_t)bh * num_splits;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, lse[s]);
  float num = 0.f, den = 0.f;
  if (M != -INFINITY) {
    for (int s = 0; s < num_splits; ++s) {
      if (lse[s] == -INFINITY) continue;  // empty split: its partial row was never written
      float w = __expf(lse[s] - M);
      num += w * part_o[((int64_t)bh * num_splits + s) * D + d];
      den += w;
    }
  }
  out[(int64_t)b * out_stride + (int64_t)h * D + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

// ---------------------------------------------------------------------------------------
// prefill (causal, varlen, cached-prefix aware)
// ---------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128)
gqa_prefill_kernel(const bf16* __restrict__ q, int64_t q_stride, const bf16* __restrict__ kv_layer,
                   const int* __restrict__ req_to_token, int64_t r2t_stride, const int* __restrict__ b_req_idx,
                   const int* __restrict__ cu_q, const int* __restrict__ b_ready_len, bf16* __restrict__ out,
                   int64_t out_stride, int Hq, int Hkv, float scale_log2) {
  constexpr int CH = D / 8;
  constexpr int BM = 64, BN = 64;
  constexpr int TILE_BYTES = BN * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_smem = smem;                 // BM x D
  uint8_t* kv_smem = smem + BM * D * 2;   // 2 stages x (K, V)

  const int b = blockIdx.z, h = blockIdx.y;
  const int kvh = h / (Hq / Hkv);
  const int q_begin = cu_q[b];
  const int q_len = cu_q[b + 1] - q_begin;
  const int tile = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int q0 = tile * BM;
  if (q0 >= q_len) return;
  const int ready = b_ready_len[b];
  const int req = LLB_CHECK_REQ(b_req_idx[b]);
  const int rows_valid = min(BM, q_len - q0);
  const int kv_end = ready + q0 + rows_valid;  // exclusive upper bound any row of this tile may see
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int64_t r2t_base = (int64_t)req * r2t_stride;

  for (int c = threadIdx.x; c < BM * CH; c += blockDim.x) {
    int r = c / CH, ch = c % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows_valid)
      v = *reinterpret_cast<const uint4*>(q + (int64_t)(q_begin + q0 + r) * q_stride + (int64_t)h * D + ch * 8);
    *reinterpret_cast<uint4*>(q_smem + swz<D>(r, ch)) = v;
  }

  auto issue = [&](int kt, int stage) {
    const uint32_t sb = smem_u32(kv_smem) + stage * 2 * TILE_BYTES;
    for (int c = threadIdx.x; c < BN * CH; c += blockDim.x) {
      int tok = c / CH, ch = c % CH;
      int pos = kt + tok;
      bool ok = pos < kv_end;
      int sl = ok ? LLB_CHECK_SLOT(req_to_token[r2t_base + pos]) : 0;
      const bf16* src = kv_layer + ((int64_t)sl * (2 * Hkv) + kvh) * D + ch * 8;
      cp_async16(sb + swz<D>(tok, ch), src, ok);
      cp_async16(sb + TILE_BYTES + swz<D>(tok, ch), src + (int64_t)Hkv * D, ok);
    }
    cp_async_commit();
  };

  const int n_kv_tiles = (kv_end + BN - 1) / BN;
  issue(0, 0);
  __syncthreads();  // Q tile visible
  uint32_t qa[D / 16][4];
  {
    const uint32_t qb = smem_u32(q_smem);
    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], qb + swz<D>(row, ks * 2 + (lane >> 4)));
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int prow0 = ready + q0 + warp * 16 + g;  // absolute position of this thread's first row

  for (int t = 0; t < n_kv_tiles; ++t) {
    if (t + 1 < n_kv_tiles) {
      issue((t + 1) * BN, (t + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int kt = t * BN;
    const uint32_t kb = smem_u32(kv_smem) + (t & 1) * 2 * TILE_BYTES;
    const uint32_t vb = kb + TILE_BYTES;
    // a warp whose rows all precede this KV tile has nothing to do in it
    const bool warp_active = kt <= ready + q0 + warp * 16 + 15;
    if (warp_active) {
      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int n2 = 0; n2 < BN / 16; ++n2) {
          uint32_t b0, b1, b2, b3;
          const int tok = n2 * 16 + (lane & 7) + (lane >> 4) * 8;
          ldmatrix_x4(b0, b1, b2, b3, kb + swz<D>(tok, ks * 2 + ((lane >> 3) & 1)));
          mma_bf16_16816(s[2 * n2], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
          mma_bf16_16816(s[2 * n2 + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int col = kt + j * 8 + tig * 2 + (e & 1);
          int prow = prow0 + (e >> 1) * 8;
          float v = (col <= prow && col < kv_end) ? s[j][e] * scale_log2 : -INFINITY;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
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
        for (int j = 0; j < BN / 8; ++j) {
          s[j][2 * r] = exp2f(s[j][2 * r] - m_use);
          s[j][2 * r + 1] = exp2f(s[j][2 * r + 1] - m_use);
          rs += s[j][2 * r] + s[j][2 * r + 1];
        }
        l_run[r] = l_run[r] * alpha[r] + rs;
      }
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        o[nt][0] *= alpha[0];
        o[nt][1] *= alpha[0];
        o[nt][2] *= alpha[1];
        o[nt][3] *= alpha[1];
      }
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
        const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                       a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        const int tok = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int n2 = 0; n2 < D / 16; ++n2) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, vb + swz<D>(tok, n2 * 2 + (lane >> 4)));
          mma_bf16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
          mma_bf16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();  // everyone done with this stage before it is refilled
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    int lr = warp * 16 + g + r * 8;
    if (lr < rows_valid) {
      float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      bf16* orow = out + (int64_t)(q_begin + q0 + lr) * out_stride + (int64_t)h * D;
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        bf162 v = __floats2bfloat162_rn(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
        *reinterpret_cast<bf162*>(orow + nt * 8 + tig * 2) = v;
      }
    }
  }
}

constexpr int kDecodeStages = 3;
template <int D>
constexpr int decode_smem_bytes() {
  return 16 * D * 2 + 4 * kDecodeStages * 2 * 16 * D * 2;
}
template <int D>
constexpr int prefill_smem_bytes() {
  return 64 * D * 2 + 2 * 2 * 64 * D * 2;
}

template <typename K>
int set_smem(K kernel, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e == cudaSuccess ? LLB_OK : (int)e;
}

}  // namespace

// Number of KV splits the decode launcher will use for a batch (the caller sizes the
// scratch buffers with it): enough CTAs to fill the GPU, at least 256 tokens per split.
LLB_EXPORT int llb_gqa_decode_num_splits(int B, int Hq, int Hkv, int max_seq_len) {
  int G = Hq / Hkv;
  int ctas = B * Hkv * ((G + 15) / 16);
  int target = 148 * 4;
  int want = (target + ctas - 1) / ctas;
  int cap = (max_seq_len + 255) / 256;
  if (cap < 1) cap = 1;
  int s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return s;
}

// q [B, Hq, D] (row stride q_stride elements), out [B, Hq, D] (row stride out_stride).
// part_o: fp32 [B, Hq, num_splits, D], part_lse: fp32 [B, Hq, num_splits]; only touched when num_splits > 1.
LLB_EXPORT int llb_gqa_decode(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                              int64_t r2t_stride, const int* b_req_idx, const int* b_seq_len, void* out,
                              int64_t out_stride, float* part_o, float* part_lse, int B, int Hq, int Hkv, int D,
                              int num_splits, float sm_scale, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (Hkv <= 0 || Hq % Hkv != 0 || num_splits < 1) return LLB_ERR_BAD_ARG;
  if (num_splits > 1 && (part_o == nullptr || part_lse == nullptr)) return LLB_ERR_BAD_ARG;
  const int G = Hq / Hkv;
  dim3 grid(num_splits, Hkv * ((G + 15) / 16), B);
  const float sl2 = sm_scale * kLog2e;
#define LAUNCH_DECODE(DD)                                                                                         \
  {                                                                                                               \
    static DeviceOnce configured;                                                                                    \
    if (!configured.done()) {                                                                                            \
      int rc = set_smem(gqa_decode_kernel<DD, kDecodeStages>, decode_smem_bytes<DD>());                           \
      if (rc) return rc;                                                                                          \
      configured.set();                                                                                            \
    }                                                                                                             \
    launch_pdl(gqa_decode_kernel<DD, kDecodeStages>, grid, dim3(128), decode_smem_bytes<DD>(), st, (const bf16*)q, \
               q_stride, (const bf16*)kv_layer, req_to_token, r2t_stride, b_req_idx, b_seq_len, (bf16*)out,       \
               out_stride, part_o, part_lse, Hq, Hkv, num_splits, sl2);                                           \
    LLB_LAUNCH_CHECK();                                                                                           \
    if (num_splits > 1) {                                                                                         \
      launch_pdl(decode_merge_kernel<DD>, dim3(B * Hq), dim3(DD), 0, st, (const float*)part_o,                    \
                 (const float*)part_lse, (bf16*)out, out_stride, Hq, num_splits);                                 \
      LLB_LAUNCH_CHECK();                                                                                         \
    }                                                                                                             \
  }
  if (D == 128)
    LAUNCH_DECODE(128)
  else if (D == 64)
    LAUNCH_DECODE(64)
  else
    return LLB_ERR_UNSUPPORTED;
#undef LAUNCH_DECODE
  return LLB_OK;
}

// tcgen05 kernel for head size 128 (attention_tc.cu); LLB_ATTN_TC=0 keeps the mma.sync kernel below
LLB_EXPORT int llb_gqa_prefill_tc(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                                  int64_t r2t_stride, const int* b_req_idx, const int* cu_q, const int* b_ready_len,
                                  void* out, int64_t out_stride, int B, int max_q_len, int Hq, int Hkv, float sm_scale,
                                  cudaStream_t st);
static bool attn_tc_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("LLB_ATTN_TC");
    on = (e == nullptr || e[0] != '0') ? 1 : 0;
  }
  return on == 1;
}

// q [T, Hq, D] new tokens of all requests back to back (cu_q [B+1]); out same layout.
LLB_EXPORT int llb_gqa_prefill(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                               int64_t r2t_stride, const int* b_req_idx, const int* cu_q, const int* b_ready_len,
                               void* out, int64_t out_stride, int B, int max_q_len, int Hq, int Hkv, int D,
                               float sm_scale, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return LLB_OK;
  if (Hkv <= 0 || Hq % Hkv != 0) return LLB_ERR_BAD_ARG;
  if (D == 128 && attn_tc_enabled() && (q_stride % 8) == 0 && (out_stride % 8) == 0 && ((uintptr_t)q & 15) == 0 &&
      ((uintptr_t)out & 15) == 0)
    return llb_gqa_prefill_tc(q, q_stride, kv_layer, req_to_token, r2t_stride, b_req_idx, cu_q, b_ready_len, out,
                              out_stride, B, max_q_len, Hq, Hkv, sm_scale, st);
  dim3 grid((max_q_len + 63) / 64, Hq, B);
  const float sl2 = sm_scale * kLog2e;
#define LAUNCH_PREFILL(DD)                                                                                       \
  {                                                                                                              \
    static DeviceOnce configured;                                                                                   \
    if (!configured.done()) {                                                                                           \
      int rc = set_smem(gqa_prefill_kernel<DD>, prefill_smem_bytes<DD>());                                       \
      if (rc) return rc;                                                                                         \
      configured.set();                                                                                           \
    }                                                                                                            \
    gqa_prefill_kernel<DD><<<grid, 128, prefill_smem_bytes<DD>(), st>>>(                                         \
        (const bf16*)q, q_stride, (const bf16*)kv_layer, req_to_token, r2t_stride, b_req_idx, cu_q, b_ready_len, \
        (bf16*)out, out_stride, Hq, Hkv, sl2);                                                                   \
    LLB_LAUNCH_CHECK();                                                                                          \
  }
  if (D == 128)
    LAUNCH_PREFILL(128)
  else if (D == 64)
    LAUNCH_PREFILL(64)
  else
    return LLB_ERR_UNSUPPORTED;
#undef LAUNCH_PREFILL
  return LLB_OK;
}

// ---------------------------------------------------------------------------------------
// Split-KV decode attention for callers that must not allocate device memory
// (declaration and contract: attention_no_alloc.h).
// ---------------------------------------------------------------------------------------
#include "attention_no_alloc.h"
#include <mutex>

namespace {
// Partial outputs [rows, 128] fp32 followed by partial log-sum-exps [rows] fp32.  Lives in the
// library image: every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) float g_no_alloc_scratch[LLB_NO_ALLOC_MAX_ROWS * 128 + LLB_NO_ALLOC_MAX_ROWS];

constexpr int kMaxDevices = 64;
float* g_no_alloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_no_alloc_mu;

// Device address of the scratch array on the current device.  In host code the array's name is only a
// stand-in for the symbol, not an address a kernel may use, so the address is asked for once per
// device (with that device current) and cached.
int no_alloc_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return LLB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_no_alloc_mu);
  if (g_no_alloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_no_alloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_no_alloc_ptr[dev] = p;
  }
  *out = g_no_alloc_ptr[dev];
  return LLB_OK;
}
}  // namespace

LLB_EXPORT int llb_gqa_decode_no_alloc(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                                       int64_t r2t_stride, const int* b_req_idx, const int* b_seq_len, void* out,
                                       int64_t out_stride, int B, int Hq, int Hkv, int D, int num_splits,
                                       float sm_scale, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (num_splits < 1 || Hq <= 0) return LLB_ERR_BAD_ARG;
  if (D > 128) return LLB_ERR_TOO_LARGE;
  const int64_t rows = (int64_t)B * Hq * num_splits;
  if (num_splits > 1 && rows > LLB_NO_ALLOC_MAX_ROWS) return LLB_ERR_TOO_LARGE;
  float* scratch = nullptr;
  int rc = no_alloc_scratch(&scratch);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: every (row, split) either gets its partial output and
  // log-sum-exp written by this call, or is marked empty (lse = -inf) and skipped by the merge.
  return llb_gqa_decode(q, q_stride, kv_layer, req_to_token, r2t_stride, b_req_idx, b_seq_len, out, out_stride,
                        scratch, scratch + (int64_t)LLB_NO_ALLOC_MAX_ROWS * 128, B, Hq, Hkv, D, num_splits, sm_scale,
                        st);
}
