// int8 KV cache: quantising store and split-KV decode attention over the quantised pool.
//
//   pool slice of a layer : kv_layer[slot, 2*Hkv, D + 16] int8   (K heads first, then V heads)
//   a (slot, head) row    : D int8 values, then one fp32 scale (x = q * scale) and 12 unused bytes, so that
//                           every row starts on a 16-byte boundary and moves as opaque bytes (prefix copies,
//                           staging pages for disaggregated serving, host offload) like a bf16 row does
//
// Decode reads half the bytes of the bf16 pool.  The kernel keeps the structure of the bf16 decode kernel
// (one private cp.async ring per warp, 16 tokens per stage, the G query heads of a KV head as one 16-row
// mma tile): the int8 rows land in shared memory as they are, are widened to fp16 there (exact; two byte
// permutes and two packed subtractions per four values) and feed the same ldmatrix / mma.sync sequence in
// fp16 (the query is converted once per CTA); the K scale of a token multiplies its score column, the V
// scale multiplies its probability column before the P.V product.
//
// The same kernel serves the fp8 pool (`FP8 = true`): rows are D e4m3 values with no scale in the row; the scales are
// static per (layer, head) numbers from a calibration file, so the K scale is folded into the softmax scale of
// the CTA's KV head and the V scale multiplies the output once; widening is the hardware e4m3 -> fp16 conversion.
//
// Behavioural counterpart in the reference: lightllm/common/kv_cache_mem_manager/ppl_int8kv_mem_manager.py
// (group-quantised pool with a scale buffer), fp8_static_per_head_quant_mem_manager.py,
// common/basemodel/attention/triton/int8kv.py, attention/fa3/fp8.py.
#include "common.cuh"
#include <cuda_fp16.h>
#include <cuda_fp8.h>

using namespace llb;

namespace {

constexpr int kPad = 16;                 // bytes after the payload of a row: fp32 scale + padding
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kStages = 2;

template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

// ---------------------------------------------------------------------------------------
// store: src [T, rows, D] bf16 (row stride src_stride elements per token) -> pool rows at slot[t]
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
kv_quant_store_int8_kernel(const bf16* __restrict__ src, int64_t src_stride, int8_t* __restrict__ pool,
                           const int* __restrict__ slot, int T, int rows, int D) {
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * 4 + warp;   // (token, row)
  if (item >= (int64_t)T * rows) return;
  const int t = (int)(item / rows), r = (int)(item % rows);
  const bf16* x = src + (int64_t)t * src_stride + (int64_t)r * D;
  float amax = 0.f;
  for (int d = lane; d < D; d += 32) amax = fmaxf(amax, fabsf(__bfloat162float(x[d])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax / 127.f : 1.f;
  int8_t* dst = pool + ((int64_t)slot[t] * rows + r) * (D + kPad);
  for (int d = lane; d < D; d += 32) {
    float q = rintf(__bfloat162float(x[d]) / scale);   // division: the same rounding as the definition
    q = fminf(fmaxf(q, -127.f), 127.f);
    dst[d] = (int8_t)q;
  }
  if (lane == 0) *reinterpret_cast<float*>(dst + D) = scale;
}

// sixteen int8 -> sixteen fp16 (two 16-byte chunks).  With the sign bit flipped a byte is u = q + 128; placing u
// in the low byte of a half whose high byte is 0x64 gives the fp16 number 1024 + u, and subtracting 1152 leaves q
// exactly: two byte permutes and two packed subtractions per four values.
__device__ __forceinline__ void widen16(const uint4& in, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t o[8];
  const __half2 bias = __halves2half2(__ushort_as_half((unsigned short)0x6480), __ushort_as_half((unsigned short)0x6480));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t x = w[i] ^ 0x80808080u;
    uint32_t p0 = __byte_perm(x, 0x64646464u, 0x4140);
    uint32_t p1 = __byte_perm(x, 0x64646464u, 0x4342);
    __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&p0), bias);
    __half2 h1 = __hsub2(*reinterpret_cast<__half2*>(&p1), bias);
    o[2 * i] = *reinterpret_cast<uint32_t*>(&h0);
    o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&h1);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// The two 16-byte chunks of one widened group.  With 8 groups per row (D = 128) the eight lanes that share a
// store instruction would hit only the even chunk slots; the upper four lanes store their odd chunk first, so
// every store covers eight distinct slots.
template <int D>
__device__ __forceinline__ void store_pair(uint8_t* tile, int tok, int ch, const uint4& lo, const uint4& hi) {
  if (D == 128) {
    const bool up = (ch & 4) != 0;
    const uint4 first = up ? hi : lo, second = up ? lo : hi;
    const int c0 = 2 * ch + (up ? 1 : 0), c1 = 2 * ch + (up ? 0 : 1);
    *reinterpret_cast<uint4*>(tile + (uint32_t)(tok * (D * 2) + ((c0 ^ (tok & 7)) << 4))) = first;
    *reinterpret_cast<uint4*>(tile + (uint32_t)(tok * (D * 2) + ((c1 ^ (tok & 7)) << 4))) = second;
  } else {
    *reinterpret_cast<uint4*>(tile + (uint32_t)(tok * (D * 2) + (((2 * ch) ^ (tok & 7)) << 4))) = lo;
    *reinterpret_cast<uint4*>(tile + (uint32_t)(tok * (D * 2) + (((2 * ch + 1) ^ (tok & 7)) << 4))) = hi;
  }
}

// sixteen e4m3 -> sixteen fp16
__device__ __forceinline__ void widen16_fp8(const uint4& in, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xffffu), __NV_E4M3);
    __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
    o[2 * i] = (uint32_t)a.x | ((uint32_t)a.y << 16);
    o[2 * i + 1] = (uint32_t)b.x | ((uint32_t)b.y << 16);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void mma_f16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// eight bf16 -> eight fp16, saturated to the fp16 range
__device__ __forceinline__ uint4 bf16x8_to_f16x8(const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
    lo = fminf(fmaxf(lo, -65504.f), 65504.f);
    hi = fminf(fmaxf(hi, -65504.f), 65504.f);
    o[i] = pack_f16x2(lo, hi);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// ---------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------
template <int D>
struct Int8DecodeSmem {
  static constexpr int Q_BYTES = 16 * D * 2;
  static constexpr int TILE8 = 16 * D;                    // one int8 tile (K or V) of 16 tokens
  static constexpr int STAGE = 2 * TILE8 + 32 * 16;        // K, V, then 32 scale chunks of 16 bytes
  static constexpr int TILE16 = 16 * D * 2;                // one widened tile
  static constexpr int WARP = kStages * STAGE + TILE16;     // one widened tile: K, then (after Q.K^T) V
  static constexpr int TOTAL = Q_BYTES + 4 * WARP;
};

template <int D, bool FP8>
__global__ void __launch_bounds__(128)
gqa_decode_int8_kernel(const bf16* __restrict__ q, int64_t q_stride, const int8_t* __restrict__ kv_layer,
                       const int* __restrict__ req_to_token, int64_t r2t_stride, const int* __restrict__ b_req_idx,
                       const int* __restrict__ b_seq_len, bf16* __restrict__ out, int64_t out_stride,
                       float* __restrict__ part_o, float* __restrict__ part_lse, int Hq, int Hkv, int num_splits,
                       float scale_log2_in, const float* __restrict__ head_scales) {
  pdl_wait();
  using S = Int8DecodeSmem<D>;
  constexpr int CH = D / 8;     // 16-byte chunks of a bf16 row
  constexpr int CH8 = D / 16;   // 16-byte chunks of an 8-bit row
  constexpr int ROW = FP8 ? D : D + kPad;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_smem = smem;
  uint8_t* warp_smem = smem + S::Q_BYTES + (threadIdx.x >> 5) * S::WARP;
  uint8_t* wide = warp_smem + kStages * S::STAGE;          // the widened tile

  const int split = blockIdx.x;
  const int G = Hq / Hkv;
  const int gc = (G + 15) >> 4;
  const int kvh = blockIdx.y / gc;
  const int chunk_id = blockIdx.y % gc;
  const int head0 = kvh * G + chunk_id * 16;
  const int nrows = min(16, G - chunk_id * 16);
  const int b = blockIdx.z;
  const int req = b_req_idx[b];
  const int L = b_seq_len[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  // fp8 pool: static scales of this KV head (K folded into the score scale, V applied to the output)
  const float scale_log2 = FP8 ? scale_log2_in * head_scales[kvh] : scale_log2_in;
  const float out_scale = FP8 ? head_scales[Hkv + kvh] : 1.f;

  const int tiles_total = (L + 15) >> 4;
  const int tiles_per_split = (tiles_total + num_splits - 1) / num_splits;
  const int s0 = split * tiles_per_split * 16;
  const int e0 = min(L, s0 + tiles_per_split * 16);

  if (s0 >= e0) {
    if (num_splits > 1) {
      for (int r = threadIdx.x; r < nrows; r += blockDim.x)
        part_lse[((int64_t)b * Hq + head0 + r) * num_splits + split] = -INFINITY;
    } else {
      for (int i = threadIdx.x; i < nrows * D; i += blockDim.x)
        out[(int64_t)b * out_stride + (int64_t)(head0 + i / D) * D + (i % D)] = __float2bfloat16(0.f);
    }
    return;
  }

  for (int c = threadIdx.x; c < 16 * CH; c += blockDim.x) {
    int r = c / CH, ch = c % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows)
      v = bf16x8_to_f16x8(*reinterpret_cast<const uint4*>(q + (int64_t)b * q_stride + (int64_t)(head0 + r) * D + ch * 8));
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

  auto load_slots = [&](int i) {
    int slot = -1;
    if (i < my_count) {
      const int p0 = s0 + (warp + 4 * i) * 16;
      if (lane < 16 && p0 + lane < e0) slot = req_to_token[r2t_base + p0 + lane];
    }
    return slot;
  };
  int slot_ahead = load_slots(0);

  auto issue = [&](int i) {
    const int slot = slot_ahead;
    slot_ahead = load_slots(i + 1);
    if (i < my_count) {
      const uint32_t sb = wbase + (i % kStages) * S::STAGE;
#pragma unroll
      for (int j = 0; j < (16 * CH8) / 32; ++j) {
        int c = lane + 32 * j;
        int tok = c / CH8, ch = c % CH8;
        int sl = __shfl_sync(0xffffffffu, slot, tok);
        bool ok = sl >= 0;
        const int8_t* src = kv_layer + ((int64_t)(ok ? sl : 0) * (2 * Hkv) + kvh) * ROW + ch * 16;
        cp_async16(sb + tok * D + ch * 16, src, ok);
        cp_async16(sb + S::TILE8 + tok * D + ch * 16, src + (int64_t)Hkv * ROW, ok);
      }
      if (!FP8) {  // scales: lanes 0..15 the K rows, lanes 16..31 the V rows
        int tok = lane & 15;
        int sl = __shfl_sync(0xffffffffu, slot, tok);
        bool ok = sl >= 0;
        const int8_t* src = kv_layer + ((int64_t)(ok ? sl : 0) * (2 * Hkv) + kvh + (lane >> 4) * Hkv) * ROW + D;
        cp_async16(sb + 2 * S::TILE8 + lane * 16, src, ok);
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
  for (int i = 0; i < kStages - 1; ++i) issue(i);

  const uint32_t kb = smem_u32(wide);
  const uint32_t vb = kb;
  for (int i = 0; i < my_count; ++i) {
    issue(i + kStages - 1);
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const uint8_t* st8 = warp_smem + (i % kStages) * S::STAGE;
    const int p0 = s0 + (warp + 4 * i) * 16;

    // widen K into the swizzled fp16 tile
#pragma unroll
    for (int j = 0; j < (16 * CH8) / 32; ++j) {
      int c = lane + 32 * j;
      int tok = c / CH8, ch = c % CH8;
      uint4 lo, hi;
      if (FP8)
        widen16_fp8(*reinterpret_cast<const uint4*>(st8 + tok * D + ch * 16), lo, hi);
      else
        widen16(*reinterpret_cast<const uint4*>(st8 + tok * D + ch * 16), lo, hi);
      store_pair<D>(wide, tok, ch, lo, hi);
    }
    __syncwarp();
    const float* sc = reinterpret_cast<const float*>(st8 + 2 * S::TILE8);   // [32] scales, 4 floats apart

    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    {
      const int tok = (lane & 7) + (lane >> 4) * 8;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kb + swz<D>(tok, ks * 2 + ((lane >> 3) & 1)));
        mma_f16_16816(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_f16_16816(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
    }
    __syncwarp();   // every lane has read its K fragments: the tile is free for V
#pragma unroll
    for (int j = 0; j < (16 * CH8) / 32; ++j) {
      int c = lane + 32 * j;
      int tok = c / CH8, ch = c % CH8;
      uint4 lo, hi;
      if (FP8)
        widen16_fp8(*reinterpret_cast<const uint4*>(st8 + S::TILE8 + tok * D + ch * 16), lo, hi);
      else
        widen16(*reinterpret_cast<const uint4*>(st8 + S::TILE8 + tok * D + ch * 16), lo, hi);
      store_pair<D>(wide, tok, ch, lo, hi);
    }
    __syncwarp();
    float vs[2][2];   // V scale of the token columns this lane holds
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        const int col = j * 8 + tig * 2 + c2;
        const float ks_ = FP8 ? 1.f : sc[col * 4];
        vs[j][c2] = FP8 ? 1.f : sc[(16 + col) * 4];
        const bool in = p0 + col < e0;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int e = 2 * r + c2;
          float v = in ? s[j][e] * ks_ * scale_log2 : -INFINITY;
          s[j][e] = v;
          mx[r] = fmaxf(mx[r], v);
        }
        if (!in) vs[j][c2] = 0.f;
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
    const uint32_t a0 = pack_f16x2(s[0][0] * vs[0][0], s[0][1] * vs[0][1]);
    const uint32_t a1 = pack_f16x2(s[0][2] * vs[0][0], s[0][3] * vs[0][1]);
    const uint32_t a2 = pack_f16x2(s[1][0] * vs[1][0], s[1][1] * vs[1][1]);
    const uint32_t a3 = pack_f16x2(s[1][2] * vs[1][0], s[1][3] * vs[1][1]);
    {
      const int tok = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int n2 = 0; n2 < D / 16; ++n2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vb + swz<D>(tok, n2 * 2 + (lane >> 4)));
        mma_f16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
        mma_f16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncwarp();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  static_assert(S::WARP >= 16 * D * 4 + 128, "warp memory too small for the merge buffer");
  float* wo = reinterpret_cast<float*>(warp_smem);
  float* wml = reinterpret_cast<float*>(warp_smem + 16 * D * 4);
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
  const uint8_t* ring0 = smem + S::Q_BYTES;
  for (int idx = threadIdx.x; idx < nrows * D; idx += blockDim.x) {
    int r = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, reinterpret_cast<const float*>(ring0 + w * S::WARP + 16 * D * 4)[r]);
    float num = 0.f, den = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* po = reinterpret_cast<const float*>(ring0 + w * S::WARP);
        const float* pml = reinterpret_cast<const float*>(ring0 + w * S::WARP + 16 * D * 4);
        float sc2 = exp2f(pml[r] - M);
        num += sc2 * po[r * D + d];
        den += sc2 * pml[16 + r];
      }
    }
    float val = den > 0.f ? num / den * out_scale : 0.f;
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

// ---------------------------------------------------------------------------------------
// decode, head size 128, mma fragments built from registers
// ---------------------------------------------------------------------------------------
// The 8-bit rows are staged as they are (row pitch 144 bytes, which also staggers the rows over the banks) and the
// mma operands are assembled straight from 16-byte shared-memory loads: no widened tile, no ldmatrix.
//  * Q.K^T: the contraction runs over the head dimension, whose order does not matter as long as Q and K agree.
//    Lane (g, tig) owns bytes [32 tig, 32 tig + 32) of a K row: k-step ks takes its bytes 4 ks .. 4 ks + 3 (two for
//    each half of the B fragment).  The Q fragments are loaded once with the same mapping.
//  * P.V: the output column order is free as long as the store undoes it.  Column g of n-tile nt stands for
//    d = 16 g + nt: lane (g, tig) reads bytes [16 g, 16 g + 16) of token rows 2 tig, 2 tig + 1, 2 tig + 8, 2 tig + 9
//    and pairs byte nt of two rows into one half2.
constexpr int kRowPitch = 144;
constexpr int kRegStages = 4;
constexpr int kRegStageBytes = 2 * 16 * kRowPitch;            // K tile + V tile
constexpr int kRegWarpBytes = kRegStages * kRegStageBytes;    // 18432
constexpr int kRegSmemBytes = 4 * kRegWarpBytes;

template <bool FP8>
__device__ __forceinline__ void cvt_k_word(uint32_t w, uint32_t& b0, uint32_t& b1) {
  if (FP8) {
    __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
    __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
    b0 = (uint32_t)a.x | ((uint32_t)a.y << 16);
    b1 = (uint32_t)b.x | ((uint32_t)b.y << 16);
  } else {
    const __half2 bias = __halves2half2(__ushort_as_half((unsigned short)0x6480), __ushort_as_half((unsigned short)0x6480));
    const uint32_t x = w ^ 0x80808080u;
    uint32_t p0 = __byte_perm(x, 0x64646464u, 0x4140);
    uint32_t p1 = __byte_perm(x, 0x64646464u, 0x4342);
    __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&p0), bias);
    __half2 h1 = __hsub2(*reinterpret_cast<__half2*>(&p1), bias);
    b0 = *reinterpret_cast<uint32_t*>(&h0);
    b1 = *reinterpret_cast<uint32_t*>(&h1);
  }
}

// byte `i` (0..3) of word a and of word b as one half2 (a first)
template <bool FP8>
__device__ __forceinline__ uint32_t cvt_v_pair(uint32_t a, uint32_t b, int i) {
  const uint32_t p = __byte_perm(a, b, (uint32_t)(i | ((4 + i) << 4)));   // low 16 bits: {a.byte i, b.byte i}
  if (FP8) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(p & 0xffffu), __NV_E4M3);
    return (uint32_t)h.x | ((uint32_t)h.y << 16);
  } else {
    const __half2 bias = __halves2half2(__ushort_as_half((unsigned short)0x6480), __ushort_as_half((unsigned short)0x6480));
    uint32_t q = __byte_perm(p ^ 0x00008080u, 0x64646464u, 0x4140);
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&q), bias);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

template <bool FP8>
__global__ void __launch_bounds__(128)
gqa_decode_q8_regs_kernel(const bf16* __restrict__ q, int64_t q_stride, const int8_t* __restrict__ kv_layer,
                          const int* __restrict__ req_to_token, int64_t r2t_stride, const int* __restrict__ b_req_idx,
                          const int* __restrict__ b_seq_len, bf16* __restrict__ out, int64_t out_stride,
                          float* __restrict__ part_o, float* __restrict__ part_lse, int Hq, int Hkv, int num_splits,
                          float scale_log2_in, const float* __restrict__ head_scales) {
  pdl_wait();
  constexpr int D = 128;
  constexpr int ROW = FP8 ? D : D + kPad;          // bytes of a row in the pool
  constexpr int CHUNKS = ROW / 16;                  // 8 or 9 (the ninth carries the int8 row's scale)
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* warp_smem = smem + (threadIdx.x >> 5) * kRegWarpBytes;

  const int split = blockIdx.x;
  const int G = Hq / Hkv;
  const int gc = (G + 15) >> 4;
  const int kvh = blockIdx.y / gc;
  const int chunk_id = blockIdx.y % gc;
  const int head0 = kvh * G + chunk_id * 16;
  const int nrows = min(16, G - chunk_id * 16);
  const int b = blockIdx.z;
  const int req = b_req_idx[b];
  const int L = b_seq_len[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const float scale_log2 = FP8 ? scale_log2_in * head_scales[kvh] : scale_log2_in;
  const float out_scale = FP8 ? head_scales[Hkv + kvh] : 1.f;

  const int tiles_total = (L + 15) >> 4;
  const int tiles_per_split = (tiles_total + num_splits - 1) / num_splits;
  const int s0 = split * tiles_per_split * 16;
  const int e0 = min(L, s0 + tiles_per_split * 16);

  if (s0 >= e0) {
    if (num_splits > 1) {
      for (int r = threadIdx.x; r < nrows; r += blockDim.x)
        part_lse[((int64_t)b * Hq + head0 + r) * num_splits + split] = -INFINITY;
    } else {
      for (int i = threadIdx.x; i < nrows * D; i += blockDim.x)
        out[(int64_t)b * out_stride + (int64_t)(head0 + i / D) * D + (i % D)] = __float2bfloat16(0.f);
    }
    return;
  }

  // ---- Q fragments: rows g and g + 8, elements [32 tig, 32 tig + 32) of each, four per k-step ----
  uint32_t qa[8][4];
  {
    uint4 r0[4], r1[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      r0[c] = make_uint4(0, 0, 0, 0);
      r1[c] = make_uint4(0, 0, 0, 0);
      if (g < nrows)
        r0[c] = bf16x8_to_f16x8(*reinterpret_cast<const uint4*>(q + (int64_t)b * q_stride + (int64_t)(head0 + g) * D +
                                                                 tig * 32 + c * 8));
      if (g + 8 < nrows)
        r1[c] = bf16x8_to_f16x8(*reinterpret_cast<const uint4*>(q + (int64_t)b * q_stride +
                                                                 (int64_t)(head0 + g + 8) * D + tig * 32 + c * 8));
    }
    // k-step ks uses elements 4 ks .. 4 ks + 3: half2 (4ks, 4ks+1) and half2 (4ks+2, 4ks+3)
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint4& a = r0[ks >> 1];
      const uint4& c = r1[ks >> 1];
      qa[ks][0] = (ks & 1) ? a.z : a.x;
      qa[ks][2] = (ks & 1) ? a.w : a.y;
      qa[ks][1] = (ks & 1) ? c.z : c.x;
      qa[ks][3] = (ks & 1) ? c.w : c.y;
    }
  }

  const int ntiles = (e0 - s0 + 15) >> 4;
  const int my_count = ntiles > warp ? (ntiles - warp + 3) / 4 : 0;
  const int64_t r2t_base = (int64_t)req * r2t_stride;
  const uint32_t wbase = smem_u32(warp_smem);

  auto load_slots = [&](int i) {
    int slot = -1;
    if (i < my_count) {
      const int p0 = s0 + (warp + 4 * i) * 16;
      if (lane < 16 && p0 + lane < e0) slot = req_to_token[r2t_base + p0 + lane];
    }
    return slot;
  };
  int slot_ahead = load_slots(0);

  auto issue = [&](int i) {
    const int slot = slot_ahead;
    slot_ahead = load_slots(i + 1);
    if (i < my_count) {
      const uint32_t sb = wbase + (i % kRegStages) * kRegStageBytes;
      // 16 rows x CHUNKS chunks per tile; lanes walk the (row, chunk) pairs
#pragma unroll
      for (int it = 0; it < (16 * CHUNKS + 31) / 32; ++it) {   // every lane takes part in the shuffle
        const int c = lane + 32 * it;
        const bool active = c < 16 * CHUNKS;
        const int tok = active ? c / CHUNKS : 0, ch = active ? c % CHUNKS : 0;
        const int sl = __shfl_sync(0xffffffffu, slot, tok);
        const bool ok = sl >= 0;
        const int8_t* src = kv_layer + ((int64_t)(ok ? sl : 0) * (2 * Hkv) + kvh) * ROW + ch * 16;
        if (active) {
          cp_async16(sb + tok * kRowPitch + ch * 16, src, ok);
          cp_async16(sb + 16 * kRowPitch + tok * kRowPitch + ch * 16, src + (int64_t)Hkv * ROW, ok);
        }
      }
    }
    cp_async_commit();
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

#pragma unroll
  for (int i = 0; i < kRegStages - 1; ++i) issue(i);

  for (int i = 0; i < my_count; ++i) {
    issue(i + kRegStages - 1);
    cp_async_wait<kRegStages - 1>();
    __syncwarp();
    const uint8_t* kt = warp_smem + (i % kRegStages) * kRegStageBytes;
    const uint8_t* vt = kt + 16 * kRowPitch;
    const int p0 = s0 + (warp + 4 * i) * 16;

    float s[2][4];
    {
      // four independent accumulation chains (two token groups x even / odd k-steps) instead of two of length eight
      float acc[2][2][4];
      uint32_t w[2][8];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint8_t* row = kt + (8 * j + g) * kRowPitch + tig * 32;
        const uint4 w0 = *reinterpret_cast<const uint4*>(row);
        const uint4 w1 = *reinterpret_cast<const uint4*>(row + 16);
        w[j][0] = w0.x, w[j][1] = w0.y, w[j][2] = w0.z, w[j][3] = w0.w;
        w[j][4] = w1.x, w[j][5] = w1.y, w[j][6] = w1.z, w[j][7] = w1.w;
#pragma unroll
        for (int h = 0; h < 2; ++h) acc[j][h][0] = acc[j][h][1] = acc[j][h][2] = acc[j][h][3] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t b0, b1;
          cvt_k_word<FP8>(w[j][ks], b0, b1);
          mma_f16_16816(acc[j][ks & 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = acc[j][0][e] + acc[j][1][e];
    }
    float vs[2][2];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        const int col = j * 8 + tig * 2 + c2;
        const float ks_ = FP8 ? 1.f : *reinterpret_cast<const float*>(kt + col * kRowPitch + D);
        vs[j][c2] = FP8 ? 1.f : *reinterpret_cast<const float*>(vt + col * kRowPitch + D);
        const bool in = p0 + col < e0;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int e = 2 * r + c2;
          float v = in ? s[j][e] * ks_ * scale_log2 : -INFINITY;
          s[j][e] = v;
          mx[r] = fmaxf(mx[r], v);
        }
        if (!in) vs[j][c2] = 0.f;
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
    for (int nt = 0; nt < 16; ++nt) {
      o[nt][0] *= alpha[0];
      o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1];
      o[nt][3] *= alpha[1];
    }
    const uint32_t a0 = pack_f16x2(s[0][0] * vs[0][0], s[0][1] * vs[0][1]);
    const uint32_t a1 = pack_f16x2(s[0][2] * vs[0][0], s[0][3] * vs[0][1]);
    const uint32_t a2 = pack_f16x2(s[1][0] * vs[1][0], s[1][1] * vs[1][1]);
    const uint32_t a3 = pack_f16x2(s[1][2] * vs[1][0], s[1][3] * vs[1][1]);
    {
      const uint8_t* base = vt + g * 16;
      const uint4 va = *reinterpret_cast<const uint4*>(base + (2 * tig) * kRowPitch);
      const uint4 vb = *reinterpret_cast<const uint4*>(base + (2 * tig + 1) * kRowPitch);
      const uint4 vc = *reinterpret_cast<const uint4*>(base + (2 * tig + 8) * kRowPitch);
      const uint4 vd = *reinterpret_cast<const uint4*>(base + (2 * tig + 9) * kRowPitch);
      const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
      const uint32_t wc[4] = {vc.x, vc.y, vc.z, vc.w}, wd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const uint32_t b0 = cvt_v_pair<FP8>(wa[nt >> 2], wb[nt >> 2], nt & 3);
        const uint32_t b1 = cvt_v_pair<FP8>(wc[nt >> 2], wd[nt >> 2], nt & 3);
        mma_f16_16816(o[nt], a0, a1, a2, a3, b0, b1);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncwarp();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  static_assert(kRegWarpBytes >= 16 * 128 * 4 + 128, "warp memory too small for the merge buffer");
  float* wo = reinterpret_cast<float*>(warp_smem);
  float* wml = reinterpret_cast<float*>(warp_smem + 16 * D * 4);
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {   // column c of n-tile nt is d = 16 c + nt
    const int d0 = (2 * tig) * 16 + nt, d1 = (2 * tig + 1) * 16 + nt;
    wo[g * D + d0] = o[nt][0];
    wo[g * D + d1] = o[nt][1];
    wo[(g + 8) * D + d0] = o[nt][2];
    wo[(g + 8) * D + d1] = o[nt][3];
  }
  if (tig == 0) {
    wml[g] = m_run[0];
    wml[g + 8] = m_run[1];
    wml[16 + g] = l_run[0];
    wml[16 + g + 8] = l_run[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * D; idx += blockDim.x) {
    int r = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, reinterpret_cast<const float*>(smem + w * kRegWarpBytes + 16 * D * 4)[r]);
    float num = 0.f, den = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* po = reinterpret_cast<const float*>(smem + w * kRegWarpBytes);
        const float* pml = reinterpret_cast<const float*>(smem + w * kRegWarpBytes + 16 * D * 4);
        float sc2 = exp2f(pml[r] - M);
        num += sc2 * po[r * D + d];
        den += sc2 * pml[16 + r];
      }
    }
    float val = den > 0.f ? num / den * out_scale : 0.f;
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
decode_merge_int8_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, bf16* __restrict__ out,
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
      if (lse[s] == -INFINITY) continue;
      float w = __expf(lse[s] - M);
      num += w * part_o[((int64_t)bh * num_splits + s) * D + d];
      den += w;
    }
  }
  out[(int64_t)b * out_stride + (int64_t)h * D + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

}  // namespace

// src [T, rows, D] bf16 -> pool[slot[t], rows, D + 16] int8 with per-row scales
LLB_EXPORT int llb_kv_quant_store_int8(const void* src, int64_t src_stride, void* pool, const int* slot, int T,
                                       int rows, int D, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (rows <= 0 || D <= 0 || (D % 16) != 0) return LLB_ERR_BAD_ARG;
  const int64_t items = (int64_t)T * rows;
  launch_pdl(kv_quant_store_int8_kernel, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, st, (const bf16*)src,
             src_stride, (int8_t*)pool, slot, T, rows, D);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

namespace {
// Head size 128 runs the register-fragment kernel; LLB_KV8_REGS=0 selects the kernel that widens the tile in shared
// memory (the one head size 64 uses) for comparison.
bool kv8_regs_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("LLB_KV8_REGS");
    on = (e == nullptr || e[0] != '0') ? 1 : 0;
  }
  return on == 1;
}

template <bool FP8>
int launch_decode8(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token, int64_t r2t_stride,
                   const int* b_req_idx, const int* b_seq_len, void* out, int64_t out_stride, float* part_o,
                   float* part_lse, int B, int Hq, int Hkv, int D, int num_splits, float sm_scale,
                   const float* head_scales, cudaStream_t st) {
  if (B <= 0) return LLB_OK;
  if (Hkv <= 0 || Hq % Hkv != 0 || num_splits < 1) return LLB_ERR_BAD_ARG;
  if (num_splits > 1 && (part_o == nullptr || part_lse == nullptr)) return LLB_ERR_BAD_ARG;
  if (FP8 && head_scales == nullptr) return LLB_ERR_BAD_ARG;
  const int G = Hq / Hkv;
  dim3 grid(num_splits, Hkv * ((G + 15) / 16), B);
  const float sl2 = sm_scale * kLog2e;
#define LAUNCH_DECODE8(DD)                                                                                          \
  {                                                                                                                 \
    static DeviceOnce configured;                                                                                      \
    if (!configured.done()) {                                                                                              \
      cudaError_t e = cudaFuncSetAttribute(gqa_decode_int8_kernel<DD, FP8>,                                         \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, Int8DecodeSmem<DD>::TOTAL); \
      if (e != cudaSuccess) return (int)e;                                                                          \
      configured.set();                                                                                              \
    }                                                                                                               \
    launch_pdl(gqa_decode_int8_kernel<DD, FP8>, grid, dim3(128), Int8DecodeSmem<DD>::TOTAL, st, (const bf16*)q,     \
               q_stride, (const int8_t*)kv_layer, req_to_token, r2t_stride, b_req_idx, b_seq_len, (bf16*)out,       \
               out_stride, part_o, part_lse, Hq, Hkv, num_splits, sl2, head_scales);                                \
    LLB_LAUNCH_CHECK();                                                                                             \
    if (num_splits > 1) {                                                                                           \
      launch_pdl(decode_merge_int8_kernel<DD>, dim3(B * Hq), dim3(DD), 0, st, (const float*)part_o,                 \
                 (const float*)part_lse, (bf16*)out, out_stride, Hq, num_splits);                                   \
      LLB_LAUNCH_CHECK();                                                                                           \
    }                                                                                                               \
  }
  if (D == 128 && kv8_regs_enabled()) {
    static DeviceOnce configured;     
    if (!configured.done()) {
      cudaError_t e = cudaFuncSetAttribute(gqa_decode_q8_regs_kernel<FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kRegSmemBytes);
      if (e != cudaSuccess) return (int)e;
      configured.set();  
    }
    launch_pdl(gqa_decode_q8_regs_kernel<FP8>, grid, dim3(128), kRegSmemBytes, st, (const bf16*)q, q_stride,
               (const int8_t*)kv_layer, req_to_token, r2t_stride, b_req_idx, b_seq_len, (bf16*)out, out_stride,
               part_o, part_lse, Hq, Hkv, num_splits, sl2, head_scales);
    LLB_LAUNCH_CHECK();
    if (num_splits > 1) {
      launch_pdl(decode_merge_int8_kernel<128>, dim3(B * Hq), dim3(128), 0, st, (const float*)part_o,
                 (const float*)part_lse, (bf16*)out, out_stride, Hq, num_splits);
      LLB_LAUNCH_CHECK();
    }
    return LLB_OK;
  }
  if (D == 128)
    LAUNCH_DECODE8(128)
  else if (D == 64)
    LAUNCH_DECODE8(64)
  else
    return LLB_ERR_UNSUPPORTED;
#undef LAUNCH_DECODE8
  return LLB_OK;
}
}  // namespace

// Same contract as llb_gqa_decode with kv_layer the int8 pool slice described at the top of this file.
LLB_EXPORT int llb_gqa_decode_int8kv(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                                     int64_t r2t_stride, const int* b_req_idx, const int* b_seq_len, void* out,
                                     int64_t out_stride, float* part_o, float* part_lse, int B, int Hq, int Hkv,
                                     int D, int num_splits, float sm_scale, cudaStream_t st) {
  return launch_decode8<false>(q, q_stride, kv_layer, req_to_token, r2t_stride, b_req_idx, b_seq_len, out, out_stride,
                               part_o, part_lse, B, Hq, Hkv, D, num_splits, sm_scale, nullptr, st);
}

// kv_layer: e4m3 rows [slot, 2*Hkv, D]; head_scales: fp32 [2*Hkv] of this layer (K heads, then V heads), x = q * scale.
LLB_EXPORT int llb_gqa_decode_fp8kv(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                                    int64_t r2t_stride, const int* b_req_idx, const int* b_seq_len, void* out,
                                    int64_t out_stride, float* part_o, float* part_lse, int B, int Hq, int Hkv, int D,
                                    int num_splits, float sm_scale, const float* head_scales, cudaStream_t st) {
  return launch_decode8<true>(q, q_stride, kv_layer, req_to_token, r2t_stride, b_req_idx, b_seq_len, out, out_stride,
                              part_o, part_lse, B, Hq, Hkv, D, num_splits, sm_scale, head_scales, st);
}
