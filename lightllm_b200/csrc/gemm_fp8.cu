// fp8 (e4m3) GEMM with 128 x 128 block scales for sm_100a:  C[M, N] = sum_kb sa[kb, m] * sw[n / g, kb] * (A_kb . W_kb^T).
//
// A [M, K] e4m3 carries one fp32 scale per token and 128-wide K group (stored K-group major, `a_scale[kb * a_scale_ld
// + m]`, so that the 128 epilogue threads of a tile read consecutive floats); W [N, K] e4m3 carries one fp32 scale
// per g weight rows and 128-wide K group (`w_scale[(n / g) * KB + kb]`, g = 128 for checkpoint layout, 32 for
// gate / up matrices interleaved in blocks of 32 rows).  This is the DeepSeek-V3 checkpoint scheme
// (`weight_scale_inv`), reference: lightllm/common/quantization/deepgemm.py:46-126 (deep_gemm.fp8_gemm_nt) and
// lightllm/common/quantization/w8a8.py:477-531.
//
// One CTA per 128 x 128 output tile (persistent over tiles).  Warp 0 streams 128 x 128-byte operand tiles with TMA
// (128B swizzle), warp 1 issues tcgen05.mma kind::f8f6f4 (four K = 32 instructions per K group) into one of two
// 128-column tensor-memory buffers, starting every K group from zero; the four epilogue warps read the finished
// group back (tcgen05.ld), multiply by the group's two scales and add into fp32 registers (one output row per
// thread) while the tensor core works on the next group in the other buffer.  Grouped (MoE) mode: M-block i
// multiplies with expert mblock_expert[i] of the stacked weights [E * N, K]; -1 skips the block.
#include "sm100_ptx.cuh"

#include <cuda_fp8.h>

using namespace llb;
using namespace llb::sm100;

namespace {

constexpr int BM = 128, BN = 128, BKB = 128;  // BKB: K elements (= bytes) per stage, one scale group
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BKB, STAGE_BYTES = A_BYTES + BN * BKB;
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t TMEM_COLS = 256;

enum { F8_STORE = 0, F8_RESIDUAL = 1, F8_GATED_SILU = 2 };

struct Fp8Params {
  bf16* C;
  const bf16* residual;
  const float* a_scale;
  const float* w_scale;
  const int* mblock_expert;
  int* status;
  int M, N, K;
  int64_t ldc, a_scale_ld;
  int ws_rows;        // weight rows per scale (128 or 32)
  int ws_total_rows;  // rows of the w_scale array (clamp for a ragged last tile)
  int num_m_blocks, num_n_blocks, group_m;
  int epi;
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int GROUP, int& mb, int& nb) {
  int per_group = GROUP * num_n;
  int grp = tile / per_group;
  int first_m = grp * GROUP;
  int gsz = min(GROUP, num_m - first_m);
  int in = tile - grp * per_group;
  mb = first_m + in % gsz;
  nb = in / gsz;
}

// Writes one output row segment (BN accumulators of row `row`, tile column block `nb`) through the epilogue.
__device__ __forceinline__ void store_row(const Fp8Params& p, const float* acc, int row, int nb) {
  const int col_tile0 = nb * BN;
  if (p.epi == F8_GATED_SILU) {  // columns are [32 gate | 32 up] pairs; N / 2 output columns
    bf16* crow = p.C + (int64_t)row * p.ldc;
#pragma unroll
    for (int c = 0; c < BN; c += 64) {
      if (col_tile0 + c < p.N) {
        const int ocol = (col_tile0 + c) / 2;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          float o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = silu_f(acc[c + j + e]) * acc[c + 32 + j + e];
          *reinterpret_cast<bf16x8*>(crow + ocol + j) = pack8(o);
        }
      }
    }
  } else {
    bf16* crow = p.C + (int64_t)row * p.ldc + col_tile0;
    const bf16* rrow = p.epi == F8_RESIDUAL ? p.residual + (int64_t)row * p.ldc + col_tile0 : nullptr;
#pragma unroll
    for (int c = 0; c < BN; c += 8) {
      const int col0 = col_tile0 + c;
      if (col0 + 8 <= p.N) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = acc[c + e];
        if (rrow != nullptr) {
          float rv[8];
          unpack8(*reinterpret_cast<const bf16x8*>(rrow + c), rv);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += rv[e];
        }
        *reinterpret_cast<bf16x8*>(crow + c) = pack8(o);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (col0 + e < p.N)
            crow[c + e] = __float2bfloat16(acc[c + e] + (rrow != nullptr ? __bfloat162float(rrow[c + e]) : 0.f));
      }
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const Fp8Params p) {
  constexpr uint32_t IDESC = umma_idesc(BM, BN, 0);  // e4m3 x e4m3 -> fp32
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8 * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8 * (2 * STAGES + 2 + a); };
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int k_blocks = (p.K + BKB - 1) / BKB;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer ----
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
        int w_row0 = nb * BN;
        if (p.mblock_expert != nullptr) {
          const int e = p.mblock_expert[mb];
          if (e < 0) continue;
          w_row0 += e * p.N;
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, p.status, 31);
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, &tmA, full_bar(stage), kb * BKB, mb * BM);
          tma_load_2d(sa + A_BYTES, &tmB, full_bar(stage), kb * BKB, w_row0);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer: one K group per tensor-memory buffer ----
      int stage = 0;
      uint32_t phase = 0;
      uint32_t blk = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (p.mblock_expert != nullptr) {
          int mb, nb;
          tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
          if (p.mblock_expert[mb] < 0) continue;
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++blk) {
          const uint32_t buf = blk & 1u, bphase = (blk >> 1) & 1u;
          mbar_wait(tempty_bar(buf), bphase ^ 1u, &abort_flag, p.status, 32);
          mbar_wait(full_bar(stage), phase, &abort_flag, p.status, 33);
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint64_t da = umma_smem_desc_sw128(sa);
          const uint64_t db = umma_smem_desc_sw128(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k)  // K = 32 per instruction: +32 bytes = +2 in 16-byte units
            umma_fp8(tmem_base + buf * BN, da + 2 * k, db + 2 * k, IDESC, k != 0);
          umma_commit(empty_bar(stage));
          umma_commit(tfull_bar(buf));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else {
    // ---- scaled accumulation + output (one row per thread) ----
    const int lane_grp = warp & 3;
    const int erow = lane_grp * 32 + lane;
    uint32_t blk = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
      int w_row0 = nb * BN;
      if (p.mblock_expert != nullptr) {
        const int e = p.mblock_expert[mb];
        if (e < 0) continue;
        w_row0 += e * p.N;
      }
      const int row = mb * BM + erow;
      const bool row_ok = row < p.M;
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      int srow[BN / 32];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) srow[c] = min((w_row0 + c * 32) / p.ws_rows, p.ws_total_rows - 1) * k_blocks;
      for (int kb = 0; kb < k_blocks; ++kb, ++blk) {
        const uint32_t buf = blk & 1u, bphase = (blk >> 1) & 1u;
        const float sa = row_ok ? p.a_scale[(int64_t)kb * p.a_scale_ld + row] : 0.f;
        float sw[BN / 32];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) sw[c] = sa * __ldg(p.w_scale + srow[c] + kb);
        mbar_wait(tfull_bar(buf), bphase, &abort_flag, p.status, 34);
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + buf * BN;
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__uint_as_float(r[j]), sw[c], acc[c * 32 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
      }
      if (row_ok) store_row(p, acc, row, nb);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Per-token, per-128-column-group quantisation of bf16 activations to e4m3: one warp per (row, group), four
// values per lane; scale = amax / 448 (reference: per_token_group_quant_fp8,
// lightllm/common/basemodel/triton_kernel/quantization/fp8act_quant_kernel.py).
__global__ void __launch_bounds__(256) quant_fp8_group128_kernel(const bf16* __restrict__ x, int64_t ldx,
                                                                 uint8_t* __restrict__ q, int64_t ldq,
                                                                 float* __restrict__ scale, int64_t scale_ld, int M,
                                                                 int K, int k_groups) {
  pdl_wait();
  const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (int64_t)M * k_groups) return;
  const int row = (int)(w / k_groups), g = (int)(w - (int64_t)row * k_groups);
  const int col = g * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (col + 4 <= K) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + (int64_t)row * ldx + col);
    const bf162* h = reinterpret_cast<const bf162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
  } else {
    for (int e = 0; e < 4; ++e)
      if (col + e < K) v[e] = __bfloat162float(x[(int64_t)row * ldx + col + e]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = fmaxf(amax, 1e-10f) / 448.f;
  const float inv = 1.f / s;
  if (lane == 0) scale[(int64_t)g * scale_ld + row] = s;
  uint32_t packed = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e)
    packed |= (uint32_t)__nv_cvt_float_to_fp8(v[e] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * e);
  if (col + 4 <= K) {
    *reinterpret_cast<uint32_t*>(q + (int64_t)row * ldq + col) = packed;
  } else {
    for (int e = 0; e < 4; ++e)
      if (col + e < K) q[(int64_t)row * ldq + col + e] = (uint8_t)(packed >> (8 * e));
  }
}

// ---------------------------------------------------------------------------------------------
// int8 GEMM (w8a8): s8 activations with one fp32 scale per token, s8 weights with one fp32 scale per output
// channel.  tcgen05.mma kind::i8 accumulates the whole K range as s32 in tensor memory (two 128-column buffers
// alternate between tiles, so the epilogue of a tile overlaps the next tile's main loop); the epilogue converts to
// fp32, multiplies by both scales and goes through the same output code as the fp8 kernel.
// Reference: lightllm/common/quantization/w8a8.py (vllm scaled_int8_quant + cutlass_scaled_mm).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8Params p) {
  // instruction descriptor: D = s32 (2 << 4), A and B = signed 8-bit (1 << 7, 1 << 10), K-major, N and M fields
  constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8 * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8 * (2 * STAGES + 2 + a); };
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int k_blocks = (p.K + BKB - 1) / BKB;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, p.status, 51);
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, &tmA, full_bar(stage), kb * BKB, mb * BM);
          tma_load_2d(sa + A_BYTES, &tmB, full_bar(stage), kb * BKB, nb * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
        const uint32_t buf = it & 1, bphase = (it >> 1) & 1;
        mbar_wait(tempty_bar(buf), bphase ^ 1u, &abort_flag, p.status, 52);
        tc_fence_after();
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(full_bar(stage), phase, &abort_flag, p.status, 53);
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint64_t da = umma_smem_desc_sw128(sa);
          const uint64_t db = umma_smem_desc_sw128(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k) umma_i8(tmem_base + buf * BN, da + 2 * k, db + 2 * k, IDESC, (kb | k) != 0);
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        umma_commit(tfull_bar(buf));
      }
    }
  } else {
    const int lane_grp = warp & 3;
    const int erow = lane_grp * 32 + lane;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      int mb, nb;
      tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
      const uint32_t buf = it & 1, bphase = (it >> 1) & 1;
      const int row = mb * BM + erow;
      const bool row_ok = row < p.M;
      const float sa = row_ok ? p.a_scale[row] : 0.f;
      mbar_wait(tfull_bar(buf), bphase, &abort_flag, p.status, 54);
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + buf * BN;
      float acc[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = nb * BN + c * 32 + j;
          const float sw = col < p.N ? __ldg(p.w_scale + col) : 0.f;
          acc[c * 32 + j] = (float)(int32_t)r[j] * sa * sw;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
      if (row_ok) store_row(p, acc, row, nb);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Per-token symmetric int8 quantisation: one warp per row, scale = amax / 127.
__global__ void __launch_bounds__(256) quant_int8_per_token_kernel(const bf16* __restrict__ x, int64_t ldx,
                                                                   int8_t* __restrict__ q, int64_t ldq,
                                                                   float* __restrict__ scale, int M, int K) {
  pdl_wait();
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const bf16* xr = x + (int64_t)row * ldx;
  float amax = 0.f;
  for (int c = lane; c < K; c += 32) amax = fmaxf(amax, fabsf(__bfloat162float(xr[c])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = fmaxf(amax, 1e-10f) / 127.f, inv = 1.f / s;
  if (lane == 0) scale[row] = s;
  int8_t* qr = q + (int64_t)row * ldq;
  for (int c = lane; c < K; c += 32) {
    const float v = rintf(__bfloat162float(xr[c]) * inv);
    qr[c] = (int8_t)fminf(fmaxf(v, -127.f), 127.f);
  }
}

struct MapKey8 {
  const void* p;
  uint64_t rows, cols, ld;
  bool operator==(const MapKey8& o) const { return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld; }
};
struct MapKey8Hash {
  size_t operator()(const MapKey8& k) const {
    size_t h = (size_t)k.p;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    return h;
  }
};
std::mutex g_map8_mu;
std::unordered_map<MapKey8, CUtensorMap, MapKey8Hash> g_maps8;

int cached_tmap8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld) {
  MapKey8 key{base, rows, cols, ld};
  std::lock_guard<std::mutex> lk(g_map8_mu);
  auto it = g_maps8.find(key);
  if (it != g_maps8.end()) {
    *out = it->second;
    return LLB_OK;
  }
  int rc = make_tmap_2d(out, base, 1, rows, cols, ld, 128, BKB);
  if (rc) return rc;
  if (g_maps8.size() > 8192) g_maps8.clear();
  g_maps8.emplace(key, *out);
  return LLB_OK;
}

}  // namespace

// x [M, K] bf16 (row pitch ldx) -> q [M, K] e4m3 (row pitch ldq bytes, a multiple of 16) and
// scale [ceil(K / 128), scale_ld] fp32 (scale_ld >= M).
LLB_EXPORT int llb_quant_fp8_group128(const void* x, int64_t ldx, void* q, int64_t ldq, float* scale,
                                      int64_t scale_ld, int M, int K, cudaStream_t st) {
  if (M <= 0 || K <= 0) return LLB_OK;
  if ((ldx % 4) || (ldq % 4) || ((uintptr_t)x & 7) || ((uintptr_t)q & 3) || scale_ld < M) return LLB_ERR_BAD_ARG;
  const int kg = cdiv(K, 128);
  const int64_t warps = (int64_t)M * kg;
  cudaError_t e = launch_pdl(quant_fp8_group128_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, st,
                             (const bf16*)x, ldx, (uint8_t*)q, ldq, scale, scale_ld, M, K, kg);
  return e == cudaSuccess ? LLB_OK : (int)e;
}

// C[M, N] (bf16; N / 2 columns for the gated epilogue) from e4m3 A [M, K] (pitch lda bytes) and W [n_rows_total, K]
// (pitch ldw bytes) with their block scales.  mblock_expert != null selects the grouped (MoE) mode, where N is the
// per-expert row count and M the padded row count (a multiple of 128).
LLB_EXPORT int llb_gemm_fp8_block(const void* A, int64_t lda, const float* a_scale, int64_t a_scale_ld, const void* W,
                                  int64_t ldw, const float* w_scale, int ws_rows, int w_rows_total, void* C,
                                  int64_t ldc, const void* residual, int M, int N, int K, int epi,
                                  const int* mblock_expert, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return LLB_OK;
  if (K <= 0 || (K % 16) || (lda % 16) || (ldw % 16) || (ldc % 8) || ((uintptr_t)C & 15)) return LLB_ERR_BAD_ARG;
  if (ws_rows != 128 && ws_rows != 32) return LLB_ERR_BAD_ARG;
  if (epi == F8_GATED_SILU && (N % 64)) return LLB_ERR_UNSUPPORTED;
  if (epi == F8_RESIDUAL && residual == nullptr) return LLB_ERR_BAD_ARG;
  if (mblock_expert != nullptr && ((N % BN) || (M % BM))) return LLB_ERR_UNSUPPORTED;
  if (epi < 0 || epi > 2) return LLB_ERR_UNSUPPORTED;
  CUtensorMap ta, tb;
  int rc = cached_tmap8(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda);
  if (rc) return rc;
  rc = cached_tmap8(&tb, W, (uint64_t)w_rows_total, (uint64_t)K, (uint64_t)ldw);
  if (rc) return rc;
  static DeviceOnce configured;     
  if (!configured.done()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured.set();  
  }
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  p.C = (bf16*)C;
  p.residual = (const bf16*)residual;
  p.a_scale = a_scale;
  p.w_scale = w_scale;
  p.mblock_expert = mblock_expert;
  p.status = status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.a_scale_ld = a_scale_ld;
  p.ws_rows = ws_rows;
  p.ws_total_rows = cdiv(w_rows_total, ws_rows);
  p.num_m_blocks = cdiv(M, BM);
  p.num_n_blocks = cdiv(N, BN);
  p.epi = epi;
  const int64_t panel_rows = (24ll << 20) / ((int64_t)BM * K);
  p.group_m = (int)(panel_rows < 4 ? 4 : (panel_rows > 64 ? 64 : panel_rows));
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  cudaError_t e = launch_pdl(gemm_fp8_block_kernel, dim3(grid), dim3(THREADS), SMEM_BYTES, st, ta, tb, p);
  return e == cudaSuccess ? LLB_OK : (int)e;
}

// x [M, K] bf16 -> q [M, K] s8 (row pitch ldq bytes) and scale [M] fp32.
LLB_EXPORT int llb_quant_int8_per_token(const void* x, int64_t ldx, void* q, int64_t ldq, float* scale, int M, int K,
                                        cudaStream_t st) {
  if (M <= 0 || K <= 0) return LLB_OK;
  cudaError_t e = launch_pdl(quant_int8_per_token_kernel, dim3((unsigned)((M + 7) / 8)), dim3(256), 0, st,
                             (const bf16*)x, ldx, (int8_t*)q, ldq, scale, M, K);
  return e == cudaSuccess ? LLB_OK : (int)e;
}

// C[M, N] bf16 = (a_scale[m] * w_scale[n]) * (A . W^T) with s8 A [M, K] (pitch lda bytes) and s8 W [N, K]
// (pitch ldw bytes); epilogues as llb_gemm_fp8_block (store / + residual / SwiGLU of interleaved columns).
LLB_EXPORT int llb_gemm_int8(const void* A, int64_t lda, const float* a_scale, const void* W, int64_t ldw,
                             const float* w_scale, void* C, int64_t ldc, const void* residual, int M, int N, int K,
                             int epi, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return LLB_OK;
  if (K <= 0 || (K % 16) || (lda % 16) || (ldw % 16) || (ldc % 8) || ((uintptr_t)C & 15)) return LLB_ERR_BAD_ARG;
  if (epi == F8_GATED_SILU && (N % 64)) return LLB_ERR_UNSUPPORTED;
  if (epi == F8_RESIDUAL && residual == nullptr) return LLB_ERR_BAD_ARG;
  if (epi < 0 || epi > 2) return LLB_ERR_UNSUPPORTED;
  CUtensorMap ta, tb;
  int rc = cached_tmap8(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda);
  if (rc) return rc;
  rc = cached_tmap8(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw);
  if (rc) return rc;
  static DeviceOnce configured;     
  if (!configured.done()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured.set();  
  }
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  p.C = (bf16*)C;
  p.residual = (const bf16*)residual;
  p.a_scale = a_scale;
  p.w_scale = w_scale;
  p.status = status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.num_m_blocks = cdiv(M, BM);
  p.num_n_blocks = cdiv(N, BN);
  p.epi = epi;
  const int64_t panel_rows = (24ll << 20) / ((int64_t)BM * K);
  p.group_m = (int)(panel_rows < 4 ? 4 : (panel_rows > 64 ? 64 : panel_rows));
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  cudaError_t e = launch_pdl(gemm_i8_kernel, dim3(grid), dim3(THREADS), SMEM_BYTES, st, ta, tb, p);
  return e == cudaSuccess ? LLB_OK : (int)e;
}
