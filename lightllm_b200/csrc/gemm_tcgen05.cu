// bf16 GEMM for sm_100a:  C[M, N] = A[M, K] . W[N, K]^T  (+ epilogue)
//
// Weights keep the checkpoint layout [out, in] (both operands K-major), which is exactly
// what tcgen05.mma wants for A and B tiles in shared memory.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: 128 x 64 A tile + BN x 64 W tile per stage, 128-byte swizzle,
//               completion counted on the stage's "full" mbarrier
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) x4 per stage into a
//               TMEM accumulator; tcgen05.commit releases the stage / publishes the accumulator
//   warps 2..5  epilogue: tcgen05.ld the fp32 accumulator (each warp its 32 TMEM lanes), apply the
//               epilogue functor, store.  Two accumulators (2 x BN TMEM columns) so the epilogue
//               of tile i overlaps the main loop of tile i+1.
// Epilogues: plain store, + bias, + residual, SiLU/GELU-gated product of interleaved
// gate/up column blocks (the SwiGLU FFN never materialises the [T, 2I] tensor), fp32 store
// (lm_head logits).
//
// Behavioural counterpart in the reference: the cuBLAS calls behind
// lightllm/common/quantization/no_quant.py (torch.mm / addmm), silu_and_mul_fwd and the
// residual adds of the layer template.
#include "sm100_ptx.cuh"

using namespace llb;
using namespace llb::sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_BUDGET = 224 * 1024;
constexpr int64_t kPanelBytes = 24ll << 20;  // A panel kept hot in L2 while W streams past it

enum Epi { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_GATED_SILU = 2, EPI_F32 = 3, EPI_GATED_GELU = 4 };

struct GemmParams {
  void* C;
  const bf16* residual;  // [M, ldc] bf16 (EPI_RESIDUAL)
  const bf16* bias;      // [N] or null
  int* status;
  int M, N, K;
  int64_t ldc;  // elements
  int num_m_blocks, num_n_blocks;
  int group_m;         // M-blocks per raster group (sized so the group's A panel stays in L2)
  int stream_k;        // 1: every CTA gets an equal share of (tile, k-block) units; split tiles are fixed up
  float* sk_partials;  // [grid][2][BM * BN] fp32 partial tiles of split tiles (stream_k only)
  int* sk_counters;    // [tiles] arrived k-blocks per tile, self-resetting (stream_k only)
  // grouped (MoE) mode: A is the expert-sorted activation, W stacks the experts along its rows
  // ([E * N, K]); M-block i multiplies with expert mblock_expert[i] (-1: padding block, skipped)
  const int* mblock_expert;
  // batched mode (per-head GEMMs of MLA): rank-3 tensor maps, tile -> (batch, m, n); C += batch * c_batch_stride
  int batch_count;
  int64_t c_batch_stride;
  // W stored as [N/128][K/64][128][64] (every 128-row x 64-column tile is 16 contiguous KB): number of
  // k-blocks per tile row, 0 for the row-major checkpoint layout
  int w_tiled_kb;
  // same tiling, every tile stored as its 128B-swizzled shared-memory image: loaded with one untiled bulk copy
  const bf16* w_swz;
  // fused all-gather of the output over NVLink peer memory (tensor-parallel partial sums): with push_world > 0 the
  // bf16 tile is stored into every rank's gather slot of this rank (push[q], same row pitch ldc) instead of C, and
  // after a CTA has stored a tile it adds the tile's column count to counter [push_rank * push_max_mb + row / 128]
  // on every rank (release, system scope): a consumer that sees N columns for a 128-row block may read it.
  bf16* push[8];
  uint32_t* push_cnt[8];
  int push_world, push_rank, push_max_mb;
};

// Output staging of the epilogue warps: a thread owns one accumulator row, so storing straight from registers
// makes every store instruction touch 32 different rows (16 bytes each).  Instead each warp parks 32 rows x 128
// bytes of finished output in shared memory and writes them back four whole 128-byte lines per instruction
// (residual rows are fetched the same way).  Rows are 144 bytes apart so that the 16-byte accesses of eight
// consecutive rows fall into distinct banks.
constexpr int EPI_ROW_PITCH = 144;
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_PITCH;
constexpr int EPI_STAGE_BYTES = 4 * EPI_WARP_BYTES;

template <int BN>
constexpr int stage_bytes() {
  return BM * BK * 2 + BN * BK * 2;
}
template <int BN>
constexpr int num_stages() {
  return (SMEM_BUDGET - EPI_STAGE_BYTES) / stage_bytes<BN>() > 8 ? 8 : (SMEM_BUDGET - EPI_STAGE_BYTES) / stage_bytes<BN>();
}
template <int BN>
constexpr int smem_bytes() {
  return num_stages<BN>() * stage_bytes<BN>() + 1024 /*align slack*/ + 256 /*barriers*/ + EPI_STAGE_BYTES;
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float gelu_tanh_f(float v) {
  return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

// Tile order: groups of `GROUP` M-blocks, M fastest inside a group, so CTAs running at the same time
// share W tiles (decode: both M-blocks of one W tile) and the group's A panel is re-read from L2
// while W streams past it once per group.

// Work of one CTA as a sequence of segments (tile, k-block range).  Data-parallel mode: whole tiles,
// round-robin.  Stream-K mode: CTA c owns units [c*U/G, (c+1)*U/G) of the U = tiles * k_blocks
// (tile, k-block) units, so a tile may be shared by neighbouring CTAs.
struct SegIter {
  int64_t u, u_end;
  int tile_rr, num_tiles, kb, G;
  bool stream_k;
  __device__ SegIter(bool sk, int cta, int grid, int tiles, int k_blocks)
      : tile_rr(cta), num_tiles(tiles), kb(k_blocks), G(grid), stream_k(sk) {
    int64_t U = (int64_t)tiles * k_blocks;
    u = (int64_t)cta * U / grid;
    u_end = (int64_t)(cta + 1) * U / grid;
  }
  __device__ bool next(int& tile, int& k0, int& k1) {
    if (stream_k) {
      if (u >= u_end) return false;
      tile = (int)(u / kb);
      k0 = (int)(u - (int64_t)tile * kb);
      int64_t left = u_end - u;
      k1 = (int)(left < (int64_t)(kb - k0) ? k0 + left : kb);
      u += k1 - k0;
      return true;
    }
    if (tile_rr >= num_tiles) return false;
    tile = tile_rr;
    tile_rr += G;
    k0 = 0;
    k1 = kb;
    return true;
  }
};
__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int GROUP, int& mb, int& nb) {
  int per_group = GROUP * num_n;
  int grp = tile / per_group;
  int first_m = grp * GROUP;
  int gsz = min(GROUP, num_m - first_m);
  int in = tile - grp * per_group;
  mb = first_m + in % gsz;
  nb = in / gsz;
}

// Called by the four epilogue warps (threads 64..191) after they stored a tile of `ncols` valid columns of the
// 128-row block `row_block`: makes the peer stores visible and advances the block's column counter on every rank.
__device__ __forceinline__ void push_signal(const GemmParams& p, int row_block, int ncols) {
  if (p.push_world <= 0) return;
  __threadfence_system();
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (threadIdx.x == 64 && ncols > 0 && row_block < p.push_max_mb) {
    for (int q = 0; q < p.push_world; ++q)
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.push_cnt[q] + p.push_rank * p.push_max_mb + row_block),
                   "r"((uint32_t)ncols)
                   : "memory");
  }
}

// Copies the warp's staged 32 x 128-byte block to global memory: `elem_bytes`-wide elements, block origin
// (row_base, col0) of a matrix with row pitch ldc elements.
template <int ELEM_BYTES>
__device__ __forceinline__ void epi_flush(const GemmParams& p, const uint8_t* stage, int lane, int row_base, int col0,
                                          bool push) {
  constexpr int EPS = 16 / ELEM_BYTES;  // elements per 16-byte segment
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int id = i * 32 + lane, r = id >> 3, seg = id & 7;
    const int grow = row_base + r;
    if (grow < p.M) {
      const uint4 v = *reinterpret_cast<const uint4*>(stage + r * EPI_ROW_PITCH + seg * 16);
      const int64_t off = (int64_t)grow * p.ldc + col0 + seg * EPS;
      if (push) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (q < p.push_world) *reinterpret_cast<uint4*>(p.push[q] + off) = v;
      } else {
        *reinterpret_cast<uint4*>((uint8_t*)p.C + off * ELEM_BYTES) = v;
      }
    }
  }
}

// 32 accumulator columns (registers r, first column col0 of the output) of this thread's row, straight from
// registers: used for ragged right edges and by kernels without a staging buffer.
template <int EPI>
__device__ __forceinline__ void epi_direct32(const GemmParams& p, const uint32_t* r, int row, bool row_ok, int col0) {
  if (!(row_ok && col0 < p.N)) return;
  const int ncols = min(32, p.N - col0);
  if (EPI == EPI_F32) {
    float* crow = (float*)p.C + (int64_t)row * p.ldc + col0;
    if (ncols == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                               __uint_as_float(r[j + 3]));
        if (p.bias) {
          v.x += __bfloat162float(p.bias[col0 + j]);
          v.y += __bfloat162float(p.bias[col0 + j + 1]);
          v.z += __bfloat162float(p.bias[col0 + j + 2]);
          v.w += __bfloat162float(p.bias[col0 + j + 3]);
        }
        *reinterpret_cast<float4*>(crow + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) crow[j] = __uint_as_float(r[j]) + (p.bias ? __bfloat162float(p.bias[col0 + j]) : 0.f);
    }
  } else {
    bf16* crow = (bf16*)p.C + (int64_t)row * p.ldc + col0;
    const bf16* rrow = EPI == EPI_RESIDUAL ? p.residual + (int64_t)row * p.ldc + col0 : nullptr;
    if (ncols == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[j + e]);
        if (p.bias) {
          float bv[8];
          unpack8(*reinterpret_cast<const bf16x8*>(p.bias + col0 + j), bv);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += bv[e];
        }
        if (EPI == EPI_RESIDUAL) {
          float rv[8];
          unpack8(*reinterpret_cast<const bf16x8*>(rrow + j), rv);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += rv[e];
        }
        if (EPI == EPI_STORE && p.push_world > 0) {
          const bf16x8 packed = pack8(o);
          const int64_t off = (int64_t)row * p.ldc + col0 + j;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (q < p.push_world) *reinterpret_cast<bf16x8*>(p.push[q] + off) = packed;
        } else {
          *reinterpret_cast<bf16x8*>(crow + j) = pack8(o);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < ncols) {
          float v = __uint_as_float(r[j]);
          if (p.bias) v += __bfloat162float(p.bias[col0 + j]);
          if (EPI == EPI_RESIDUAL) v += __bfloat162float(rrow[j]);
          crow[j] = __float2bfloat16(v);
        }
      }
    }
  }
}

// Drains one accumulator tile (this thread's row, BN columns starting at TMEM address t_row) through the
// epilogue functor EPI into C.  `add_partials(regs, col)` adds other CTAs' partial sums (stream-K) when
// `has_add` is set.  `stage`: this warp's EPI_WARP_BYTES of shared memory (null: store from registers).
template <int BN, int EPI, typename AddFn>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, uint32_t t_row, int row, bool row_ok, int col_tile0,
                                               bool has_add, AddFn add_partials, uint8_t* stage = nullptr) {
  const int lane = threadIdx.x & 31;
  const int row_base = row - lane;
  uint8_t* my = stage + lane * EPI_ROW_PITCH;
  if (EPI == EPI_GATED_SILU || EPI == EPI_GATED_GELU) {
    // columns come as [32 gate | 32 up] pairs; output has N/2 columns
    bf16* crow = (bf16*)p.C + (int64_t)row * p.ldc;
    constexpr int STEP = (BN % 128 == 0) ? 128 : 64;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += STEP) {
      const bool staged = stage != nullptr && STEP == 128 && col_tile0 + c0 + 128 <= p.N;
#pragma unroll
      for (int sub = 0; sub < STEP / 64; ++sub) {
        const int c = c0 + sub * 64;
        uint32_t gr[32], ur[32];
        tmem_ld_32x32(t_row + c, gr);
        tmem_ld_32x32(t_row + c + 32, ur);
        tmem_wait_ld();
        if (has_add) {
          add_partials(gr, c);
          add_partials(ur, c + 32);
        }
        const int ocol = (col_tile0 + c) / 2;
        if (staged || (row_ok && col_tile0 + c < p.N)) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float gv = __uint_as_float(gr[j + e]);
              float uv = __uint_as_float(ur[j + e]);
              o[e] = (EPI == EPI_GATED_SILU ? silu_f(gv) : gelu_tanh_f(gv)) * uv;
            }
            if (staged)
              *reinterpret_cast<bf16x8*>(my + sub * 64 + j * 2) = pack8(o);
            else
              *reinterpret_cast<bf16x8*>(crow + ocol + j) = pack8(o);
          }
        }
      }
      if (staged) {
        __syncwarp();
        epi_flush<2>(p, stage, lane, row_base, (col_tile0 + c0) / 2, false);
        __syncwarp();
      }
    }
  } else if (EPI == EPI_F32) {
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t r[32];
      tmem_ld_32x32(t_row + c, r);
      tmem_wait_ld();
      if (has_add) add_partials(r, c);
      const int col0 = col_tile0 + c;
      if (stage != nullptr && col0 + 32 <= p.N) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                 __uint_as_float(r[j + 3]));
          if (p.bias) {
            v.x += __bfloat162float(p.bias[col0 + j]);
            v.y += __bfloat162float(p.bias[col0 + j + 1]);
            v.z += __bfloat162float(p.bias[col0 + j + 2]);
            v.w += __bfloat162float(p.bias[col0 + j + 3]);
          }
          *reinterpret_cast<float4*>(my + j * 4) = v;
        }
        __syncwarp();
        epi_flush<4>(p, stage, lane, row_base, col0, false);
        __syncwarp();
      } else {
        epi_direct32<EPI>(p, r, row, row_ok, col0);
      }
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < BN; c += 64) {
      const int col0 = col_tile0 + c;
      const bool staged = stage != nullptr && col0 + 64 <= p.N;
      if (staged && EPI == EPI_RESIDUAL) {  // residual rows: whole lines into the staging block
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int id = i * 32 + lane, r = id >> 3, seg = id & 7;
          const int grow = row_base + r;
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (grow < p.M) v = *reinterpret_cast<const uint4*>(p.residual + (int64_t)grow * p.ldc + col0 + seg * 8);
          *reinterpret_cast<uint4*>(stage + r * EPI_ROW_PITCH + seg * 16) = v;
        }
        __syncwarp();
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c + half * 32, r);
        tmem_wait_ld();
        if (has_add) add_partials(r, c + half * 32);
        if (!staged) {
          epi_direct32<EPI>(p, r, row, row_ok, col0 + half * 32);
          continue;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          float o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[j + e]);
          if (p.bias) {
            float bv[8];
            unpack8(*reinterpret_cast<const bf16x8*>(p.bias + col0 + half * 32 + j), bv);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += bv[e];
          }
          bf16x8* slot = reinterpret_cast<bf16x8*>(my + half * 64 + j * 2);
          if (EPI == EPI_RESIDUAL) {
            float rv[8];
            unpack8(*slot, rv);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += rv[e];
          }
          *slot = pack8(o);
        }
      }
      if (staged) {
        __syncwarp();
        epi_flush<2>(p, stage, lane, row_base, col0, EPI == EPI_STORE && p.push_world > 0);
        __syncwarp();
      }
    }
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  constexpr int STAGES = num_stages<BN>();
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int STAGE_BYTES = stage_bytes<BN>();
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // power of two for BN in {32,64,128,256}
  constexpr uint32_t IDESC = umma_idesc(BM, BN, 1);

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
  const int num_tiles = p.num_m_blocks * p.num_n_blocks * (p.batch_count > 1 ? p.batch_count : 1);
  const int k_blocks = (p.K + BK - 1) / BK;

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
  pdl_wait();  // barrier set-up and tensor-memory allocation overlapped the previous kernel's tail
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      SegIter segs(p.stream_k != 0, blockIdx.x, gridDim.x, num_tiles, k_blocks);
      int tile, k0, k1;
      while (segs.next(tile, k0, k1)) {
        int mb, nb;
        const int tpb = p.num_m_blocks * p.num_n_blocks;
        const int batch = p.batch_count > 1 ? tile / tpb : 0;
        tile_coords(p.batch_count > 1 ? tile - batch * tpb : tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
        int w_row0 = nb * BN;
        if (p.mblock_expert != nullptr) {
          const int e = p.mblock_expert[mb];
          if (e < 0) continue;
          w_row0 += e * p.N;
        }
        for (int kb = k0; kb < k1; ++kb) {
          mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, p.status, 1);
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          if (p.batch_count > 1) {
            tma_load_3d(sa, &tmA, full_bar(stage), kb * BK, mb * BM, batch);
            tma_load_3d(sa + A_BYTES, &tmB, full_bar(stage), kb * BK, w_row0, batch);
          } else if (p.w_swz != nullptr) {
            tma_load_2d(sa, &tmA, full_bar(stage), kb * BK, mb * BM);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              bulk_load(sa + A_BYTES + j * 16384,
                        p.w_swz + ((int64_t)((w_row0 >> 7) + j) * p.w_tiled_kb + kb) * (128 * BK), 16384,
                        full_bar(stage));
          } else {
            tma_load_2d(sa, &tmA, full_bar(stage), kb * BK, mb * BM);
            tma_load_2d(sa + A_BYTES, &tmB, full_bar(stage), kb * BK, w_row0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      SegIter segs(p.stream_k != 0, blockIdx.x, gridDim.x, num_tiles, k_blocks);
      int tile, k0, k1;
      while (segs.next(tile, k0, k1)) {
        if (p.mblock_expert != nullptr) {
          int mb, nb;
          tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
          if (p.mblock_expert[mb] < 0) continue;
        }
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        mbar_wait(tempty_bar(acc), acc_phase ^ 1, &abort_flag, p.status, 2);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = k0; kb < k1; ++kb) {
          mbar_wait(full_bar(stage), phase, &abort_flag, p.status, 3);
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint64_t da = umma_smem_desc_sw128(sa);
          const uint64_t db = umma_smem_desc_sw128(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K inside the 128-byte swizzle row: +32 bytes = +2 in 16-byte units
            umma_bf16(d_tmem, da + 2 * k, db + 2 * k, IDESC, ((kb - k0) | k) != 0);
          }
          umma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        umma_commit(tfull_bar(acc));  // accumulator complete
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int lane_grp = warp & 3;  // TMEM lanes 32*lane_grp .. +31 are the ones this warp may read
    const int erow = lane_grp * 32 + lane;  // row inside the tile owned by this thread
    const int etid = threadIdx.x - 64;      // 0..127 among the epilogue threads
    uint8_t* epi_stage = smem_raw + (bar_base + 256 - smem_u32(smem_raw)) + lane_grp * EPI_WARP_BYTES;
    __shared__ int sk_last_flag;
    int it = 0;
    SegIter segs(p.stream_k != 0, blockIdx.x, gridDim.x, num_tiles, k_blocks);
    int tile, k0, k1;
    while (segs.next(tile, k0, k1)) {
      int mb, nb;
      const int tpb = p.num_m_blocks * p.num_n_blocks;
      const int batch = p.batch_count > 1 ? tile / tpb : 0;
      tile_coords(p.batch_count > 1 ? tile - batch * tpb : tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
      if (p.mblock_expert != nullptr && p.mblock_expert[mb] < 0) continue;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      mbar_wait(tfull_bar(acc), acc_phase, &abort_flag, p.status, 4);
      tc_fence_after();
      const int row = mb * BM + erow;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + acc * BN;

      // ---- stream-K: a tile split over several CTAs is summed by whichever CTA arrives last ----
      int n_other = 0;        // partial tiles of other CTAs to add (only the last arriver has any)
      int other_first = 0;    // first contributing CTA of this tile
      bool do_epilogue = true;
      const bool full_tile = (k0 == 0 && k1 == k_blocks);
      if (!full_tile) {
        const int slot = k0 > 0 ? 0 : 1;
        float* mine = p.sk_partials + ((int64_t)blockIdx.x * 2 + slot) * (BM * BN) + (int64_t)erow * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<uint4*>(mine + c + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (etid == 0) {
          int prev = atomicAdd(p.sk_counters + tile, k1 - k0);
          sk_last_flag = (prev + (k1 - k0) == k_blocks) ? 1 : 0;
          if (sk_last_flag) p.sk_counters[tile] = 0;  // every contributor has arrived: ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        do_epilogue = sk_last_flag != 0;
        if (do_epilogue) {
          __threadfence();
          const int64_t U = (int64_t)num_tiles * k_blocks;
          const int64_t ts = (int64_t)tile * k_blocks;
          other_first = (int)(((ts + 1) * gridDim.x - 1) / U);
          const int other_last = (int)(((ts + k_blocks) * gridDim.x - 1) / U);
          n_other = other_last - other_first + 1;
        }
      }

      // adds the partial tiles of the other contributors to 32 accumulator columns starting at `c`
      auto add_partials = [&](uint32_t* r, int c) {
        const int64_t U = (int64_t)num_tiles * k_blocks;
        const int64_t ts = (int64_t)tile * k_blocks;
        for (int q = 0; q < n_other; ++q) {
          const int cta = other_first + q;
          if (cta == (int)blockIdx.x) continue;
          const int64_t cta_start = (int64_t)cta * U / gridDim.x;
          const int oslot = cta_start > ts ? 0 : 1;
          const float* src = p.sk_partials + ((int64_t)cta * 2 + oslot) * (BM * BN) + (int64_t)erow * BN + c;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 v = __ldcg(reinterpret_cast<const float4*>(src + j));
            r[j] = __float_as_uint(__uint_as_float(r[j]) + v.x);
            r[j + 1] = __float_as_uint(__uint_as_float(r[j + 1]) + v.y);
            r[j + 2] = __float_as_uint(__uint_as_float(r[j + 2]) + v.z);
            r[j + 3] = __float_as_uint(__uint_as_float(r[j + 3]) + v.w);
          }
        }
      };

      if (do_epilogue) {
        if (p.batch_count > 1) {
          GemmParams pb = p;
          pb.C = (bf16*)p.C + (int64_t)batch * p.c_batch_stride;
          epilogue_store<BN, EPI>(pb, t_row, row, row_ok, nb * BN, false, add_partials, epi_stage);
        } else {
          epilogue_store<BN, EPI>(p, t_row, row, row_ok, nb * BN, n_other != 0, add_partials, epi_stage);
          if (EPI == EPI_STORE) push_signal(p, mb, min(BN, p.N - nb * BN));
        }
      }
      // accumulator drained: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ----
struct MapKey {
  const void* p;
  uint64_t rows, cols, ld;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.p;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ k.box_rows;
    return h;
  }
};
std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

int cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  MapKey key{base, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lk(g_map_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return LLB_OK;
  }
  int rc = make_tmap_2d(out, base, 2, rows, cols, ld, box_rows, BK);
  if (rc) return rc;
  if (g_maps.size() > 8192) g_maps.clear();
  g_maps.emplace(key, *out);
  return LLB_OK;
}

template <int BN, int EPI>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, cudaStream_t st) {
  static DeviceOnce configured;     
  if (!configured.done()) {
    cudaError_t e =
        cudaFuncSetAttribute(gemm_bf16_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<BN>());
    if (e != cudaSuccess) return (int)e;
    configured.set();  
  }
  p.num_m_blocks = cdiv(p.M, BM);
  p.num_n_blocks = cdiv(p.N, BN);
  int tiles = p.num_m_blocks * p.num_n_blocks * (p.batch_count > 1 ? p.batch_count : 1);
  int64_t panel_rows = kPanelBytes / ((int64_t)BM * p.K * 2);
  p.group_m = (int)(panel_rows < 4 ? 4 : (panel_rows > 64 ? 64 : panel_rows));
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (p.stream_k) {
    int64_t units = (int64_t)tiles * cdiv(p.K, BK);
    grid = units < sm_count() ? (int)units : sm_count();
    p.group_m = p.num_m_blocks;  // M fastest: neighbouring CTAs share a W tile
  }
  cudaError_t le = launch_pdl(gemm_bf16_kernel<BN, EPI>, dim3(grid), dim3(GEMM_THREADS), smem_bytes<BN>(), st, ta, tb, p);
  if (le != cudaSuccess) return (int)le;
  return LLB_OK;
}

template <int BN>
int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, cudaStream_t st) {
  switch (epi) {
    case EPI_STORE:
      return launch_gemm<BN, EPI_STORE>(ta, tb, p, st);
    case EPI_RESIDUAL:
      return launch_gemm<BN, EPI_RESIDUAL>(ta, tb, p, st);
    case EPI_GATED_SILU:
      return launch_gemm<BN, EPI_GATED_SILU>(ta, tb, p, st);
    case EPI_F32:
      return launch_gemm<BN, EPI_F32>(ta, tb, p, st);
    case EPI_GATED_GELU:
      return launch_gemm<BN, EPI_GATED_GELU>(ta, tb, p, st);
  }
  return LLB_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2) for large M: the two CTAs of a cluster compute one 256 x 256 tile.
// Each CTA loads its own 128 rows of A and 128 of the 256 W rows per stage (32 KB instead of 48 KB for
// the same 128 x 256 x 64 of math per CTA, which is what the SM's L2 port can feed at full tensor
// rate); the leader CTA's MMA thread issues tcgen05.mma.cta_group::2 (M = 256), the accumulator rows
// 0-127 land in the leader's TMEM and 128-255 in the peer's.  All loads are plain per-CTA TMA loads.
//   full[s]      (leader)    TMA bytes of stage s of BOTH CTAs landed (the peer's loads name the leader's
//                            barrier through its cluster address)
//   empty[s]     (each CTA)  leader's tcgen05.commit, issued once per CTA (local + mapped address)
//   tfull[a]     (each CTA)  accumulator a complete (same two commits)
//   tempty[a]    (leader)    8 arrivals: the 4 epilogue warps of both CTAs
// ---------------------------------------------------------------------------------------
constexpr int PAIR_BN = 256;       // tile width (W rows per pair tile)
constexpr int PAIR_HALF = 128;     // W rows loaded by each CTA
constexpr int PAIR_STAGE_BYTES = BM * BK * 2 + PAIR_HALF * BK * 2;  // 32 KB
constexpr int PAIR_STAGES = 6;
constexpr int pair_smem_bytes() { return PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 512 + EPI_STAGE_BYTES; }

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmParams p) {
  constexpr int STAGES = PAIR_STAGES;
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int STAGE_BYTES = PAIR_STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t IDESC = umma_idesc(256, PAIR_BN, 1);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  auto pfull_bar = [&](int s) { return bar_base + 8 * (2 * STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8 * (3 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8 * (3 * STAGES + 2 + a); };
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + 255) / 256, num_n = (p.N + PAIR_BN - 1) / PAIR_BN;
  const int num_tiles = num_m * num_n;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(pfull_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc_pair(smem_u32(&tmem_base_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  pdl_wait();          // everything above overlapped the previous kernel's tail
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---- TMA producer (both CTAs) ----
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        int mb, nb;
        tile_coords(tile, num_m, num_n, p.group_m, mb, nb);
        for (int kb = 0; kb < k_blocks; ++kb) {
          mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, p.status, 11);
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          // both CTAs' bytes are counted on the leader's barrier (the only one the MMA thread waits on)
          const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
          if (cta == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          tma_load_2d_pair(sa, &tmA, lead_full, kb * BK, mb * 256 + (int)cta * BM);
          tma_load_2d_pair(sa + A_BYTES, &tmB, lead_full, kb * BK, nb * PAIR_BN + (int)cta * PAIR_HALF);
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
      if (cta == 0) {
        // ---- leader: MMA issuer for the pair ----
        int it = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
          const int acc = it & 1;
          const uint32_t acc_phase = (it >> 1) & 1;
          mbar_wait(tempty_bar(acc), acc_phase ^ 1, &abort_flag, p.status, 13);
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
          for (int kb = 0; kb < k_blocks; ++kb) {
            mbar_wait(full_bar(stage), phase, &abort_flag, p.status, 14);
            tc_fence_after();
            const uint32_t sa = smem_base + stage * STAGE_BYTES;
            const uint64_t da = umma_smem_desc_sw128(sa);
            const uint64_t db = umma_smem_desc_sw128(sa + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, IDESC, (kb | k) != 0);
            umma_commit_pair(empty_bar(stage));                 // my stage is free ...
            umma_commit_pair(map_to_cta(empty_bar(stage), 1));  // ... and the peer's
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          umma_commit_pair(tfull_bar(acc));
          umma_commit_pair(map_to_cta(tfull_bar(acc), 1));
        }
      }
    }
  } else {
    // ---- epilogue (both CTAs): this CTA's 128 rows of the pair tile ----
    const int lane_grp = warp & 3;
    const int erow = lane_grp * 32 + lane;
    const uint32_t tempty_leader = map_to_cta(tempty_bar(0), 0);
    uint8_t* epi_stage = smem_raw + (bar_base + 256 - smem_u32(smem_raw)) + lane_grp * EPI_WARP_BYTES;
    int it = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, p.group_m, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      mbar_wait(tfull_bar(acc), acc_phase, &abort_flag, p.status, 16);
      tc_fence_after();
      const int row = mb * 256 + (int)cta * BM + erow;
      const uint32_t t_row = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + acc * PAIR_BN;
      epilogue_store<PAIR_BN, EPI>(p, t_row, row, row < p.M, nb * PAIR_BN, false, [](uint32_t*, int) {}, epi_stage);
      if (EPI == EPI_STORE) push_signal(p, mb * 2 + (int)cta, min(PAIR_BN, p.N - nb * PAIR_BN));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * acc);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the peer may still signal into this CTA
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int EPI>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, cudaStream_t st) {
  static DeviceOnce configured;     
  if (!configured.done()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         pair_smem_bytes());
    if (e != cudaSuccess) return (int)e;
    configured.set();  
  }
  const int num_m = cdiv(p.M, 256), num_n = cdiv(p.N, PAIR_BN);
  p.num_m_blocks = num_m;
  p.num_n_blocks = num_n;
  int64_t panel_rows = kPanelBytes / ((int64_t)256 * p.K * 2);
  p.group_m = (int)(panel_rows < 2 ? 2 : (panel_rows > 32 ? 32 : panel_rows));
  int pairs = num_m * num_n;
  int max_pairs = sm_count() / 2;
  if (pairs > max_pairs) pairs = max_pairs;
  cudaError_t le = launch_pdl(gemm_bf16_pair_kernel<EPI>, dim3(pairs * 2), dim3(GEMM_THREADS), pair_smem_bytes(), st, ta,
                              tb, p);
  if (le != cudaSuccess) return (int)le;
  return LLB_OK;
}

int dispatch_pair(int epi, const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, cudaStream_t st) {
  switch (epi) {
    case EPI_STORE:
      return launch_pair<EPI_STORE>(ta, tb, p, st);
    case EPI_RESIDUAL:
      return launch_pair<EPI_RESIDUAL>(ta, tb, p, st);
    case EPI_GATED_SILU:
      return launch_pair<EPI_GATED_SILU>(ta, tb, p, st);
    case EPI_F32:
      return launch_pair<EPI_F32>(ta, tb, p, st);
    case EPI_GATED_GELU:
      return launch_pair<EPI_GATED_GELU>(ta, tb, p, st);
  }
  return LLB_ERR_UNSUPPORTED;
}

// Tile width for the data-parallel schedule: modelled time = waves x measured per-k-block cost of a
// full wave of that tile width (L2-bound figures from B200 runs: 0.27 / 0.34 / 0.56 us).
int pick_bn(int M, int N) {
  const int sms = sm_count();
  const int cands[3] = {256, 128, 64};
  const double cost[3] = {0.556, 0.343, 0.27};
  double best_t = 1e30;
  int best = 256;
  for (int i = 0; i < 3; ++i) {
    int bn = cands[i];
    if (bn > 64 && N < bn) continue;
    int64_t tiles = (int64_t)cdiv(M, BM) * cdiv(N, bn);
    int64_t waves = (tiles + sms - 1) / sms;
    double t = (double)waves * cost[i];
    if (t < best_t * 0.97) {
      best_t = t;
      best = bn;
    }
  }
  return best;
}

// ---------------------------------------------------------------------------------------------
// Skinny GEMM for decode (M <= 256): the weight matrix is streamed once, tokens are the small operand.
//
// One cluster of 2*S CTAs computes one output tile of 256 x (NB*256): S CTA pairs split the K range, each pair
// runs cta_group::2 MMAs of M = 256 (CTA h supplies token rows h*128.. and 128 of every 256 weight rows), so a
// CTA stages 16 KB of activations per 16 KB * NB of weights and k-block.  With S > 1 the fp32 partial tiles
// are summed through distributed shared memory: every CTA spills its 128 x 256 accumulator to its own
// shared memory (the drained pipeline stages), and after a cluster barrier each CTA reduces the column slice
// 256/S that it owns from all S peers and writes the final values.  NB = 2 (both halves of the tensor
// memory) is for wide N without split; S > 1 requires NB = 1.
// ---------------------------------------------------------------------------------------------
constexpr int SK_RSTRIDE = 260;  // floats per spilled row: 16-byte stores of 8 consecutive rows hit distinct banks

// TW: tile width per accumulator (256, or 128 to spread a narrow output over twice as many SMs; NB = 1 only)
template <int NB, int TW>
constexpr int sk_stage_bytes() { return BM * BK * 2 + NB * (TW / 2) * BK * 2; }
template <int NB, int TW>
constexpr int sk_stages() { return NB == 1 ? (TW == 128 ? 8 : 6) : 4; }
template <int NB, int TW>
constexpr int sk_smem_bytes() { return sk_stages<NB, TW>() * sk_stage_bytes<NB, TW>() + 1024 + 512 + EPI_STAGE_BYTES; }

// No memory clobber: the caller orders these loads after the cluster barrier (both are volatile asm), and
// several of them must be allowed in flight at once.
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr));
  return v;
}

template <int NB, int EPI, int TW>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const GemmParams p, const int splits) {
  static_assert(TW == 256 || (TW == 128 && NB == 1), "tile width");
  constexpr int STAGES = sk_stages<NB, TW>();
  constexpr int HALF = TW / 2;  // weight rows loaded by each CTA of a pair
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = HALF * BK * 2;
  constexpr int STAGE_BYTES = sk_stage_bytes<NB, TW>();
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t IDESC = umma_idesc(256, TW, 1);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8 * (2 * STAGES);
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t half = rank & 1u, split = rank >> 1;
  const uint32_t leader_rank = rank & ~1u, peer_rank = rank | 1u;
  int mb, nbk;
  tile_coords(blockIdx.y, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nbk);
  const int m0 = mb * 256;
  const int n0 = nbk * TW * NB;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int kb0 = (int)split * kb_per;
  const int nk = max(min(kb_total, kb0 + kb_per) - kb0, 0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc_pair(smem_u32(&tmem_base_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer (every CTA) ----
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nk; ++i) {
        const int kb = kb0 + i;
        mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, p.status, 21);
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint32_t lead_full = map_to_cta(full_bar(stage), leader_rank);
        if (half == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
        tma_load_2d_pair(sa, &tmA, lead_full, kb * BK, m0 + (int)half * BM);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const int wrow = n0 + j * TW + (int)half * HALF;
          if (p.w_tiled_kb)
            tma_load_2d_pair(sa + A_BYTES + j * B_BYTES, &tmB, lead_full, 0,
                             ((wrow >> 7) * p.w_tiled_kb + kb) * 128 + (wrow & 127));
          else
            tma_load_2d_pair(sa + A_BYTES + j * B_BYTES, &tmB, lead_full, kb * BK, wrow);
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && half == 0) {  // ---- MMA issuer of the pair ----
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nk; ++i) {
        mbar_wait(full_bar(stage), phase, &abort_flag, p.status, 22);
        tc_fence_after();
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint64_t da = umma_smem_desc_sw128(sa);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const uint64_t db = umma_smem_desc_sw128(sa + A_BYTES + j * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(tmem_base + j * TW, da + 2 * k, db + 2 * k, IDESC, (i | k) != 0);
        }
        umma_commit_pair(empty_bar(stage));
        umma_commit_pair(map_to_cta(empty_bar(stage), peer_rank));
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      umma_commit_pair(tfull_bar);
      umma_commit_pair(map_to_cta(tfull_bar, peer_rank));
    }
  } else {
    // ---- accumulator drain (every CTA): its 128 token rows ----
    const int lane_grp = warp & 3;
    const int erow = lane_grp * 32 + lane;
    mbar_wait(tfull_bar, 0, &abort_flag, p.status, 23);
    tc_fence_after();
    const int row = m0 + (int)half * BM + erow;
    const uint32_t t_row = tmem_base + ((uint32_t)(lane_grp * 32) << 16);
    if (splits == 1) {
      uint8_t* epi_stage = smem_raw + (bar_base + 256 - smem_u32(smem_raw)) + lane_grp * EPI_WARP_BYTES;
#pragma unroll
      for (int j = 0; j < NB; ++j)
        epilogue_store<TW, EPI>(p, t_row + j * TW, row, row < p.M, n0 + j * TW, false, [](uint32_t*, int) {},
                                epi_stage);
      if (EPI == EPI_STORE) push_signal(p, mb * 2 + (int)half, max(0, min(TW * NB, p.N - n0)));
    } else {
      float* R = reinterpret_cast<float*>(smem_gen) + (size_t)erow * SK_RSTRIDE;
#pragma unroll 1
      for (int c = 0; c < TW; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(R + c + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                              __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  cluster_sync_all();  // every CTA's partial tile is in its shared memory

  if (splits > 1) {
    // all six warps reduce: thread t owns float4 column groups of the slice, two rows per iteration, and
    // issues every peer load of an iteration before the first add
    const int W = TW / splits, W4 = W / 4;
    const uint32_t r_base = smem_base;
    uint32_t peer_base[4];
#pragma unroll
    for (int s2 = 0; s2 < 4; ++s2) peer_base[s2] = map_to_cta(r_base, (uint32_t)(2 * (s2 < splits ? s2 : 0)) + half);
    for (int i = threadIdx.x; i < BM * W4; i += GEMM_THREADS) {
      const int r = i / W4, c4 = i - r * W4;
      const int col_local = (int)split * W + c4 * 4;
      const uint32_t off = (uint32_t)(r * SK_RSTRIDE + col_local) * 4u;
      float4 v[4];
#pragma unroll
      for (int s2 = 0; s2 < 4; ++s2)
        if (s2 < splits) v[s2] = ld_dsmem_f4(peer_base[s2] + off);
      float4 acc = v[0];
#pragma unroll
      for (int s2 = 1; s2 < 4; ++s2) {
        if (s2 < splits) {
          acc.x += v[s2].x;
          acc.y += v[s2].y;
          acc.z += v[s2].z;
          acc.w += v[s2].w;
        }
      }
      const int grow = m0 + (int)half * BM + r, gcol = n0 + col_local;
      if (grow < p.M && gcol < p.N) {
        if (p.bias) {
          acc.x += __bfloat162float(p.bias[gcol]);
          acc.y += __bfloat162float(p.bias[gcol + 1]);
          acc.z += __bfloat162float(p.bias[gcol + 2]);
          acc.w += __bfloat162float(p.bias[gcol + 3]);
        }
        if (EPI == EPI_F32) {
          *reinterpret_cast<float4*>((float*)p.C + (int64_t)grow * p.ldc + gcol) = acc;
        } else {
          if (EPI == EPI_RESIDUAL) {
            const bf162* rr = reinterpret_cast<const bf162*>(p.residual + (int64_t)grow * p.ldc + gcol);
            const float2 r0 = __bfloat1622float2(rr[0]), r1 = __bfloat1622float2(rr[1]);
            acc.x += r0.x;
            acc.y += r0.y;
            acc.z += r1.x;
            acc.w += r1.y;
          }
          bf162 o0 = __floats2bfloat162_rn(acc.x, acc.y), o1 = __floats2bfloat162_rn(acc.z, acc.w);
          uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&o0), *reinterpret_cast<uint32_t*>(&o1));
          if (EPI == EPI_STORE && p.push_world > 0) {
            const int64_t off = (int64_t)grow * p.ldc + gcol;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (q < p.push_world) *reinterpret_cast<uint2*>(p.push[q] + off) = packed;
          } else {
            *reinterpret_cast<uint2*>((bf16*)p.C + (int64_t)grow * p.ldc + gcol) = packed;
          }
        }
      }
    }
    if (EPI == EPI_STORE && p.push_world > 0) {  // this CTA wrote its column slice of its 128 rows
      __threadfence_system();
      __syncthreads();
      const int c0 = n0 + (int)split * W;
      const int valid = max(0, min(W, p.N - c0));
      const int row_block = mb * 2 + (int)half;
      if (threadIdx.x == 0 && valid > 0 && row_block < p.push_max_mb) {
        for (int q = 0; q < p.push_world; ++q)
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.push_cnt[q] + p.push_rank * p.push_max_mb +
                                                                          row_block),
                       "r"((uint32_t)valid)
                       : "memory");
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while a peer may still read its shared memory or signal into it
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int NB, int EPI, int TW = 256>
int launch_skinny(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p_in, int splits, cudaStream_t st) {
  GemmParams p = p_in;
  p.num_m_blocks = cdiv(p.M, 256);
  p.num_n_blocks = cdiv(p.N, TW * NB);
  int64_t panel_rows = kPanelBytes / ((int64_t)256 * p.K * 2);
  p.group_m = (int)(panel_rows < 2 ? 2 : (panel_rows > 32 ? 32 : panel_rows));
  static DeviceOnce configured;     
  if (!configured.done()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_skinny_kernel<NB, EPI, TW>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, sk_smem_bytes<NB, TW>());
    if (e != cudaSuccess) return (int)e;
    configured.set();  
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * splits, p.num_m_blocks * p.num_n_blocks, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = sk_smem_bytes<NB, TW>();
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2 * splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_skinny_kernel<NB, EPI, TW>, ta, tb, p, splits);
  return e == cudaSuccess ? LLB_OK : (int)e;
}

// nb: 1 or 2 accumulators; splits: 1, 2 or 4 (nb must be 1 when splits > 1; gated epilogues need splits == 1);
// tw: 256, or 128 (nb == 1, plain epilogues only)
int dispatch_skinny(int epi, int nb, int splits, int tw, const CUtensorMap& ta, const CUtensorMap& tb,
                    const GemmParams& p, cudaStream_t st) {
  if (splits > 1 && (nb != 1 || epi == EPI_GATED_SILU || epi == EPI_GATED_GELU)) return LLB_ERR_UNSUPPORTED;
  if (tw == 128) {
    if (nb != 1) return LLB_ERR_UNSUPPORTED;
    switch (epi) {
      case EPI_STORE: return launch_skinny<1, EPI_STORE, 128>(ta, tb, p, splits, st);
      case EPI_RESIDUAL: return launch_skinny<1, EPI_RESIDUAL, 128>(ta, tb, p, splits, st);
      case EPI_F32: return launch_skinny<1, EPI_F32, 128>(ta, tb, p, splits, st);
    }
    return LLB_ERR_UNSUPPORTED;
  }
  if (nb == 1) {
    switch (epi) {
      case EPI_STORE: return launch_skinny<1, EPI_STORE>(ta, tb, p, splits, st);
      case EPI_RESIDUAL: return launch_skinny<1, EPI_RESIDUAL>(ta, tb, p, splits, st);
      case EPI_GATED_SILU: return launch_skinny<1, EPI_GATED_SILU>(ta, tb, p, splits, st);
      case EPI_GATED_GELU: return launch_skinny<1, EPI_GATED_GELU>(ta, tb, p, splits, st);
      case EPI_F32: return launch_skinny<1, EPI_F32>(ta, tb, p, splits, st);
    }
  } else {
    switch (epi) {
      case EPI_STORE: return launch_skinny<2, EPI_STORE>(ta, tb, p, 1, st);
      case EPI_RESIDUAL: return launch_skinny<2, EPI_RESIDUAL>(ta, tb, p, 1, st);
      case EPI_GATED_SILU: return launch_skinny<2, EPI_GATED_SILU>(ta, tb, p, 1, st);
      case EPI_GATED_GELU: return launch_skinny<2, EPI_GATED_GELU>(ta, tb, p, 1, st);
      case EPI_F32: return launch_skinny<2, EPI_F32>(ta, tb, p, 1, st);
    }
  }
  return LLB_ERR_UNSUPPORTED;
}

// Shape rule for M <= 256 (measured on B200, CUDA-graph replays): at M = 256 these GEMMs sit on the roofline ridge,
// so what matters is how many SMs work.  Up to 74 tiles of 256 columns: one accumulator, K split over 2 pairs
// (4 pairs = clusters of 8 only for very narrow outputs: few of those clusters are co-resident).  Wider, up to
// one wave of 512-column tiles: both accumulators, no split.  Beyond that the persistent pair kernel
// (returns nb = 0, use_pair = true) overlaps its epilogues with the next tile.
bool g_skinny_auto = true;
bool g_skinny_tw128 = true;

void skinny_plan(int M, int N, int K, int epi, int* nb, int* splits, bool* use_pair, int* tw) {
  const bool gated = epi == EPI_GATED_SILU || epi == EPI_GATED_GELU;
  const int sms = sm_count();
  const int tiles = cdiv(N, 256), kb = cdiv(K, BK);
  *nb = 0;
  *splits = 1;
  *use_pair = false;
  *tw = 256;
  if (tiles * 2 <= sms) {
    *nb = 1;
    if (gated) return;
    if (tiles <= 8 && kb >= 32) {
      *splits = 4;
    } else if (tiles * 4 <= sms && kb >= 16) {
      *splits = 2;
      // clusters of 4: about sms / 4 of them are co-resident; half-width tiles double the SMs at work
      if (g_skinny_tw128 && cdiv(N, 128) <= sms / 4 && (N % 128) == 0) *tw = 128;
    } else if (g_skinny_tw128 && cdiv(N, 128) * 2 <= sms && tiles * 4 <= sms && (N % 128) == 0) {
      *tw = 128;  // short K (no split): still twice the SMs
    }
    return;
  }
  if (cdiv(N, 512) * 2 <= sms) {
    *nb = 2;
    return;
  }
  if (M > 128) *use_pair = true;
}


// ---------------------------------------------------------------------------------------------
// Split-K GEMM for M <= 256 without clusters: CTA (tile, split) multiplies all token rows (one or two 128-row
// blocks, one tensor-memory accumulator each) with 128 weight rows over its share of K, so every weight byte is
// staged once and the grid is tiles x splits CTAs whatever the shape (a narrow output with a long K fills the GPU
// through the split).  The fp32 partial sums meet in an L2-resident workspace: a tile is cut into units of 128
// rows x 32 columns (64 for the gated epilogues: one gate / up column group), unit u is finished by split
// u % splits, every CTA stores the units it does not own ([column][row] order: a warp stores 32 consecutive
// rows of a column per instruction), adds 1 to the tile's arrival counter and waits until all splits have arrived;
// then it adds the other splits' values to its own accumulator columns of the units it owns and runs the epilogue
// on them.  The work after the K loop is the same on every CTA.  All CTAs of a tile must be co-resident: the host
// only uses this kernel with tiles x splits <= number of SMs (one CTA per SM by shared memory).  The wait is
// bounded (status code 31).  Counters only grow; counter arrays are separate per split count so that a tile's
// counter is always a multiple of `splits` when a launch starts.
// ---------------------------------------------------------------------------------------------
constexpr int SPK_BN = 128;
constexpr int SPK_MAX_TILES = 2048;  // counters per split count
template <int MBLK>
constexpr int spk_stage_bytes() { return (MBLK * BM + SPK_BN) * BK * 2; }
template <int MBLK>
constexpr int spk_stages() { return MBLK == 2 ? 4 : 6; }
template <int MBLK>
constexpr int spk_smem_bytes() { return spk_stages<MBLK>() * spk_stage_bytes<MBLK>() + 1024 + 256 + EPI_STAGE_BYTES; }

template <int MBLK, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const GemmParams p, const int splits) {
  constexpr int STAGES = spk_stages<MBLK>();
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int STAGE_BYTES = spk_stage_bytes<MBLK>();
  constexpr uint32_t TMEM_COLS = MBLK * SPK_BN;
  constexpr uint32_t IDESC = umma_idesc(BM, SPK_BN, 1);
  constexpr bool GATED = EPI == EPI_GATED_SILU || EPI == EPI_GATED_GELU;
  constexpr int UW = GATED ? 64 : 32;     // unit width in accumulator columns
  constexpr int UPB = SPK_BN / UW;        // units per 128-row block
  constexpr int U = MBLK * UPB;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8 * (2 * STAGES);
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int spk_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / splits, split = blockIdx.x - tile * splits;
  const int n0 = tile * SPK_BN;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int kb0 = split * kb_per;
  const int nk = max(min(kb_total, kb0 + kb_per) - kb0, 0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer ----
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      // The weights do not depend on the kernel before this one: the first stages' weight tiles are requested while
      // that kernel is still draining; the activations (its output) follow after the dependency wait.
      const int pre = min(nk, STAGES);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), STAGE_BYTES);
        tma_load_2d(smem_base + i * STAGE_BYTES + MBLK * A_BYTES, &tmB, full_bar(i), (kb0 + i) * BK, n0);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) {
#pragma unroll
        for (int m = 0; m < MBLK; ++m)
          tma_load_2d(smem_base + i * STAGE_BYTES + m * A_BYTES, &tmA, full_bar(i), (kb0 + i) * BK, m * BM);
      }
      int stage = pre == STAGES ? 0 : pre;
      uint32_t phase = pre == STAGES ? 1 : 0;
      for (int i = pre; i < nk; ++i) {
        const int kb = kb0 + i;
        mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, p.status, 31);
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        mbar_expect_tx(full_bar(stage), STAGE_BYTES);
        tma_load_2d(sa + MBLK * A_BYTES, &tmB, full_bar(stage), kb * BK, n0);
#pragma unroll
        for (int m = 0; m < MBLK; ++m) tma_load_2d(sa + m * A_BYTES, &tmA, full_bar(stage), kb * BK, m * BM);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {  // ---- MMA issuer ----
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nk; ++i) {
        mbar_wait(full_bar(stage), phase, &abort_flag, p.status, 32);
        tc_fence_after();
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint64_t db = umma_smem_desc_sw128(sa + MBLK * A_BYTES);
#pragma unroll
        for (int m = 0; m < MBLK; ++m) {
          const uint64_t da = umma_smem_desc_sw128(sa + m * A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_base + m * SPK_BN, da + 2 * k, db + 2 * k, IDESC, (i | k) != 0);
        }
        umma_commit(empty_bar(stage));
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      umma_commit(tfull_bar);
    }
  } else {
    // ---- epilogue warps: thread = one row of every 128-row block ----
    pdl_wait();
    const int lane_grp = warp & 3;
    const int erow = lane_grp * 32 + lane;
    const int etid = threadIdx.x - 64;
    mbar_wait(tfull_bar, 0, &abort_flag, p.status, 33);
    tc_fence_after();
    const uint32_t t_lane = tmem_base + ((uint32_t)(lane_grp * 32) << 16);
    if (splits == 1) {
      uint8_t* epi_stage = smem_raw + (bar_base + 256 - smem_u32(smem_raw)) + lane_grp * EPI_WARP_BYTES;
#pragma unroll 1
      for (int m = 0; m < MBLK; ++m) {
        const int row = m * BM + erow;
        epilogue_store<SPK_BN, EPI>(p, t_lane + m * SPK_BN, row, row < p.M, n0, false, [](uint32_t*, int) {}, epi_stage);
        if (EPI == EPI_STORE) push_signal(p, m, max(0, min(SPK_BN, p.N - n0)));
      }
    } else {
      float* ws_mine = p.sk_partials + (int64_t)blockIdx.x * (U * UW * BM);
      uint32_t* counter = reinterpret_cast<uint32_t*>(p.sk_counters) + tile;
      if (nk > 0) {
#pragma unroll 1
        for (int u = 0; u < U; ++u) {
          if (u % splits == split) continue;
          const int m = u / UPB, c = (u % UPB) * UW;
          float* dst = ws_mine + (int64_t)u * (UW * BM) + erow;
#pragma unroll 1
          for (int cc = 0; cc < UW; cc += 32) {
            uint32_t r[32];
            tmem_ld_32x32(t_lane + m * SPK_BN + c + cc, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(dst + (cc + j) * BM, __uint_as_float(r[j]));
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (etid == 0) {
        const uint32_t prev = atomicAdd(counter, 1u);
        const uint32_t target = (prev / (uint32_t)splits + 1u) * (uint32_t)splits;
        int ok = 1;
        uint64_t t0 = 0;
        for (uint32_t spin = 0;; ++spin) {
          uint32_t v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
          if ((int32_t)(v - target) >= 0) break;
          if ((spin & 0xff) == 0xff) {
            const uint64_t now = global_timer_ns();
            if (t0 == 0) {
              t0 = now;
            } else if (now - t0 > 1000000000ull) {
              if (p.status) atomicCAS(p.status, 0, 34);
              ok = 0;
              break;
            }
          }
        }
        spk_ok = ok;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      __threadfence();
      int pushed[MBLK];
#pragma unroll
      for (int m = 0; m < MBLK; ++m) pushed[m] = 0;
      if (spk_ok) {
#pragma unroll 1
        for (int u = split; u < U; u += splits) {
          const int m = u / UPB, c = (u % UPB) * UW;
          const int row = m * BM + erow;
          const bool row_ok = row < p.M;
          uint32_t r[GATED ? 64 : 32];
#pragma unroll
          for (int cc = 0; cc < UW; cc += 32) {
            if (nk > 0) {
              tmem_ld_32x32(t_lane + m * SPK_BN + c + cc, r + cc);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[cc + j] = 0u;
            }
          }
          tmem_wait_ld();
          for (int s2 = 0; s2 < splits; ++s2) {
            if (s2 == split) continue;
            // a split without k-blocks (K not a multiple of splits * 64) stored nothing
            if (min(kb_total, s2 * kb_per + kb_per) - s2 * kb_per <= 0) continue;
            const float* src = p.sk_partials + ((int64_t)(tile * splits + s2) * U + u) * (UW * BM) + erow;
#pragma unroll
            for (int j = 0; j < UW; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldcg(src + j * BM));
          }
          const int col0 = n0 + c;
          if (GATED) {
            // accumulator columns [32 gate | 32 up] -> 32 output columns starting at col0 / 2
            if (row_ok && col0 < p.N) {
              bf16* crow = (bf16*)p.C + (int64_t)row * p.ldc + col0 / 2;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float gv = __uint_as_float(r[j + e]), uv = __uint_as_float(r[32 + j + e]);
                  o[e] = (EPI == EPI_GATED_SILU ? silu_f(gv) : gelu_tanh_f(gv)) * uv;
                }
                *reinterpret_cast<bf16x8*>(crow + j) = pack8(o);
              }
            }
          } else {
            epi_direct32<EPI>(p, r, row, row_ok, col0);
            pushed[m] += max(0, min(32, p.N - col0));
          }
        }
      }
      if (EPI == EPI_STORE && p.push_world > 0) {
#pragma unroll
        for (int m = 0; m < MBLK; ++m) push_signal(p, m, pushed[m]);
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int MBLK, int EPI>
int launch_splitk(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int splits, cudaStream_t st) {
  static DeviceOnce configured;
  if (!configured.done()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_splitk_kernel<MBLK, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         spk_smem_bytes<MBLK>());
    if (e != cudaSuccess) return (int)e;
    configured.set();
  }
  const int tiles = cdiv(p.N, SPK_BN);
  cudaError_t le = launch_pdl(gemm_bf16_splitk_kernel<MBLK, EPI>, dim3(tiles * splits), dim3(GEMM_THREADS),
                              spk_smem_bytes<MBLK>(), st, ta, tb, p, splits);
  return le == cudaSuccess ? LLB_OK : (int)le;
}

template <int MBLK>
int dispatch_splitk(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int splits,
                    cudaStream_t st) {
  switch (epi) {
    case EPI_STORE: return launch_splitk<MBLK, EPI_STORE>(ta, tb, p, splits, st);
    case EPI_RESIDUAL: return launch_splitk<MBLK, EPI_RESIDUAL>(ta, tb, p, splits, st);
    case EPI_GATED_SILU: return launch_splitk<MBLK, EPI_GATED_SILU>(ta, tb, p, splits, st);
    case EPI_GATED_GELU: return launch_splitk<MBLK, EPI_GATED_GELU>(ta, tb, p, splits, st);
    case EPI_F32: return launch_splitk<MBLK, EPI_F32>(ta, tb, p, splits, st);
  }
  return LLB_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// The same split through the L2 workspace, on CTA-pair tiles: a cluster of two CTAs computes a 256 x 256 tile
// slice with cta_group::2 MMAs (CTA h stages token rows h*128.. and 128 of the 256 weight rows per k-block, i.e.
// 16 KB of activations per 16 KB of weights, against 32 KB per 16 KB in the kernel above), and `splits` such
// pairs share the K range of a tile.  What an SM can pull from L2 per microsecond is what bounds these launches,
// so bytes staged per CTA is the figure of merit; the pair layout has the lowest.  CTA (tile, split, h) owns
// 128 accumulator rows x 256 columns, cut into units of 32 (gated: 64) columns; the units are shared out among
// the splits exactly as above, with one arrival counter per (tile, h).
// ---------------------------------------------------------------------------------------------
constexpr int PSK_TW = 256;
constexpr int PSK_STAGES = 6;
constexpr int PSK_STAGE_BYTES = BM * BK * 2 + (PSK_TW / 2) * BK * 2;  // 32 KB
constexpr int psk_smem_bytes() { return PSK_STAGES * PSK_STAGE_BYTES + 1024 + 256 + EPI_STAGE_BYTES; }

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pairsplit_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const GemmParams p, const int splits) {
  constexpr int STAGES = PSK_STAGES;
  constexpr int HALF = PSK_TW / 2;
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int STAGE_BYTES = PSK_STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = PSK_TW;
  constexpr uint32_t IDESC = umma_idesc(256, PSK_TW, 1);
  constexpr bool GATED = EPI == EPI_GATED_SILU || EPI == EPI_GATED_GELU;
  constexpr int UW = GATED ? 64 : 32;
  constexpr int U = PSK_TW / UW;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (STAGES + s); };
  const uint32_t tfull_bar = bar_base + 8 * (2 * STAGES);
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int spk_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t half = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1;                  // (m block, tile, split)
  const int per_m = p.num_n_blocks * splits;
  const int mb = pair / per_m;
  const int tile = (pair - mb * per_m) / splits, split = pair - mb * per_m - tile * splits;
  const int m0 = mb * 256;
  const int n0 = tile * PSK_TW;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int kb0 = split * kb_per;
  const int nk = max(min(kb_total, kb0 + kb_per) - kb0, 0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc_pair(smem_u32(&tmem_base_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer (both CTAs; transaction bytes are counted on the leader's barrier) ----
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      const int wrow = n0 + (int)half * HALF;
      const int pre = min(nk, STAGES);
      for (int i = 0; i < pre; ++i) {  // weights first: they do not depend on the previous kernel
        if (half == 0) mbar_expect_tx(full_bar(i), 2 * STAGE_BYTES);
        tma_load_2d_pair(smem_base + i * STAGE_BYTES + A_BYTES, &tmB, map_to_cta(full_bar(i), 0), (kb0 + i) * BK, wrow);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d_pair(smem_base + i * STAGE_BYTES, &tmA, map_to_cta(full_bar(i), 0), (kb0 + i) * BK,
                         m0 + (int)half * BM);
      int stage = pre == STAGES ? 0 : pre;
      uint32_t phase = pre == STAGES ? 1 : 0;
      for (int i = pre; i < nk; ++i) {
        const int kb = kb0 + i;
        mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, p.status, 35);
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
        if (half == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
        tma_load_2d_pair(sa + A_BYTES, &tmB, lead_full, kb * BK, wrow);
        tma_load_2d_pair(sa, &tmA, lead_full, kb * BK, m0 + (int)half * BM);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0 && half == 0) {  // ---- MMA issuer of the pair ----
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nk; ++i) {
        mbar_wait(full_bar(stage), phase, &abort_flag, p.status, 36);
        tc_fence_after();
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        const uint64_t da = umma_smem_desc_sw128(sa);
        const uint64_t db = umma_smem_desc_sw128(sa + A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_pair(tmem_base, da + 2 * k, db + 2 * k, IDESC, (i | k) != 0);
        umma_commit_pair(empty_bar(stage));
        umma_commit_pair(map_to_cta(empty_bar(stage), 1));
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      umma_commit_pair(tfull_bar);
      umma_commit_pair(map_to_cta(tfull_bar, 1));
    }
  } else {
    pdl_wait();
    const int lane_grp = warp & 3;
    const int erow = lane_grp * 32 + lane;
    const int etid = threadIdx.x - 64;
    if (nk > 0) mbar_wait(tfull_bar, 0, &abort_flag, p.status, 37);
    tc_fence_after();
    const int row = m0 + (int)half * BM + erow;
    const bool row_ok = row < p.M;
    const uint32_t t_lane = tmem_base + ((uint32_t)(lane_grp * 32) << 16);
    const int row_block = mb * 2 + (int)half;
    if (splits == 1) {
      uint8_t* epi_stage = smem_raw + (bar_base + 256 - smem_u32(smem_raw)) + lane_grp * EPI_WARP_BYTES;
      epilogue_store<PSK_TW, EPI>(p, t_lane, row, row_ok, n0, false, [](uint32_t*, int) {}, epi_stage);
      if (EPI == EPI_STORE) push_signal(p, row_block, max(0, min(PSK_TW, p.N - n0)));
    } else {
      // workspace slot of CTA (m block, tile, half, split): U units of [UW columns][128 rows] floats
      const int64_t slot0 = ((int64_t)(mb * p.num_n_blocks + tile) * 2 + half) * splits;
      float* ws_mine = p.sk_partials + (slot0 + split) * (int64_t)(PSK_TW * BM);
      uint32_t* counter = reinterpret_cast<uint32_t*>(p.sk_counters) + (mb * p.num_n_blocks + tile) * 2 + half;
      if (nk > 0) {
#pragma unroll 1
        for (int u = 0; u < U; ++u) {
          if (u % splits == split) continue;
          float* dst = ws_mine + (int64_t)u * (UW * BM) + erow;
#pragma unroll 1
          for (int cc = 0; cc < UW; cc += 32) {
            uint32_t r[32];
            tmem_ld_32x32(t_lane + u * UW + cc, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(dst + (cc + j) * BM, __uint_as_float(r[j]));
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (etid == 0) {
        const uint32_t prev = atomicAdd(counter, 1u);
        const uint32_t target = (prev / (uint32_t)splits + 1u) * (uint32_t)splits;
        int ok = 1;
        uint64_t t0 = 0;
        for (uint32_t spin = 0;; ++spin) {
          uint32_t v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
          if ((int32_t)(v - target) >= 0) break;
          if ((spin & 0xff) == 0xff) {
            const uint64_t now = global_timer_ns();
            if (t0 == 0) {
              t0 = now;
            } else if (now - t0 > 1000000000ull) {
              if (p.status) atomicCAS(p.status, 0, 38);
              ok = 0;
              break;
            }
          }
        }
        spk_ok = ok;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      __threadfence();
      int pushed = 0;
      if (spk_ok) {
#pragma unroll 1
        for (int u = split; u < U; u += splits) {
          uint32_t r[GATED ? 64 : 32];
#pragma unroll
          for (int cc = 0; cc < UW; cc += 32) {
            if (nk > 0) {
              tmem_ld_32x32(t_lane + u * UW + cc, r + cc);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[cc + j] = 0u;
            }
          }
          tmem_wait_ld();
          for (int s2 = 0; s2 < splits; ++s2) {
            if (s2 == split) continue;
            if (min(kb_total, s2 * kb_per + kb_per) - s2 * kb_per <= 0) continue;
            const float* src = p.sk_partials + (slot0 + s2) * (int64_t)(PSK_TW * BM) + (int64_t)u * (UW * BM) + erow;
#pragma unroll
            for (int j = 0; j < UW; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldcg(src + j * BM));
          }
          const int col0 = n0 + u * UW;
          if (GATED) {
            if (row_ok && col0 < p.N) {
              bf16* crow = (bf16*)p.C + (int64_t)row * p.ldc + col0 / 2;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float gv = __uint_as_float(r[j + e]), uv = __uint_as_float(r[32 + j + e]);
                  o[e] = (EPI == EPI_GATED_SILU ? silu_f(gv) : gelu_tanh_f(gv)) * uv;
                }
                *reinterpret_cast<bf16x8*>(crow + j) = pack8(o);
              }
            }
          } else {
            epi_direct32<EPI>(p, r, row, row_ok, col0);
            pushed += max(0, min(32, p.N - col0));
          }
        }
      }
      if (EPI == EPI_STORE && p.push_world > 0) push_signal(p, row_block, pushed);
    }
    tc_fence_before();
  }

  __syncthreads();
  cluster_sync_all();  // the leader's MMAs read the peer's shared memory and commit into its barriers
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int EPI>
int launch_pairsplit(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p_in, int splits, cudaStream_t st) {
  GemmParams p = p_in;
  p.num_m_blocks = cdiv(p.M, 256);
  p.num_n_blocks = cdiv(p.N, PSK_TW);
  static DeviceOnce configured;
  if (!configured.done()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_pairsplit_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         psk_smem_bytes());
    if (e != cudaSuccess) return (int)e;
    configured.set();
  }
  cudaError_t le = launch_pdl(gemm_bf16_pairsplit_kernel<EPI>, dim3(2 * p.num_m_blocks * p.num_n_blocks * splits),
                              dim3(GEMM_THREADS), psk_smem_bytes(), st, ta, tb, p, splits);
  return le == cudaSuccess ? LLB_OK : (int)le;
}

int dispatch_pairsplit(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int splits,
                       cudaStream_t st) {
  switch (epi) {
    case EPI_STORE: return launch_pairsplit<EPI_STORE>(ta, tb, p, splits, st);
    case EPI_RESIDUAL: return launch_pairsplit<EPI_RESIDUAL>(ta, tb, p, splits, st);
    case EPI_GATED_SILU: return launch_pairsplit<EPI_GATED_SILU>(ta, tb, p, splits, st);
    case EPI_GATED_GELU: return launch_pairsplit<EPI_GATED_GELU>(ta, tb, p, splits, st);
    case EPI_F32: return launch_pairsplit<EPI_F32>(ta, tb, p, splits, st);
  }
  return LLB_ERR_UNSUPPORTED;
}

// Largest usable split count of the pair split-K kernel (0: the shape does not fit it): every split needs a
// k-block, the units of a tile must divide among the splits, and all CTAs must be resident at once.
int pairsplit_max_splits(int M, int N, int K, int epi) {
  if ((N % 8) != 0) return 0;
  const bool gated = epi == EPI_GATED_SILU || epi == EPI_GATED_GELU;
  const int units = gated ? 4 : 8;
  const int pairs = cdiv(M, 256) * cdiv(N, PSK_TW), kb = cdiv(K, BK);
  if (pairs * 2 > sm_count() || pairs * 2 > SPK_MAX_TILES) return 0;
  int s = 1;
  while (s * 2 <= units && pairs * 2 * s * 2 <= sm_count() && (int64_t)cdiv(kb, s * 2) * (s * 2 - 1) < kb) s *= 2;
  return s;
}

// Largest usable split count for the split-K kernel (0: the shape does not fit it).
int splitk_max_splits(int M, int N, int K, int epi) {
  if (M > 256 || (N % 8) != 0) return 0;
  const bool gated = epi == EPI_GATED_SILU || epi == EPI_GATED_GELU;
  const int mblk = M > 128 ? 2 : 1;
  const int units = mblk * (gated ? 2 : 4);
  const int tiles = cdiv(N, SPK_BN), kb = cdiv(K, BK);
  if (tiles > sm_count() || tiles > SPK_MAX_TILES) return 0;
  int s = 1;
  while (s * 2 <= units && tiles * s * 2 <= sm_count() && (int64_t)cdiv(kb, s * 2) * (s * 2 - 1) < kb) s *= 2;
  return s;
}

// one-shot configuration of the next llb_gemm_bf16 call (set by llb_gemm_set_push, cleared by the call)
struct PushCfg {
  bf16* push[8];
  uint32_t* cnt[8];
  int world, rank, max_mb;
} g_push = {{nullptr}, {nullptr}, 0, 0, 0};

void apply_push(GemmParams& p) {
  p.push_world = g_push.world;
  p.push_rank = g_push.rank;
  p.push_max_mb = g_push.max_mb;
  for (int q = 0; q < 8; ++q) {
    p.push[q] = g_push.push[q];
    p.push_cnt[q] = g_push.cnt[q];
  }
  g_push.world = 0;
}
bool g_pair_auto = true;  // measured faster than one-CTA tiles for M >= 1024, K <= 8192 on B200

}  // namespace

LLB_EXPORT void llb_gemm_set_pair_auto(int on) { g_pair_auto = on != 0; }
LLB_EXPORT void llb_gemm_set_skinny_auto(int on) { g_skinny_auto = on != 0; }
LLB_EXPORT void llb_gemm_set_skinny_tw128(int on) { g_skinny_tw128 = on != 0; }
// The next llb_gemm_bf16 call (epilogue "store", N % 32 == 0, no stream-K) writes its output into the gather slots
// `push[q]` of all `world` ranks and advances their per-row-block column counters `cnt[q]` (see GemmParams).
LLB_EXPORT int llb_gemm_set_push(void** push, void** cnt, int rank, int world, int max_mb) {
  if (world < 1 || world > 8) return LLB_ERR_BAD_ARG;
  for (int q = 0; q < 8; ++q) {
    g_push.push[q] = q < world ? (bf16*)push[q] : nullptr;
    g_push.cnt[q] = q < world ? (uint32_t*)cnt[q] : nullptr;
  }
  g_push.world = world;
  g_push.rank = rank;
  g_push.max_mb = max_mb;
  return LLB_OK;
}

// C[M,N] (ldc) = A[M,K] (lda) . W[N,K]^T (ldw)  with epilogue `epi`:
//   0 store bf16 (+bias)          1 store bf16 of acc (+bias) + residual[M,N] (same ldc)
//   2 SiLU-gated: W rows interleaved as [32 gate | 32 up] blocks; C is [M, N/2]
//   3 store fp32 (+bias)          4 GELU(tanh)-gated, layout as 2
// bn: 0 = choose, else 64/128/256, or 512 = the CTA-pair (cta_group::2) kernel with 256x256 tiles.  status: optional device int receiving a wait-timeout code.
// stream_k: 0 = whole tiles per CTA, 1 = equal (tile, k-block) shares with fix-up of split tiles,
// -1 = choose (stream-K when the tiles would fill fewer than three waves).  Stream-K needs
// sk_partials (>= SMs * 2 * 128 * bn floats) and sk_counters (>= tiles ints, zero before first use;
// the kernel leaves them zero); launches that share them must not overlap on the GPU.
LLB_EXPORT int llb_gemm_bf16(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                             const void* residual, const void* bias, int M, int N, int K, int epi, int bn,
                             int stream_k, float* sk_partials, int64_t sk_partials_floats, int* sk_counters,
                             int sk_counters_len, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return LLB_OK;
  if (K <= 0 || (K % 8) != 0) return LLB_ERR_UNSUPPORTED;
  if ((epi == EPI_GATED_SILU || epi == EPI_GATED_GELU) && (N % 64) != 0) return LLB_ERR_UNSUPPORTED;
  if (epi != EPI_F32 && (((uintptr_t)C & 15) || (ldc % 8))) return LLB_ERR_BAD_ARG;
  if (epi == EPI_F32 && (((uintptr_t)C & 15) || (ldc % 4))) return LLB_ERR_BAD_ARG;
  if (epi == EPI_RESIDUAL && (residual == nullptr || ((uintptr_t)residual & 15))) return LLB_ERR_BAD_ARG;
  const int kblocks = cdiv(K, BK);
  if (stream_k != 0) {
    int sk_bn = bn ? bn : (N >= 256 ? 256 : (N >= 128 ? 128 : 64));
    int64_t tiles = (int64_t)cdiv(M, BM) * cdiv(N, sk_bn);
    bool fits = sk_partials != nullptr && sk_counters != nullptr &&
                sk_partials_floats >= (int64_t)sm_count() * 2 * BM * sk_bn && sk_counters_len >= tiles && tiles <= 8192;
    bool want = stream_k == 1 || (tiles < 3ll * sm_count() && tiles % sm_count() != 0 && kblocks >= 4);
    if (fits && want) {
      stream_k = 1;
      bn = sk_bn;
    } else {
      if (stream_k == 1 && !fits) return LLB_ERR_BAD_ARG;
      stream_k = 0;
    }
  }
  // split-K kernel without clusters: explicit (bn = 2000 + splits, 2000 = as many splits as fit)
  if (bn >= 2000 && bn < 2100) {
    int splits = bn - 2000;
    const int smax = splitk_max_splits(M, N, K, epi);
    if (smax == 0 || ldw < 0 || stream_k != 0) return LLB_ERR_UNSUPPORTED;
    if (splits == 0) splits = smax;
    if (splits > smax || (splits & (splits - 1)) != 0) return LLB_ERR_UNSUPPORTED;
    const int mblk = M > 128 ? 2 : 1;
    const int tiles = cdiv(N, SPK_BN);
    int log2s = 0;
    while ((1 << log2s) < splits) ++log2s;
    if (splits > 1 && (sk_partials == nullptr || sk_counters == nullptr ||
                       sk_partials_floats < (int64_t)tiles * splits * mblk * BM * SPK_BN ||
                       sk_counters_len < 8192 + 4 * SPK_MAX_TILES))
      return LLB_ERR_BAD_ARG;
    CUtensorMap ta, tb;
    int rc = cached_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM);
    if (rc) return rc;
    rc = cached_tmap(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, SPK_BN);
    if (rc) return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    apply_push(p);
    if (p.push_world > 0 && (epi != EPI_STORE || (N % 32))) return LLB_ERR_UNSUPPORTED;
    p.C = C;
    p.residual = (const bf16*)residual;
    p.bias = (const bf16*)bias;
    p.status = status;
    p.M = M;
    p.N = N;
    p.K = K;
    p.ldc = ldc;
    p.batch_count = 1;
    p.sk_partials = sk_partials;
    p.sk_counters = sk_counters ? sk_counters + 8192 + log2s * SPK_MAX_TILES : nullptr;
    return mblk == 2 ? dispatch_splitk<2>(epi, ta, tb, p, splits, st) : dispatch_splitk<1>(epi, ta, tb, p, splits, st);
  }
  // the same split on CTA-pair tiles: explicit (bn = 3000 + splits, 3000 = as many splits as fit)
  if (bn >= 3000 && bn < 3100) {
    int splits = bn - 3000;
    const int smax = pairsplit_max_splits(M, N, K, epi);
    if (smax == 0 || ldw < 0 || stream_k != 0) return LLB_ERR_UNSUPPORTED;
    if (splits == 0) splits = smax;
    if (splits > smax || (splits & (splits - 1)) != 0) return LLB_ERR_UNSUPPORTED;
    const int pairs = cdiv(M, 256) * cdiv(N, PSK_TW);
    int log2s = 0;
    while ((1 << log2s) < splits) ++log2s;
    if (splits > 1 && (sk_partials == nullptr || sk_counters == nullptr ||
                       sk_partials_floats < (int64_t)pairs * 2 * splits * BM * PSK_TW ||
                       sk_counters_len < 8192 + 4 * SPK_MAX_TILES))
      return LLB_ERR_BAD_ARG;
    CUtensorMap ta, tb;
    int rc = cached_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM);
    if (rc) return rc;
    rc = cached_tmap(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, PSK_TW / 2);
    if (rc) return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    apply_push(p);
    if (p.push_world > 0 && (epi != EPI_STORE || (N % 32))) return LLB_ERR_UNSUPPORTED;
    p.C = C;
    p.residual = (const bf16*)residual;
    p.bias = (const bf16*)bias;
    p.status = status;
    p.M = M;
    p.N = N;
    p.K = K;
    p.ldc = ldc;
    p.batch_count = 1;
    p.sk_partials = sk_partials;
    p.sk_counters = sk_counters ? sk_counters + 8192 + log2s * SPK_MAX_TILES : nullptr;
    return dispatch_pairsplit(epi, ta, tb, p, splits, st);
  }
  // skinny (decode) kernel: explicit (bn = 1000 + 10 * nb + splits) or chosen for M <= 256
  int sk_nb = 0, sk_splits = 0, sk_tw = 256;
  if (bn >= 1000) {
    if (bn >= 1100) {  // 1100 + 10 + splits: half-width tiles
      sk_tw = 128;
      bn -= 100;
    }
    sk_nb = (bn - 1000) / 10;
    sk_splits = (bn - 1000) % 10;
    if ((sk_nb != 1 && sk_nb != 2) || (sk_tw == 128 && sk_nb != 1) || (sk_splits != 1 && sk_splits != 2 && sk_splits != 4) || (N % 8) ||
        (int64_t)cdiv(kblocks, sk_splits) * (sk_splits - 1) >= kblocks)
      return LLB_ERR_UNSUPPORTED;
  } else if (bn == 0 && stream_k == 0 && g_skinny_auto && M >= 1024 && K >= 8192 && (N % 512) == 0 && ldw >= 0 &&
             (int64_t)cdiv(M, 256) * (N / 512) >= 2ll * (sm_count() / 2)) {
    sk_nb = 2;  // long K: one 256 x 512 tile per CTA pair measured faster than the persistent 256 x 256 schedule
    sk_splits = 1;
  } else if (bn == 0 && stream_k == 0 && g_skinny_auto && M <= 256 && N >= 1024 && (N % 8) == 0 && K >= 1024) {
    bool plan_pair = false;
    skinny_plan(M, N, K, epi, &sk_nb, &sk_splits, &plan_pair, &sk_tw);
    if (plan_pair && ldw >= 0) bn = 512;
  }
  const bool w_swz = ldw == -2;   // tiled and pre-swizzled (one-CTA kernels, bn 128 / 256)
  const bool w_tiled = ldw == -1;  // W is [N/128][K/64][128][64]
  if (w_tiled && ((N % 128) || (K % 64) || !sk_nb)) return LLB_ERR_UNSUPPORTED;
  if (w_swz && ((N % 256) || (K % 64) || sk_nb || (bn != 128 && bn != 256) || stream_k)) return LLB_ERR_UNSUPPORTED;
  if (sk_nb) {
    CUtensorMap ta, tb;
    int rc = cached_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM);
    if (rc) return rc;
    if (w_tiled)
      rc = cached_tmap(&tb, W, (uint64_t)N * (K / 64), 64, 64, (uint32_t)(sk_tw / 2));
    else
      rc = cached_tmap(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)(sk_tw / 2));
    if (rc) return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.w_tiled_kb = w_tiled ? K / 64 : 0;
    apply_push(p);
    if (p.push_world > 0 && (epi != EPI_STORE || (N % 32))) return LLB_ERR_UNSUPPORTED;
    p.C = C;
    p.residual = (const bf16*)residual;
    p.bias = (const bf16*)bias;
    p.status = status;
    p.M = M;
    p.N = N;
    p.K = K;
    p.ldc = ldc;
    p.batch_count = 1;
    return dispatch_skinny(epi, sk_nb, sk_splits, sk_tw, ta, tb, p, st);
  }
  // CTA-pair kernel: explicit (bn == 512) or chosen for big problems (at least two waves of pair tiles)
  bool use_pair = bn == 512;
  if (bn == 0 && stream_k == 0 && g_pair_auto && M >= 1024 && N >= 512 &&
      (int64_t)cdiv(M, 256) * cdiv(N, 256) >= 2ll * (sm_count() / 2))
    use_pair = true;
  if (bn == 0 || bn == 512) bn = use_pair ? PAIR_HALF : pick_bn(M, N);
  CUtensorMap ta, tb;
  int rc = cached_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM);
  if (rc) return rc;
  if (w_swz)
    tb = ta;  // unused: W comes by untiled bulk copies
  else
    rc = cached_tmap(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn);
  if (rc) return rc;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.w_tiled_kb = w_swz ? K / 64 : 0;
  p.w_swz = w_swz ? (const bf16*)W : nullptr;
  apply_push(p);
  if (p.push_world > 0 && (epi != EPI_STORE || (N % 32) || stream_k)) return LLB_ERR_UNSUPPORTED;
  p.C = C;
  p.residual = (const bf16*)residual;
  p.bias = (const bf16*)bias;
  p.status = status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.stream_k = stream_k;
  p.sk_partials = sk_partials;
  p.sk_counters = sk_counters;
  p.mblock_expert = nullptr;
  p.batch_count = 1;
  p.c_batch_stride = 0;
  if (use_pair) {
    p.stream_k = 0;
    return dispatch_pair(epi, ta, tb, p, st);
  }
  switch (bn) {
    case 256:
      return dispatch_epi<256>(epi, ta, tb, p, st);
    case 128:
      return dispatch_epi<128>(epi, ta, tb, p, st);
    case 64:
      return dispatch_epi<64>(epi, ta, tb, p, st);
  }
  return LLB_ERR_UNSUPPORTED;
}

// Grouped GEMM for MoE experts.  A [M_pad, K] holds the routed tokens sorted by expert, every expert's
// rows padded to a multiple of 128; W [E * N, K] stacks the expert weights; mblock_expert[M_pad / 128]
// (device) names the expert of each 128-row block, -1 for blocks beyond the routed rows (skipped).
// C [M_pad, N] (or [M_pad, N/2] for the gated epilogues).  N must be a multiple of the tile width.
LLB_EXPORT int llb_gemm_bf16_grouped(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                                     const int* mblock_expert, int M_pad, int N, int K, int E, int epi, int bn,
                                     int* status, cudaStream_t st) {
  if (M_pad <= 0 || N <= 0 || E <= 0) return LLB_OK;
  if (K <= 0 || (K % 8) != 0 || (M_pad % BM) != 0) return LLB_ERR_UNSUPPORTED;
  if (epi == EPI_RESIDUAL) return LLB_ERR_UNSUPPORTED;
  if (bn == 0) bn = (N % 256 == 0) ? 256 : ((N % 128 == 0) ? 128 : 64);
  if (N % bn != 0) return LLB_ERR_UNSUPPORTED;
  if (((uintptr_t)C & 15) || (ldc % 8)) return LLB_ERR_BAD_ARG;
  CUtensorMap ta, tb;
  int rc = cached_tmap(&ta, A, (uint64_t)M_pad, (uint64_t)K, (uint64_t)lda, BM);
  if (rc) return rc;
  rc = cached_tmap(&tb, W, (uint64_t)E * (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn);
  if (rc) return rc;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = C;
  p.residual = nullptr;
  p.bias = nullptr;
  p.status = status;
  p.M = M_pad;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.stream_k = 0;
  p.sk_partials = nullptr;
  p.sk_counters = nullptr;
  p.mblock_expert = mblock_expert;
  p.batch_count = 1;
  p.c_batch_stride = 0;
  switch (bn) {
    case 256:
      return dispatch_epi<256>(epi, ta, tb, p, st);
    case 128:
      return dispatch_epi<128>(epi, ta, tb, p, st);
    case 64:
      return dispatch_epi<64>(epi, ta, tb, p, st);
  }
  return LLB_ERR_UNSUPPORTED;
}

// Batched GEMM: for every batch index h:  C[:, h, :] = A[:, h, :] . W[h]^T
//   A [M, batch, K] with element strides (a_row_stride, a_batch_stride), inner stride 1
//   W [batch, N, K] contiguous;  C [M, batch, N] with element strides (c_row_stride, c_batch_stride)
// Strides in bytes must be multiples of 16 (TMA).  Used for the W_UK / W_UV absorption steps of MLA.
LLB_EXPORT int llb_gemm_bf16_batched(const void* A, int64_t a_row_stride, int64_t a_batch_stride, const void* W,
                                     void* C, int64_t c_row_stride, int64_t c_batch_stride, int M, int N, int K,
                                     int batch, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || batch <= 0) return LLB_OK;
  if (K % 8 != 0 || N % 8 != 0) return LLB_ERR_UNSUPPORTED;
  if ((a_row_stride % 8) || (a_batch_stride % 8) || (c_row_stride % 8) || (c_batch_stride % 8)) return LLB_ERR_BAD_ARG;
  int bn = N >= 256 && N % 256 == 0 ? 256 : (N % 128 == 0 ? 128 : 64);
  if ((int64_t)cdiv(M, BM) * cdiv(N, bn) * batch < sm_count() && bn > 64) bn = bn / 2;
  CUtensorMap ta, tb;
  int rc = make_tmap_3d(&ta, A, 2, (uint64_t)batch, (uint64_t)M, (uint64_t)K, (uint64_t)a_row_stride,
                        (uint64_t)a_batch_stride, BM, BK);
  if (rc) return rc;
  rc = make_tmap_3d(&tb, W, 2, (uint64_t)batch, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint64_t)N * K, (uint32_t)bn, BK);
  if (rc) return rc;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = C;
  p.residual = nullptr;
  p.bias = nullptr;
  p.status = status;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = c_row_stride;
  p.stream_k = 0;
  p.sk_partials = nullptr;
  p.sk_counters = nullptr;
  p.mblock_expert = nullptr;
  p.batch_count = batch;
  p.c_batch_stride = c_batch_stride;
  switch (bn) {
    case 256:
      return launch_gemm<256, EPI_STORE>(ta, tb, p, st);
    case 128:
      return launch_gemm<128, EPI_STORE>(ta, tb, p, st);
    case 64:
      return launch_gemm<64, EPI_STORE>(ta, tb, p, st);
  }
  return LLB_ERR_UNSUPPORTED;
}
