// Prefill attention on the 5th-generation tensor cores (tcgen05 + tensor memory), head size 128, causal, varlen,
// aware of an already cached prefix, K/V read through the token-granular slot table of the KV pool.
//
// One CTA computes 128 query rows of one (request, query head).  Per 128-key tile:
//   S  = Q . K^T            tcgen05.mma 128 x 128 x 128 into one of two tensor-memory buffers
//   P  = exp2(S - m)        the four softmax warps (one query row per thread) read S back, keep the running
//                           maximum / sum and write P as bf16 into shared memory in the operand layout
//   PV = P . V              tcgen05.mma into a third buffer, started from zero for every tile; the softmax
//                           threads add it to their fp32 output row in registers, rescaled when the maximum moves
// The MMA thread issues S of tile j + 1 before it waits for P of tile j, so the tensor core works on the next
// scores while the softmax of the current tile runs.  K and V tiles are gathered row by row (one 256-byte row per
// token and KV head) with 16-byte asynchronous copies straight into the 128-byte-swizzled operand layout; each
// of the two stages has its own K warp and V warp, so two tiles are always in flight.  V is consumed in the
// layout it has in memory (keys x head-dim, head-dim contiguous) as an MN-major B operand, 64 head-dim columns
// per instruction so that one swizzle atom spans the whole MN extent.
//
// Behavioural counterpart in the reference: lightllm/common/basemodel/triton_kernel/att/prefill_att/
// context_flashattention_nopad.py and the FlashInfer paged prefill wrapper
// (lightllm/common/basemodel/attention/flashinfer/).
#include "sm100_ptx.cuh"

using namespace llb;
using namespace llb::sm100;
LLB_DEBUG_BOUNDS_STORAGE(attention_tc)


namespace {

constexpr int D = 128;
constexpr int BM = 128, BN = 128;
constexpr int BLOCK_BYTES = 128 * 128;      // 128 rows x 64 bf16 (one swizzle-wide column block)
constexpr int TILE_BYTES = 2 * BLOCK_BYTES;  // 128 rows x 128 bf16
constexpr int THREADS = 11 * 32;  // warp 0, 10: K/V gather of stage 0, 1; warp 1: MMA; warps 2..9: softmax
// shared memory: Q | P | 2 stages x (K, V) | barriers | row-maximum / row-sum exchange
constexpr int OFF_Q = 0, OFF_P = TILE_BYTES, OFF_KV = 2 * TILE_BYTES;
constexpr int OFF_BAR = OFF_KV + 4 * TILE_BYTES;
constexpr int OFF_XCH = OFF_BAR + 256;               // float [2 tile parities][2 halves][128 rows]
constexpr int SMEM_BYTES = OFF_XCH + 2 * 2 * 128 * 4 + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint64_t kIssueWaitNs = 2000000000ull;

__device__ int g_attn_tc_status = 0;

// byte offset of 16-byte chunk `ch` (0..15: 8 head-dim / key elements each) of row `r` inside a 128 x 128 tile
__device__ __forceinline__ uint32_t tile_off(int r, int ch) {
  return (uint32_t)((ch >> 3) * BLOCK_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4));
}

// shared-memory descriptor for an MN-major operand block (rows = K index, 128 bytes of MN elements per row,
// 128-byte swizzle): groups of 8 rows are 1024 bytes apart.  Both offset fields carry that stride: the MN extent
// of one instruction (64 elements) fits the swizzle width, so no second stride is ever applied.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128_mn(uint32_t smem_addr) {
  uint64_t d = (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)(1024 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ float ex2_fast(float x) {  // 2^x, one MUFU instruction (x = -inf gives 0)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const bf162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(THREADS, 1)
gqa_prefill_tc_kernel(const bf16* __restrict__ q, int64_t q_stride, const bf16* __restrict__ kv_layer,
                      const int* __restrict__ req_to_token, int64_t r2t_stride, const int* __restrict__ b_req_idx,
                      const int* __restrict__ cu_q, const int* __restrict__ b_ready_len, bf16* __restrict__ out,
                      int64_t out_stride, int Hq, int Hkv, float scale_log2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + OFF_BAR;
  auto k_full = [&](int s) { return bar_base + 8 * s; };
  auto v_full = [&](int s) { return bar_base + 8 * (2 + s); };
  auto k_empty = [&](int s) { return bar_base + 8 * (4 + s); };
  auto v_empty = [&](int s) { return bar_base + 8 * (6 + s); };
  auto s_full = [&](int b) { return bar_base + 8 * (8 + b); };
  const uint32_t p_full = bar_base + 8 * 10, pv_full = bar_base + 8 * 11, q_full = bar_base + 8 * 12;
  float* xch = reinterpret_cast<float*>(smem_gen + OFF_XCH);
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int b = blockIdx.z, h = blockIdx.y;
  const int kvh = h / (Hq / Hkv);
  const int q_begin = cu_q[b];
  const int q_len = cu_q[b + 1] - q_begin;
  const int tile = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int q0 = tile * BM;
  if (q0 >= q_len) return;  // whole CTA: nothing allocated yet
  const int ready = b_ready_len[b];
  const int req = LLB_CHECK_REQ(b_req_idx[b]);
  const int rows_valid = min(BM, q_len - q0);
  const int kv_end = ready + q0 + rows_valid;  // exclusive bound on the keys any row of this tile may see
  const int n_tiles = (kv_end + BN - 1) / BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r2t_base = (int64_t)req * r2t_stride;
  int* status = &g_attn_tc_status;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
    }
    mbar_init(p_full, 8);
    mbar_init(pv_full, 1);
    mbar_init(q_full, 8);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  if (warp >= 2 && warp <= 9) {
    // Q tile -> shared memory in operand layout (rows beyond the request's tokens are zero), by the softmax warps
    // while the gather warps already fetch the first K / V tiles
    for (int c = threadIdx.x - 64; c < BM * 16; c += 256) {
      const int r = c >> 4, ch = c & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows_valid)
        v = *reinterpret_cast<const uint4*>(q + (int64_t)(q_begin + q0 + r) * q_stride + (int64_t)h * D + ch * 8);
      *reinterpret_cast<uint4*>(smem_gen + OFF_Q + tile_off(r, ch)) = v;
    }
    fence_proxy_async();  // the tensor core reads Q through the async proxy
    __syncwarp();
    if (lane == 0) mbar_arrive(q_full);
  }

  if (warp == 0 || warp == 10) {
    // ---- K / V gather of one stage: tiles stage, stage + 2, ...  K is released as soon as its scores are done,
    // V after P.V, so the K copy of tile j + 2 is in flight while tile j + 1 is being worked on ----
    const int stage = warp == 0 ? 0 : 1;
    const uint32_t k_dst = smem_base + OFF_KV + stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
    const bf16* k_src = kv_layer + (int64_t)kvh * D;
    const bf16* v_src = kv_layer + (int64_t)(kvh + Hkv) * D;
    for (int j = stage; j < n_tiles; j += 2) {
      const uint32_t par = (((uint32_t)j >> 1) & 1u) ^ 1u;
      const int kt = j * BN;
      int slots[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int pos = kt + u * 32 + lane;
        slots[u] = pos < kv_end ? LLB_CHECK_SLOT(req_to_token[r2t_base + pos]) : -1;
      }
      const int ch = lane & 15;
      mbar_wait(k_empty(stage), par, &abort_flag, status, 41);
#pragma unroll
      for (int u = 0; u < 4; ++u) {  // keys 32 u .. 32 u + 31; a half-warp copies the 16 chunks of one key's row
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int kk = 2 * i + (lane >> 4);
          const int sl = __shfl_sync(0xffffffffu, slots[u], kk);
          cp_async16(k_dst + tile_off(u * 32 + kk, ch), k_src + (int64_t)(sl >= 0 ? sl : 0) * (2 * Hkv) * D + ch * 8,
                     sl >= 0);
        }
      }
      cp_async_commit();
      mbar_wait(v_empty(stage), par, &abort_flag, status, 48);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int kk = 2 * i + (lane >> 4);
          const int sl = __shfl_sync(0xffffffffu, slots[u], kk);
          cp_async16(v_dst + tile_off(u * 32 + kk, ch), v_src + (int64_t)(sl >= 0 ? sl : 0) * (2 * Hkv) * D + ch * 8,
                     sl >= 0);
        }
      }
      cp_async_commit();
      cp_async_wait<1>();  // K landed
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(k_full(stage));
      cp_async_wait<0>();  // V landed
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(v_full(stage));
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer: scores of tile s and P.V of tile t are issued in whichever order their inputs arrive ----
      constexpr uint32_t IDESC_S = umma_idesc(BM, BN, 1);
      constexpr uint32_t IDESC_PV = umma_idesc(BM, 64, 1) | (1u << 16);  // B operand MN-major
      const uint32_t q_addr = smem_base + OFF_Q, p_addr = smem_base + OFF_P;
      int s_next = 0, pv_next = 0;
      mbar_wait(q_full, 0, &abort_flag, status, 40);
      uint64_t t0 = 0;
      uint32_t spins = 0;
      while (pv_next < n_tiles) {
        // score buffer s_next & 1 was last read for tile s_next - 2: free once that tile's P has been seen
        if (s_next < n_tiles && s_next < pv_next + 2 && mbar_test_wait(k_full(s_next & 1), ((uint32_t)s_next >> 1) & 1u)) {
          tc_fence_after();
          const uint32_t k_addr = smem_base + OFF_KV + (s_next & 1) * 2 * TILE_BYTES;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks >> 2) * BLOCK_BYTES + (ks & 3) * 32;
            umma_bf16(tmem_base + (s_next & 1) * BN, umma_smem_desc_sw128(q_addr + off),
                      umma_smem_desc_sw128(k_addr + off), IDESC_S, ks != 0);
          }
          umma_commit(s_full(s_next & 1));
          umma_commit(k_empty(s_next & 1));
          ++s_next;
          spins = 0;
          t0 = 0;
          continue;
        }
        if (pv_next < s_next && mbar_test_wait(p_full, (uint32_t)pv_next & 1u) &&
            mbar_test_wait(v_full(pv_next & 1), ((uint32_t)pv_next >> 1) & 1u)) {
          tc_fence_after();
          const uint32_t v_addr = smem_base + OFF_KV + (pv_next & 1) * 2 * TILE_BYTES + TILE_BYTES;
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {  // head-dim columns 64 hb .. 64 hb + 63
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks) {  // 16 keys per instruction
              const uint32_t a_off = (ks >> 2) * BLOCK_BYTES + (ks & 3) * 32;
              umma_bf16(tmem_base + 2 * BN + hb * 64, umma_smem_desc_sw128(p_addr + a_off),
                        umma_smem_desc_sw128_mn(v_addr + hb * BLOCK_BYTES + ks * 2048), IDESC_PV, ks != 0);
            }
          }
          umma_commit(pv_full);
          umma_commit(v_empty(pv_next & 1));
          ++pv_next;
          spins = 0;
          t0 = 0;
          continue;
        }
        if ((++spins & 0xff) == 0) {  // bounded: give up after two seconds without progress
          if (abort_flag) break;
          const uint64_t now = global_timer_ns();
          if (t0 == 0) {
            t0 = now;
          } else if (now - t0 > kIssueWaitNs) {
            abort_flag = 1;
            atomicCAS(status, 0, 49);
            break;
          }
        }
      }
    }
  } else {
    // ---- softmax + output accumulation: warps 2..9.  Two threads per query row: `half` 0 owns keys 0..63 of every
    // score tile and head-dim columns 0..63 of the output, half 1 the rest; they exchange the row maximum ----
    const int lane_grp = warp & 3;
    const int half = (warp - 2) >> 2;
    const int erow = lane_grp * 32 + lane;
    const int prow = ready + q0 + erow;  // absolute position of this row's token
    const uint32_t t_lane = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + half * 64;
    uint8_t* p_tile = smem_gen + OFF_P;
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    for (int j = 0; j < n_tiles; ++j) {
      const int kt = j * BN + half * 64;
      mbar_wait(s_full(j & 1), ((uint32_t)j >> 1) & 1u, &abort_flag, status, 45);
      tc_fence_after();
      uint32_t sr[64];
      tmem_ld_32x32(t_lane + (j & 1) * BN, sr);
      tmem_ld_32x32(t_lane + (j & 1) * BN + 32, sr + 32);
      tmem_wait_ld();
      const int lim = min(prow, kv_end - 1) - kt;  // my columns 0..lim are visible to this row
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (lim >= 63) {  // whole tile visible (every tile but the ones on the diagonal / at the end)
#pragma unroll
        for (int e = 0; e < 64; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sr[e]));
      } else {
#pragma unroll
        for (int e = 0; e < 64; ++e)
          if (e <= lim) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sr[e]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float* x = xch + (j & 1) * 256;
      x[half * 128 + erow] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(mx, x[(half ^ 1) * 128 + erow]);
      const float m_new = fmaxf(m_run, mx * scale_log2);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ex2_fast(m_run - m_use);
      m_run = m_new;
      if (j > 0) {  // o = (o + P V of the previous tile), then rescaled to the new maximum
        mbar_wait(pv_full, (uint32_t)(j - 1) & 1u, &abort_flag, status, 46);
        tc_fence_after();
        uint32_t r[64];
        tmem_ld_32x32(t_lane + 2 * BN, r);
        tmem_ld_32x32(t_lane + 2 * BN + 32, r + 32);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 64; ++e) o[e] = (o[e] + __uint_as_float(r[e])) * alpha;
      }
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      const bool all_visible = lim >= 63;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float pv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float pe = ex2_fast(fmaf(__uint_as_float(sr[g * 8 + e]), scale_log2, -m_use));
          pv[e] = (all_visible || g * 8 + e <= lim) ? pe : 0.f;
          rs4[e & 3] += pv[e];
        }
        *reinterpret_cast<uint4*>(p_tile + tile_off(erow, half * 8 + g)) =
            make_uint4(pack2(pv[0], pv[1]), pack2(pv[2], pv[3]), pack2(pv[4], pv[5]), pack2(pv[6], pv[7]));
      }
      l_run = l_run * alpha + (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tc_fence_before();    // my reads of S and of the previous P V are done
      fence_proxy_async();  // my P stores are visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    mbar_wait(pv_full, (uint32_t)(n_tiles - 1) & 1u, &abort_flag, status, 47);
    tc_fence_after();
    // total row sum = my keys + the other half's keys
    float* x = xch + (n_tiles & 1) * 256;
    x[half * 128 + erow] = l_run;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float l_tot = l_run + x[(half ^ 1) * 128 + erow];
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
    // output: every warp parks its 32 rows x 64 columns in its own part of the (now idle) Q / P buffers and
    // writes whole 128-byte lines
    uint8_t* stg = smem_gen + OFF_Q + (warp - 2) * (32 * 144);
    {
      uint32_t r[64];
      tmem_ld_32x32(t_lane + 2 * BN, r);
      tmem_ld_32x32(t_lane + 2 * BN + 32, r + 32);
      tmem_wait_ld();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (o[g * 8 + e] + __uint_as_float(r[g * 8 + e])) * inv;
        *reinterpret_cast<uint4*>(stg + lane * 144 + g * 16) =
            make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
      }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int id = i * 32 + lane, r = id >> 3, seg = id & 7;
      const int lr = lane_grp * 32 + r;
      if (lr < rows_valid) {
        const uint4 v = *reinterpret_cast<const uint4*>(stg + r * 144 + seg * 16);
        *reinterpret_cast<uint4*>(out + (int64_t)(q_begin + q0 + lr) * out_stride + (int64_t)h * D + half * 64 +
                                  seg * 8) = v;
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

LLB_EXPORT int llb_attn_tc_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_attn_tc_status, sizeof(int));
  return v;
}

// Same contract as llb_gqa_prefill (head size 128 only): q [T, Hq, 128] new tokens of all requests back to back.
LLB_EXPORT int llb_gqa_prefill_tc(const void* q, int64_t q_stride, const void* kv_layer, const int* req_to_token,
                                  int64_t r2t_stride, const int* b_req_idx, const int* cu_q, const int* b_ready_len,
                                  void* out, int64_t out_stride, int B, int max_q_len, int Hq, int Hkv, float sm_scale,
                                  cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return LLB_OK;
  if (Hkv <= 0 || Hq % Hkv != 0 || (q_stride % 8) || (out_stride % 8) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15))
    return LLB_ERR_BAD_ARG;
  static DeviceOnce configured;     
  if (!configured.done()) {
    cudaError_t e = cudaFuncSetAttribute(gqa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured.set();  
  }
  dim3 grid((max_q_len + BM - 1) / BM, Hq, B);
  gqa_prefill_tc_kernel<<<grid, THREADS, SMEM_BYTES, st>>>((const bf16*)q, q_stride, (const bf16*)kv_layer, req_to_token,
                                                          r2t_stride, b_req_idx, cu_q, b_ready_len, (bf16*)out,
                                                          out_stride, Hq, Hkv, sm_scale * kLog2e);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
