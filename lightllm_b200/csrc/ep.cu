// Expert-parallel dispatch / combine over NVLink peer memory (data-parallel attention + expert-parallel MoE).
//
// Every rank holds its own tokens [T, H] with their top-k expert ids / weights; expert e lives on rank
// e / E_local.  One MoE layer runs three kernels per rank, all writing / reading symmetric buffers of the peers:
//
//   ep_count   one CTA: per token the set of destination ranks (a token goes to a rank once, however many of
//              its experts live there), per-destination counts and the token's slot inside this rank's block
//              for each destination; the count row is stored into every peer's count matrix, then a flag.
//   ep_push    waits for all count rows; block base of (me -> r) = sum of counts of lower ranks to r; copies
//              every token's hidden row, id row and weight row into the peers' receive buffers with 16-byte
//              stores, remembers where each copy went, clears the id rows of its own receive buffer beyond the
//              total it will receive, and (last CTA) releases a "pushed" flag on every peer.
//   [ep_wait + the grouped expert GEMMs of this rank over its receive buffer: rows whose ids are not local drop out]
//   ep_combine releases "results ready" to all peers, waits for theirs, and for every own token sums the partial
//              results it finds in the peers' result buffers at the remembered rows (16-byte peer loads).
//
// Nothing returns to the host in between: the launches have fixed worst-case grids, which keeps a decode step
// capturable in a CUDA graph.  Waits are bounded (1 s) and record a code in a status word.
#include "common.cuh"

using namespace llb;

namespace {
constexpr int EP_MAX_WORLD = 8;
constexpr uint64_t kEpWaitNs = 1000000000ull;

struct EpView {
  // symmetric buffers as seen from this rank, index = peer rank
  bf16* h_recv[EP_MAX_WORLD];      // [max_recv, H]
  int* ids_recv[EP_MAX_WORLD];     // [max_recv, k]
  float* w_recv[EP_MAX_WORLD];     // [max_recv, k]
  bf16* out_recv[EP_MAX_WORLD];    // [max_recv, H]  partial results computed by that rank
  int* counts[EP_MAX_WORLD];       // [world, world] count matrix copy on that rank: counts[src][dst]
  uint32_t* flags[EP_MAX_WORLD];   // [3, world]: count flags, pushed flags, result flags (index by source rank)
  int rank, world;
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ bool ep_wait_flag(const uint32_t* flag, uint32_t want, int* status, int code) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if ((int32_t)(ld_acquire_sys_u32(flag) - want) >= 0) return true;
    if ((spin & 0x3f) == 0x3f) {
      if (status && *(volatile int*)status != 0) return false;
      uint64_t now = timer_ns();
      if (t0 == 0)
        t0 = now;
      else if (now - t0 > kEpWaitNs) {
        if (status) atomicCAS(status, 0, code);
        return false;
      }
      __nanosleep(64);
    }
  }
}

// ---- count: one CTA ----
__global__ void __launch_bounds__(1024) ep_count_kernel(EpView v, const int* __restrict__ topk_ids, int T, int k,
                                                        int experts_per_rank, uint8_t* __restrict__ dest_mask,
                                                        int* __restrict__ slot_in_block, const uint32_t* epoch_ptr) {
  const uint32_t epoch = *(volatile const uint32_t*)epoch_ptr + 1;
  __shared__ int s_cnt[EP_MAX_WORLD];
  if (threadIdx.x < EP_MAX_WORLD) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    uint32_t mask = 0;
    for (int j = 0; j < k; ++j) {
      const int e = topk_ids[(int64_t)t * k + j];
      if (e >= 0) {
        const int r = e / experts_per_rank;
        if (r < v.world) mask |= 1u << r;
      }
    }
    dest_mask[t] = (uint8_t)mask;
    for (int r = 0; r < v.world; ++r)
      slot_in_block[(int64_t)t * EP_MAX_WORLD + r] = (mask >> r) & 1u ? atomicAdd(&s_cnt[r], 1) : -1;
  }
  __syncthreads();
  if (threadIdx.x < v.world) {
    const int dst = threadIdx.x;
    for (int q = 0; q < v.world; ++q) v.counts[q][v.rank * v.world + dst] = s_cnt[dst];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < v.world) st_release_sys_u32(v.flags[threadIdx.x] + 0 * v.world + v.rank, epoch);
}

// ---- push ----
__global__ void __launch_bounds__(256) ep_push_kernel(EpView v, const bf16* __restrict__ h,
                                                      const int* __restrict__ topk_ids,
                                                      const float* __restrict__ topk_w, int T, int H, int k,
                                                      const uint8_t* __restrict__ dest_mask,
                                                      const int* __restrict__ slot_in_block, int* __restrict__ where,
                                                      int max_recv, unsigned* __restrict__ arrive, int* status,
                                                      int* __restrict__ recv_total_out, const uint32_t* epoch_ptr) {
  const uint32_t epoch = *(volatile const uint32_t*)epoch_ptr + 1;
  __shared__ int s_base[EP_MAX_WORLD];
  __shared__ int s_total;
  if (threadIdx.x < v.world) ep_wait_flag(v.flags[v.rank] + 0 * v.world + threadIdx.x, epoch, status, 300 + threadIdx.x);
  __syncthreads();
  if (threadIdx.x < v.world) {
    const int dst = threadIdx.x;
    int base = 0;
    const volatile int* C = v.counts[v.rank];
    for (int s = 0; s < v.rank; ++s) base += C[s * v.world + dst];
    s_base[dst] = base;
  }
  if (threadIdx.x == 0) {
    int tot = 0;
    const volatile int* C = v.counts[v.rank];
    for (int s = 0; s < v.world; ++s) tot += C[s * v.world + v.rank];
    s_total = tot < max_recv ? tot : max_recv;
    if (blockIdx.x == 0) *recv_total_out = s_total;
  }
  __syncthreads();
  // rows of my own receive buffer that nobody writes in this exchange carry no expert
  for (int64_t i = (int64_t)s_total * k + blockIdx.x * blockDim.x + threadIdx.x; i < (int64_t)max_recv * k;
       i += (int64_t)gridDim.x * blockDim.x)
    v.ids_recv[v.rank][i] = -1;
  const int nvec = H >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const uint32_t mask = dest_mask[t];
    for (int r = 0; r < v.world; ++r) {
      if (!((mask >> r) & 1u)) {
        if (threadIdx.x == 0) where[(int64_t)t * EP_MAX_WORLD + r] = -1;
        continue;
      }
      const int row = s_base[r] + slot_in_block[(int64_t)t * EP_MAX_WORLD + r];
      if (row >= max_recv) {  // receive buffer too small for this exchange: recorded, the token's share is lost
        if (threadIdx.x == 0) {
          where[(int64_t)t * EP_MAX_WORLD + r] = -1;
          atomicCAS(status, 0, 390);
        }
        continue;
      }
      const uint4* src = reinterpret_cast<const uint4*>(h + (int64_t)t * H);
      uint4* dst = reinterpret_cast<uint4*>(v.h_recv[r] + (int64_t)row * H);
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
      if (threadIdx.x < k) {
        v.ids_recv[r][(int64_t)row * k + threadIdx.x] = topk_ids[(int64_t)t * k + threadIdx.x];
        v.w_recv[r][(int64_t)row * k + threadIdx.x] = topk_w[(int64_t)t * k + threadIdx.x];
      }
      if (threadIdx.x == 0) where[(int64_t)t * EP_MAX_WORLD + r] = row;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(arrive, 1u);
    if (prev == gridDim.x - 1) {
      *arrive = 0;
      __threadfence_system();
      for (int r = 0; r < v.world; ++r) st_release_sys_u32(v.flags[r] + 1 * v.world + v.rank, epoch);
    }
  }
}

// ---- wait for every source's push (runs right before this rank's expert GEMMs) ----
__global__ void ep_wait_pushed_kernel(EpView v, int* status, const uint32_t* epoch_ptr) {
  const uint32_t epoch = *(volatile const uint32_t*)epoch_ptr + 1;
  if (threadIdx.x < v.world) ep_wait_flag(v.flags[v.rank] + 1 * v.world + threadIdx.x, epoch, status, 400 + threadIdx.x);
}

// ---- combine ----
__global__ void __launch_bounds__(256) ep_combine_kernel(EpView v, bf16* __restrict__ out, int T, int H,
                                                         const int* __restrict__ where, int accumulate, int* status,
                                                         uint32_t* epoch_ptr, unsigned* arrive) {
  const uint32_t epoch = *(volatile uint32_t*)epoch_ptr + 1;
  if (blockIdx.x == 0 && threadIdx.x < v.world) {
    __threadfence_system();
    st_release_sys_u32(v.flags[threadIdx.x] + 2 * v.world + v.rank, epoch);
  }
  if (threadIdx.x < v.world) ep_wait_flag(v.flags[v.rank] + 2 * v.world + threadIdx.x, epoch, status, 500 + threadIdx.x);
  __syncthreads();
  const int nvec = H >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    int rows[EP_MAX_WORLD];
#pragma unroll
    for (int r = 0; r < EP_MAX_WORLD; ++r) rows[r] = r < v.world ? where[(int64_t)t * EP_MAX_WORLD + r] : -1;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float acc[8];
      if (accumulate) {
        unpack8(reinterpret_cast<const bf16x8*>(out + (int64_t)t * H)[i], acc);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      }
      uint4 raw[EP_MAX_WORLD];
#pragma unroll
      for (int r = 0; r < EP_MAX_WORLD; ++r)
        if (rows[r] >= 0) raw[r] = reinterpret_cast<const uint4*>(v.out_recv[r] + (int64_t)rows[r] * H)[i];
#pragma unroll
      for (int r = 0; r < EP_MAX_WORLD; ++r) {
        if (rows[r] >= 0) {
          float f[8];
          unpack8(*reinterpret_cast<const bf16x8*>(&raw[r]), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += f[e];
        }
      }
      reinterpret_cast<bf16x8*>(out + (int64_t)t * H)[i] = pack8(acc);
    }
  }
  // the last CTA closes the round: the next layer's kernels of this rank read epoch + 1
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(arrive, 1u);
    if (prev == gridDim.x - 1) {
      *arrive = 0;
      __threadfence();
      *epoch_ptr = epoch;
    }
  }
}

EpView make_view(void** h_recv, void** ids_recv, void** w_recv, void** out_recv, void** counts, void** flags, int rank,
                 int world) {
  EpView v;
  memset(&v, 0, sizeof(v));
  for (int q = 0; q < world; ++q) {
    v.h_recv[q] = (bf16*)h_recv[q];
    v.ids_recv[q] = (int*)ids_recv[q];
    v.w_recv[q] = (float*)w_recv[q];
    v.out_recv[q] = (bf16*)out_recv[q];
    v.counts[q] = (int*)counts[q];
    v.flags[q] = (uint32_t*)flags[q];
  }
  v.rank = rank;
  v.world = world;
  return v;
}
}  // namespace

// dispatch = count + push + wait.  Tables hold `world` peer pointers.  scratch: dest_mask [T] bytes,
// slot_in_block [T, 8] ints, where [T, 8] ints (kept until combine), arrive (1 unsigned, zeroed once).
// `epoch` is a device counter of finished rounds (advanced by llb_ep_combine), so a captured graph replays correctly.
LLB_EXPORT int llb_ep_dispatch(void** h_recv, void** ids_recv, void** w_recv, void** out_recv, void** counts,
                               void** flags, int rank, int world, const void* h, const int* topk_ids,
                               const float* topk_w, int T, int H, int k, int experts_per_rank, int max_recv,
                               void* dest_mask, int* slot_in_block, int* where, unsigned* arrive, int* recv_total,
                               int* status, const unsigned* epoch, int ctas, cudaStream_t st) {
  if (world < 1 || world > EP_MAX_WORLD || (H % 8) || k < 1 || k > 32) return LLB_ERR_UNSUPPORTED;
  EpView v = make_view(h_recv, ids_recv, w_recv, out_recv, counts, flags, rank, world);
  ep_count_kernel<<<1, 1024, 0, st>>>(v, topk_ids, T, k, experts_per_rank, (uint8_t*)dest_mask, slot_in_block, epoch);
  LLB_LAUNCH_CHECK();
  if (ctas < 1) ctas = 1;
  ep_push_kernel<<<ctas, 256, 0, st>>>(v, (const bf16*)h, topk_ids, topk_w, T, H, k, (const uint8_t*)dest_mask,
                                       slot_in_block, where, max_recv, arrive, status, recv_total, epoch);
  LLB_LAUNCH_CHECK();
  ep_wait_pushed_kernel<<<1, 32, 0, st>>>(v, status, epoch);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

LLB_EXPORT int llb_ep_combine(void** h_recv, void** ids_recv, void** w_recv, void** out_recv, void** counts,
                              void** flags, int rank, int world, void* out, int T, int H, const int* where,
                              int accumulate, int* status, unsigned* epoch, unsigned* arrive, int ctas, cudaStream_t st) {
  if (world < 1 || world > EP_MAX_WORLD || (H % 8)) return LLB_ERR_UNSUPPORTED;
  EpView v = make_view(h_recv, ids_recv, w_recv, out_recv, counts, flags, rank, world);
  if (ctas < 1) ctas = 1;
  ep_combine_kernel<<<ctas, 256, 0, st>>>(v, (bf16*)out, T, H, where, accumulate, status, epoch, arrive);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
