// Tensor-parallel reduction over NVLink peer memory, fused with the residual add and the RMSNorm
// that follow every row-parallel GEMM (o_proj, down_proj).
//
//   residual += sum_over_ranks(partial_r)        h = rmsnorm(residual) * w
//
// Every rank owns one "symmetric" region with the same layout, mapped into all peers (CUDA IPC):
//   partial[2][maxT, H]   the rank's GEMM output (the GEMM writes straight into it), double-buffered
//   sums   [2][maxT, H]   reduced rows pushed by their owner ranks (two-shot mode), double-buffered
//   ready  [world]        ready[q] = epoch of the last call for which rank q's partial is complete
//   rowflag[maxT]         rowflag[i] = epoch of the last call for which row i of `sums` is complete
//
// One kernel per rank and call, no NCCL, no host round trip:
//   one-shot  (small T): wait ready[*] -> every rank pulls all peers' rows with P2P loads, sums in
//             fp32, adds the residual, normalises.  (tp-1) * T * H * 2 bytes in per rank, one hop.
//   two-shot  (larger T): rank r reduces the rows it owns (row % world == r) from the peers' partials
//             and pushes the bf16 sums into every rank's `sums` with P2P stores + a per-row flag;
//             then every rank adds the residual and normalises all rows from its own memory.
//             2 * (tp-1)/tp * T * H * 2 bytes per rank (the all-reduce minimum), rows stream through
//             as they complete, no global barrier.
// Flags carry a call epoch that only grows, so nothing is ever reset; the epoch lives in device memory
// and is advanced by the last CTA to finish, which keeps CUDA-graph replays correct.  A rank can run at
// most one call ahead of its slowest peer (it needs that peer's rows of the current call to finish), so
// two buffers per kind are enough.  Every wait is bounded: on expiry the kernel records a code in the
// status word and carries on, so it always terminates.
//
// The same kernel can be launched cooperatively with gridDim.y = world on ONE GPU (all "ranks" are
// slices of that GPU's memory): that is how the protocol is tested where only one GPU is available.
//
// Reference behaviour: lightllm/distributed/communication_op.py (all_reduce dispatch: FlashInfer one-shot,
// torch symmetric memory, NCCL) followed by separate add and rmsnorm kernels
// (lightllm/common/basemodel/layer_infer/base_layer_infer.py:63-84).
#include "common.cuh"
#include <cooperative_groups.h>

using namespace llb;

namespace {

constexpr int MAX_WORLD = 8;
constexpr uint64_t kCommWaitNs = 1000000000ull;

struct RankView {
  // pointers as seen from THIS rank; index = peer rank
  const bf16* partial[MAX_WORLD];  // peers' partial buffers (current parity)
  bf16* sums[MAX_WORLD];           // peers' sums buffers (current parity)
  uint32_t* ready[MAX_WORLD];      // peers' ready arrays
  uint32_t* rowflag[MAX_WORLD];    // peers' row flag arrays
  bf16* residual;                  // local [T, H]
  bf16* out;                       // local [T, H] normed output
  const bf16* norm_w;              // local [H]
  uint32_t* epoch;                 // local device counter (value of the previous call)
  uint32_t* arrive;                // local CTA arrival counter
  int* status;                     // local status word
  int rank;
};

struct CommParams {
  RankView v[MAX_WORLD];  // v[0] in a real multi-GPU launch; v[blockIdx.y] in the one-GPU emulation
  int world, T, H;
  float eps, w_offset;
  int one_shot;
  int do_norm;  // 0: plain all-reduce (out = sum over ranks, residual untouched)
  int rows_per_chunk;  // two-shot: owned rows reduced and flagged together (about 1024 vectors of 16 bytes)
  int max_chunks;      // flag slots per owner rank in every rank's flag array
  // pushed mode (one_shot == 2): the producing GEMMs of all ranks stored their partial tiles into this rank's
  // gather slots (partial[q] are LOCAL here) and advance push_cnt[q * push_max_mb + row / 128] by the columns
  // stored; a 128-row block is complete when every rank's counter reached (*push_epoch + 1) * H.
  const uint32_t* push_cnt[MAX_WORLD];  // per emulated rank: that rank's local counter array
  uint32_t* push_epoch[MAX_WORLD];      // per emulated rank: rounds finished on this buffer
  int push_max_mb;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Wait until *flag >= want (wrap-safe).  Called by one thread; returns false on timeout.
// Once any wait of this rank has expired (status != 0) the later ones give up at their first check, so a
// broken link costs one timeout per launch, not one per row.
__device__ bool wait_flag(const uint32_t* flag, uint32_t want, int* status, int code) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
    if ((spin & 0x3f) == 0x3f) {
      if (status && *(volatile int*)status != 0) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0)
        t0 = now;
      else if (now - t0 > kCommWaitNs) {
        if (status) atomicCAS(status, 0, code);
        return false;
      }
      __nanosleep(64);
    }
  }
}

__device__ __forceinline__ void add8(float* acc, const uint4& raw) {
  const bf16x8* p = reinterpret_cast<const bf16x8*>(&raw);
  float f[8];
  unpack8(*p, f);
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] += f[k];
}

// sum over ranks of row `row` (vector v) read from the peers' partial buffers
__device__ __forceinline__ void reduce_vec(const RankView& me, int world, int64_t off, float* acc) {
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  uint4 raw[MAX_WORLD];
#pragma unroll
  for (int q = 0; q < MAX_WORLD; ++q)
    if (q < world) raw[q] = ld_cg_16(me.partial[q] + off);
#pragma unroll
  for (int q = 0; q < MAX_WORLD; ++q)
    if (q < world) add8(acc, raw[q]);
}

// Two-shot phase 1: reduce the rows this rank owns (row % world == rank), chunk by chunk, and push the sums to
// every rank.  All of a thread's peer loads of an iteration are issued before the first use (8 x 16 bytes in
// flight per thread); a chunk's flag is released to all ranks after its sums are globally visible.
template <int W>
__device__ __forceinline__ void two_shot_phase1(const CommParams& p, const RankView& me, uint32_t epoch) {
  constexpr int U = 8 / W;
  const int world = p.world, T = p.T, H = p.H, nvec = H >> 3, G = gridDim.x;
  const int n_owned = (T - me.rank + world - 1) / world;
  const int rpc = p.rows_per_chunk;
  const int n_chunks = (n_owned + rpc - 1) / rpc;
  for (int c = blockIdx.x; c < n_chunks; c += G) {
    const int i0 = c * rpc;
    const int nv = (min(n_owned, i0 + rpc) - i0) * nvec;
    for (int base = 0; base < nv; base += 256 * U) {
      uint4 raw[U][W];
      int64_t offs[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * 256 + threadIdx.x;
        offs[u] = -1;
        if (idx < nv) {
          const int row = me.rank + (i0 + idx / nvec) * world;
          offs[u] = (int64_t)row * H + (idx % nvec) * 8;
#pragma unroll
          for (int q = 0; q < W; ++q)
            if (q < world) raw[u][q] = ld_cg_16(me.partial[q] + offs[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (offs[u] >= 0) {
          float acc[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
          for (int q = 0; q < W; ++q)
            if (q < world) add8(acc, raw[u][q]);
          bf16x8 packed = pack8(acc);
          const uint4 o = *reinterpret_cast<uint4*>(&packed);
#pragma unroll
          for (int q = 0; q < W; ++q)
            if (q < world) *reinterpret_cast<uint4*>(me.sums[q] + offs[u]) = o;
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) st_release_sys(me.rowflag[threadIdx.x] + me.rank * p.max_chunks + c, epoch);
  }
}

template <int MAX_VEC>
__global__ void __launch_bounds__(256) tp_reduce_norm_kernel(const CommParams p) {
  __shared__ float red[33];
  __shared__ int s_ok;
  const RankView& me = p.v[blockIdx.y];
  const int world = p.world, T = p.T, H = p.H;
  const int nvec = H >> 3;
  const uint32_t epoch = *me.epoch + 1;  // this call
  const int G = gridDim.x;

  const bool pushed = p.one_shot == 2;
  const uint32_t push_target = pushed ? (*(volatile uint32_t*)p.push_epoch[blockIdx.y] + 1u) * (uint32_t)H : 0u;
  if (!pushed) {
    // ---- announce: my partial (written by the GEMM that ran before this kernel) is complete ----
    if (blockIdx.x == 0 && threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(me.ready[threadIdx.x] + me.rank, epoch);
    }
    // ---- wait for every peer's partial ----
    if (threadIdx.x < world) wait_flag(me.ready[me.rank] + threadIdx.x, epoch, me.status, 100 + threadIdx.x);
    __syncthreads();
  }

  if (p.one_shot == 0) {
    if (world <= 2)
      two_shot_phase1<2>(p, me, epoch);
    else if (world <= 4)
      two_shot_phase1<4>(p, me, epoch);
    else
      two_shot_phase1<8>(p, me, epoch);
  }

  // token-sharded mode (one_shot == 3: reduce-scatter + residual + RMSNorm on the rows this rank owns, then
  // all-gather of the normalised rows): only rows with row % world == rank are reduced here, their residual
  // rows are the only ones kept up to date, and the normalised rows are pushed into every rank's `sums` buffer.
  const bool tpsp = p.one_shot == 3;
  const int row0 = tpsp ? me.rank + (int)blockIdx.x * world : (int)blockIdx.x;
  const int row_step = tpsp ? G * world : G;

  // ---- phase 2: residual add + RMSNorm over all rows (one-shot: reduce here from the peers) ----
  for (int row = row0; row < T; row += row_step) {
    if (pushed) {
      if (threadIdx.x < world)
        wait_flag(p.push_cnt[blockIdx.y] + threadIdx.x * p.push_max_mb + (row >> 7), push_target, me.status,
                  600 + threadIdx.x);
      __syncthreads();
    }
    if (p.one_shot == 0) {
      if (threadIdx.x == 0) {
        const int owner = row % world, chunk = (row / world) / p.rows_per_chunk;
        s_ok = wait_flag(me.rowflag[me.rank] + owner * p.max_chunks + chunk, epoch, me.status, 200) ? 1 : 0;
      }
      __syncthreads();
    }
    float vals[MAX_VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int v = threadIdx.x + i * 256;
      if (v < nvec) {
        const int64_t off = (int64_t)row * H + v * 8;
        if (p.one_shot) {
          reduce_vec(me, world, off, vals[i]);
        } else {
          uint4 raw = ld_cg_16(me.sums[me.rank] + off);
          unpack8(*reinterpret_cast<bf16x8*>(&raw), vals[i]);
        }
        if (p.do_norm) {
          float r[8];
          unpack8(*reinterpret_cast<const bf16x8*>(me.residual + off), r);
#pragma unroll
          for (int k = 0; k < 8; ++k) vals[i][k] += r[k];
          bf16x8 s = pack8(vals[i]);
          *reinterpret_cast<bf16x8*>(me.residual + off) = s;
          unpack8(s, vals[i]);
#pragma unroll
          for (int k = 0; k < 8; ++k) ss += vals[i][k] * vals[i][k];
        } else {
          *reinterpret_cast<bf16x8*>(me.out + off) = pack8(vals[i]);
        }
      }
    }
    if (p.do_norm) {
      ss = block_sum(ss, red);
      const float inv = rsqrtf(ss / (float)H + p.eps);
#pragma unroll
      for (int i = 0; i < MAX_VEC; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nvec) {
          float wf[8], o[8];
          unpack8(reinterpret_cast<const bf16x8*>(me.norm_w)[v], wf);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] = vals[i][k] * inv * (wf[k] + p.w_offset);
          if (tpsp) {
            const bf16x8 packed = pack8(o);
#pragma unroll
            for (int q = 0; q < MAX_WORLD; ++q)
              if (q < world) *reinterpret_cast<bf16x8*>(me.sums[q] + (int64_t)row * H + v * 8) = packed;
          } else {
            *reinterpret_cast<bf16x8*>(me.out + (int64_t)row * H + v * 8) = pack8(o);
          }
        }
      }
    }
    if (tpsp) {
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < world) st_release_sys(me.rowflag[threadIdx.x] + me.rank * p.max_chunks + row / world, epoch);
    }
    __syncthreads();
  }
  if (tpsp) {  // all-gather completion: every row of the other owners has landed in my buffer
    for (int row = blockIdx.x; row < T; row += G) {
      const int owner = row % world;
      if (owner != me.rank && threadIdx.x == 0)
        wait_flag(me.rowflag[me.rank] + owner * p.max_chunks + row / world, epoch, me.status, 700);
    }
  }

  // ---- the last CTA of this rank advances the epoch ----
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned prev = atomicAdd(me.arrive, 1u);
    if (prev == (unsigned)G - 1) {
      *me.arrive = 0;
      __threadfence();
      *me.epoch = epoch;
      if (pushed) *p.push_epoch[blockIdx.y] = *p.push_epoch[blockIdx.y] + 1u;
    }
  }
}

int launch(const CommParams& p, int ranks_in_grid, int ctas, cudaStream_t st) {
  if (p.H % 8 != 0 || p.H > 8 * 256 * 8 || p.world > MAX_WORLD || p.world < 1) return LLB_ERR_UNSUPPORTED;
  int per = cdiv(p.H / 8, 256);
  dim3 grid(ctas, ranks_in_grid);
  void* args[] = {(void*)&p};
  const void* fn = per <= 1   ? (const void*)tp_reduce_norm_kernel<1>
                   : per <= 2 ? (const void*)tp_reduce_norm_kernel<2>
                   : per <= 4 ? (const void*)tp_reduce_norm_kernel<4>
                              : (const void*)tp_reduce_norm_kernel<8>;
  // CTAs of one launch wait on CTAs of the peers' launches (two-shot), so all of them must be resident
  static int max_resident_tab[DeviceOnce::kMaxDevices][4] = {};
  const int slot = per <= 1 ? 0 : per <= 2 ? 1 : per <= 4 ? 2 : 3;
  int dev = DeviceOnce::current();
  if (dev < 0) dev = 0;
  int* max_resident = max_resident_tab[dev];
  if (max_resident[slot] == 0) {
    int occ = 0, sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, 256, 0) != cudaSuccess || occ < 1) occ = 1;
    max_resident[slot] = sms * occ;
  }
  if ((int)grid.x * ranks_in_grid > max_resident[slot]) grid.x = max_resident[slot] / ranks_in_grid;
  if (grid.x < 1) grid.x = 1;
  cudaError_t e;
  if (ranks_in_grid > 1) {
    // one-GPU emulation: CTAs of different "ranks" wait on one another, so they must be co-resident
    e = cudaLaunchCooperativeKernel(fn, grid, dim3(256), args, 0, st);
  } else {
    e = cudaLaunchKernel(fn, grid, dim3(256), args, 0, st);
  }
  return e == cudaSuccess ? LLB_OK : (int)e;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Copy-engine path for prompt-sized reductions.  The bytes of a reduce-scatter / all-gather are moved by
// cudaMemcpyAsync over NVLink (DMA engines, no SM), so that the transfer can run under the GEMMs of another
// micro-batch; the kernels here are only the glue: a flag exchange ("my buffer of call e is complete" / "I have
// seen everybody's") and the local sum of the gathered slices fused with the residual add and the RMSNorm.
// ---------------------------------------------------------------------------------------------
namespace {

struct CeFlagPtrs {
  uint32_t* peer[MAX_WORLD];  // flag array [world] of every rank, as seen from this rank
};

// Writes `value` into slot `rank` of every rank's flag array (release: everything this stream did before is
// visible to a peer that sees the flag), then waits until every slot of the local array has reached `value`.
// The wait is bounded by `timeout_ns` (prompt passes of different ranks can be far apart when a process is still
// warming up, so the limit is a parameter and longer than the decode kernels' one second); on expiry the code is
// recorded in `status` and the kernel returns.
// `mode`: bit 0 = signal, bit 1 = wait (both in a real run; one at a time where several ranks are emulated on one
// stream, whose kernels run one after the other).
__global__ void ce_signal_wait_kernel(CeFlagPtrs f, const uint32_t* local, int rank, int world, uint32_t value,
                                      int* status, int code, uint64_t timeout_ns, int mode) {
  const int t = threadIdx.x;
  if (t >= world) return;
  if (mode & 1) {
    __threadfence_system();
    st_release_sys(f.peer[t] + rank, value);
  }
  if (!(mode & 2)) return;
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if ((int32_t)(ld_acquire_sys(local + t) - value) >= 0) return;
    if ((spin & 0x3f) == 0x3f) {
      if (status && *(volatile int*)status != 0) return;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, code + t);
        return;
      }
      __nanosleep(128);
    }
  }
}

struct CeReduceParams {
  const bf16* src[MAX_WORLD];  // [rows, H] partial sums: this rank's own rows and the slices pulled from the peers
  bf16* residual;              // [rows, H] updated in place
  bf16* out;                   // [rows, H] normalised rows
  const bf16* norm_w;
  int nsrc, rows, H;
  float eps, w_offset;
};

template <int MAX_VEC>
__global__ void __launch_bounds__(256) ce_reduce_norm_kernel(const CeReduceParams p) {
  __shared__ float red[33];
  const int nvec = p.H >> 3;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    float vals[MAX_VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int v = threadIdx.x + i * 256;
      if (v < nvec) {
        const int64_t off = (int64_t)row * p.H + v * 8;
        uint4 raw[MAX_WORLD];
#pragma unroll
        for (int q = 0; q < MAX_WORLD; ++q)
          if (q < p.nsrc) raw[q] = ld_cg_16(p.src[q] + off);
        float r[8];
        unpack8(*reinterpret_cast<const bf16x8*>(p.residual + off), r);
#pragma unroll
        for (int k = 0; k < 8; ++k) vals[i][k] = 0.f;
#pragma unroll
        for (int q = 0; q < MAX_WORLD; ++q)
          if (q < p.nsrc) add8(vals[i], raw[q]);
#pragma unroll
        for (int k = 0; k < 8; ++k) vals[i][k] += r[k];
        const bf16x8 sres = pack8(vals[i]);
        *reinterpret_cast<bf16x8*>(p.residual + off) = sres;
        unpack8(sres, vals[i]);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += vals[i][k] * vals[i][k];
      }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)p.H + p.eps);
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int v = threadIdx.x + i * 256;
      if (v < nvec) {
        float wf[8], o[8];
        unpack8(reinterpret_cast<const bf16x8*>(p.norm_w)[v], wf);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = vals[i][k] * inv * (wf[k] + p.w_offset);
        *reinterpret_cast<bf16x8*>(p.out + (int64_t)row * p.H + v * 8) = pack8(o);
      }
    }
    __syncthreads();
  }
}

}  // namespace

LLB_EXPORT int llb_ce_signal_wait(void** peer_flags, const void* local_flags, int rank, int world, uint32_t value,
                                  int* status, int code, int64_t timeout_ms, int mode, cudaStream_t st) {
  if (world < 1 || world > MAX_WORLD) return LLB_ERR_BAD_ARG;
  CeFlagPtrs f;
  for (int q = 0; q < MAX_WORLD; ++q) f.peer[q] = q < world ? (uint32_t*)peer_flags[q] : nullptr;
  ce_signal_wait_kernel<<<1, 32, 0, st>>>(f, (const uint32_t*)local_flags, rank, world, value, status, code,
                                          (uint64_t)(timeout_ms > 0 ? timeout_ms : 1000) * 1000000ull, mode);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// residual[rows, H] += sum of the `nsrc` partial slices; out = rmsnorm(residual) * (norm_w + w_offset)
LLB_EXPORT int llb_ce_reduce_norm(const void** srcs, int nsrc, void* residual, void* out, const void* norm_w, int rows,
                                  int H, float eps, float w_offset, cudaStream_t st) {
  if (rows <= 0) return LLB_OK;
  if (nsrc < 1 || nsrc > MAX_WORLD || H % 8 != 0 || H > 8 * 256 * 8) return LLB_ERR_UNSUPPORTED;
  CeReduceParams p;
  memset(&p, 0, sizeof(p));
  for (int q = 0; q < nsrc; ++q) p.src[q] = (const bf16*)srcs[q];
  p.residual = (bf16*)residual;
  p.out = (bf16*)out;
  p.norm_w = (const bf16*)norm_w;
  p.nsrc = nsrc;
  p.rows = rows;
  p.H = H;
  p.eps = eps;
  p.w_offset = w_offset;
  const int per = cdiv(H / 8, 256);
  const int grid = rows < 1184 ? rows : 1184;
  if (per <= 1)
    ce_reduce_norm_kernel<1><<<grid, 256, 0, st>>>(p);
  else if (per <= 2)
    ce_reduce_norm_kernel<2><<<grid, 256, 0, st>>>(p);
  else if (per <= 4)
    ce_reduce_norm_kernel<4><<<grid, 256, 0, st>>>(p);
  else
    ce_reduce_norm_kernel<8><<<grid, 256, 0, st>>>(p);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// One stream-ordered copy between any two device ranges this process can address (local memory, or a peer's
// block opened through IPC: the driver routes it over NVLink on a copy engine).
LLB_EXPORT int llb_memcpy_async(void* dst, const void* src, int64_t bytes, cudaStream_t st) {
  if (bytes <= 0) return LLB_OK;
  cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, st);
  return e == cudaSuccess ? LLB_OK : (int)e;
}

// ---- symmetric memory helpers (plain cudaMalloc + legacy IPC handles; one process per GPU) ----
LLB_EXPORT int llb_symm_alloc(void** out, int64_t bytes) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*out, 0, (size_t)bytes);
  return e == cudaSuccess ? LLB_OK : (int)e;
}
LLB_EXPORT int llb_symm_free(void* p) { return (int)cudaFree(p); }
LLB_EXPORT int llb_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return LLB_OK;
}
LLB_EXPORT int llb_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? LLB_OK : (int)e;
}
LLB_EXPORT int llb_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// Pointer tables (arrays of `world` device pointers as seen from the calling rank).  In the one-GPU
// emulation (`emulate_ranks` = world) the tables hold world x world entries, rank-major.
LLB_EXPORT int llb_tp_reduce_norm(const void** partial, void** sums, void** ready, void** rowflag, void** residual,
                                  void** out, const void* norm_w, void** epoch, void** arrive, int* status, int rank,
                                  int world, int emulate_ranks, int T, int H, float eps, float w_offset, int one_shot,
                                  int do_norm, int ctas, int max_chunks, void** push_cnt, void** push_epoch,
                                  int push_max_mb, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  CommParams p;
  memset(&p, 0, sizeof(p));
  p.world = world;
  p.T = T;
  p.H = H;
  p.eps = eps;
  p.w_offset = w_offset;
  p.one_shot = one_shot;
  p.do_norm = do_norm;
  p.rows_per_chunk = (H / 8) >= 1024 ? 1 : 1024 / (H / 8);
  p.max_chunks = max_chunks;
  p.push_max_mb = push_max_mb;
  if (one_shot == 2 && (push_cnt == nullptr || push_epoch == nullptr || push_max_mb < cdiv(T, 128))) return LLB_ERR_BAD_ARG;
  const int nr = emulate_ranks > 1 ? emulate_ranks : 1;
  for (int r = 0; r < nr; ++r) {
    RankView& v = p.v[r];
    for (int q = 0; q < world; ++q) {
      v.partial[q] = (const bf16*)partial[r * world + q];
      v.sums[q] = (bf16*)sums[r * world + q];
      v.ready[q] = (uint32_t*)ready[r * world + q];
      v.rowflag[q] = (uint32_t*)rowflag[r * world + q];
    }
    v.residual = (bf16*)residual[r];
    v.out = (bf16*)out[r];
    v.norm_w = (const bf16*)norm_w;
    v.epoch = (uint32_t*)epoch[r];
    v.arrive = (uint32_t*)arrive[r];
    v.status = status;
    v.rank = emulate_ranks > 1 ? r : rank;
    p.push_cnt[r] = one_shot == 2 ? (const uint32_t*)push_cnt[r] : nullptr;
    p.push_epoch[r] = one_shot == 2 ? (uint32_t*)push_epoch[r] : nullptr;
  }
  return launch(p, nr, ctas, st);
}
