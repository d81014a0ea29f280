// Shared device/host helpers for the sm_100a kernels of this package.
//
// Conventions used by every exported entry point:
//   * C ABI (`extern "C"`), raw device pointers, an explicit cudaStream_t;
//     the Python side passes `tensor.data_ptr()` and the current torch stream.
//   * return value: 0 on success, a negative LLB_ERR_* code on a rejected
//     argument, or the (positive) cudaError_t of a failed launch.
//   * device-side waits are bounded; a wait that runs out records a code in
//     the caller-provided status word and the kernel returns normally.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define LLB_OK 0
#define LLB_ERR_BAD_ARG (-1)
#define LLB_ERR_UNSUPPORTED (-2)
#define LLB_ERR_TOO_LARGE (-3)
#define LLB_ERR_DRIVER (-4)

#define LLB_EXPORT extern "C" __attribute__((visibility("default")))

#define LLB_LAUNCH_CHECK()                                  \
  do {                                                      \
    cudaError_t _e = cudaGetLastError();                    \
    if (_e != cudaSuccess) return (int)_e;                  \
  } while (0)

namespace llb {

// Programmatic dependent launch: a kernel launched through launch_pdl() may be scheduled while the previous
// kernel of the stream is still draining; it must call pdl_wait() before it touches global memory (the call
// returns once the previous kernel has completed and flushed).  Its own prologue (barrier set-up, tensor
// memory allocation, index arithmetic) overlaps the predecessor's tail.  LLB_PDL=0 turns the attribute off.
// After its own wait the kernel lets the next kernel of the stream be scheduled (launch_dependents): that kernel's
// CTAs start on every SM as soon as this kernel's CTA there has exited and run their prologue up to their own
// pdl_wait(), instead of waiting for the whole grid to drain plus a launch latency.
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LLB_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// One-time per-device set-up (function attributes such as the dynamic shared-memory limit belong to the device
// that was current when they were set): `static DeviceOnce once; if (!once.done()) { ...; once.set(); }`.
struct DeviceOnce {
  static constexpr int kMaxDevices = 64;
  bool flags[kMaxDevices] = {};
  static int current() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return -1;
    return d;
  }
  bool done() const {
    int d = current();
    return d >= 0 && flags[d];
  }
  void set() {
    int d = current();
    if (d >= 0) flags[d] = true;
  }
};

// ---------------------------------------------------------------------------------------
// Debug build with index checks (compile with -DLLB_DEBUG_BOUNDS: `LLB_DEBUG_BOUNDS=1 python -m lightllm_b200.build`
// produces libllb_kernels_dbg.so next to the regular library; LLB_DEBUG_BOUNDS=1 at run time loads it).
// The kernels that turn an index read from memory into an address (KV pool slots, request-table rows and
// columns, expert ids) compare it with the declared size first; an index outside records a code in a status
// word and the access goes to entry 0 instead, so a wrong index is reported without touching memory beyond the
// table.  The declared sizes live in a __constant__ struct per translation unit (no relocatable device code is
// linked), set through the unit's exported setter; 0 = unknown = unchecked.
//   901 pool slot   902 request row   903 request-table column   904 expert id
// ---------------------------------------------------------------------------------------
struct DebugBounds {
  int pool_slots;   // valid slots are [0, pool_slots)  (the HOLD slot included)
  int req_rows;     // valid request rows are [0, req_rows)  (the HOLD row included)
  int r2t_cols;     // valid positions inside a request row
  int num_experts;  // valid expert ids (negative ids mean "no expert" and pass)
  int* status;
};
#ifdef LLB_DEBUG_BOUNDS
#define LLB_DEBUG_BOUNDS_STORAGE(unit)                                                                      \
  __constant__ llb::DebugBounds g_dbg_bounds = {0, 0, 0, 0, nullptr};                                      \
  LLB_EXPORT int llb_debug_set_bounds_##unit(int pool_slots, int req_rows, int r2t_cols, int num_experts,  \
                                             int* status) {                                                \
    llb::DebugBounds b = {pool_slots, req_rows, r2t_cols, num_experts, status};                            \
    cudaError_t e = cudaMemcpyToSymbol(g_dbg_bounds, &b, sizeof(b));                                       \
    return e == cudaSuccess ? 0 : (int)e;                                                                  \
  }
#define LLB_DBG_CHECK(idx, field, code) llb::dbg_check((idx), g_dbg_bounds.field, g_dbg_bounds.status, (code))
__device__ __forceinline__ int dbg_check(int idx, int limit, int* status, int code) {
  if (limit > 0 && (idx < 0 || idx >= limit)) {
    if (status) atomicCAS(status, 0, code);
    return 0;
  }
  return idx;
}
#else
#define LLB_DEBUG_BOUNDS_STORAGE(unit)
#define LLB_DBG_CHECK(idx, field, code) (idx)
#endif
#define LLB_CHECK_SLOT(x) LLB_DBG_CHECK((x), pool_slots, 901)
#define LLB_CHECK_REQ(x) LLB_DBG_CHECK((x), req_rows, 902)
#define LLB_CHECK_POS(x) LLB_DBG_CHECK((x), r2t_cols, 903)
#define LLB_CHECK_EXPERT(x) LLB_DBG_CHECK((x), num_experts, 904)

__host__ __device__ __forceinline__ int cdiv(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// 16-byte vector of 8 bf16 values.  Plain words, so that the type is trivially copyable and a load or store of
// it is one 128-bit access (a member of type bf162 has user-provided copy operations, which made every struct
// assignment four separate 32-bit stores).
struct alignas(16) bf16x8 {
  uint32_t w[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
  const uint4 raw = *reinterpret_cast<const uint4*>(&p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // a bf16 is the upper half of an fp32
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bf162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    p.w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` is a shared array of >= 33 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// cp.async helpers (16-byte, L2-only caching: streaming KV / weights)
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, bool pred) {
  int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// ldmatrix / mma.sync (legacy tensor path; used by the bandwidth-bound attention kernels)
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  bf162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

}  // namespace llb
