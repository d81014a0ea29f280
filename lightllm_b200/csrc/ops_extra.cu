// Kernels for the model families that are not RMSNorm + gated-SiLU decoders: LayerNorm with bias
// (Bloom, StarCoder, StarCoder2, StableLM), the plain (non-gated) activations of their MLPs, optional
// residual add fused into the norm, and an element scale (MiniCPM / Gemma embedding and logit scales).
#include "common.cuh"

using namespace llb;

// out = LayerNorm(x (+ residual)) * w + b ; when ADD the sum is also stored back into `residual`.
template <bool ADD>
__global__ void __launch_bounds__(256) layernorm_kernel(bf16* __restrict__ out, bf16* __restrict__ residual,
                                                        const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                        const bf16* __restrict__ b, int H, float eps) {
  extern __shared__ float row[];  // H floats
  __shared__ float red[33];
  const int64_t base = (int64_t)blockIdx.x * H;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = __bfloat162float(x[base + i]);
    if (ADD) {
      v += __bfloat162float(residual[base + i]);
      bf16 r = __float2bfloat16(v);
      residual[base + i] = r;
      v = __bfloat162float(r);
    }
    row[i] = v;
    s += v;
  }
  s = block_sum(s, red);
  const float mean = s / (float)H;
  __syncthreads();
  float q = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float d = row[i] - mean;
    q += d * d;
  }
  q = block_sum(q, red);
  const float inv = rsqrtf(q / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = (row[i] - mean) * inv * __bfloat162float(w[i]);
    if (b != nullptr) v += __bfloat162float(b[i]);
    out[base + i] = __float2bfloat16(v);
  }
}

LLB_EXPORT int llb_layernorm(void* out, void* residual, const void* x, const void* w, const void* b, int T, int H,
                             float eps, cudaStream_t st) {
  if (T <= 0) return LLB_OK;
  if (H <= 0 || (size_t)H * 4 > 96 * 1024) return LLB_ERR_UNSUPPORTED;
  size_t smem = (size_t)H * 4;
  if (residual != nullptr) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    layernorm_kernel<true><<<T, 256, smem, st>>>((bf16*)out, (bf16*)residual, (const bf16*)x, (const bf16*)w,
                                                 (const bf16*)b, H, eps);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    layernorm_kernel<false><<<T, 256, smem, st>>>((bf16*)out, nullptr, (const bf16*)x, (const bf16*)w, (const bf16*)b,
                                                  H, eps);
  }
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}

// In-place activation: 0 = SiLU, 1 = GELU(tanh), 2 = GELU(erf), 3 = ReLU, 4 = scale by `alpha`.
__global__ void __launch_bounds__(256) act_kernel(bf16* __restrict__ x, int64_t n, int kind, float alpha) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = __bfloat162float(x[i]);
  if (kind == 0) {
    v = v / (1.f + __expf(-v));
  } else if (kind == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    v = 0.5f * v * (1.f + tanhf(k0 * (v + k1 * v * v * v)));
  } else if (kind == 2) {
    v = 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
  } else if (kind == 3) {
    v = fmaxf(v, 0.f);
  } else {
    v *= alpha;
  }
  x[i] = __float2bfloat16(v);
}

LLB_EXPORT int llb_act_(void* x, int64_t n, int kind, float alpha, cudaStream_t st) {
  if (n <= 0) return LLB_OK;
  if (kind < 0 || kind > 4) return LLB_ERR_BAD_ARG;
  act_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((bf16*)x, n, kind, alpha);
  LLB_LAUNCH_CHECK();
  return LLB_OK;
}
