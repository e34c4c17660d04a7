// One pass over a flat fp32 gradient bucket after the data-parallel all-reduce:
// unscale, finite check and squared-norm partial (sm_100a), HBM-bound.
// The reference does these as separate passes: scaler.unscale_ then
// clip_grad_norm_ (train.py:2364-2365).
#include "common.cuh"

namespace ulm {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
unscale_sumsq_kernel(float* __restrict__ g, int64_t n, const float* __restrict__ inv_scale_dev, float* __restrict__ out) {
  const float inv = inv_scale_dev ? *inv_scale_dev : 1.f;
  const int64_t nvec = n / 4;
  float ss = 0.f;
  bool bad = false;
  float4* g4 = reinterpret_cast<float4*>(g);
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * kThreads) {
    float4 v = g4[i];
    v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    g4[i] = v;
  }
  for (int64_t i = nvec * 4 + (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
    const float v = g[i] * inv;
    ss += v * v;
    g[i] = v;
  }
  bad = !isfinite(ss);                     // any inf/nan element makes the partial non-finite
  ss = warp_sum(ss);
  __shared__ float part[kThreads / 32];
  __shared__ int anybad;
  if (threadIdx.x == 0) anybad = 0;
  __syncthreads();
  if (bad) anybad = 1;
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) t += part[w];
    atomicAdd(out, t);
    if (anybad || !isfinite(t)) out[1] = 1.f;
  }
}

}  // namespace
}  // namespace ulm

extern "C" int ulm_grad_unscale_sumsq(float* grad, int64_t n, const float* inv_scale_dev, float* out, void* stream) {
  using namespace ulm;
  if (n < 0) return fail(ULM_ERR_ARG, "ulm_grad_unscale_sumsq: negative n");
  if (n == 0) return ULM_OK;
  if (!grad || !out) return fail(ULM_ERR_ARG, "ulm_grad_unscale_sumsq: null pointer");
  if (reinterpret_cast<uintptr_t>(grad) & 15) return fail(ULM_ERR_ARG, "ulm_grad_unscale_sumsq: grad must be 16-byte aligned");
  int64_t blocks = (n / 4 + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > 4 * kNumSMs) blocks = 4 * kNumSMs;
  unscale_sumsq_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(grad, n, inv_scale_dev, out);
  return check_launch("ulm_grad_unscale_sumsq");
}
