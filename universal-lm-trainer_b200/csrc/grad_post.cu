// One pass over a flat fp32 gradient bucket after the data-parallel all-reduce:
// unscale, finite check and squared-norm partial (sm_100a), HBM-bound.
// The reference does these as separate passes: scaler.unscale_ then
// clip_grad_norm_ (train.py:2364-2365).
// Every CTA writes its partial sum to caller scratch and a second one-CTA kernel adds
// the partials in index order: the squared norm is then bit-identical on every run and
// on every data-parallel rank (all ranks hold the same reduced gradients and must
// derive the same clip factor from them, or their weights drift apart).
#include "common.cuh"

namespace ulm {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxBlocks = 4 * kNumSMs;

__global__ void __launch_bounds__(kThreads)
unscale_sumsq_kernel(float* __restrict__ g, int64_t n, const float* __restrict__ inv_scale_dev,
                     float* __restrict__ partial, float* __restrict__ out) {
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
    partial[blockIdx.x] = t;
    if (anybad || !isfinite(t)) out[1] = 1.f;
  }
}

// out[0] += partial[0] + partial[1] + ... in a fixed tree order (one CTA)
__global__ void __launch_bounds__(kThreads)
sumsq_reduce_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out) {
  __shared__ float sh[kThreads];
  float t = 0.f;
  for (int i = threadIdx.x; i < nparts; i += kThreads) t += partial[i];
  sh[threadIdx.x] = t;
  __syncthreads();
  for (int o = kThreads / 2; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] += sh[0];
}

}  // namespace
}  // namespace ulm

extern "C" int64_t ulm_grad_sumsq_partial_count(void) { return ulm::kMaxBlocks; }

extern "C" int ulm_grad_unscale_sumsq(float* grad, int64_t n, const float* inv_scale_dev, float* out, float* partial, void* stream) {
  using namespace ulm;
  if (n < 0) return fail(ULM_ERR_ARG, "ulm_grad_unscale_sumsq: negative n");
  if (n == 0) return ULM_OK;
  if (!grad || !out || !partial) return fail(ULM_ERR_ARG, "ulm_grad_unscale_sumsq: null pointer");
  if (reinterpret_cast<uintptr_t>(grad) & 15) return fail(ULM_ERR_ARG, "ulm_grad_unscale_sumsq: grad must be 16-byte aligned");
  int64_t blocks = (n / 4 + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  unscale_sumsq_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(grad, n, inv_scale_dev, partial, out);
  int rc = check_launch("ulm_grad_unscale_sumsq");
  if (rc) return rc;
  sumsq_reduce_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(partial, (int)blocks, out);
  return check_launch("ulm_grad_unscale_sumsq(reduce)");
}
