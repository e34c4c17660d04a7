// Row kernels of the chunked cross-entropy (sm_100a), HBM-bound.
//
// The reference computes, per chunk of rows, logits = fc_out(h) and
// F.cross_entropy(logits, target, ignore_index, reduction='sum')
// (train.py:2075-2079); autocast runs the CE in fp32 on the 16-bit logits.
// Here one CTA owns one row of the [rows, V] logits tile:
//   fwd: single pass, online (max, sum of exp) per thread over 16-byte vectors,
//        block reduction, lse and the row's loss written in fp32;
//   bwd: logits <- (exp(logit - lse) - onehot) * g in place, rounded once to the
//        tile's dtype, so no fp32 [rows, V] array ever exists.
#include "common.cuh"

namespace ulm {
namespace {

constexpr int kThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <typename T> struct VecN { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void unpack(const uint4& u, float (&f)[VecN<T>::N]) {
  if constexpr (sizeof(T) == 4) {
    const float* p = reinterpret_cast<const float*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = p[i];
  } else {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = Cvt<T>::unpack2(w[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
}

template <typename T>
__device__ __forceinline__ uint4 pack(const float (&f)[VecN<T>::N]) {
  uint4 u;
  if constexpr (sizeof(T) == 4) {
    float* p = reinterpret_cast<float*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = f[i];
  } else {
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = Cvt<T>::pack2(f[2 * i], f[2 * i + 1]);
  }
  return u;
}

// (m, s) pairs in the log2 domain: value = s * 2^m
__device__ __forceinline__ void combine(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  if (mn == -INFINITY) { m = mn; s = 0.f; return; }
  s = s * exp2f(m - mn) + s2 * exp2f(m2 - mn);
  m = mn;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
ce_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target,
              float* __restrict__ lse, float* __restrict__ loss,
              int64_t row_stride, int V, int64_t ignore_index) {
  constexpr int N = VecN<T>::N;
  const int64_t r = blockIdx.x;
  const T* row = logits + r * row_stride;
  const int nvec = V / N;
  float m = -INFINITY, s = 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
    float f[N];
    unpack<T>(*reinterpret_cast<const uint4*>(row + (int64_t)vi * N), f);
    float mx = f[0];
#pragma unroll
    for (int j = 1; j < N; ++j) mx = fmaxf(mx, f[j]);
    mx *= kLog2e;
    const float mn = fmaxf(m, mx);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) acc += exp2f(fmaf(f[j], kLog2e, -mn));
    s = s * exp2f(m - mn) + acc;
    m = mn;
  }
  for (int c = nvec * N + threadIdx.x; c < V; c += kThreads) {   // ragged tail of the vocabulary
    combine(m, s, Cvt<T>::to_f(row[c]) * kLog2e, 1.f);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    combine(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  __shared__ float sm[kThreads / 32], ss[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    m = sm[0]; s = ss[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) combine(m, s, sm[w], ss[w]);
    const float l = (m + log2f(s)) * kLn2;
    lse[r] = l;
    const int64_t t = target[r];
    float out = 0.f;
    if (t != ignore_index && t >= 0 && t < V) out = l - Cvt<T>::to_f(row[t]);
    loss[r] = out;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
ce_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ target, const float* __restrict__ lse,
              const float* __restrict__ gscale_dev, float gscale,
              int64_t row_stride, int V, int64_t ignore_index) {
  constexpr int N = VecN<T>::N;
  const int64_t r = blockIdx.x;
  T* row = logits + r * row_stride;
  const int64_t t = target[r];
  const bool valid = (t != ignore_index && t >= 0 && t < V);
  const float g = valid ? gscale * (gscale_dev ? *gscale_dev : 1.f) : 0.f;
  const float l2 = lse[r] * kLog2e;
  const int nvec = V / N;
  for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
    uint4* p = reinterpret_cast<uint4*>(row + (int64_t)vi * N);
    float f[N];
    unpack<T>(*p, f);
    const int c0 = vi * N;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float sm = exp2f(fmaf(f[j], kLog2e, -l2));
      if ((int64_t)(c0 + j) == t) sm -= 1.f;
      f[j] = sm * g;
    }
    *p = pack<T>(f);
  }
  for (int c = nvec * N + threadIdx.x; c < V; c += kThreads) {
    float sm = exp2f(fmaf(Cvt<T>::to_f(row[c]), kLog2e, -l2));
    if ((int64_t)c == t) sm -= 1.f;
    row[c] = Cvt<T>::from_f(sm * g);
  }
}

int check(const char* who, const void* logits, const void* target, const void* lse, int64_t row_stride,
          int64_t rows, int V, int dtype) {
  if (dtype != ULM_F16 && dtype != ULM_BF16 && dtype != ULM_F32) return fail(ULM_ERR_ARG, "%s: bad dtype", who);
  const int n = dtype == ULM_F32 ? 4 : 8;
  if (rows < 0 || V <= 0) return fail(ULM_ERR_ARG, "%s: bad shape", who);
  if (rows > 0x7fffffffLL) return fail(ULM_ERR_TOO_LARGE, "%s: more than 2^31-1 rows in one tile", who);
  if (rows == 0) return ULM_OK;
  if (!logits || !target || !lse) return fail(ULM_ERR_ARG, "%s: null tensor", who);
  if ((reinterpret_cast<uintptr_t>(logits) & 15) || row_stride % n) return fail(ULM_ERR_ARG, "%s: rows must be 16-byte aligned", who);
  if (row_stride < V) return fail(ULM_ERR_ARG, "%s: row stride shorter than V", who);
  return ULM_OK;
}

}  // namespace
}  // namespace ulm

extern "C" int ulm_ce_fwd(const ulm_ce_fwd_args* a) {
  using namespace ulm;
  if (!a) return fail(ULM_ERR_ARG, "ulm_ce_fwd: null args");
  int rc = check("ulm_ce_fwd", a->logits, a->target, a->lse, a->row_stride, a->rows, a->V, a->dtype);
  if (rc || a->rows == 0) return rc;
  if (!a->loss) return fail(ULM_ERR_ARG, "ulm_ce_fwd: null loss");
  cudaStream_t st = (cudaStream_t)a->stream;
#define ULM_CE_FWD(T) ce_fwd_kernel<T><<<(unsigned)a->rows, kThreads, 0, st>>>((const T*)a->logits, a->target, a->lse, a->loss, a->row_stride, a->V, a->ignore_index)
  if (a->dtype == ULM_F16) ULM_CE_FWD(__half); else if (a->dtype == ULM_BF16) ULM_CE_FWD(__nv_bfloat16); else ULM_CE_FWD(float);
#undef ULM_CE_FWD
  return check_launch("ulm_ce_fwd");
}

extern "C" int ulm_ce_bwd(const ulm_ce_bwd_args* a) {
  using namespace ulm;
  if (!a) return fail(ULM_ERR_ARG, "ulm_ce_bwd: null args");
  int rc = check("ulm_ce_bwd", a->logits, a->target, a->lse, a->row_stride, a->rows, a->V, a->dtype);
  if (rc || a->rows == 0) return rc;
  cudaStream_t st = (cudaStream_t)a->stream;
#define ULM_CE_BWD(T) ce_bwd_kernel<T><<<(unsigned)a->rows, kThreads, 0, st>>>((T*)a->logits, a->target, a->lse, a->gscale_dev, a->gscale, a->row_stride, a->V, a->ignore_index)
  if (a->dtype == ULM_F16) ULM_CE_BWD(__half); else if (a->dtype == ULM_BF16) ULM_CE_BWD(__nv_bfloat16); else ULM_CE_BWD(float);
#undef ULM_CE_BWD
  return check_launch("ulm_ce_bwd");
}
