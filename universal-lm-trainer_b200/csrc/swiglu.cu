// SwiGLU gate of the feed-forward block (sm_100a), HBM-bound elementwise work.
//
// The reference computes  w2( silu(w1 x) * (w3 x) )  (train.py:1966-1975) with
// three PyTorch kernels in the forward (silu, mul) and five in the backward.  Here
// one kernel each way, over the two GEMM outputs a = w1 x and b = w3 x:
//   fwd:  y  = r(r(silu(a)) * b)
//   bwd:  db = r(dy * r(silu(a))),  da = r(r(dy * b) * silu'(a)),
//         silu'(a) = s (1 + a (1 - s)),  s = 1 / (1 + exp(-a)),
// where r() rounds to the tensors' dtype: the intermediate roundings are the ones
// eager PyTorch makes between its kernels (each kernel computes in fp32 and writes
// the tensor dtype), so 16-bit results agree with the reference's path to the last
// bit except where exp() itself differs by an ulp.
// 16-byte vectors, grid-stride, grid capped at a small multiple of the SM count;
// bytes moved: fwd 3 per element pair (2 reads + 1 write) x elem size, bwd 5.
#include "common.cuh"

namespace ulm {
namespace {

constexpr int kThreads = 256;

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

template <typename T>
__device__ __forceinline__ float rnd(float v) { return Cvt<T>::to_f(Cvt<T>::from_f(v)); }

__device__ __forceinline__ float sigmoid(float a) { return 1.f / (1.f + expf(-a)); }
__device__ __forceinline__ float silu(float a) { return a / (1.f + expf(-a)); }   // the form ATen's kernel uses

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, int64_t nvec, int64_t n) {
  constexpr int N = VecN<T>::N;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
    float fa[N], fb[N], fy[N];
    unpack<T>(reinterpret_cast<const uint4*>(a)[v], fa);
    unpack<T>(reinterpret_cast<const uint4*>(b)[v], fb);
#pragma unroll
    for (int i = 0; i < N; ++i) fy[i] = rnd<T>(silu(fa[i])) * fb[i];
    reinterpret_cast<uint4*>(y)[v] = pack<T>(fy);
  }
  // tail shorter than a vector
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nvec * N)) {
    const int64_t i = nvec * N + threadIdx.x;
    const float fa = Cvt<T>::to_f(a[i]);
    y[i] = Cvt<T>::from_f(rnd<T>(silu(fa)) * Cvt<T>::to_f(b[i]));
  }
}

template <typename T>
__device__ __forceinline__ void bwd_one(float fa, float fb, float fg, float& da, float& db) {
  const float s = sigmoid(fa);
  db = fg * rnd<T>(silu(fa));
  da = rnd<T>(fg * fb) * (s * (1.f + fa * (1.f - s)));
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_bwd_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ dy,
                  T* __restrict__ da, T* __restrict__ db, int64_t nvec, int64_t n) {
  constexpr int N = VecN<T>::N;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
    float fa[N], fb[N], fg[N], oa[N], ob[N];
    unpack<T>(reinterpret_cast<const uint4*>(a)[v], fa);
    unpack<T>(reinterpret_cast<const uint4*>(b)[v], fb);
    unpack<T>(reinterpret_cast<const uint4*>(dy)[v], fg);
#pragma unroll
    for (int i = 0; i < N; ++i) bwd_one<T>(fa[i], fb[i], fg[i], oa[i], ob[i]);
    reinterpret_cast<uint4*>(da)[v] = pack<T>(oa);
    reinterpret_cast<uint4*>(db)[v] = pack<T>(ob);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nvec * N)) {
    const int64_t i = nvec * N + threadIdx.x;
    float oa, ob;
    bwd_one<T>(Cvt<T>::to_f(a[i]), Cvt<T>::to_f(b[i]), Cvt<T>::to_f(dy[i]), oa, ob);
    da[i] = Cvt<T>::from_f(oa);
    db[i] = Cvt<T>::from_f(ob);
  }
}

unsigned grid_for(int64_t nvec) {
  int64_t blocks = (nvec + kThreads - 1) / kThreads;
  const int64_t cap = 16 * kNumSMs;
  if (blocks > cap) blocks = cap;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

bool aligned16(const void* p) { return p && !(reinterpret_cast<uintptr_t>(p) & 15); }

}  // namespace
}  // namespace ulm

extern "C" int ulm_swiglu_fwd(const ulm_swiglu_args* p) {
  using namespace ulm;
  if (!p) return fail(ULM_ERR_ARG, "ulm_swiglu_fwd: null args");
  if (p->dtype != ULM_F16 && p->dtype != ULM_BF16 && p->dtype != ULM_F32) return fail(ULM_ERR_ARG, "ulm_swiglu_fwd: bad dtype");
  if (p->n < 0) return fail(ULM_ERR_ARG, "ulm_swiglu_fwd: negative size");
  if (p->n == 0) return ULM_OK;
  if (!aligned16(p->a) || !aligned16(p->b) || !aligned16(p->y)) return fail(ULM_ERR_ARG, "ulm_swiglu_fwd: a, b, y must be non-null and 16-byte aligned");
  cudaStream_t st = (cudaStream_t)p->stream;
#define ULM_GO(T)                                                                                   \
  do {                                                                                              \
    const int64_t nvec = p->n / VecN<T>::N;                                                          \
    swiglu_fwd_kernel<T><<<grid_for(nvec), kThreads, 0, st>>>((const T*)p->a, (const T*)p->b, (T*)p->y, nvec, p->n); \
  } while (0)
  if (p->dtype == ULM_F16) ULM_GO(__half); else if (p->dtype == ULM_BF16) ULM_GO(__nv_bfloat16); else ULM_GO(float);
#undef ULM_GO
  return check_launch("ulm_swiglu_fwd");
}

extern "C" int ulm_swiglu_bwd(const ulm_swiglu_args* p) {
  using namespace ulm;
  if (!p) return fail(ULM_ERR_ARG, "ulm_swiglu_bwd: null args");
  if (p->dtype != ULM_F16 && p->dtype != ULM_BF16 && p->dtype != ULM_F32) return fail(ULM_ERR_ARG, "ulm_swiglu_bwd: bad dtype");
  if (p->n < 0) return fail(ULM_ERR_ARG, "ulm_swiglu_bwd: negative size");
  if (p->n == 0) return ULM_OK;
  if (!aligned16(p->a) || !aligned16(p->b) || !aligned16(p->dy) || !aligned16(p->da) || !aligned16(p->db))
    return fail(ULM_ERR_ARG, "ulm_swiglu_bwd: a, b, dy, da, db must be non-null and 16-byte aligned");
  cudaStream_t st = (cudaStream_t)p->stream;
#define ULM_GO(T)                                                                                   \
  do {                                                                                              \
    const int64_t nvec = p->n / VecN<T>::N;                                                          \
    swiglu_bwd_kernel<T><<<grid_for(nvec), kThreads, 0, st>>>((const T*)p->a, (const T*)p->b, (const T*)p->dy, \
                                                               (T*)p->da, (T*)p->db, nvec, p->n);    \
  } while (0)
  if (p->dtype == ULM_F16) ULM_GO(__half); else if (p->dtype == ULM_BF16) ULM_GO(__nv_bfloat16); else ULM_GO(float);
#undef ULM_GO
  return check_launch("ulm_swiglu_bwd");
}
