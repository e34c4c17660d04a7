// RMSNorm forward / backward (sm_100a), HBM-bound.
//
// y = w * x * rsqrt(mean(x^2) + eps) with the reduction in fp32 (the reference
// calls F.rms_norm, train.py:1862-1875; manual form inf.py:58-67).
// One warp per row; a lane keeps its part of the row in registers (16-byte
// loads), so x is read once.  The backward accumulates dw per warp across a
// grid-stride loop over rows, reduces across the CTA in shared memory and writes
// one partial row per CTA into caller-provided scratch; a second small kernel
// sums the partials in a fixed order (deterministic, no atomics).
#include "common.cuh"

#include <mutex>

namespace ulm {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxVec = 8;   // 16-byte vectors a lane keeps in registers (forward)
constexpr int kMaxD = 1024;  // widest row the backward keeps in registers

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[Vec<T>::N]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  if constexpr (sizeof(T) == 4) {
    const float* f = reinterpret_cast<const float*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = f[i];
  } else {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = Cvt<T>::unpack2(w[i]);
      out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
  }
}

template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[Vec<T>::N]) {
  uint4 u;
  if constexpr (sizeof(T) == 4) {
    float* f = reinterpret_cast<float*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = v[i];
  } else {
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = Cvt<T>::pack2(v[2 * i], v[2 * i + 1]);
  }
  *reinterpret_cast<uint4*>(p) = u;
}

// N consecutive elements of type TY (N * sizeof(TY) is 16 bytes, or 8 when a 16-bit y / dy
// accompanies an fp32 x)
template <typename TY, int N>
__device__ __forceinline__ void load_n(const TY* p, float (&out)[N]) {
  if constexpr (N * sizeof(TY) == 16) {
    load_vec<TY>(p, out);
  } else {
    static_assert(N == 4 && sizeof(TY) == 2, "8-byte vectors: four 16-bit elements");
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = Cvt<TY>::unpack2(u.x), b = Cvt<TY>::unpack2(u.y);
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
  }
}
template <typename TY, int N>
__device__ __forceinline__ void store_n(TY* p, const float (&v)[N]) {
  if constexpr (N * sizeof(TY) == 16) {
    store_vec<TY>(p, v);
  } else {
    static_assert(N == 4 && sizeof(TY) == 2, "8-byte vectors: four 16-bit elements");
    uint2 u;
    u.x = Cvt<TY>::pack2(v[0], v[1]);
    u.y = Cvt<TY>::pack2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = u;
  }
}

// weight element i..i+N-1 as floats, for either weight dtype
template <typename TW, int N>
__device__ __forceinline__ void load_w(const TW* w, int i, float (&out)[N]) {
#pragma unroll
  for (int j = 0; j < N; ++j) out[j] = Cvt<TW>::to_f(w[i + j]);
}

template <typename T, typename TW, typename TY>
__global__ void __launch_bounds__(kThreads)
rmsnorm_fwd_kernel(const T* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y,
                   float* __restrict__ rstd, int64_t x_stride, int64_t y_stride,
                   int64_t rows, int d, float eps) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarps;
  const int nvec = d / N;                              // vectors per row
  for (int64_t r = warp0; r < rows; r += nwarps) {
    const T* xr = x + r * x_stride;
    float v[kMaxVec][N];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int vi = it * 32 + lane;
      if (vi < nvec) {
        load_vec<T>(xr + vi * N, v[it]);
#pragma unroll
        for (int j = 0; j < N; ++j) ss += v[it][j] * v[it][j];
      }
    }
    for (int vi = kMaxVec * 32 + lane; vi < nvec; vi += 32) {   // rows wider than the register tile
      float t[N];
      load_vec<T>(xr + vi * N, t);
#pragma unroll
      for (int j = 0; j < N; ++j) ss += t[j] * t[j];
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps);
    if (rstd && lane == 0) rstd[r] = inv;
    TY* yr = y + r * y_stride;
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int vi = it * 32 + lane;
      if (vi < nvec) {
        float wv[N], o[N];
        load_w<TW, N>(w, vi * N, wv);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = v[it][j] * inv * wv[j];
        store_n<TY, N>(yr + vi * N, o);
      }
    }
    for (int vi = kMaxVec * 32 + lane; vi < nvec; vi += 32) {
      float t[N], wv[N], o[N];
      load_vec<T>(xr + vi * N, t);
      load_w<TW, N>(w, vi * N, wv);
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = t[j] * inv * wv[j];
      store_n<TY, N>(yr + vi * N, o);
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w,  xhat = x * rstd
// dw[c] = sum_rows dy * xhat.  Rows wider than kMaxD are rejected on the host.
template <typename T, typename TW, typename TY>
__global__ void __launch_bounds__(kThreads)
rmsnorm_bwd_kernel(const T* __restrict__ x, const TW* __restrict__ w, const TY* __restrict__ dy,
                   const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ partial,
                   int64_t x_stride, int64_t dy_stride, int64_t dx_stride,
                   int64_t rows, int d, float eps) {
  constexpr int N = Vec<T>::N;
  constexpr int kMaxVec = kMaxD / (32 * N);            // shadows the forward's constant: 32 floats per array
  extern __shared__ float s_dw[];                      // [kWarps][d]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t nwarps = (int64_t)gridDim.x * kWarps;
  const int nvec = d / N;
  float acc[kMaxVec][N];
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it)
#pragma unroll
    for (int j = 0; j < N; ++j) acc[it][j] = 0.f;
  for (int64_t r = warp0; r < rows; r += nwarps) {
    const T* xr = x + r * x_stride;
    const TY* gr = dy + r * dy_stride;
    float xv[kMaxVec][N], gv[kMaxVec][N];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int vi = it * 32 + lane;
      if (vi < nvec) {
        load_vec<T>(xr + vi * N, xv[it]);
        load_n<TY, N>(gr + vi * N, gv[it]);
#pragma unroll
        for (int j = 0; j < N; ++j) ss += xv[it][j] * xv[it][j];
      }
    }
    float inv;
    if (rstd) inv = rstd[r];
    else inv = rsqrtf(warp_sum(ss) / (float)d + eps);
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int vi = it * 32 + lane;
      if (vi < nvec) {
        float wv[N];
        load_w<TW, N>(w, vi * N, wv);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float xh = xv[it][j] * inv;
          acc[it][j] += gv[it][j] * xh;
          gv[it][j] *= wv[j];
          xv[it][j] = xh;
          dot += gv[it][j] * xh;
        }
      }
    }
    dot = warp_sum(dot) / (float)d;
    T* dr = dx + r * dx_stride;
#pragma unroll
    for (int it = 0; it < kMaxVec; ++it) {
      const int vi = it * 32 + lane;
      if (vi < nvec) {
        float o[N];
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = inv * (gv[it][j] - xv[it][j] * dot);
        store_vec<T>(dr + vi * N, o);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < kMaxVec; ++it) {
    const int vi = it * 32 + lane;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < N; ++j) s_dw[warp * d + vi * N + j] = acc[it][j];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += kThreads) {
    float t = 0.f;
#pragma unroll
    for (int wi = 0; wi < kWarps; ++wi) t += s_dw[wi * d + c];
    partial[(int64_t)blockIdx.x * d + c] = t;
  }
}

__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                         int nparts, int d) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float t = 0.f;
  for (int p = 0; p < nparts; ++p) t += partial[(int64_t)p * d + c];
  dw[c] = t;
}

// y / dy may be 16-bit next to an fp32 x (autocast's layout); otherwise they have x's dtype
int check_kind(const char* who, int kind, int x_dtype) {
  if (kind == ULM_Y_SAME) return ULM_OK;
  if (kind != ULM_Y_F16 && kind != ULM_Y_BF16) return fail(ULM_ERR_ARG, "%s: bad y/dy kind %d", who, kind);
  if (x_dtype != ULM_F32) return fail(ULM_ERR_ARG, "%s: a 16-bit y/dy kind needs an fp32 x", who);
  return ULM_OK;
}

int64_t bwd_grid(int64_t rows) {
  const int64_t want = (rows + kWarps - 1) / kWarps;
  const int64_t cap = 2 * kNumSMs;
  return want < 1 ? 1 : (want < cap ? want : cap);
}

int check_common(const char* who, int x_dtype, int w_dtype, int d, int64_t rows, const void* x, const void* w,
                 int64_t s0, int64_t s1, int64_t s2) {
  if (x_dtype != ULM_F16 && x_dtype != ULM_BF16 && x_dtype != ULM_F32) return fail(ULM_ERR_ARG, "%s: bad x dtype", who);
  if (w_dtype != x_dtype && w_dtype != ULM_F32) return fail(ULM_ERR_ARG, "%s: weight must be fp32 or x's dtype", who);
  const int n = x_dtype == ULM_F32 ? 4 : 8;
  if (d <= 0 || d % n) return fail(ULM_ERR_ARG, "%s: d must be a positive multiple of %d", who, n);
  if (rows < 0) return fail(ULM_ERR_ARG, "%s: negative rows", who);
  if (s0 % n || s1 % n || s2 % n) return fail(ULM_ERR_ARG, "%s: row strides must keep rows 16-byte aligned", who);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || !w) return fail(ULM_ERR_ARG, "%s: x must be 16-byte aligned, w non-null", who);
  return ULM_OK;
}

}  // namespace
}  // namespace ulm

extern "C" int64_t ulm_rmsnorm_bwd_partial_rows(int64_t rows) { return ulm::bwd_grid(rows); }

extern "C" int ulm_rmsnorm_fwd(const ulm_rmsnorm_fwd_args* a) {
  using namespace ulm;
  if (!a) return fail(ULM_ERR_ARG, "ulm_rmsnorm_fwd: null args");
  int rc = check_common("ulm_rmsnorm_fwd", a->x_dtype, a->w_dtype, a->d, a->rows, a->x, a->w, a->x_stride, a->y_stride, 0);
  if (rc) return rc;
  if ((rc = check_kind("ulm_rmsnorm_fwd", a->y_kind, a->x_dtype))) return rc;
  if (a->rows == 0) return ULM_OK;
  if (!a->y || (reinterpret_cast<uintptr_t>(a->y) & 15)) return fail(ULM_ERR_ARG, "ulm_rmsnorm_fwd: y must be 16-byte aligned");
  int64_t blocks = (a->rows + kWarps - 1) / kWarps;
  if (blocks > 8 * kNumSMs) blocks = 8 * kNumSMs;
  cudaStream_t st = (cudaStream_t)a->stream;
#define ULM_RMS_FWD3(T, TW, TY)                                                                  \
  rmsnorm_fwd_kernel<T, TW, TY><<<(unsigned)blocks, kThreads, 0, st>>>(                          \
      (const T*)a->x, (const TW*)a->w, (TY*)a->y, a->rstd, a->x_stride, a->y_stride, a->rows, a->d, a->eps)
#define ULM_RMS_FWD(T, TW) ULM_RMS_FWD3(T, TW, T)
  if (a->x_dtype == ULM_F32 && a->y_kind == ULM_Y_F16) ULM_RMS_FWD3(float, float, __half);
  else if (a->x_dtype == ULM_F32 && a->y_kind == ULM_Y_BF16) ULM_RMS_FWD3(float, float, __nv_bfloat16);
  else if (a->x_dtype == ULM_F32) ULM_RMS_FWD(float, float);
  else if (a->x_dtype == ULM_F16) { if (a->w_dtype == ULM_F32) ULM_RMS_FWD(__half, float); else ULM_RMS_FWD(__half, __half); }
  else { if (a->w_dtype == ULM_F32) ULM_RMS_FWD(__nv_bfloat16, float); else ULM_RMS_FWD(__nv_bfloat16, __nv_bfloat16); }
#undef ULM_RMS_FWD
#undef ULM_RMS_FWD3
  return check_launch("ulm_rmsnorm_fwd");
}

namespace ulm {
// Shared by the entry points that differ only in where `partial` lives.
int rmsnorm_bwd_launch(const ulm_rmsnorm_bwd_args* a, float* partial, const char* who) {
  int rc = check_common(who, a->x_dtype, a->w_dtype, a->d, a->rows, a->x, a->w, a->x_stride, a->dy_stride, a->dx_stride);
  if (rc) return rc;
  if ((rc = check_kind(who, a->dy_kind, a->x_dtype))) return rc;
  if (a->d > kMaxD) return fail(ULM_ERR_TOO_LARGE, "%s: d=%d exceeds %d", who, a->d, kMaxD);
  if (!a->dy || !a->dx || !a->dw || !partial) return fail(ULM_ERR_ARG, "%s: null tensor", who);
  if ((reinterpret_cast<uintptr_t>(a->dy) & 15) || (reinterpret_cast<uintptr_t>(a->dx) & 15))
    return fail(ULM_ERR_ARG, "%s: dy and dx must be 16-byte aligned", who);
  cudaStream_t st = (cudaStream_t)a->stream;
  const int64_t blocks = bwd_grid(a->rows);
  const size_t smem = (size_t)kWarps * a->d * sizeof(float);
  if (a->rows > 0) {
#define ULM_RMS_BWD3(T, TW, TY)                                                                  \
  do {                                                                                           \
    if (smem > 48 * 1024)                                                                        \
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<T, TW, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    rmsnorm_bwd_kernel<T, TW, TY><<<(unsigned)blocks, kThreads, smem, st>>>(                     \
        (const T*)a->x, (const TW*)a->w, (const TY*)a->dy, a->rstd, (T*)a->dx, partial,          \
        a->x_stride, a->dy_stride, a->dx_stride, a->rows, a->d, a->eps);                         \
  } while (0)
#define ULM_RMS_BWD(T, TW) ULM_RMS_BWD3(T, TW, T)
    if (a->x_dtype == ULM_F32 && a->dy_kind == ULM_Y_F16) ULM_RMS_BWD3(float, float, __half);
    else if (a->x_dtype == ULM_F32 && a->dy_kind == ULM_Y_BF16) ULM_RMS_BWD3(float, float, __nv_bfloat16);
    else if (a->x_dtype == ULM_F32) ULM_RMS_BWD(float, float);
    else if (a->x_dtype == ULM_F16) { if (a->w_dtype == ULM_F32) ULM_RMS_BWD(__half, float); else ULM_RMS_BWD(__half, __half); }
    else { if (a->w_dtype == ULM_F32) ULM_RMS_BWD(__nv_bfloat16, float); else ULM_RMS_BWD(__nv_bfloat16, __nv_bfloat16); }
#undef ULM_RMS_BWD
#undef ULM_RMS_BWD3
    rc = check_launch(who);
    if (rc) return rc;
  }
  rmsnorm_dw_reduce_kernel<<<(a->d + 127) / 128, 128, 0, st>>>(partial, a->dw, a->rows > 0 ? (int)blocks : 0, a->d);
  return check_launch(who);
}
}  // namespace ulm

extern "C" int ulm_rmsnorm_bwd(const ulm_rmsnorm_bwd_args* a) {
  using namespace ulm;
  if (!a) return fail(ULM_ERR_ARG, "ulm_rmsnorm_bwd: null args");
  return rmsnorm_bwd_launch(a, a->partial, "ulm_rmsnorm_bwd");
}

// ---------------------------------------------------------------------------
// Variant for callers that may not allocate device memory.
//
// ulm_rmsnorm_bwd needs one fp32 row of partial weight gradients per CTA, and
// normally the caller allocates that.  Some callers cannot: a training loop
// whose memory pool is frozen after warm-up, code running while a stream is
// being captured, a host language binding that owns no allocator.  For them the
// scratch lives in the library image instead: a fixed array in device global
// memory, present once on every GPU that loads the library and held until the
// process exits.
//
// The array's name below is only a handle in host code, not a device address;
// the address is looked up once per device with cudaGetSymbolAddress (with that
// device current) and cached.
// ---------------------------------------------------------------------------
namespace ulm {
namespace {

constexpr int kStaticMaxParts = 2 * kNumSMs;             // the backward never launches more CTAs than this
constexpr int kStaticMaxD = kMaxD;                       // widest row the backward kernel accepts
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_rms_partial[kStaticMaxParts * kStaticMaxD];   // 1.16 MiB

std::mutex g_static_mu;
float* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (set up on first use).
int static_scratch(float** out, const char* who) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ULM_ERR_CUDA, "%s: cudaGetDevice: %s", who, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(ULM_ERR_TOO_LARGE, "%s: device index %d beyond %d", who, dev, kMaxDevices - 1);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_rms_partial);
    if (e != cudaSuccess || !p) return fail(ULM_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", who, cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return ULM_OK;
}

}  // namespace
}  // namespace ulm

extern "C" int ulm_rmsnorm_bwd_static(const ulm_rmsnorm_bwd_args* a) {
  using namespace ulm;
  const char* who = "ulm_rmsnorm_bwd_static";
  if (!a) return fail(ULM_ERR_ARG, "%s: null args", who);
  if (a->d > kStaticMaxD)
    return fail(ULM_ERR_TOO_LARGE, "%s: d=%d exceeds the built-in scratch (rows of at most %d elements)", who, a->d, kStaticMaxD);
  if (bwd_grid(a->rows) > kStaticMaxParts)
    return fail(ULM_ERR_TOO_LARGE, "%s: %lld partial rows exceed the built-in scratch (%d)", who, (long long)bwd_grid(a->rows), kStaticMaxParts);
  if (a->rows > 0 && a->x) {                              // the tensors must live on the current device
    cudaPointerAttributes at;
    int dev = -1;
    if (cudaPointerGetAttributes(&at, a->x) == cudaSuccess && cudaGetDevice(&dev) == cudaSuccess &&
        at.type == cudaMemoryTypeDevice && at.device != dev)
      return fail(ULM_ERR_ARG, "%s: x is on device %d but device %d is current", who, at.device, dev);
    cudaGetLastError();
  }
  float* scratch = nullptr;
  int rc = static_scratch(&scratch, who);
  if (rc) return rc;
  // Every element the reduction reads (bwd_grid(rows) x d) is written by the backward
  // kernel of this same call first, so nothing left over from an earlier call is used
  // and nothing needs clearing.
  return rmsnorm_bwd_launch(a, scratch, who);
}
