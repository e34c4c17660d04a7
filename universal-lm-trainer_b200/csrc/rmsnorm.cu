// RMSNorm forward / backward (sm_100a), HBM-bound, optionally fused with the residual add
// in front of it.
//
// y = w * x * rsqrt(mean(x^2) + eps) with the reduction in fp32 (the reference calls
// F.rms_norm, train.py:1862-1875; manual form inf.py:58-67).  With a `branch` tensor the
// kernel first forms x_new = x + branch (the residual add of train.py:1989 / 1993), writes
// it out and normalises it in the same pass; the backward then also adds the gradient
// that reaches x_new from later layers and writes the sum once for both inputs of the add.
//
// One warp per row; a lane keeps its part of the row in registers (16-byte loads), so x is
// read once.  To keep enough bytes in flight per SM a warp works on several rows at a time
// (all their loads are issued before the first reduction), and the per-lane register tile is
// sized by the row width (template parameter NV = 16-byte vectors per lane), not by a fixed
// maximum.  The backward accumulates dw per warp across a grid-stride loop over rows,
// reduces across the CTA in shared memory and writes one partial row per CTA into
// caller-provided scratch; a second small kernel sums the partials in a fixed order
// (deterministic, no atomics).
#include "common.cuh"

#include <mutex>

namespace ulm {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxD = 1024;  // widest row the backward accepts (and the static scratch is sized for)

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

// N consecutive elements of type TE as floats; N * sizeof(TE) is 16 bytes, or 8 (four 16-bit
// elements beside an fp32 row)
template <typename TE, int N>
__device__ __forceinline__ void load_n(const TE* p, float (&out)[N]) {
  if constexpr (sizeof(TE) == 4) {
    static_assert(N == 4, "fp32 vectors hold four elements");
    const float4 f = *reinterpret_cast<const float4*>(p);
    out[0] = f.x; out[1] = f.y; out[2] = f.z; out[3] = f.w;
  } else if constexpr (N == 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = Cvt<TE>::unpack2(w[i]);
      out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
  } else {
    static_assert(N == 4 && sizeof(TE) == 2, "8-byte vectors: four 16-bit elements");
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = Cvt<TE>::unpack2(u.x), b = Cvt<TE>::unpack2(u.y);
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
  }
}
template <typename TE, int N>
__device__ __forceinline__ void store_n(TE* p, const float (&v)[N]) {
  if constexpr (sizeof(TE) == 4) {
    static_assert(N == 4, "fp32 vectors hold four elements");
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if constexpr (N == 8) {
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = Cvt<TE>::pack2(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  } else {
    static_assert(N == 4 && sizeof(TE) == 2, "8-byte vectors: four 16-bit elements");
    uint2 u;
    u.x = Cvt<TE>::pack2(v[0], v[1]);
    u.y = Cvt<TE>::pack2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = u;
  }
}

// 16 raw bytes of a row (N = 16 / sizeof(TE) elements) as floats.  The kernels keep rows in registers in
// this raw form -- half the registers of the unpacked floats for 16-bit data -- and unpack where they use them.
template <typename TE, int N>
__device__ __forceinline__ void unpack_raw(const uint4& u, float (&out)[N]) {
  if constexpr (sizeof(TE) == 4) {
    out[0] = __uint_as_float(u.x); out[1] = __uint_as_float(u.y); out[2] = __uint_as_float(u.z); out[3] = __uint_as_float(u.w);
  } else {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = Cvt<TE>::unpack2(w[i]);
      out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
  }
}

// Makes the compiler forget what it knows about a raw vector, so that values unpacked from it earlier are
// not kept alive (as twice as many registers) for the next use but unpacked again.
__device__ __forceinline__ void forget(uint4& u) { asm volatile("" : "+r"(u.x), "+r"(u.y), "+r"(u.z), "+r"(u.w)); }
__device__ __forceinline__ void forget(uint2& u) { asm volatile("" : "+r"(u.x), "+r"(u.y)); }

// weight elements i..i+N-1 as floats, for either weight dtype, with vector loads (w is 16-byte aligned, i a
// multiple of N)
template <typename TW, int N>
__device__ __forceinline__ void load_w(const TW* w, int i, float (&out)[N]) {
  if constexpr (sizeof(TW) == 4) {
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(w + i + j));
      out[j] = f.x; out[j + 1] = f.y; out[j + 2] = f.z; out[j + 3] = f.w;
    }
  } else {
    static_assert(N == 8, "16-bit weights go with 16-bit rows");
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(w + i));
    unpack_raw<TW, 8>(u, out);
  }
}

// Rows a warp works on at a time (measured on B200 at 32768 x 768: two rows and three CTAs per SM reach the
// speed of a plain copy; four rows or more CTAs are slower).
__host__ __device__ constexpr int rows_per_iter(int nv) { return nv <= 6 ? 2 : 1; }

struct FwdParams {
  const void* x; const void* branch; const void* w; void* x_out; void* y; float* rstd;
  int64_t x_stride, branch_stride, xout_stride, y_stride, rows;
  int d; float eps;
};

// T: dtype of x (and x_out); TY: dtype of y (and of branch); NV: vectors of N = 16/sizeof(T) elements per lane.
template <typename T, typename TW, typename TY, int NV, bool ADD>
__global__ void __launch_bounds__(kThreads, 3)
rmsnorm_fwd_kernel(const FwdParams p) {
  constexpr int N = Vec<T>::N;
  constexpr int R = rows_per_iter(NV);
  const T* __restrict__ x = static_cast<const T*>(p.x);
  const TY* __restrict__ br = static_cast<const TY*>(p.branch);
  const TW* __restrict__ w = static_cast<const TW*>(p.w);
  T* __restrict__ xo = static_cast<T*>(p.x_out);
  TY* __restrict__ y = static_cast<TY*>(p.y);
  const int lane = threadIdx.x & 31;
  const int nvec = p.d / N;                            // vectors per row
  const float inv_d = 1.f / (float)p.d;
  const int64_t warp0 = ((int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5)) * R;
  const int64_t step = (int64_t)gridDim.x * kWarps * R;
  for (int64_t r0 = warp0; r0 < p.rows; r0 += step) {
    uint4 raw[R][NV];                                  // ADD: already x + branch, as fp32 bits
    // every load of the R rows first: this is what keeps enough bytes in flight
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int64_t r = r0 + i;
#pragma unroll
      for (int it = 0; it < NV; ++it) {
        const int vi = it * 32 + lane;
        raw[i][it] = make_uint4(0u, 0u, 0u, 0u);
        if (r < p.rows && vi < nvec) {
          raw[i][it] = *reinterpret_cast<const uint4*>(x + r * p.x_stride + vi * N);
          if constexpr (ADD) {
            float a[N], b[N];
            unpack_raw<T, N>(raw[i][it], a);
            load_n<TY, N>(br + r * p.branch_stride + vi * N, b);
            raw[i][it] = make_uint4(__float_as_uint(a[0] + b[0]), __float_as_uint(a[1] + b[1]),
                                    __float_as_uint(a[2] + b[2]), __float_as_uint(a[3] + b[3]));
          }
        }
      }
    }
    float ss[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      ss[i] = 0.f;
#pragma unroll
      for (int it = 0; it < NV; ++it) {
        float v[N];
        unpack_raw<T, N>(raw[i][it], v);
#pragma unroll
        for (int j = 0; j < N; ++j) ss[i] += v[j] * v[j];
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int it = 0; it < NV; ++it) forget(raw[i][it]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int i = 0; i < R; ++i) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
    float inv[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      inv[i] = rsqrtf(ss[i] * inv_d + p.eps);
      if (p.rstd && lane == 0 && r0 + i < p.rows) p.rstd[r0 + i] = inv[i];
    }
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int vi = it * 32 + lane;
      if (vi < nvec) {
        float wv[N];
        load_w<TW, N>(w, vi * N, wv);                  // once per column block, for all R rows
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int64_t r = r0 + i;
          if (r < p.rows) {
            float v[N], o[N];
            unpack_raw<T, N>(raw[i][it], v);
            if constexpr (ADD) *reinterpret_cast<uint4*>(xo + r * p.xout_stride + vi * N) = raw[i][it];
#pragma unroll
            for (int j = 0; j < N; ++j) o[j] = v[j] * inv[i] * wv[j];
            store_n<TY, N>(y + r * p.y_stride + vi * N, o);
          }
        }
      }
    }
  }
}

// Rows wider than the largest register tile: two passes over x (forward only, no fused add).
template <typename T, typename TW, typename TY>
__global__ void __launch_bounds__(kThreads)
rmsnorm_fwd_wide_kernel(const FwdParams p) {
  constexpr int N = Vec<T>::N;
  const T* __restrict__ x = static_cast<const T*>(p.x);
  const TW* __restrict__ w = static_cast<const TW*>(p.w);
  TY* __restrict__ y = static_cast<TY*>(p.y);
  const int lane = threadIdx.x & 31;
  const int nvec = p.d / N;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarps;
  for (int64_t r = warp0; r < p.rows; r += nwarps) {
    const T* xr = x + r * p.x_stride;
    float ss = 0.f;
    for (int vi = lane; vi < nvec; vi += 32) {
      float t[N];
      load_n<T, N>(xr + vi * N, t);
#pragma unroll
      for (int j = 0; j < N; ++j) ss += t[j] * t[j];
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)p.d + p.eps);
    if (p.rstd && lane == 0) p.rstd[r] = inv;
    TY* yr = y + r * p.y_stride;
    for (int vi = lane; vi < nvec; vi += 32) {
      float t[N], wv[N], o[N];
      load_n<T, N>(xr + vi * N, t);
      load_w<TW, N>(w, vi * N, wv);
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = t[j] * inv * wv[j];
      store_n<TY, N>(yr + vi * N, o);
    }
  }
}

// rows a warp of the backward works on at a time: one, with the next one prefetched (raw x and dy tiles of both
// plus the fp32 dw accumulators must fit 128 registers so that two CTAs share an SM)
__host__ __device__ constexpr int bwd_rows_per_iter(int elems_per_lane) { return 1; }

template <size_t BYTES> struct GradRaw { using type = uint4; };
template <> struct GradRaw<8> { using type = uint2; };
template <typename TY, int N>
__device__ __forceinline__ void unpack_graw(const uint4& u, float (&out)[N]) { unpack_raw<TY, N>(u, out); }
template <typename TY, int N>
__device__ __forceinline__ void unpack_graw(const uint2& u, float (&out)[N]) {
  static_assert(N == 4 && sizeof(TY) == 2, "8-byte vectors: four 16-bit elements");
  const float2 a = Cvt<TY>::unpack2(u.x), b = Cvt<TY>::unpack2(u.y);
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}

struct BwdParams {
  const void* x; const void* w; const void* dy; const float* rstd; const void* g_add;
  void* dx; void* d_branch; float* partial;
  int64_t x_stride, dy_stride, gadd_stride, dx_stride, dbranch_stride, rows;
  int d; float eps;
};

// dx = rstd * (g - xhat * mean(g * xhat)) [+ g_add],  g = dy * w,  xhat = x * rstd
// dw[c] = sum_rows dy * xhat.  ADD: g_add (dtype T, may be NULL at run time) is the gradient reaching the
// normalised tensor from elsewhere; d_branch (dtype TY, may be NULL) receives the same sum rounded to 16 bits.
template <typename T, typename TW, typename TY, int NV, bool ADD>
__global__ void __launch_bounds__(kThreads, 2)
rmsnorm_bwd_kernel(const BwdParams p) {
  constexpr int N = Vec<T>::N;
  constexpr int R = bwd_rows_per_iter(NV * N);
  extern __shared__ float s_dw[];                      // [kWarps][d]
  const T* __restrict__ x = static_cast<const T*>(p.x);
  const TW* __restrict__ w = static_cast<const TW*>(p.w);
  const TY* __restrict__ dy = static_cast<const TY*>(p.dy);
  const T* __restrict__ ga = static_cast<const T*>(p.g_add);
  T* __restrict__ dx = static_cast<T*>(p.dx);
  TY* __restrict__ db = static_cast<TY*>(p.d_branch);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = p.d / N;
  const float inv_d = 1.f / (float)p.d;
  const int64_t warp0 = ((int64_t)blockIdx.x * kWarps + warp) * R;
  const int64_t step = (int64_t)gridDim.x * kWarps * R;
  using GRaw = typename GradRaw<sizeof(TY) * N>::type;  // dy vector: 16 bytes, or 8 (16-bit dy beside an fp32 x)
  float acc[NV][N];
#pragma unroll
  for (int it = 0; it < NV; ++it)
#pragma unroll
    for (int j = 0; j < N; ++j) acc[it][j] = 0.f;
  // The rows of the NEXT iteration are fetched while the current ones are worked on (the grid-stride loop is
  // otherwise one dependent chain per warp: load, reduce, store, load ...), register tile permitting.
  // (an fp32 row of more than 16 elements per lane plus its prefetched successor no longer fits 128 registers:
  // the spills cost the fused-add backward 5 % at d = 768)
  constexpr bool kPrefetch = NV * N <= (sizeof(T) == 4 ? 16 : 24);
  auto load_rows = [&](int64_t r0, uint4 (&xr)[R][NV], GRaw (&gr)[R][NV]) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int64_t r = r0 + i;
#pragma unroll
      for (int it = 0; it < NV; ++it) {
        const int vi = it * 32 + lane;
        xr[i][it] = make_uint4(0u, 0u, 0u, 0u);
        gr[i][it] = GRaw{};
        if (r < p.rows && vi < nvec) {
          xr[i][it] = *reinterpret_cast<const uint4*>(x + r * p.x_stride + vi * N);
          gr[i][it] = *reinterpret_cast<const GRaw*>(dy + r * p.dy_stride + vi * N);
        }
      }
    }
  };
  uint4 xraw[R][NV], xnext[kPrefetch ? R : 1][kPrefetch ? NV : 1];
  GRaw graw[R][NV], gnext[kPrefetch ? R : 1][kPrefetch ? NV : 1];
  if constexpr (kPrefetch) load_rows(warp0, xraw, graw);
  for (int64_t r0 = warp0; r0 < p.rows; r0 += step) {
    if constexpr (kPrefetch) load_rows(r0 + step, xnext, gnext);
    else load_rows(r0, xraw, graw);
    float inv[R], dot[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int64_t r = r0 + i;
      if (p.rstd) {
        inv[i] = r < p.rows ? p.rstd[r] : 0.f;
      } else {
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < NV; ++it) {
          float xv[N];
          unpack_raw<T, N>(xraw[i][it], xv);
#pragma unroll
          for (int j = 0; j < N; ++j) ss += xv[j] * xv[j];
        }
        inv[i] = rsqrtf(warp_sum(ss) * inv_d + p.eps);
      }
      dot[i] = 0.f;
    }
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int vi = it * 32 + lane;
      float wv[N];
#pragma unroll
      for (int j = 0; j < N; ++j) wv[j] = 0.f;
      if (vi < nvec) load_w<TW, N>(w, vi * N, wv);     // once per column block, for all R rows
#pragma unroll
      for (int i = 0; i < R; ++i) {
        float xv[N], gv[N];
        unpack_raw<T, N>(xraw[i][it], xv);
        unpack_graw<TY, N>(graw[i][it], gv);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float xh = xv[j] * inv[i];
          acc[it][j] += gv[j] * xh;                    // rows past the end carry zeros
          dot[i] += gv[j] * wv[j] * xh;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int it = 0; it < NV; ++it) { forget(xraw[i][it]); forget(graw[i][it]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int i = 0; i < R; ++i) dot[i] += __shfl_xor_sync(0xffffffffu, dot[i], o);
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int vi = it * 32 + lane;
      if (vi < nvec) {
        float wv[N];
        load_w<TW, N>(w, vi * N, wv);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int64_t r = r0 + i;
          if (r < p.rows) {
            float xv[N], gv[N], o[N];
            unpack_raw<T, N>(xraw[i][it], xv);
            unpack_graw<TY, N>(graw[i][it], gv);
            const float dm = dot[i] * inv_d;
#pragma unroll
            for (int j = 0; j < N; ++j) o[j] = inv[i] * (gv[j] * wv[j] - xv[j] * inv[i] * dm);
            if constexpr (ADD) {
              if (ga) {
                float g2[N];
                load_n<T, N>(ga + r * p.gadd_stride + vi * N, g2);
#pragma unroll
                for (int j = 0; j < N; ++j) o[j] += g2[j];
              }
              if (db) store_n<TY, N>(db + r * p.dbranch_stride + vi * N, o);
            }
            store_n<T, N>(dx + r * p.dx_stride + vi * N, o);
          }
        }
      }
    }
    if constexpr (kPrefetch) {
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int it = 0; it < NV; ++it) { xraw[i][it] = xnext[i][it]; graw[i][it] = gnext[i][it]; }
    }
  }
#pragma unroll
  for (int it = 0; it < NV; ++it) {
    const int vi = it * 32 + lane;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < N; ++j) s_dw[warp * p.d + vi * N + j] = acc[it][j];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < p.d; c += kThreads) {
    float t = 0.f;
#pragma unroll
    for (int wi = 0; wi < kWarps; ++wi) t += s_dw[wi * p.d + c];
    p.partial[(int64_t)blockIdx.x * p.d + c] = t;
  }
}

// The same backward for wide fp32 rows (more than 16 elements per lane: d = 768, 1024 in the training layout, an
// fp32 residual stream with a 16-bit dy).  One warp per row needs the raw x, dy and g_add of the row plus the dw
// accumulators in registers at once, which at 128 registers leaves no room for a second row in flight; here TWO
// warps share a row (NVH vectors per lane each), twelve warps a CTA, so that 24 warps per SM each have a whole
// row's loads outstanding.  The two halves of the row's dot product meet through shared memory and a
// 64-thread named barrier (double-buffered slot, one barrier per row).
constexpr int kSplitWarps = 12;
constexpr int kSplitThreads = kSplitWarps * 32;

template <typename TW, typename TY, int NVH, bool ADD>
__global__ void __launch_bounds__(kSplitThreads, 2)
rmsnorm_bwd_split_kernel(const BwdParams p) {
  constexpr int N = 4;
  extern __shared__ float s_dw[];                      // [kSplitWarps][d], then the pairs' exchange slots
  float* s_red = s_dw + (size_t)kSplitWarps * p.d;     // [2 phases][2 quantities][kSplitWarps]
  const float* __restrict__ x = static_cast<const float*>(p.x);
  const TW* __restrict__ w = static_cast<const TW*>(p.w);
  const TY* __restrict__ dy = static_cast<const TY*>(p.dy);
  const float* __restrict__ ga = static_cast<const float*>(p.g_add);
  float* __restrict__ dx = static_cast<float*>(p.dx);
  TY* __restrict__ db = static_cast<TY*>(p.d_branch);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = warp >> 1, half = warp & 1;
  const int nvec = p.d / N;
  const float inv_d = 1.f / (float)p.d;
  float acc[NVH][N];
#pragma unroll
  for (int it = 0; it < NVH; ++it)
#pragma unroll
    for (int j = 0; j < N; ++j) acc[it][j] = 0.f;
  auto pair_sum = [&](float v, int phase, int q) {     // sum of v over the two warps of the pair
    v = warp_sum(v);
    float* slot = s_red + ((phase * 2 + q) * kSplitWarps);
    if (lane == 0) slot[warp] = v;
    asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
    return slot[2 * pair] + slot[2 * pair + 1];
  };
  int phase = 0;
  const int64_t step = (int64_t)gridDim.x * (kSplitWarps / 2);
  for (int64_t r = (int64_t)blockIdx.x * (kSplitWarps / 2) + pair; r < p.rows; r += step, phase ^= 1) {
    uint4 xr[NVH];
    uint2 gr[NVH];
    [[maybe_unused]] float4 ar[NVH];
#pragma unroll
    for (int it = 0; it < NVH; ++it) {                 // everything the row needs, requested at once
      const int vi = (half * NVH + it) * 32 + lane;
      xr[it] = make_uint4(0u, 0u, 0u, 0u);
      gr[it] = make_uint2(0u, 0u);
      if constexpr (ADD) ar[it] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (vi < nvec) {
        xr[it] = *reinterpret_cast<const uint4*>(x + r * p.x_stride + vi * N);
        gr[it] = *reinterpret_cast<const uint2*>(dy + r * p.dy_stride + vi * N);
        if constexpr (ADD) {
          if (ga) ar[it] = *reinterpret_cast<const float4*>(ga + r * p.gadd_stride + vi * N);
        }
      }
    }
    float inv;
    if (p.rstd) {
      inv = p.rstd[r];
    } else {
      float ss = 0.f;
#pragma unroll
      for (int it = 0; it < NVH; ++it) {
        float xv[N];
        unpack_raw<float, N>(xr[it], xv);
#pragma unroll
        for (int j = 0; j < N; ++j) ss += xv[j] * xv[j];
      }
      inv = rsqrtf(pair_sum(ss, phase, 0) * inv_d + p.eps);
    }
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < NVH; ++it) {
      const int vi = (half * NVH + it) * 32 + lane;
      float wv[N], xv[N], gv[N];
#pragma unroll
      for (int j = 0; j < N; ++j) wv[j] = 0.f;
      if (vi < nvec) load_w<TW, N>(w, vi * N, wv);
      unpack_raw<float, N>(xr[it], xv);
      unpack_graw<TY, N>(gr[it], gv);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float xh = xv[j] * inv;
        acc[it][j] += gv[j] * xh;                      // vectors past the end carry zeros
        dot += gv[j] * wv[j] * xh;
      }
    }
    const float dm = pair_sum(dot, phase, 1) * inv_d;
#pragma unroll
    for (int it = 0; it < NVH; ++it) {
      const int vi = (half * NVH + it) * 32 + lane;
      if (vi < nvec) {
        float wv[N], xv[N], gv[N], o[N];
        load_w<TW, N>(w, vi * N, wv);
        unpack_raw<float, N>(xr[it], xv);
        unpack_graw<TY, N>(gr[it], gv);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = inv * (gv[j] * wv[j] - xv[j] * inv * dm);
        if constexpr (ADD) {
          o[0] += ar[it].x; o[1] += ar[it].y; o[2] += ar[it].z; o[3] += ar[it].w;
          if (db) store_n<TY, N>(db + r * p.dbranch_stride + vi * N, o);
        }
        store_n<float, N>(dx + r * p.dx_stride + vi * N, o);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < NVH; ++it) {
    const int vi = (half * NVH + it) * 32 + lane;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < N; ++j) s_dw[warp * p.d + vi * N + j] = acc[it][j];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < p.d; c += kSplitThreads) {
    const int h = (c / N) / (32 * NVH);                // the half of every pair that owns this column
    float t = 0.f;
#pragma unroll
    for (int pi = 0; pi < kSplitWarps / 2; ++pi) t += s_dw[(2 * pi + h) * p.d + c];
    p.partial[(int64_t)blockIdx.x * p.d + c] = t;
  }
}

// dw[c] = sum over the partial rows, in a fixed order: a CTA takes 32 columns, its 32 x 32 threads each add
// every 32nd partial row of one column (coalesced 128-byte reads, short independent chains), and the 32
// sub-sums of a column are added in index order.
__global__ void __launch_bounds__(1024)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nparts, int d) {
  __shared__ float sub[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float t = 0.f;
  if (c < d)
    for (int p = threadIdx.y; p < nparts; p += 32) t += partial[(int64_t)p * d + c];
  sub[threadIdx.y][threadIdx.x] = t;
  __syncthreads();
  if (threadIdx.y == 0 && c < d) {
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < 32; ++g) sum += sub[g][threadIdx.x];
    dw[c] = sum;
  }
}

// y / dy may be 16-bit next to an fp32 x (autocast's layout); otherwise they have x's dtype
int check_kind(const char* who, int kind, int x_dtype) {
  if (kind == ULM_Y_SAME) return ULM_OK;
  if (kind != ULM_Y_F16 && kind != ULM_Y_BF16) return fail(ULM_ERR_ARG, "%s: bad y/dy kind %d", who, kind);
  if (x_dtype != ULM_F32) return fail(ULM_ERR_ARG, "%s: a 16-bit y/dy kind needs an fp32 x", who);
  return ULM_OK;
}

// upper bound on the CTAs of the backward = partial rows the caller provides
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
  if ((reinterpret_cast<uintptr_t>(x) & 15) || !w || (reinterpret_cast<uintptr_t>(w) & 15))
    return fail(ULM_ERR_ARG, "%s: x and w must be 16-byte aligned, w non-null", who);
  return ULM_OK;
}

// smallest instantiated register tile that holds `need` vectors per lane (0: none does)
int pick_nv(int need) {
  for (int nv : {1, 2, 3, 4, 6, 8}) if (need <= nv) return nv;
  return 0;
}

template <typename T, typename TW, typename TY, bool ADD>
void launch_fwd(const FwdParams& p, int nv, cudaStream_t st) {
  auto go = [&](auto kern, int nv_) {
    const int64_t per_cta = (int64_t)kWarps * rows_per_iter(nv_);
    int64_t blocks = (p.rows + per_cta - 1) / per_cta;
    if (blocks > 8 * kNumSMs) blocks = 8 * kNumSMs;
    kern<<<(unsigned)blocks, kThreads, 0, st>>>(p);
  };
  switch (nv) {
    case 1: go(rmsnorm_fwd_kernel<T, TW, TY, 1, ADD>, 1); break;
    case 2: go(rmsnorm_fwd_kernel<T, TW, TY, 2, ADD>, 2); break;
    case 3: go(rmsnorm_fwd_kernel<T, TW, TY, 3, ADD>, 3); break;
    case 4: go(rmsnorm_fwd_kernel<T, TW, TY, 4, ADD>, 4); break;
    case 6: go(rmsnorm_fwd_kernel<T, TW, TY, 6, ADD>, 6); break;
    case 8: go(rmsnorm_fwd_kernel<T, TW, TY, 8, ADD>, 8); break;
    default:
      if constexpr (!ADD) {
        int64_t blocks = (p.rows + kWarps - 1) / kWarps;
        if (blocks > 8 * kNumSMs) blocks = 8 * kNumSMs;
        rmsnorm_fwd_wide_kernel<T, TW, TY><<<(unsigned)blocks, kThreads, 0, st>>>(p);
      }
  }
}

template <typename T, typename TW, typename TY, bool ADD>
void launch_bwd(const BwdParams& p, int nv, int64_t blocks, size_t smem, cudaStream_t st) {
  if constexpr (sizeof(T) == 4 && sizeof(TY) == 2) {
    if (nv == 6 || nv == 8) {                          // wide fp32 rows: two warps per row
      const int64_t want = (p.rows + kSplitWarps / 2 - 1) / (kSplitWarps / 2);
      const int64_t grid = want < blocks ? want : blocks;       // never more CTAs than partial rows were provided
      const size_t sm = ((size_t)kSplitWarps * p.d + 4 * kSplitWarps) * sizeof(float);
      auto launch = [&](auto kern) {
        if (sm > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        kern<<<(unsigned)grid, kSplitThreads, sm, st>>>(p);
      };
      if (nv == 6) launch(rmsnorm_bwd_split_kernel<TW, TY, 3, ADD>); else launch(rmsnorm_bwd_split_kernel<TW, TY, 4, ADD>);
      return;
    }
  }
  auto go = [&](auto kern) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<(unsigned)blocks, kThreads, smem, st>>>(p);
  };
  switch (nv) {
    case 1: go(rmsnorm_bwd_kernel<T, TW, TY, 1, ADD>); break;
    case 2: go(rmsnorm_bwd_kernel<T, TW, TY, 2, ADD>); break;
    case 3: go(rmsnorm_bwd_kernel<T, TW, TY, 3, ADD>); break;
    case 4: go(rmsnorm_bwd_kernel<T, TW, TY, 4, ADD>); break;
    case 6: go(rmsnorm_bwd_kernel<T, TW, TY, 6, ADD>); break;
    default: go(rmsnorm_bwd_kernel<T, TW, TY, 8, ADD>); break;
  }
}

}  // namespace
}  // namespace ulm

extern "C" int64_t ulm_rmsnorm_bwd_partial_rows(int64_t rows) { return ulm::bwd_grid(rows); }

extern "C" int ulm_rmsnorm_fwd(const ulm_rmsnorm_fwd_args* a) {
  using namespace ulm;
  const char* who = "ulm_rmsnorm_fwd";
  if (!a) return fail(ULM_ERR_ARG, "%s: null args", who);
  int rc = check_common(who, a->x_dtype, a->w_dtype, a->d, a->rows, a->x, a->w, a->x_stride, a->y_stride, 0);
  if (rc) return rc;
  if ((rc = check_kind(who, a->y_kind, a->x_dtype))) return rc;
  const bool add = a->branch != nullptr;
  if (add) {
    if (a->x_dtype != ULM_F32 || a->y_kind == ULM_Y_SAME)
      return fail(ULM_ERR_ARG, "%s: the fused residual add takes an fp32 x and a 16-bit branch and y", who);
    if (!a->x_out || (reinterpret_cast<uintptr_t>(a->x_out) & 15) || (reinterpret_cast<uintptr_t>(a->branch) & 7) ||
        a->branch_stride % 4 || a->xout_stride % 4)
      return fail(ULM_ERR_ARG, "%s: x_out must be 16-byte aligned, branch 8-byte aligned, their row strides multiples of 4", who);
  }
  if (a->rows == 0) return ULM_OK;
  if (!a->y || (reinterpret_cast<uintptr_t>(a->y) & 15)) return fail(ULM_ERR_ARG, "%s: y must be 16-byte aligned", who);
  const int n = a->x_dtype == ULM_F32 ? 4 : 8;
  const int nv = pick_nv((a->d / n + 31) / 32);
  if (add && !nv) return fail(ULM_ERR_TOO_LARGE, "%s: the fused residual add takes rows of at most %d elements", who, 8 * 32 * n);
  FwdParams p{a->x, a->branch, a->w, a->x_out, a->y, a->rstd, a->x_stride, a->branch_stride, a->xout_stride, a->y_stride,
              a->rows, a->d, a->eps};
  cudaStream_t st = (cudaStream_t)a->stream;
  if (a->x_dtype == ULM_F32 && a->y_kind == ULM_Y_F16) {
    if (add) launch_fwd<float, float, __half, true>(p, nv, st); else launch_fwd<float, float, __half, false>(p, nv, st);
  } else if (a->x_dtype == ULM_F32 && a->y_kind == ULM_Y_BF16) {
    if (add) launch_fwd<float, float, __nv_bfloat16, true>(p, nv, st); else launch_fwd<float, float, __nv_bfloat16, false>(p, nv, st);
  } else if (a->x_dtype == ULM_F32) {
    launch_fwd<float, float, float, false>(p, nv, st);
  } else if (a->x_dtype == ULM_F16) {
    if (a->w_dtype == ULM_F32) launch_fwd<__half, float, __half, false>(p, nv, st); else launch_fwd<__half, __half, __half, false>(p, nv, st);
  } else {
    if (a->w_dtype == ULM_F32) launch_fwd<__nv_bfloat16, float, __nv_bfloat16, false>(p, nv, st);
    else launch_fwd<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, false>(p, nv, st);
  }
  return check_launch(who);
}

namespace ulm {
// Shared by the entry points that differ only in where `partial` lives.
int rmsnorm_bwd_launch(const ulm_rmsnorm_bwd_args* a, float* partial, const char* who) {
  int rc = check_common(who, a->x_dtype, a->w_dtype, a->d, a->rows, a->x, a->w, a->x_stride, a->dy_stride, a->dx_stride);
  if (rc) return rc;
  if ((rc = check_kind(who, a->dy_kind, a->x_dtype))) return rc;
  if (a->d > kMaxD) return fail(ULM_ERR_TOO_LARGE, "%s: d=%d exceeds %d", who, a->d, kMaxD);
  if (!a->dy || !a->dx || !a->dw || !partial) return fail(ULM_ERR_ARG, "%s: null tensor", who);
  const uintptr_t dy_mask = a->dy_kind == ULM_Y_SAME ? 15 : 7;      // four 16-bit elements beside an fp32 vector
  if ((reinterpret_cast<uintptr_t>(a->dy) & dy_mask) || (reinterpret_cast<uintptr_t>(a->dx) & 15))
    return fail(ULM_ERR_ARG, "%s: dy and dx must be 16-byte aligned (a 16-bit dy beside an fp32 x: 8-byte)", who);
  const bool add = a->g_add != nullptr || a->d_branch != nullptr;
  if (add) {
    if (a->x_dtype != ULM_F32 || a->dy_kind == ULM_Y_SAME)
      return fail(ULM_ERR_ARG, "%s: the fused gradient add takes an fp32 x and a 16-bit dy", who);
    if ((reinterpret_cast<uintptr_t>(a->g_add) & 15) || (reinterpret_cast<uintptr_t>(a->d_branch) & 7) ||
        a->gadd_stride % 4 || a->dbranch_stride % 4)
      return fail(ULM_ERR_ARG, "%s: g_add must be 16-byte aligned, d_branch 8-byte aligned, their row strides multiples of 4", who);
  }
  cudaStream_t st = (cudaStream_t)a->stream;
  const int n = a->x_dtype == ULM_F32 ? 4 : 8;
  const int nv = pick_nv((a->d / n + 31) / 32);          // d <= 1024: at most 8 vectors per lane
  const int r_iter = bwd_rows_per_iter(nv * n);
  int64_t blocks = (a->rows + (int64_t)kWarps * r_iter - 1) / ((int64_t)kWarps * r_iter);
  const int64_t cap = bwd_grid(a->rows);
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const size_t smem = (size_t)kWarps * a->d * sizeof(float);
  if (a->rows > 0) {
    BwdParams p{a->x, a->w, a->dy, a->rstd, a->g_add, a->dx, a->d_branch, partial,
                a->x_stride, a->dy_stride, a->gadd_stride, a->dx_stride, a->dbranch_stride, a->rows, a->d, a->eps};
    if (a->x_dtype == ULM_F32 && a->dy_kind == ULM_Y_F16) {
      if (add) launch_bwd<float, float, __half, true>(p, nv, blocks, smem, st); else launch_bwd<float, float, __half, false>(p, nv, blocks, smem, st);
    } else if (a->x_dtype == ULM_F32 && a->dy_kind == ULM_Y_BF16) {
      if (add) launch_bwd<float, float, __nv_bfloat16, true>(p, nv, blocks, smem, st);
      else launch_bwd<float, float, __nv_bfloat16, false>(p, nv, blocks, smem, st);
    } else if (a->x_dtype == ULM_F32) {
      launch_bwd<float, float, float, false>(p, nv, blocks, smem, st);
    } else if (a->x_dtype == ULM_F16) {
      if (a->w_dtype == ULM_F32) launch_bwd<__half, float, __half, false>(p, nv, blocks, smem, st);
      else launch_bwd<__half, __half, __half, false>(p, nv, blocks, smem, st);
    } else {
      if (a->w_dtype == ULM_F32) launch_bwd<__nv_bfloat16, float, __nv_bfloat16, false>(p, nv, blocks, smem, st);
      else launch_bwd<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, false>(p, nv, blocks, smem, st);
    }
    rc = check_launch(who);
    if (rc) return rc;
  }
  rmsnorm_dw_reduce_kernel<<<(a->d + 31) / 32, dim3(32, 32), 0, st>>>(partial, a->dw, a->rows > 0 ? (int)blocks : 0, a->d);
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
  // Every element the reduction reads (one row of d floats per launched CTA) is written by the backward
  // kernel of this same call first, so nothing left over from an earlier call is used
  // and nothing needs clearing.
  return rmsnorm_bwd_launch(a, scratch, who);
}
