// Fused RoPE forward / adjoint for head_dim 64 (sm_100a).
//
// The arithmetic (rope_math.cuh) follows the reference's eager path
// (train.py:1914-1918) as its fused kernel reproduces it
// (csrc/flash_attn_v100/fast_ops.cu:31-68).
// HBM-bound: each thread owns 8 columns of the low half and their 8 partners in
// the high half of a row (two 16-byte loads, two 16-byte stores), so a row is
// read and written exactly once; q and k go through the same launch.  Either of
// the two may be absent (NULL): the attention forward rotates Q itself when it is
// given the tables, and then only K needs this kernel.
#include "rope_math.cuh"

namespace ulm {
namespace {

constexpr int kThreads = 256;   // 4 threads per (position, head group) -> 64 of them per CTA
constexpr int kHeadsPerThread = 4;

// A thread owns 8 columns of the low half and their 8 partners in the high half (two 16-byte
// vectors each way) of up to kHeadsPerThread heads of ONE position: the cos / sin values depend on
// the position only, so they are loaded once and reused for every head -- per row two 16-byte loads
// of data and two of tables instead of two and eight.
template <typename T, bool BWD>
__global__ void __launch_bounds__(kThreads)
rope_kernel(const T* __restrict__ q, const T* __restrict__ k, T* __restrict__ qo, T* __restrict__ ko,
            const float* __restrict__ cs, const float* __restrict__ sn,
            int64_t q_sb, int64_t q_sh, int64_t q_ss, int64_t k_sb, int64_t k_sh, int64_t k_ss,
            int64_t qo_sb, int64_t qo_sh, int64_t qo_ss, int64_t ko_sb, int64_t ko_sh, int64_t ko_ss,
            int64_t cs_stride, int64_t sn_stride, int B, int H, int S, int first) {
  const int hg_count = (H + kHeadsPerThread - 1) / kHeadsPerThread;
  const int64_t tasks = (int64_t)B * S * hg_count;
  const int64_t task = (int64_t)blockIdx.x * (kThreads / 4) + (threadIdx.x >> 2);
  const int which = first + (int)blockIdx.y;          // 0 = q, 1 = k
  if (task >= tasks) return;
  const int hg = (int)(task % hg_count);
  const int s = (int)((task / hg_count) % S);
  const int b = (int)(task / ((int64_t)hg_count * S));
  const int d0 = (threadIdx.x & 3) * 8;               // low-half columns d0..d0+7, partners +32
  const T* src = which ? k + b * k_sb + s * k_ss : q + b * q_sb + s * q_ss;
  T* dst = which ? ko + b * ko_sb + s * ko_ss : qo + b * qo_sb + s * qo_ss;
  const int64_t src_sh = which ? k_sh : q_sh, dst_sh = which ? ko_sh : qo_sh;
  const int h0 = hg * kHeadsPerThread;
  const int nh = H - h0 < kHeadsPerThread ? H - h0 : kHeadsPerThread;

  uint4 lo[kHeadsPerThread], hi[kHeadsPerThread];
#pragma unroll
  for (int i = 0; i < kHeadsPerThread; ++i) {
    if (i < nh) {
      lo[i] = *reinterpret_cast<const uint4*>(src + (h0 + i) * src_sh + d0);
      hi[i] = *reinterpret_cast<const uint4*>(src + (h0 + i) * src_sh + d0 + 32);
    }
  }
  RopeChunk tab;                                       // cos / sin of this position: columns d0..d0+7 and partners
  rope_load_chunk(tab, cs + (int64_t)s * cs_stride, sn + (int64_t)s * sn_stride, d0 >> 3);
#pragma unroll
  for (int i = 0; i < kHeadsPerThread; ++i) {
    if (i < nh) {
      uint4 olo, ohi;
      rope_apply_chunk<T, BWD>(tab, lo[i], hi[i], olo, ohi);
      *reinterpret_cast<uint4*>(dst + (h0 + i) * dst_sh + d0) = olo;
      *reinterpret_cast<uint4*>(dst + (h0 + i) * dst_sh + d0 + 32) = ohi;
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
bool mult8(int64_t a, int64_t b, int64_t c) { return (a % 8 == 0) && (b % 8 == 0) && (c % 8 == 0); }

}  // namespace
}  // namespace ulm

extern "C" int ulm_rope(const ulm_rope_args* a) {
  using namespace ulm;
  if (!a) return fail(ULM_ERR_ARG, "ulm_rope: null args");
  if (a->dtype != ULM_F16 && a->dtype != ULM_BF16) return fail(ULM_ERR_ARG, "ulm_rope: dtype must be f16 or bf16");
  if (a->B < 0 || a->H < 0 || a->S < 0) return fail(ULM_ERR_ARG, "ulm_rope: negative size");
  if (a->B == 0 || a->H == 0 || a->S == 0) return ULM_OK;
  const bool has_q = a->q || a->qo, has_k = a->k || a->ko;
  if (!has_q && !has_k) return ULM_OK;
  if ((has_q && (!a->q || !a->qo)) || (has_k && (!a->k || !a->ko)) || !a->cos_tab || !a->sin_tab)
    return fail(ULM_ERR_ARG, "ulm_rope: null tensor");
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->qo) || !aligned16(a->ko) ||
      !aligned16(a->cos_tab) || !aligned16(a->sin_tab))
    return fail(ULM_ERR_ARG, "ulm_rope: base pointers must be 16-byte aligned");
  if ((has_q && (!mult8(a->q_sb, a->q_sh, a->q_ss) || !mult8(a->qo_sb, a->qo_sh, a->qo_ss))) ||
      (has_k && (!mult8(a->k_sb, a->k_sh, a->k_ss) || !mult8(a->ko_sb, a->ko_sh, a->ko_ss))))
    return fail(ULM_ERR_ARG, "ulm_rope: strides must be multiples of 8 elements");
  if (a->cos_stride % 4 || a->sin_stride % 4) return fail(ULM_ERR_ARG, "ulm_rope: table row stride must be a multiple of 4 floats");
  const int64_t tasks = (int64_t)a->B * a->S * ((a->H + kHeadsPerThread - 1) / kHeadsPerThread);
  const int64_t blocks = (tasks + kThreads / 4 - 1) / (kThreads / 4);
  if (blocks > 0x7fffffffLL) return fail(ULM_ERR_TOO_LARGE, "ulm_rope: too many rows");
  dim3 grid((unsigned)blocks, (has_q ? 1u : 0u) + (has_k ? 1u : 0u));
  const int first = has_q ? 0 : 1;
  cudaStream_t st = (cudaStream_t)a->stream;
#define ULM_ROPE_LAUNCH(T, BWD)                                                                 \
  rope_kernel<T, BWD><<<grid, kThreads, 0, st>>>(                                               \
      (const T*)a->q, (const T*)a->k, (T*)a->qo, (T*)a->ko, a->cos_tab, a->sin_tab,             \
      a->q_sb, a->q_sh, a->q_ss, a->k_sb, a->k_sh, a->k_ss, a->qo_sb, a->qo_sh, a->qo_ss,       \
      a->ko_sb, a->ko_sh, a->ko_ss, a->cos_stride, a->sin_stride, a->B, a->H, a->S, first)
  if (a->dtype == ULM_F16) {
    if (a->backward) ULM_ROPE_LAUNCH(__half, true); else ULM_ROPE_LAUNCH(__half, false);
  } else {
    if (a->backward) ULM_ROPE_LAUNCH(__nv_bfloat16, true); else ULM_ROPE_LAUNCH(__nv_bfloat16, false);
  }
#undef ULM_ROPE_LAUNCH
  return check_launch("ulm_rope");
}
