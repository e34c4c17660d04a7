// Fused RoPE forward / adjoint for head_dim 64 (sm_100a).
//
// The arithmetic (rope_math.cuh) follows the reference's eager path
// (train.py:1914-1918) as its fused kernel reproduces it
// (csrc/flash_attn_v100/fast_ops.cu:31-68).
// HBM-bound: each thread owns 8 columns of the low half and their 8 partners in
// the high half of one row (two 16-byte loads, two 16-byte stores), so a row is
// read and written exactly once; q and k go through the same launch.  Either of
// the two may be absent (NULL): the attention forward rotates Q itself when it is
// given the tables, and then only K needs this kernel.
#include "rope_math.cuh"

namespace ulm {
namespace {

constexpr int kThreads = 256;   // 4 threads per row -> 64 rows per CTA

template <typename T, bool BWD>
__global__ void __launch_bounds__(kThreads)
rope_kernel(const T* __restrict__ q, const T* __restrict__ k, T* __restrict__ qo, T* __restrict__ ko,
            const float* __restrict__ cs, const float* __restrict__ sn,
            int64_t q_sb, int64_t q_sh, int64_t q_ss, int64_t k_sb, int64_t k_sh, int64_t k_ss,
            int64_t qo_sb, int64_t qo_sh, int64_t qo_ss, int64_t ko_sb, int64_t ko_sh, int64_t ko_ss,
            int64_t cs_stride, int64_t sn_stride, int B, int H, int S, int h_inner, int first) {
  const int64_t rows = (int64_t)B * H * S;
  const int64_t row = (int64_t)blockIdx.x * (kThreads / 4) + (threadIdx.x >> 2);
  const int which = first + (int)blockIdx.y;          // 0 = q, 1 = k
  if (row >= rows) return;
  int b, h, s;
  if (h_inner) {                                       // memory order (b, s, h): fused-qkv views
    h = (int)(row % H); s = (int)((row / H) % S); b = (int)(row / ((int64_t)H * S));
  } else {                                             // memory order (b, h, s)
    s = (int)(row % S); h = (int)((row / S) % H); b = (int)(row / ((int64_t)H * S));
  }
  const int d0 = (threadIdx.x & 3) * 8;               // low-half columns d0..d0+7, partners +32
  const T* src = which ? k + b * k_sb + h * k_sh + s * k_ss : q + b * q_sb + h * q_sh + s * q_ss;
  T* dst = which ? ko + b * ko_sb + h * ko_sh + s * ko_ss : qo + b * qo_sb + h * qo_sh + s * qo_ss;

  const uint4 lo = *reinterpret_cast<const uint4*>(src + d0);
  const uint4 hi = *reinterpret_cast<const uint4*>(src + d0 + 32);
  uint4 olo, ohi;
  rope_vec8<T, BWD>(lo, hi, cs + (int64_t)s * cs_stride, sn + (int64_t)s * sn_stride, d0, olo, ohi);
  *reinterpret_cast<uint4*>(dst + d0) = olo;
  *reinterpret_cast<uint4*>(dst + d0 + 32) = ohi;
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
  const int64_t rows = (int64_t)a->B * a->H * a->S;
  const int64_t blocks = (rows + kThreads / 4 - 1) / (kThreads / 4);
  if (blocks > 0x7fffffffLL) return fail(ULM_ERR_TOO_LARGE, "ulm_rope: too many rows");
  dim3 grid((unsigned)blocks, (has_q ? 1u : 0u) + (has_k ? 1u : 0u));
  const int h_inner = has_q ? ((a->q_sh < a->q_ss) ? 1 : 0) : ((a->k_sh < a->k_ss) ? 1 : 0);
  const int first = has_q ? 0 : 1;
  cudaStream_t st = (cudaStream_t)a->stream;
#define ULM_ROPE_LAUNCH(T, BWD)                                                                 \
  rope_kernel<T, BWD><<<grid, kThreads, 0, st>>>(                                               \
      (const T*)a->q, (const T*)a->k, (T*)a->qo, (T*)a->ko, a->cos_tab, a->sin_tab,             \
      a->q_sb, a->q_sh, a->q_ss, a->k_sb, a->k_sh, a->k_ss, a->qo_sb, a->qo_sh, a->qo_ss,       \
      a->ko_sb, a->ko_sh, a->ko_ss, a->cos_stride, a->sin_stride, a->B, a->H, a->S, h_inner, first)
  if (a->dtype == ULM_F16) {
    if (a->backward) ULM_ROPE_LAUNCH(__half, true); else ULM_ROPE_LAUNCH(__half, false);
  } else {
    if (a->backward) ULM_ROPE_LAUNCH(__nv_bfloat16, true); else ULM_ROPE_LAUNCH(__nv_bfloat16, false);
  }
#undef ULM_ROPE_LAUNCH
  return check_launch("ulm_rope");
}
