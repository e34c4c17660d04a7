// The RoPE arithmetic shared by the stand-alone kernel (rope.cu) and the fused forms
// inside the attention kernels (rotation of the resident Q tile in the forward,
// adjoint in the dQ / dK epilogues of the backward).
//
// Math follows the reference's eager path (train.py:1914-1918) as its fused kernel
// reproduces it (csrc/flash_attn_v100/fast_ops.cu:31-68): fp32 products and sum
// WITHOUT fma contraction, one rounding to the 16-bit type.
//   fwd: out[d] = x[d] cos[d] - x[d+32] sin[d]        (d <  32)
//        out[d] = x[d] cos[d] + x[d-32] sin[d]        (d >= 32)
//   bwd: dx[d]  = g[d] cos[d] + g[d+32] sin[d+32]     (d <  32)
//        dx[d]  = g[d] cos[d] - g[d-32] sin[d-32]     (d >= 32)
// Every user feeds 16-bit inputs through the same sequence of operations, so the
// fused forms are bit-identical to the stand-alone kernel.
#pragma once

#include "common.cuh"

namespace ulm {

// One packed pair of low-half elements (columns d, d+1 with d < 32) and their partners
// (columns d+32, d+33): cl/sl = cos/sin at d, d+1; ch/sh = cos/sin at d+32, d+33.
template <typename T, bool BWD>
__device__ __forceinline__ void rope_pair(uint32_t lo_in, uint32_t hi_in, const float* cl, const float* sl,
                                          const float* ch, const float* sh, uint32_t& lo_out, uint32_t& hi_out) {
  const float2 a = Cvt<T>::unpack2(lo_in);            // x[d], d < 32
  const float2 p = Cvt<T>::unpack2(hi_in);            // x[d + 32]
  float l0, l1, h0, h1;
  if (!BWD) {
    l0 = __fadd_rn(__fmul_rn(a.x, cl[0]), __fmul_rn(-p.x, sl[0]));
    l1 = __fadd_rn(__fmul_rn(a.y, cl[1]), __fmul_rn(-p.y, sl[1]));
    h0 = __fadd_rn(__fmul_rn(p.x, ch[0]), __fmul_rn(a.x, sh[0]));
    h1 = __fadd_rn(__fmul_rn(p.y, ch[1]), __fmul_rn(a.y, sh[1]));
  } else {
    l0 = __fadd_rn(__fmul_rn(a.x, cl[0]), __fmul_rn(p.x, sh[0]));
    l1 = __fadd_rn(__fmul_rn(a.y, cl[1]), __fmul_rn(p.y, sh[1]));
    h0 = __fadd_rn(__fmul_rn(p.x, ch[0]), __fmul_rn(-a.x, sl[0]));
    h1 = __fadd_rn(__fmul_rn(p.y, ch[1]), __fmul_rn(-a.y, sl[1]));
  }
  lo_out = Cvt<T>::pack2(l0, l1);
  hi_out = Cvt<T>::pack2(h0, h1);
}

// Eight low-half columns d0..d0+7 (one 16-byte vector) and their eight partners, tables
// read from global memory (rows of `c` and `n` are this position's cos / sin rows).
template <typename T, bool BWD>
__device__ __forceinline__ void rope_vec8(const uint4& lo, const uint4& hi, const float* __restrict__ c,
                                          const float* __restrict__ n, int d0, uint4& olo, uint4& ohi) {
  float cl[8], ch[8], sl[8], sh[8];
#pragma unroll
  for (int i = 0; i < 8; i += 4) {
    *reinterpret_cast<float4*>(cl + i) = *reinterpret_cast<const float4*>(c + d0 + i);
    *reinterpret_cast<float4*>(ch + i) = *reinterpret_cast<const float4*>(c + d0 + 32 + i);
    *reinterpret_cast<float4*>(sl + i) = *reinterpret_cast<const float4*>(n + d0 + i);
    *reinterpret_cast<float4*>(sh + i) = *reinterpret_cast<const float4*>(n + d0 + 32 + i);
  }
  const uint32_t* lw = reinterpret_cast<const uint32_t*>(&lo);
  const uint32_t* hw = reinterpret_cast<const uint32_t*>(&hi);
  uint32_t* ol = reinterpret_cast<uint32_t*>(&olo);
  uint32_t* oh = reinterpret_cast<uint32_t*>(&ohi);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    rope_pair<T, BWD>(lw[i], hw[i], cl + 2 * i, sl + 2 * i, ch + 2 * i, sh + 2 * i, ol[i], oh[i]);
}

}  // namespace ulm
