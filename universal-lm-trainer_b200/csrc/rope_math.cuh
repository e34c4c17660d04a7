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

// The table values of one vector position v (low-half columns [8v, 8v+8) and their partners) held in
// registers, so that one load serves several rows of the same position (the stand-alone kernel rotates
// several heads per thread with them).
struct RopeChunk {               // 32 registers
  float4 cl[2], ch[2], sl[2], sh[2];
};
__device__ __forceinline__ void rope_load_chunk(RopeChunk& t, const float* __restrict__ c, const float* __restrict__ n, int v) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    t.cl[i] = __ldg(reinterpret_cast<const float4*>(c + 8 * v) + i);
    t.ch[i] = __ldg(reinterpret_cast<const float4*>(c + 8 * v + 32) + i);
    t.sl[i] = __ldg(reinterpret_cast<const float4*>(n + 8 * v) + i);
    t.sh[i] = __ldg(reinterpret_cast<const float4*>(n + 8 * v + 32) + i);
  }
}
template <typename T, bool BWD>
__device__ __forceinline__ void rope_apply_chunk(const RopeChunk& t, const uint4& lo, const uint4& hi, uint4& olo, uint4& ohi) {
  const float* cl = reinterpret_cast<const float*>(t.cl);
  const float* ch = reinterpret_cast<const float*>(t.ch);
  const float* sl = reinterpret_cast<const float*>(t.sl);
  const float* sh = reinterpret_cast<const float*>(t.sh);
  const uint32_t* lw = reinterpret_cast<const uint32_t*>(&lo);
  const uint32_t* hw = reinterpret_cast<const uint32_t*>(&hi);
  uint32_t* ol = reinterpret_cast<uint32_t*>(&olo);
  uint32_t* oh = reinterpret_cast<uint32_t*>(&ohi);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    rope_pair<T, BWD>(lw[i], hw[i], cl + 2 * i, sl + 2 * i, ch + 2 * i, sh + 2 * i, ol[i], oh[i]);
}

// ---------------------------------------------------------------------------
// Form used inside the attention kernels: EIGHT threads per row.  Thread `cg` (0..7) of a row
// owns low-half columns [4 cg, 4 cg + 4) and their partners [32 + 4 cg, 36 + 4 cg).  Eight
// neighbouring lanes then read one full 128-byte line of a table row per load instruction
// (a thread-per-row mapping would touch 32 different lines per instruction and make the
// load/store unit, not the arithmetic, the cost of the rotation).  The table values are held
// in registers so that their loads can be issued long before the data they multiply exists
// (the kernels prefetch them while they wait for a barrier).
// ---------------------------------------------------------------------------
struct RopeQuad {                // 16 registers
  float4 cl, ch, sl, sh;         // cos / sin of the four low columns and of their partners
};
__device__ __forceinline__ void rope_load_quad(RopeQuad& t, const float* __restrict__ c, const float* __restrict__ n, int cg) {
  t.cl = __ldg(reinterpret_cast<const float4*>(c + 4 * cg));
  t.ch = __ldg(reinterpret_cast<const float4*>(c + 32 + 4 * cg));
  t.sl = __ldg(reinterpret_cast<const float4*>(n + 4 * cg));
  t.sh = __ldg(reinterpret_cast<const float4*>(n + 32 + 4 * cg));
}
// lo / hi: the four low columns and their four partners as two packed pairs each
template <typename T, bool BWD>
__device__ __forceinline__ void rope_apply_quad(const RopeQuad& t, const uint2& lo, const uint2& hi, uint2& olo, uint2& ohi) {
  const float* cl = reinterpret_cast<const float*>(&t.cl);
  const float* ch = reinterpret_cast<const float*>(&t.ch);
  const float* sl = reinterpret_cast<const float*>(&t.sl);
  const float* sh = reinterpret_cast<const float*>(&t.sh);
  rope_pair<T, BWD>(lo.x, hi.x, cl, sl, ch, sh, olo.x, ohi.x);
  rope_pair<T, BWD>(lo.y, hi.y, cl + 2, sl + 2, ch + 2, sh + 2, olo.y, ohi.y);
}

// Byte offset, inside a tile of 128-byte rows laid out with the 128-byte swizzle (16-byte chunk c of
// row r sits at chunk position c ^ (r & 7) -- what TMA writes and what the kernels' own staging tiles
// use), of the 8 bytes holding 16-bit columns [4 q, 4 q + 4) of row r (q = 0..15).
__device__ __forceinline__ uint32_t swz_quad_offset(int r, int q) {
  return (uint32_t)(r * 128 + ((((q >> 1) ^ (r & 7))) << 4) + ((q & 1) << 3));
}

}  // namespace ulm
