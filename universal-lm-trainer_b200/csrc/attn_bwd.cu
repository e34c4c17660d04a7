// Causal FlashAttention-2 backward for head_dim 64 on sm_100a.
//
// Replaces fa_bwd of the reference (csrc/flash_attn_v100/flash_attn_v100_bwd.cu:
// delta pre-pass :42-61, dQ kernel :66-219, dK/dV kernel :224-428) with the same
// three-kernel split and the same formulas (flash_attn_v100_bwd.cu:10-15):
//   P = exp2(S*scale*log2e - lse*log2e),  P_d = keep * P / (1-p),
//   delta = rowsum(O * dO),  dP = dO V^T,  dS = P_d * dP - P * delta,
//   dV = P_d^T dO,  dQ = scale * dS K,  dK = scale * dS^T Q,
// P and dS rounded to the 16-bit type before their MMAs.
//
// Machine mapping (both tensor-core kernels): TMA-staged 128-byte-swizzled
// tiles, tcgen05.mma with fp32 accumulators in TMEM, the 16-bit P / dS operands
// written back into TMEM over the scores they came from and consumed as the A
// operand, so no intermediate ever touches shared or global memory.
//   dQ kernel:   CTA = 128 query rows (thread r of a group = row r = TMEM lane r),
//                walks key tiles of 64: S and dP (128x64 each) -> dS -> dQ += dS K.
//   dK/dV kernel: CTA = 128 keys (thread r = key r), walks query tiles of 64 from
//                the diagonal down, transposed view: S^T = K Q^T, dP^T = V dO^T,
//                dV += P^T dO, dK += dS^T Q.
// One CTA per SM owns all 512 TMEM columns.  Streamed tiles are independent of
// each other (the softmax statistics come from the forward pass), so tile t lives
// in score buffer pair t % kBufs and is turned into P/dS by compute group
// t % kGroups (kGW warps each).  MMAs are issued by single-purpose threads, one
// warp each: one issues S, one dP, into a buffer pair as soon as it is free; one
// (dK/dV kernel: optionally two) issues the gradient MMAs out of it as soon as the
// group has written P/dS.  tcgen05.mma blocks its issuing thread while the tensor
// pipe is busy, so a thread's barrier waits add to its MMAs' time; with one issuer
// per operand stream those waits overlap the other issuers' MMAs (one thread for
// everything left the pipe idle during every hand-off; S and dP on one thread
// cost the dQ kernel 12 %).  Each accumulator has exactly one issuer, so the
// summation order, and with it the result, is the same on every run.  All barrier
// waits are bounded (status bit + clean exit on expiry); the compute warps make the
// outcome of a wait warp-uniform by a vote, because warp-wide TMEM loads follow.
//
// Fused RoPE adjoint (template parameter ROPE): q and k are the rotated tensors; the
// dQ and dK epilogues round their result to 16 bits, hand the accumulator back, and
// then apply the adjoint rotation (rope_math.cuh: the stand-alone kernel's arithmetic
// on the same 16-bit values, so the bits are equal) before the one store each row
// gets anyway -- the separate RoPE-backward launch and its read+write of dQ and dK
// disappear.
#include <type_traits>

#include "tc.cuh"
#include "rope_math.cuh"

namespace ulm {
namespace {

using namespace tc;

constexpr int HD = 64;
constexpr int BR = 128;                 // rows owned by a CTA (queries or keys)
constexpr int BT = 64;                  // rows of the streamed tile
constexpr int kBufs = 3;                // score buffer pairs in TMEM; tile t lives in pair t % kBufs
constexpr int kGroups = 3;              // compute groups; tile t is worked on by group t % kGroups
constexpr int kGradIssuers = 1;         // dK/dV kernel: 1 = one thread issues dV and dK, 2 = one thread each
constexpr int kStages = 6;              // streamed-tile ring (must exceed kBufs)
static_assert(128 * kBufs + 128 <= 512, "score buffer pairs and accumulators must fit 512 TMEM columns");
static_assert(kBufs == kGroups, "a buffer pair's barriers are awaited by one group only: successive phases of an mbarrier must be awaited in order");
// Warps per compute group: 4 (a thread per row of the tile) or 8 (two threads per row, 32 columns each).
// A single warp issues about one instruction every two clocks on its dependent chains, so a second
// warp per sub-partition nearly halves the time a group holds a tile; measured at B=8,H=12,S=4096:
// the dK/dV kernel gains 8 % with 8, the dQ kernel (less work per element, 72 instead of 128
// registers) loses 2 %.
constexpr int kGWdQ = 4, kGWdKV = 8;
// Single-thread roles, one warp each, after the compute warps: TMA producer, the S issuer, the dP issuer,
// then kGradIssuers gradient issuers (dK/dV kernel: dV and dK on one thread or on two; the dQ kernel uses
// the first).
template <int GW>
struct Roles {
  static_assert(GW == 4 || GW == 8, "a compute group is one or two warps per TMEM sub-partition");
  static constexpr int kGroupThreads = 32 * GW;
  static constexpr int kProducerWarp = GW * kGroups, kMmaWarp = kProducerWarp + 1, kMma2Warp = kProducerWarp + 2,
                       kGradWarp = kProducerWarp + 3, kGrad2Warp = kProducerWarp + 4;
  static constexpr int kThreads = kGroupThreads * kGroups + (3 + kGradIssuers) * 32;
};
constexpr uint32_t kBigTile = BR * HD * 2;    // 16 KB
constexpr uint32_t kSmallTile = BT * HD * 2;  //  8 KB
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU;
  x ^= x >> 15; x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}
// keep mask of the reference (fa_common.cuh:30-38)
__device__ __forceinline__ bool dropout_keep(uint32_t seed_mix, int row, int col, float p) {
  uint32_t h = seed_mix ^ ((uint32_t)(row + 1) * 0x85EBCA6Bu) ^ ((uint32_t)(col + 1) * 0xC2B2AE35u);
  h = hash_u32(h);
  return ((h >> 8) * (1.0f / 16777216.0f)) >= p;
}

// TMEM column (relative to the buffer) of the packed 16-bit A operand for k-step kk: 8 columns per 16
// streamed rows.  With one thread per row the 64 rows pack into columns [0,32); with two threads per
// row each half packs over its own scores, rows [0,32) into columns [0,16) and rows [32,64) into [32,48).
template <int GW>
__device__ __forceinline__ constexpr uint32_t packed_col(int kk) {
  return GW == 8 ? (uint32_t)((kk >> 1) * 32 + (kk & 1) * 8) : (uint32_t)(kk * 8);
}

// dS of two neighbouring score elements without dropout, two-wide fp32 arithmetic (one issue slot per pair, same
// rounding as the scalar operations): p = 2^(s*scale2 - lse2), dS = p * (dP - delta); nl and nd hold the NEGATED
// statistics of the two elements.  keep(e) says whether element e is inside the mask.
template <typename Keep>
__device__ __forceinline__ void pair_ds(uint32_t s0, uint32_t s1, uint32_t dp0, uint32_t dp1, uint64_t sc2, uint64_t nl, uint64_t nd,
                                        Keep keep, float (&d)[2], float* p_out = nullptr) {
  float x0, x1;
  f2_unpack(f2_fma(f2_pack(__uint_as_float(s0), __uint_as_float(s1)), sc2, nl), x0, x1);
  float p0 = ex2(x0), p1 = ex2(x1);
  p0 = keep(0) ? p0 : 0.f;
  p1 = keep(1) ? p1 : 0.f;
  if (p_out) { p_out[0] = p0; p_out[1] = p1; }
  f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack(__uint_as_float(dp0), __uint_as_float(dp1)), nd)), d[0], d[1]);
}

template <typename T> struct Fmt { static constexpr int v = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr int v = 1; };

template <int GW>
__device__ __forceinline__ void group_sync(int g) {      // the threads of compute group g
  asm volatile("bar.sync %0, %1;" ::"r"(g + 1), "n"(32 * GW) : "memory");
}

// A compute group's wait for an mbarrier.  One warp polls; the others block in the group's named barrier.  The
// barrier's OR-reduction hands every thread of the group the same verdict, so a group leaves as a whole and no
// warp is left behind in a later group barrier when a wait times out.  (Eight warps polling issued more than half
// of the kernel's instructions; taking them away did not change the run time, so the polling was not what the
// working groups were short of.)
template <int GW>
__device__ __forceinline__ bool group_wait(int g, bool poller, uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                           uint32_t* fail_bits, uint32_t bit) {
  uint32_t fail = 0;
  if (poller) {
    if (!mbar_wait(bar, parity, abort_flag)) {
      fail = 1;
      if ((threadIdx.x & 31) == 0) atomicOr(fail_bits, bit);
    } else if (*abort_flag) {
      fail = 1;
    }
  }
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(any) : "r"(fail), "r"(g + 1), "n"(32 * GW) : "memory");
  return any == 0;
}

template <typename T>
__device__ __forceinline__ void store_row_16bit(T* dst, const uint32_t (&v)[32], float f) {
#pragma unroll
  for (int v4 = 0; v4 < 4; ++v4) {
    uint4 u;
    u.x = Cvt<T>::pack2(__uint_as_float(v[v4 * 8 + 0]) * f, __uint_as_float(v[v4 * 8 + 1]) * f);
    u.y = Cvt<T>::pack2(__uint_as_float(v[v4 * 8 + 2]) * f, __uint_as_float(v[v4 * 8 + 3]) * f);
    u.z = Cvt<T>::pack2(__uint_as_float(v[v4 * 8 + 4]) * f, __uint_as_float(v[v4 * 8 + 5]) * f);
    u.w = Cvt<T>::pack2(__uint_as_float(v[v4 * 8 + 6]) * f, __uint_as_float(v[v4 * 8 + 7]) * f);
    *reinterpret_cast<uint4*>(dst + v4 * 8) = u;
  }
}

// Tables of the fused RoPE adjoint (unused when ROPE is false).
struct RopeTab {
  const float* cos_tab; const float* sin_tab;
  int64_t cos_stride, sin_stride;
};

// 32 accumulator columns of this thread's row, scaled and rounded to 16 bits: four 16-byte vectors
template <typename T>
__device__ __forceinline__ void acc_to_16bit(uint32_t taddr, float f, uint4 (&out)[4]) {
  uint32_t ov[32];
  tmem_ld32(taddr, ov);
  tmem_wait_ld();
#pragma unroll
  for (int v4 = 0; v4 < 4; ++v4) {
    out[v4].x = Cvt<T>::pack2(__uint_as_float(ov[v4 * 8 + 0]) * f, __uint_as_float(ov[v4 * 8 + 1]) * f);
    out[v4].y = Cvt<T>::pack2(__uint_as_float(ov[v4 * 8 + 2]) * f, __uint_as_float(ov[v4 * 8 + 3]) * f);
    out[v4].z = Cvt<T>::pack2(__uint_as_float(ov[v4 * 8 + 4]) * f, __uint_as_float(ov[v4 * 8 + 5]) * f);
    out[v4].w = Cvt<T>::pack2(__uint_as_float(ov[v4 * 8 + 6]) * f, __uint_as_float(ov[v4 * 8 + 7]) * f);
  }
}

// 32 consecutive 16-bit columns of a gradient row held as four 16-byte vectors
template <typename T>
__device__ __forceinline__ void store_32(T* dst, const uint4 (&v)[4]) {
#pragma unroll
  for (int v4 = 0; v4 < 4; ++v4) *reinterpret_cast<uint4*>(dst + v4 * 8) = v[v4];
}

// ---------------------------------------------------------------------------
// Fused RoPE adjoint of a 128-row gradient tile held one row per thread (or per thread pair).
// A thread that owned a row would have to read its own table row: 32 different 128-byte lines per warp
// load, which makes the load/store unit the cost.  So the rounded 16-bit rows go through a small shared
// staging tile (64 rows x 128 bytes per compute group, 128-byte swizzle) and are picked up again with
// eight threads per row (rope_math.cuh): table loads and the final global stores are then fully
// coalesced.  Two passes of 64 rows; the tables of pass 0 are prefetched into registers before the wait
// for the accumulator (see the callers), those of pass 1 while pass 0 is being worked on.
// ---------------------------------------------------------------------------
constexpr int kRopeStageRows = 64;
constexpr uint32_t kRopeStageBytes = kRopeStageRows * 128;          // per compute group
template <int GW> struct RopeTasks { static constexpr int n = kRopeStageRows * 8 / (32 * GW); };   // per thread and pass

template <int GW>
__device__ __forceinline__ void rope_prefetch_pass(RopeQuad (&tab)[RopeTasks<GW>::n], const RopeTab& rt, int row0, int pass, int tg, int S) {
#pragma unroll
  for (int j = 0; j < RopeTasks<GW>::n; ++j) {
    const int idx = j * 32 * GW + tg;
    const int row = row0 + kRopeStageRows * pass + (idx >> 3);
    const int pos = row < S ? row : S - 1;
    rope_load_quad(tab[j], rt.cos_tab + (int64_t)pos * rt.cos_stride, rt.sin_tab + (int64_t)pos * rt.sin_stride, idx & 7);
  }
}

// `lo` / `hi`: columns [0,32) / [32,64) of this thread's row r (GW == 4), or `lo` alone = the 32 columns of half
// `my_half` (GW == 8).  `item_out` points at row 0 of the item in the output tensor.
template <typename T, int GW>
__device__ __forceinline__ void rope_adjoint_store(uint8_t* stage, int g, int tg, int r, int my_half, const uint4 (&lo)[4], const uint4 (&hi)[4],
                                                   T* item_out, int64_t row_stride, int row0, int S, const RopeTab& rt,
                                                   RopeQuad (&tab)[RopeTasks<GW>::n]) {
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    if ((r >> 6) == pass) {
      const int rr = r & 63;
      uint8_t* srow = stage + rr * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if constexpr (GW == 4) {
          *reinterpret_cast<uint4*>(srow + ((c ^ (rr & 7)) << 4)) = lo[c];
          *reinterpret_cast<uint4*>(srow + (((4 + c) ^ (rr & 7)) << 4)) = hi[c];
        } else {
          *reinterpret_cast<uint4*>(srow + (((my_half * 4 + c) ^ (rr & 7)) << 4)) = lo[c];
        }
      }
    }
    group_sync<GW>(g);
#pragma unroll
    for (int j = 0; j < RopeTasks<GW>::n; ++j) {
      const int idx = j * 32 * GW + tg;
      const int row = idx >> 3, cg = idx & 7;
      const uint2 glo = *reinterpret_cast<const uint2*>(stage + swz_quad_offset(row, cg));
      const uint2 ghi = *reinterpret_cast<const uint2*>(stage + swz_quad_offset(row, cg + 8));
      uint2 olo, ohi;
      rope_apply_quad<T, true>(tab[j], glo, ghi, olo, ohi);
      const int trow = kRopeStageRows * pass + row;
      if (row0 + trow < S) {
        T* dst = item_out + (int64_t)trow * row_stride;
        *reinterpret_cast<uint2*>(dst + 4 * cg) = olo;
        *reinterpret_cast<uint2*>(dst + 32 + 4 * cg) = ohi;
      }
    }
    if (pass == 0) rope_prefetch_pass<GW>(tab, rt, row0, 1, tg, S);
    group_sync<GW>(g);                                    // the tile is rewritten by the next pass / the next epilogue
  }
}

// ---------------------------------------------------------------------------
// delta[bh, s] = sum_d O[s, d] * dO[s, d]   (fp32), 8 threads per row
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const T* __restrict__ O, const T* __restrict__ dO, float* __restrict__ delta,
                  int64_t o_sb, int64_t o_sh, int64_t o_ss, int64_t do_sb, int64_t do_sh, int64_t do_ss,
                  int S, int H) {
  const int part = threadIdx.x & 7;
  const int row = blockIdx.x * 32 + (threadIdx.x >> 3);
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  float sum = 0.f;
  if (row < S) {
    const uint4 ov = *reinterpret_cast<const uint4*>(O + b * o_sb + h * o_sh + (int64_t)row * o_ss + part * 8);
    const uint4 gv = *reinterpret_cast<const uint4*>(dO + b * do_sb + h * do_sh + (int64_t)row * do_ss + part * 8);
    const uint32_t* ow = reinterpret_cast<const uint32_t*>(&ov);
    const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = Cvt<T>::unpack2(ow[i]), g = Cvt<T>::unpack2(gw[i]);
      sum += a.x * g.x + a.y * g.y;
    }
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  sum += __shfl_xor_sync(0xffffffffu, sum, 4);
  if (part == 0 && row < S) delta[(int64_t)bh * S + row] = sum;
}

// ---------------------------------------------------------------------------
// Persistent CTAs.  Both tensor-core kernels launch one CTA per SM, which walks a static list of
// work items (one item = one (batch*head, tile of 128 rows)).  Items are numbered heaviest first
// and dealt to the CTAs in boustrophedon order -- round r gives CTA c item r*G + c on even rounds
// and r*G + G-1-c on odd ones -- which balances the CTAs' totals to within one item of the mean
// without a global counter.  Every role walks the same list, and all ring / buffer indices run on a
// tile counter that keeps counting across items, so the producer prefetches the next item's resident
// tiles (double-buffered) and first streamed tiles, and the S and dP issuers fill free score buffers
// with them, while the last tiles of the current item are still being worked on.  Only the gradient
// issuer pauses between items, until the epilogue group has read the accumulators out of TMEM.
// ---------------------------------------------------------------------------
// ---------------------------------------------------------------------------
// dQ kernel
// TMEM columns: buffer pair b holds S at 128b and dP at 128b+64 (dS is packed over S);
// the dQ accumulator sits at 128*kBufs.
// ---------------------------------------------------------------------------
struct CtlQ {
  uint64_t qdo_full[2], qdo_free[2], kv_full[kStages], kv_empty[kStages], sdp_full[kBufs], ds_ready[kBufs], buf_free[kBufs],
      dq_done[kGroups], acc_free;
  uint32_t tmem_base;
  int abort;
  uint32_t fail_bits;
};
constexpr size_t kCtlBytes = 4096;        // control block (barriers, per-tile statistics), padded so that what follows stays 128-byte aligned
static_assert(sizeof(CtlQ) <= kCtlBytes, "control block");
constexpr size_t kRopeStage = (size_t)kGroups * kRopeStageBytes;   // extra shared memory of the ROPE variants
constexpr size_t kSmemQ = 1024 + 6 * (size_t)kBigTile + (size_t)kStages * 2 * kSmallTile + kCtlBytes;

// FUSE_DELTA: the kernel also loads the item's O tile, computes delta = rowsum(O * dO) for its 128 rows
// itself (each compute group for its own use, from shared memory) and writes it to DELTA for the dK/dV
// kernel that follows on the stream; otherwise DELTA is an input.
template <typename T, bool CAUSAL, bool DROPOUT, bool FUSE_DELTA, bool ROPE>
__global__ void __launch_bounds__(Roles<kGWdQ>::kThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmO,
                   const float* __restrict__ LSE, float* __restrict__ DELTA, T* __restrict__ dQ,
                   int64_t dq_sb, int64_t dq_sh, int64_t dq_ss, int S, int H, int BH, float scale, float scale2,
                   float dropout_p, uint32_t seed, uint32_t* status, const RopeTab rt) {
  constexpr int kGW = kGWdQ;
  using R = Roles<kGW>;
  [[maybe_unused]] constexpr int kGroupThreads = R::kGroupThreads, kProducerWarp = R::kProducerWarp, kMmaWarp = R::kMmaWarp,
                kMma2Warp = R::kMma2Warp, kGradWarp = R::kGradWarp, kGrad2Warp = R::kGrad2Warp;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQdObig = base;                               // [slot][Q|dO|O], 16 KB each; item n uses slot n & 1
  uint8_t* sKV = base + 6 * kBigTile;                    // [stage][K|V], 8 KB each
  CtlQ* ctl = reinterpret_cast<CtlQ*>(sKV + (size_t)kStages * 2 * kSmallTile);
  [[maybe_unused]] uint8_t* stage = reinterpret_cast<uint8_t*>(ctl) + kCtlBytes;   // ROPE only: kGroups staging tiles
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_all = (S + BT - 1) / BT;
  const int n_qt = (S + BR - 1) / BR;
  const int n_items = BH * n_qt;
  // item -> (batch*head, first query row, key tiles): the last query tile is the heaviest under the causal mask
  auto decode = [&](int idx, int& bh, int& m0, int& nkv) {
    const int lvl = idx / BH;
    bh = idx - lvl * BH;
    m0 = (n_qt - 1 - lvl) * BR;
    const int n_causal = (m0 + BR) / BT;
    nkv = CAUSAL ? (n_causal < n_all ? n_causal : n_all) : n_all;
  };

  if (threadIdx.x == 0) {
    // a slot is free again once the S and dP issuers' MMAs have read it and, when the compute threads read it
    // too (FUSE_DELTA), once every one of them is done with the item
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->qdo_full[i], 1); mbar_init(&ctl->qdo_free[i], 2 + (FUSE_DELTA ? kGroups * kGroupThreads : 0)); }
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->kv_full[s], 1); mbar_init(&ctl->kv_empty[s], 1); }
    for (int g = 0; g < kBufs; ++g) { mbar_init(&ctl->sdp_full[g], 2); mbar_init(&ctl->ds_ready[g], kGroupThreads); mbar_init(&ctl->buf_free[g], 1); }
    for (int g = 0; g < kGroups; ++g) mbar_init(&ctl->dq_done[g], 1);
    mbar_init(&ctl->acc_free, kGroupThreads);
    ctl->abort = 0;
    ctl->fail_bits = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) { tmem_alloc(&ctl->tmem_base, kTmemCols); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  constexpr uint32_t cQ = 128 * kBufs;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      if (FUSE_DELTA) tma_prefetch_desc(&tmO);
      ItemIter items(n_items);
      uint32_t t = 0;                                     // tiles issued so far, over all items
      int n = 0, idx;
      bool ok = true;
      for (; ok && items.next(idx); ++n) {
        int bh, m0, nkv;
        decode(idx, bh, m0, nkv);
        const int b = bh / H, h = bh - b * H, slot = n & 1;
        // the slot's previous Q/dO (item n-2) must have been read by the last S and dP MMAs of that item
        if (n >= 2 && !mbar_wait(&ctl->qdo_free[slot], ((n >> 1) - 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA); break; }
        uint8_t* big = sQdObig + (size_t)slot * 3 * kBigTile;
        mbar_expect_tx(&ctl->qdo_full[slot], (FUSE_DELTA ? 3 : 2) * kBigTile);
        tma_load_4d(big, &tmQ, &ctl->qdo_full[slot], 0, m0, h, b);
        tma_load_4d(big + kBigTile, &tmdO, &ctl->qdo_full[slot], 0, m0, h, b);
        if (FUSE_DELTA) tma_load_4d(big + 2 * kBigTile, &tmO, &ctl->qdo_full[slot], 0, m0, h, b);
        for (int j = 0; j < nkv; ++j, ++t) {
          const uint32_t s = t % kStages;
          if (t >= kStages && !mbar_wait(&ctl->kv_empty[s], ((t / kStages) - 1) & 1, abort_flag)) {
            atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA);
            ok = false;
            break;
          }
          uint8_t* dst = sKV + (size_t)s * 2 * kSmallTile;
          mbar_expect_tx(&ctl->kv_full[s], 2 * kSmallTile);
          tma_load_4d(dst, &tmK, &ctl->kv_full[s], 0, j * BT, h, b);
          tma_load_4d(dst + kSmallTile, &tmV, &ctl->kv_full[s], 0, j * BT, h, b);
        }
      }
      if (*abort_flag) {   // let our own copies land before the CTA's shared memory goes away
        const int n_loaded = ok ? n : n + 1;              // items whose Q/dO loads were issued
        for (int m = n_loaded > 2 ? n_loaded - 2 : 0; m < n_loaded; ++m) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try(&ctl->qdo_full[m & 1], (m >> 1) & 1))
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
        }
        for (uint32_t u = t > (uint32_t)kStages ? t - kStages : 0; u < t; ++u) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try(&ctl->kv_full[u % kStages], (u / kStages) & 1))
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
        }
      }
    }
  } else if (warp == kMmaWarp || warp == kMma2Warp) {
    if (lane == 0) {                                     // score MMAs: S_j = Q K_j^T (first issuer), dP_j = dO V_j^T (second)
      const bool second = warp == kMma2Warp;
      constexpr uint32_t idesc_s = make_idesc(Fmt<T>::v, BR, BT, 0);   // 128 x 64, both K-major
      ItemIter items(n_items);
      uint32_t t = 0;
      int n = 0, idx;
      bool ok = true;
      for (; ok && items.next(idx); ++n) {
        int bh, m0, nkv;
        decode(idx, bh, m0, nkv);
        const int slot = n & 1;
        if (!mbar_wait(&ctl->qdo_full[slot], (n >> 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD); break; }
        const uint64_t da = make_sdesc_sw128(smem_u32(sQdObig + (size_t)slot * 3 * kBigTile + (second ? kBigTile : 0)));
        for (int j = 0; j < nkv; ++j, ++t) {
          const uint32_t s = t % kStages, g = t % kBufs;
          // the buffer pair still holds dS of tile t-kBufs until the gradient MMAs have read it
          if (t >= kBufs && !mbar_wait(&ctl->buf_free[g], ((t / kBufs) - 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA); ok = false; break; }
          if (!mbar_wait(&ctl->kv_full[s], (t / kStages) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD); ok = false; break; }
          fence_after_sync();
          const uint64_t db = make_sdesc_sw128(smem_u32(sKV + (size_t)s * 2 * kSmallTile + (second ? kSmallTile : 0)));
          const uint32_t t_dst = tmem_base + 128 * g + (second ? 64 : 0);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) mma_ss(t_dst, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc_s, kk > 0);
          mma_commit(&ctl->sdp_full[g]);
        }
        mma_commit(&ctl->qdo_free[slot]);                 // arrives once this thread's MMAs of the item have read Q (dO)
      }
    }
  } else if (warp == kGradWarp) {
    if (lane == 0) {                                     // gradient MMAs: dQ += dS_j K_j
      constexpr uint32_t idesc_q = make_idesc(Fmt<T>::v, BR, HD, 1);   // 128 x 64, B = K tile read MN-major
      ItemIter items(n_items);
      uint32_t t = 0;
      int n = 0, idx;
      bool ok = true;
      for (; ok && items.next(idx); ++n) {
        int bh, m0, nkv;
        decode(idx, bh, m0, nkv);
        // the accumulator still holds the previous item's dQ until its epilogue has read it
        if (n >= 1 && !mbar_wait(&ctl->acc_free, (n - 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_SOFTMAX); break; }
        fence_after_sync();
        for (int j = 0; j < nkv; ++j, ++t) {
          const uint32_t s = t % kStages, g = t % kBufs;
          if (!mbar_wait(&ctl->ds_ready[g], (t / kBufs) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_SOFTMAX); ok = false; break; }
          fence_after_sync();
          const uint64_t dk = make_sdesc_sw128(smem_u32(sKV + (size_t)s * 2 * kSmallTile));
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)           // 16 keys = 2048 bytes of K, 8 TMEM columns of dS
            mma_ts(tmem_base + cQ, tmem_base + 128 * g + packed_col<kGW>(kk), dk + (uint64_t)(kk * (2048 >> 4)), idesc_q, (j > 0 || kk > 0) ? 1u : 0u);
          mma_commit(&ctl->buf_free[g]);
          mma_commit(&ctl->kv_empty[s]);
        }
        // the group that took the item's last tile runs its epilogue; one barrier per group, because a
        // barrier's successive phases must be awaited by the same threads in order
        if (ok) mma_commit(&ctl->dq_done[(t - 1) % kGroups]);
      }
    }
  } else if (warp < kProducerWarp) {
    const int g = warp / kGW;                            // compute group
    const int r = ((warp & 3) << 5) | lane;              // query row within the tile == TMEM lane
    const int my_half = (warp % kGW) >> 2;               // with two threads per row: which 32 of the tile's 64 columns
    const bool poller = warp % kGW == 0;                 // the group's warp that polls barriers (group_wait)
    const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float inv_keep = DROPOUT ? 1.f / (1.f - dropout_p) : 1.f;
    ItemIter items(n_items);
    uint32_t t0 = 0;                                     // tile counter at the start of the item
    uint32_t epilogues = 0;                              // epilogues this group has run: the phase of its dq_done barrier
    int n = 0, idx;
    bool ok = true;
    for (; ok && items.next(idx); ++n) {
      int bh, m0, nkv;
      decode(idx, bh, m0, nkv);
      const int b = bh / H, h = bh - b * H;
      const int grow = m0 + r;
      const uint32_t seed_mix = (seed * 0x9E3779B1u) ^ (((uint32_t)bh + 1u) * 0x27D4EB2Fu);
      const float lse2 = grow < S ? LSE[(int64_t)bh * S + grow] * kLog2e : INFINITY;
      const int j_first = (int)((g + kGroups - t0 % kGroups) % kGroups);   // tile t belongs to group t % kGroups, counted over all items
      float dlt = 0.f;
      if (FUSE_DELTA) {
        // Every compute thread awaits every item's load and then releases the slot (qdo_free counts all of
        // them), whether its group has a tile in the item or not: the producer cannot refill a slot before
        // the slowest group is past it, so no thread ever meets a barrier two phases ahead of the one it
        // waits for (it would wait for the wrong one -- a deadlock seen with >3 short items per CTA).
        if (!group_wait<kGW>(g, poller, &ctl->qdo_full[n & 1], (n >> 1) & 1, abort_flag, &ctl->fail_bits, ULM_STATUS_TIMEOUT_LOAD)) { ok = false; break; }
        if (j_first < nkv) {
          // row r of a 128-byte-swizzled tile: 16-byte chunk c sits at chunk position c ^ (r & 7)
          const uint8_t* go = sQdObig + (size_t)(n & 1) * 3 * kBigTile + kBigTile + (size_t)r * 128;
          const uint8_t* oo = go + kBigTile;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int off = (c ^ (r & 7)) << 4;
            const uint4 gv = *reinterpret_cast<const uint4*>(go + off);
            const uint4 ov = *reinterpret_cast<const uint4*>(oo + off);
            const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gv);
            const uint32_t* ow = reinterpret_cast<const uint32_t*>(&ov);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 a2 = Cvt<T>::unpack2(ow[i]), g2 = Cvt<T>::unpack2(gw[i]);
              dlt = fmaf(a2.x, g2.x, dlt);
              dlt = fmaf(a2.y, g2.y, dlt);
            }
          }
          // the group that owns the item's first tile publishes delta for the dK/dV kernel
          if (j_first == 0 && (kGW == 4 || my_half == 0) && grow < S) DELTA[(int64_t)bh * S + grow] = dlt;
        }
        mbar_arrive(&ctl->qdo_free[n & 1]);
      } else {
        dlt = grow < S ? DELTA[(int64_t)bh * S + grow] : 0.f;
      }
      [[maybe_unused]] const uint64_t sc2 = f2_pack(scale2, scale2), nl2 = f2_pack(-lse2, -lse2), nd2 = f2_pack(-dlt, -dlt);
      for (int j = j_first; j < nkv; j += kGroups) {
        const uint32_t t = t0 + (uint32_t)j;
        const uint32_t bf = t % kBufs;
        const uint32_t cS = 128 * bf, cP = 128 * bf + 64;
        if (!group_wait<kGW>(g, poller, &ctl->sdp_full[bf], (t / kBufs) & 1, abort_flag, &ctl->fail_bits, ULM_STATUS_TIMEOUT_MMA)) { ok = false; break; }
        fence_after_sync();
        const int c0 = j * BT;
        const bool edge = (CAUSAL && c0 + BT - 1 > m0) || (c0 + BT > S);
        // The masked and the unmasked form of a tile are separate code: as one body the compiler predicates the
        // mask's compare-and-select per element, and predicated-off instructions still take issue slots in the
        // tiles that need no mask (all but one or two per item).
        auto tile_body = [&](auto edge_c) {
        constexpr bool EDGE = decltype(edge_c)::value;
        if constexpr (kGW == 8) {
          // two threads per row: this one takes columns [32 my_half, +32) in two chunks of 16 and packs dS
          // over its own scores
  #pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t sv[16], pv[16], pk[8];
            const int col0 = my_half * 32 + ch * 16;
            tmem_ld16(t_row + cS + col0, sv);
            tmem_ld16(t_row + cP + col0, pv);
            tmem_wait_ld();
  #pragma unroll
            for (int c = 0; c < 16; c += 2) {
              float d2[2];
              if constexpr (!DROPOUT) {
                pair_ds(sv[c], sv[c + 1], pv[c], pv[c + 1], sc2, nl2, nd2,
                        [&](int e) { const int col = c0 + col0 + c + e; return !EDGE || ((col < S) && (!CAUSAL || col <= grow)); }, d2);
              } else {
  #pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int col = c0 + col0 + c + e;
                float p = ex2(fmaf(__uint_as_float(sv[c + e]), scale2, -lse2));
                if constexpr (EDGE) p = ((col < S) && (!CAUSAL || col <= grow)) ? p : 0.f;
                float dp = __uint_as_float(pv[c + e]);
                dp = dropout_keep(seed_mix, grow, col, dropout_p) ? dp * inv_keep : 0.f;
                d2[e] = p * (dp - dlt);
              }
              }
              pk[c >> 1] = Cvt<T>::pack2(d2[0], d2[1]);
            }
            st8(t_row + cS + my_half * 32 + ch * 8, pk);
          }
        } else {
  #pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t sv[32], pv[32], pk[16];
          tmem_ld32(t_row + cS + hf * 32, sv);
          tmem_ld32(t_row + cP + hf * 32, pv);
          tmem_wait_ld();
  #pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float d2[2];
            if constexpr (!DROPOUT) {
              pair_ds(sv[c], sv[c + 1], pv[c], pv[c + 1], sc2, nl2, nd2,
                      [&](int e) { const int col = c0 + hf * 32 + c + e; return !EDGE || ((col < S) && (!CAUSAL || col <= grow)); }, d2);
            } else {
  #pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int col = c0 + hf * 32 + c + e;
              float p = ex2(fmaf(__uint_as_float(sv[c + e]), scale2, -lse2));
              if constexpr (EDGE) p = ((col < S) && (!CAUSAL || col <= grow)) ? p : 0.f;
              float dp = __uint_as_float(pv[c + e]);
              dp = dropout_keep(seed_mix, grow, col, dropout_p) ? dp * inv_keep : 0.f;
              d2[e] = p * (dp - dlt);
            }
            }
            pk[c >> 1] = Cvt<T>::pack2(d2[0], d2[1]);
          }
          st16(t_row + cS + hf * 16, pk);   // packed dS columns [hf*16, hf*16+16)
        }
        }
        };
        if (edge) tile_body(std::true_type{}); else tile_body(std::false_type{});
        tmem_wait_st();
        fence_before_sync();
        mbar_arrive(&ctl->ds_ready[bf]);
      }
      t0 += (uint32_t)nkv;
      if (!ok) break;
      // The group that worked on the item's last tile runs the epilogue: its next tile reuses that tile's buffer
      // pair, which is free no sooner than the item's last gradient MMA, so it has nothing else to do meanwhile.
      if ((t0 - 1) % kGroups == (uint32_t)g) {
        // Fused RoPE adjoint: the first pass's table values are fetched into registers BEFORE the wait for the
        // last gradient MMA (the group has nothing else to do then), so their latency is off the path between
        // "accumulator complete" and "accumulator released".
        const int tg = (int)threadIdx.x - g * kGroupThreads;
        [[maybe_unused]] RopeQuad tab[RopeTasks<kGW>::n];
        if constexpr (ROPE) rope_prefetch_pass<kGW>(tab, rt, m0, 0, tg, S);
        if (!group_wait<kGW>(g, poller, &ctl->dq_done[g], epilogues++ & 1, abort_flag, &ctl->fail_bits, ULM_STATUS_TIMEOUT_MMA)) { ok = false; break; }
        fence_after_sync();
        // read and round everything first, hand the accumulator back, rotate (ROPE) and store afterwards
        T* item_out = dQ + (int64_t)b * dq_sb + (int64_t)h * dq_sh + (int64_t)m0 * dq_ss;
        uint4 lo[4];
        [[maybe_unused]] uint4 hi[4];
        if constexpr (kGW == 4) {
          acc_to_16bit<T>(t_row + cQ, scale, lo);
          acc_to_16bit<T>(t_row + cQ + 32, scale, hi);
        } else {
          acc_to_16bit<T>(t_row + cQ + my_half * 32, scale, lo);
        }
        fence_before_sync();
        mbar_arrive(&ctl->acc_free);
        if constexpr (ROPE) {
          rope_adjoint_store<T, kGW>(stage + (size_t)g * kRopeStageBytes, g, tg, r, my_half, lo, hi, item_out, dq_ss, m0, S, rt, tab);
        } else if (grow < S) {
          T* orow = item_out + (int64_t)r * dq_ss;
          if constexpr (kGW == 4) { store_32<T>(orow, lo); store_32<T>(orow + 32, hi); }
          else store_32<T>(orow + my_half * 32, lo);
        }
      }
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ctl->fail_bits && status) atomicOr(status, ctl->fail_bits);
}

// ---------------------------------------------------------------------------
// dK / dV kernel
// A work item is one (batch*head, key tile of 128); key tile 0 meets the most query tiles under the
// causal mask, so items are numbered by key tile, ascending.
// TMEM columns: buffer pair b holds S^T at 128b and dP^T at 128b+64 (P^T and dS^T
// are packed over them); the dV and dK accumulators sit at 128*kBufs and +64, so
// kBufs = 3 uses all 512 columns.
// ---------------------------------------------------------------------------
struct CtlKV {
  uint64_t kv_full[2], kv_free[2], qdo_full[kStages], qdo_empty[kStages], sdp_full[kBufs], pds_ready[kBufs], buf_free[kBufs],
      dkv_done[kGroups], acc_free;
  uint32_t tmem_base;
  int abort;
  uint32_t fail_bits;
  alignas(16) float lse2[kGroups][BT];   // per-query statistics of each group's current tile (read as float4)
  alignas(16) float dlt[kGroups][BT];
};
static_assert(sizeof(CtlKV) <= kCtlBytes, "control block");
constexpr size_t kSmemKV = 1024 + 4 * (size_t)kBigTile + (size_t)kStages * 2 * kSmallTile + kCtlBytes;

template <typename T, bool CAUSAL, bool DROPOUT, bool ROPE>
__global__ void __launch_bounds__(Roles<kGWdKV>::kThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const float* __restrict__ LSE, const float* __restrict__ DELTA,
                    T* __restrict__ dK, T* __restrict__ dV,
                    int64_t dk_sb, int64_t dk_sh, int64_t dk_ss, int64_t dv_sb, int64_t dv_sh, int64_t dv_ss,
                    int S, int H, int BH, float scale, float scale2, float dropout_p, uint32_t seed, uint32_t* status,
                    const RopeTab rt) {
  constexpr int kGW = kGWdKV;
  using R = Roles<kGW>;
  [[maybe_unused]] constexpr int kGroupThreads = R::kGroupThreads, kProducerWarp = R::kProducerWarp, kMmaWarp = R::kMmaWarp,
                kMma2Warp = R::kMma2Warp, kGradWarp = R::kGradWarp, kGrad2Warp = R::kGrad2Warp;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKVbig = base;                                 // [slot][K|V], 16 KB each; item n uses slot n & 1
  uint8_t* sQdO = base + 4 * kBigTile;                    // [stage][Q|dO], 8 KB each
  CtlKV* ctl = reinterpret_cast<CtlKV*>(sQdO + (size_t)kStages * 2 * kSmallTile);
  [[maybe_unused]] uint8_t* stage = reinterpret_cast<uint8_t*>(ctl) + kCtlBytes;   // ROPE only: kGroups staging tiles
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_all = (S + BT - 1) / BT;
  const int n_items = BH * ((S + BR - 1) / BR);
  // item -> (batch*head, first key, first query tile, query tiles): key tile 0 is the heaviest under the causal mask
  auto decode = [&](int idx, int& bh, int& n0, int& i_begin, int& nq) {
    const int kt = idx / BH;
    bh = idx - kt * BH;
    n0 = kt * BR;
    i_begin = CAUSAL ? n0 / BT : 0;
    nq = n_all - i_begin;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->kv_full[i], 1); mbar_init(&ctl->kv_free[i], 2); }
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->qdo_full[s], 1); mbar_init(&ctl->qdo_empty[s], kGradIssuers); }
    for (int g = 0; g < kBufs; ++g) { mbar_init(&ctl->sdp_full[g], 2); mbar_init(&ctl->pds_ready[g], kGroupThreads); mbar_init(&ctl->buf_free[g], kGradIssuers); }
    for (int g = 0; g < kGroups; ++g) mbar_init(&ctl->dkv_done[g], kGradIssuers);
    mbar_init(&ctl->acc_free, kGroupThreads);
    ctl->abort = 0;
    ctl->fail_bits = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) { tmem_alloc(&ctl->tmem_base, kTmemCols); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  constexpr uint32_t cV = 128 * kBufs, cK = 128 * kBufs + 64;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      ItemIter items(n_items);
      uint32_t t = 0;                                     // tiles issued so far, over all items
      int n = 0, idx;
      bool ok = true;
      for (; ok && items.next(idx); ++n) {
        int bh, n0, i_begin, nq;
        decode(idx, bh, n0, i_begin, nq);
        const int b = bh / H, h = bh - b * H, slot = n & 1;
        // the slot's previous K/V (item n-2) must have been read by the last S and dP MMAs of that item
        if (n >= 2 && !mbar_wait(&ctl->kv_free[slot], ((n >> 1) - 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA); break; }
        uint8_t* big = sKVbig + (size_t)slot * 2 * kBigTile;
        mbar_expect_tx(&ctl->kv_full[slot], 2 * kBigTile);
        tma_load_4d(big, &tmK, &ctl->kv_full[slot], 0, n0, h, b);
        tma_load_4d(big + kBigTile, &tmV, &ctl->kv_full[slot], 0, n0, h, b);
        for (int it = 0; it < nq; ++it, ++t) {
          const uint32_t s = t % kStages;
          if (t >= kStages && !mbar_wait(&ctl->qdo_empty[s], ((t / kStages) - 1) & 1, abort_flag)) {
            atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA);
            ok = false;
            break;
          }
          uint8_t* dst = sQdO + (size_t)s * 2 * kSmallTile;
          mbar_expect_tx(&ctl->qdo_full[s], 2 * kSmallTile);
          tma_load_4d(dst, &tmQ, &ctl->qdo_full[s], 0, (i_begin + it) * BT, h, b);
          tma_load_4d(dst + kSmallTile, &tmdO, &ctl->qdo_full[s], 0, (i_begin + it) * BT, h, b);
        }
      }
      if (*abort_flag) {   // let our own copies land before the CTA's shared memory goes away
        const int n_loaded = ok ? n : n + 1;              // items whose K/V loads were issued
        for (int m = n_loaded > 2 ? n_loaded - 2 : 0; m < n_loaded; ++m) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try(&ctl->kv_full[m & 1], (m >> 1) & 1))
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
        }
        for (uint32_t u = t > (uint32_t)kStages ? t - kStages : 0; u < t; ++u) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try(&ctl->qdo_full[u % kStages], (u / kStages) & 1))
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
        }
      }
    }
  } else if (warp == kMmaWarp || warp == kMma2Warp) {
    if (lane == 0) {                                     // score MMAs: S^T = K Q_i^T (first issuer), dP^T = V dO_i^T (second)
      const bool second = warp == kMma2Warp;
      constexpr uint32_t idesc_s = make_idesc(Fmt<T>::v, BR, BT, 0);   // 128 keys x 64 queries
      ItemIter items(n_items);
      uint32_t t = 0;
      int n = 0, idx;
      bool ok = true;
      for (; ok && items.next(idx); ++n) {
        int bh, n0, i_begin, nq;
        decode(idx, bh, n0, i_begin, nq);
        const int slot = n & 1;
        if (!mbar_wait(&ctl->kv_full[slot], (n >> 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD); break; }
        const uint64_t da = make_sdesc_sw128(smem_u32(sKVbig + (size_t)slot * 2 * kBigTile + (second ? kBigTile : 0)));
        for (int it = 0; it < nq; ++it, ++t) {
          const uint32_t s = t % kStages, g = t % kBufs;
          // the buffer pair still holds P/dS of tile t-kBufs until the gradient MMAs have read it
          if (t >= kBufs && !mbar_wait(&ctl->buf_free[g], ((t / kBufs) - 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA); ok = false; break; }
          if (!mbar_wait(&ctl->qdo_full[s], (t / kStages) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD); ok = false; break; }
          fence_after_sync();
          const uint64_t db = make_sdesc_sw128(smem_u32(sQdO + (size_t)s * 2 * kSmallTile + (second ? kSmallTile : 0)));
          const uint32_t t_dst = tmem_base + 128 * g + (second ? 64 : 0);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) mma_ss(t_dst, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc_s, kk > 0);
          mma_commit(&ctl->sdp_full[g]);
        }
        mma_commit(&ctl->kv_free[slot]);                  // arrives once this thread's MMAs of the item have read K (V)
      }
    }
  } else if (warp == kGradWarp || (warp == kGrad2Warp && kGradIssuers == 2)) {
    if (lane == 0) {                                     // gradient MMAs: dV += P^T dO_i (first issuer), dK += dS^T Q_i (second)
      const bool second = warp == kGrad2Warp;
      constexpr uint32_t idesc_a = make_idesc(Fmt<T>::v, BR, HD, 1);   // B = dO / Q tile read MN-major
      ItemIter items(n_items);
      uint32_t t = 0;
      int n = 0, idx;
      bool ok = true;
      for (; ok && items.next(idx); ++n) {
        int bh, n0, i_begin, nq;
        decode(idx, bh, n0, i_begin, nq);
        // the accumulators still hold the previous item's dK/dV until its epilogue has read them
        if (n >= 1 && !mbar_wait(&ctl->acc_free, (n - 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_SOFTMAX); break; }
        fence_after_sync();
        for (int it = 0; it < nq; ++it, ++t) {
          const uint32_t s = t % kStages, g = t % kBufs;
          if (!mbar_wait(&ctl->pds_ready[g], (t / kBufs) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_SOFTMAX); ok = false; break; }
          fence_after_sync();
#pragma unroll
          for (int w = 0; w < 3 - kGradIssuers; ++w) {
            // dV reads P^T (packed over S^T) against the dO tile; dK reads dS^T (packed over dP^T) against the Q tile
            const bool sec = kGradIssuers == 2 ? second : (w == 1);
            const uint64_t db = make_sdesc_sw128(smem_u32(sQdO + (size_t)s * 2 * kSmallTile + (sec ? 0 : kSmallTile)));
            const uint32_t t_acc = tmem_base + (sec ? cK : cV), t_a = tmem_base + 128 * g + (sec ? 64 : 0);
#pragma unroll
            for (int kk = 0; kk < BT / 16; ++kk)
              mma_ts(t_acc, t_a + packed_col<kGW>(kk), db + (uint64_t)(kk * (2048 >> 4)), idesc_a, (it > 0 || kk > 0) ? 1u : 0u);
          }
          mma_commit(&ctl->buf_free[g]);
          mma_commit(&ctl->qdo_empty[s]);
        }
        // the group that took the item's last tile runs its epilogue (see there); one barrier per group, because a
        // barrier's successive phases must be awaited by the same threads in order
        if (ok) mma_commit(&ctl->dkv_done[(t - 1) % kGroups]);
      }
    }
  } else if (warp < kProducerWarp) {
    const int g = warp / kGW;
    const int r = ((warp & 3) << 5) | lane;               // key row within the tile == TMEM lane
    const int tg = (int)threadIdx.x - g * kGroupThreads;  // thread index within the group
    const int my_half = (warp % kGW) >> 2;                // with two threads per row: which 32 of the tile's 64 columns
    const bool poller = warp % kGW == 0;                  // the group's warp that polls barriers (group_wait)
    const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    [[maybe_unused]] const uint64_t sc2 = f2_pack(scale2, scale2);
    const float inv_keep = DROPOUT ? 1.f / (1.f - dropout_p) : 1.f;
    ItemIter items(n_items);
    uint32_t t0 = 0;                                      // tile counter at the start of the item
    uint32_t epilogues = 0;                               // epilogues this group has run: the phase of its dkv_done barrier
    int n = 0, idx;
    bool ok = true;
    for (; ok && items.next(idx); ++n) {
      int bh, n0, i_begin, nq;
      decode(idx, bh, n0, i_begin, nq);
      const int b = bh / H, h = bh - b * H;
      const int kc = n0 + r;                              // this thread's key
      const uint32_t seed_mix = (seed * 0x9E3779B1u) ^ (((uint32_t)bh + 1u) * 0x27D4EB2Fu);
      // tile t belongs to group t % kGroups, counted over all items
      for (int it = (int)((g + kGroups - t0 % kGroups) % kGroups); it < nq; it += kGroups) {
        const uint32_t t = t0 + (uint32_t)it;
        const int i0 = (i_begin + it) * BT;
        const uint32_t bf = t % kBufs;
        const uint32_t cS = 128 * bf, cP = 128 * bf + 64;
        {   // per-query softmax statistics of this tile, shared by the group's key rows
          const int c = tg & (BT - 1);
          const int q = i0 + c;
          group_sync<kGW>(g);                                  // everyone is done with the previous tile's values
          if (tg < BT) ctl->lse2[g][c] = q < S ? -(LSE[(int64_t)bh * S + q] * kLog2e) : -INFINITY;   // both stored negated
          else if (tg < 2 * BT) ctl->dlt[g][c] = q < S ? -DELTA[(int64_t)bh * S + q] : 0.f;
        }
        // the group barrier inside the wait also publishes the statistics
        if (!group_wait<kGW>(g, poller, &ctl->sdp_full[bf], (t / kBufs) & 1, abort_flag, &ctl->fail_bits, ULM_STATUS_TIMEOUT_MMA)) { ok = false; break; }
        fence_after_sync();
        const bool edge = CAUSAL && (i0 < n0 + BR - 1);   // some query of the tile precedes some key of the CTA
        auto tile_body = [&](auto edge_c) {                // masked / unmasked tiles as separate code (see the dQ kernel)
        constexpr bool EDGE = decltype(edge_c)::value;
        if constexpr (kGW == 8) {
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t sv[16], pv[16], pp[8], pd[8];
            const int col0 = my_half * 32 + ch * 16;
            tmem_ld16(t_row + cS + col0, sv);
            tmem_ld16(t_row + cP + col0, pv);
            tmem_wait_ld();
            float l4[4], d4[4];                            // statistics of 4 queries per 16-byte shared load
#pragma unroll
            for (int c = 0; c < 16; c += 2) {
              float p2[2], d2[2];
              if ((c & 3) == 0) {
                *reinterpret_cast<float4*>(l4) = *reinterpret_cast<const float4*>(&ctl->lse2[g][col0 + c]);
                *reinterpret_cast<float4*>(d4) = *reinterpret_cast<const float4*>(&ctl->dlt[g][col0 + c]);
              }
#pragma unroll
              if constexpr (!DROPOUT) {
                pair_ds(sv[c], sv[c + 1], pv[c], pv[c + 1], sc2, f2_pack(l4[c & 3], l4[(c + 1) & 3]), f2_pack(d4[c & 3], d4[(c + 1) & 3]),
                        [&](int e) { return !EDGE || (i0 + col0 + c + e >= kc); }, d2, p2);
              } else {
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int q = i0 + col0 + c + e;
                float p = ex2(fmaf(__uint_as_float(sv[c + e]), scale2, l4[(c + e) & 3]));
                if constexpr (EDGE) p = (q >= kc) ? p : 0.f;
                float dp = __uint_as_float(pv[c + e]);
                const bool keep = dropout_keep(seed_mix, q, kc, dropout_p);
                p2[e] = keep ? p * inv_keep : 0.f;
                dp = keep ? dp * inv_keep : 0.f;
                d2[e] = p * (dp + d4[(c + e) & 3]);
              }
              }
              pp[c >> 1] = Cvt<T>::pack2(p2[0], p2[1]);
              pd[c >> 1] = Cvt<T>::pack2(d2[0], d2[1]);
            }
            st8(t_row + cS + my_half * 32 + ch * 8, pp);
            st8(t_row + cP + my_half * 32 + ch * 8, pd);
          }
        } else {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t sv[32], pv[32], pp[16], pd[16];
          tmem_ld32(t_row + cS + hf * 32, sv);
          tmem_ld32(t_row + cP + hf * 32, pv);
          tmem_wait_ld();
          float l4[4], d4[4];                              // statistics of 4 queries per 16-byte shared load
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float p2[2], d2[2];
            if ((c & 3) == 0) {
              *reinterpret_cast<float4*>(l4) = *reinterpret_cast<const float4*>(&ctl->lse2[g][hf * 32 + c]);
              *reinterpret_cast<float4*>(d4) = *reinterpret_cast<const float4*>(&ctl->dlt[g][hf * 32 + c]);
            }
#pragma unroll
            if constexpr (!DROPOUT) {
              pair_ds(sv[c], sv[c + 1], pv[c], pv[c + 1], sc2, f2_pack(l4[c & 3], l4[(c + 1) & 3]), f2_pack(d4[c & 3], d4[(c + 1) & 3]),
                      [&](int e) { return !EDGE || (i0 + hf * 32 + c + e >= kc); }, d2, p2);
            } else {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int q = i0 + hf * 32 + c + e;
              float p = ex2(fmaf(__uint_as_float(sv[c + e]), scale2, l4[(c + e) & 3]));
              if constexpr (EDGE) p = (q >= kc) ? p : 0.f;
              float dp = __uint_as_float(pv[c + e]);
              const bool keep = dropout_keep(seed_mix, q, kc, dropout_p);
              p2[e] = keep ? p * inv_keep : 0.f;
              dp = keep ? dp * inv_keep : 0.f;
              d2[e] = p * (dp + d4[(c + e) & 3]);
            }
            }
            pp[c >> 1] = Cvt<T>::pack2(p2[0], p2[1]);
            pd[c >> 1] = Cvt<T>::pack2(d2[0], d2[1]);
          }
          st16(t_row + cS + hf * 16, pp);
          st16(t_row + cP + hf * 16, pd);
        }
        }
        };
        if (edge) tile_body(std::true_type{}); else tile_body(std::false_type{});
        tmem_wait_st();
        fence_before_sync();
        mbar_arrive(&ctl->pds_ready[bf]);
      }
      t0 += (uint32_t)nq;
      if (!ok) break;
      // The group that worked on the item's last tile runs the epilogue: its next tile reuses that tile's buffer
      // pair, which is free no sooner than the item's last gradient MMA, so it has nothing else to do meanwhile.
      if ((t0 - 1) % kGroups == (uint32_t)g) {
        // Fused RoPE adjoint on dK: the first pass's table values are fetched into registers BEFORE the wait for
        // the last gradient MMAs (see the dQ kernel's epilogue).
        [[maybe_unused]] RopeQuad tab[RopeTasks<kGW>::n];
        if constexpr (ROPE) rope_prefetch_pass<kGW>(tab, rt, n0, 0, tg, S);
        if (!group_wait<kGW>(g, poller, &ctl->dkv_done[g], epilogues++ & 1, abort_flag, &ctl->fail_bits, ULM_STATUS_TIMEOUT_MMA)) { ok = false; break; }
        fence_after_sync();
        // read and round everything first, hand the accumulators back, rotate dK (ROPE) and store afterwards
        T* vrow = dV + (int64_t)b * dv_sb + (int64_t)h * dv_sh + (int64_t)kc * dv_ss;
        T* k_item = dK + (int64_t)b * dk_sb + (int64_t)h * dk_sh + (int64_t)n0 * dk_ss;
        uint4 vlo[4], klo[4];
        [[maybe_unused]] uint4 vhi[4], khi[4];
        if constexpr (kGW == 4) {
          acc_to_16bit<T>(t_row + cV, 1.f, vlo);
          acc_to_16bit<T>(t_row + cV + 32, 1.f, vhi);
          acc_to_16bit<T>(t_row + cK, scale, klo);
          acc_to_16bit<T>(t_row + cK + 32, scale, khi);
        } else {
          acc_to_16bit<T>(t_row + cV + my_half * 32, 1.f, vlo);
          acc_to_16bit<T>(t_row + cK + my_half * 32, scale, klo);
        }
        fence_before_sync();
        mbar_arrive(&ctl->acc_free);
        if (kc < S) {
          if constexpr (kGW == 4) { store_32<T>(vrow, vlo); store_32<T>(vrow + 32, vhi); }
          else store_32<T>(vrow + my_half * 32, vlo);
        }
        if constexpr (ROPE) {
          rope_adjoint_store<T, kGW>(stage + (size_t)g * kRopeStageBytes, g, tg, r, my_half, klo, khi, k_item, dk_ss, n0, S, rt, tab);
        } else if (kc < S) {
          T* krow = k_item + (int64_t)r * dk_ss;
          if constexpr (kGW == 4) { store_32<T>(krow, klo); store_32<T>(krow + 32, khi); }
          else store_32<T>(krow + my_half * 32, klo);
        }
      }
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ctl->fail_bits && status) atomicOr(status, ctl->fail_bits);
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
struct Maps { CUtensorMap q128, q64, k128, k64, v128, v64, do128, do64, o128; };

// SMs of the current device (the persistent kernels launch one CTA on each)
int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return kNumSMs;
  return n;
}

template <typename T, bool CAUSAL, bool DROPOUT, bool ROPE>
int launch_bwd(const ulm_attn_bwd_args* a, int device, const Maps& m) {
  cudaStream_t st = (cudaStream_t)a->stream;
  const unsigned BH = (unsigned)(a->B * a->H);
  const unsigned nt = (unsigned)((a->S + BR - 1) / BR);
  const float scale2 = a->softmax_scale * kLog2e;
  RopeTab rt{};
  if (ROPE) rt = RopeTab{a->cos_tab, a->sin_tab, a->cos_stride, a->sin_stride};
  int rc = ULM_OK;
  const bool fuse_delta = (a->mode & 3) == 3;            // delta wanted and the dQ kernel runs: it computes delta itself
  if ((a->mode & 1) && !fuse_delta) {
    dim3 g((unsigned)((a->S + 31) / 32), BH);
    attn_delta_kernel<T><<<g, 256, 0, st>>>((const T*)a->o, (const T*)a->d_o, a->delta, a->o_sb, a->o_sh, a->o_ss,
                                            a->do_sb, a->do_sh, a->do_ss, a->S, a->H);
    if ((rc = check_launch("ulm_attn_bwd(delta)"))) return rc;
  }
  const unsigned items = BH * nt;
  const unsigned grid = items < (unsigned)sm_count() ? items : (unsigned)sm_count();
  if (a->mode & 2) {
    auto go = [&](auto kern, std::atomic<bool>* attr) -> int {
      const size_t smem = kSmemQ + (ROPE ? kRopeStage : 0);
      if (int r = ensure_smem_attr(kern, smem, device, attr, "ulm_attn_bwd(dq)")) return r;
      kern<<<grid, Roles<kGWdQ>::kThreads, smem, st>>>(m.q128, m.k64, m.v64, m.do128, m.o128, a->lse, a->delta, (T*)a->dq,
                                                          a->dq_sb, a->dq_sh, a->dq_ss, a->S, a->H, (int)BH, a->softmax_scale, scale2,
                                                          a->dropout_p, a->seed, a->status_dev, rt);
      return check_launch("ulm_attn_bwd(dq)");
    };
    static std::atomic<bool> attr_fused[kMaxDevices], attr_plain[kMaxDevices];
    rc = fuse_delta ? go(attn_bwd_dq_kernel<T, CAUSAL, DROPOUT, true, ROPE>, attr_fused)
                    : go(attn_bwd_dq_kernel<T, CAUSAL, DROPOUT, false, ROPE>, attr_plain);
    if (rc) return rc;
  }
  if (a->mode & 4) {
    auto kern = attn_bwd_dkv_kernel<T, CAUSAL, DROPOUT, ROPE>;
    static std::atomic<bool> attr[kMaxDevices];
    const size_t smem = kSmemKV + (ROPE ? kRopeStage : 0);
    if ((rc = ensure_smem_attr(kern, smem, device, attr, "ulm_attn_bwd(dkv)"))) return rc;
    kern<<<grid, Roles<kGWdKV>::kThreads, smem, st>>>(m.q64, m.k128, m.v128, m.do64, a->lse, a->delta, (T*)a->dk, (T*)a->dv,
                                          a->dk_sb, a->dk_sh, a->dk_ss, a->dv_sb, a->dv_sh, a->dv_ss,
                                          a->S, a->H, (int)BH, a->softmax_scale, scale2, a->dropout_p, a->seed, a->status_dev, rt);
    if ((rc = check_launch("ulm_attn_bwd(dkv)"))) return rc;
  }
  return rc;
}

template <typename T, bool ROPE>
int dispatch_bwd(const ulm_attn_bwd_args* a, int device, const Maps& m) {
  const bool drop = a->dropout_p > 0.f;
  if (a->causal) return drop ? launch_bwd<T, true, true, ROPE>(a, device, m) : launch_bwd<T, true, false, ROPE>(a, device, m);
  return drop ? launch_bwd<T, false, true, ROPE>(a, device, m) : launch_bwd<T, false, false, ROPE>(a, device, m);
}

bool ok_out(const void* p, int64_t sb, int64_t sh, int64_t ss) {
  return p && !(reinterpret_cast<uintptr_t>(p) & 15) && sb % 8 == 0 && sh % 8 == 0 && ss % 8 == 0;
}

}  // namespace
}  // namespace ulm

extern "C" int ulm_attn_bwd(const ulm_attn_bwd_args* a) {
  using namespace ulm;
  if (!a) return fail(ULM_ERR_ARG, "ulm_attn_bwd: null args");
  if (a->dtype != ULM_F16 && a->dtype != ULM_BF16) return fail(ULM_ERR_ARG, "ulm_attn_bwd: dtype must be f16 or bf16");
  if (a->B < 0 || a->H < 0 || a->S < 0) return fail(ULM_ERR_ARG, "ulm_attn_bwd: negative size");
  if (a->B == 0 || a->H == 0 || a->S == 0 || (a->mode & 7) == 0) return ULM_OK;
  if (!a->q || !a->k || !a->v || !a->d_o || !a->lse || !a->delta) return fail(ULM_ERR_ARG, "ulm_attn_bwd: null tensor");
  if (!(a->softmax_scale > 0.f)) return fail(ULM_ERR_ARG, "ulm_attn_bwd: softmax_scale must be positive");
  if (a->dropout_p < 0.f || a->dropout_p >= 1.f) return fail(ULM_ERR_ARG, "ulm_attn_bwd: dropout_p must be in [0,1)");
  if ((a->mode & 1) && !ok_out(a->o, a->o_sb, a->o_sh, a->o_ss)) return fail(ULM_ERR_ARG, "ulm_attn_bwd: o must be 16-byte aligned, strides multiples of 8");
  if ((a->mode & 2) && !ok_out(a->dq, a->dq_sb, a->dq_sh, a->dq_ss)) return fail(ULM_ERR_ARG, "ulm_attn_bwd: dq must be 16-byte aligned, strides multiples of 8");
  if ((a->mode & 4) && (!ok_out(a->dk, a->dk_sb, a->dk_sh, a->dk_ss) || !ok_out(a->dv, a->dv_sb, a->dv_sh, a->dv_ss)))
    return fail(ULM_ERR_ARG, "ulm_attn_bwd: dk/dv must be 16-byte aligned, strides multiples of 8");
  if ((int64_t)a->B * a->H > 0x7fffffffLL || (a->S + 31) / 32 > 65535 * 4) return fail(ULM_ERR_TOO_LARGE, "ulm_attn_bwd: grid too large");
  const bool rope = a->cos_tab || a->sin_tab;
  if (rope) {
    if (!a->cos_tab || !a->sin_tab) return fail(ULM_ERR_ARG, "ulm_attn_bwd: cos_tab and sin_tab must be given together");
    if ((reinterpret_cast<uintptr_t>(a->cos_tab) & 15) || (reinterpret_cast<uintptr_t>(a->sin_tab) & 15) || a->cos_stride % 4 || a->sin_stride % 4 ||
        a->cos_stride < 64 || a->sin_stride < 64)
      return fail(ULM_ERR_ARG, "ulm_attn_bwd: RoPE tables must be 16-byte aligned with row strides that are multiples of 4 floats, at least 64");
  }
  tc::DeviceScope dev(a->q, "ulm_attn_bwd");
  if (dev.rc) return dev.rc;
  Maps m{};
  int rc;
#define ULM_MAP(dst, ptr, sb, sh, ss, rows, what) \
  if ((rc = tc::encode_bhsd_map(&m.dst, a->ptr, a->dtype, a->B, a->H, a->S, a->sb, a->sh, a->ss, rows, what))) return rc
  if (a->mode & 2) {
    ULM_MAP(q128, q, q_sb, q_sh, q_ss, BR, "ulm_attn_bwd(q)");
    ULM_MAP(k64, k, k_sb, k_sh, k_ss, BT, "ulm_attn_bwd(k)");
    ULM_MAP(v64, v, v_sb, v_sh, v_ss, BT, "ulm_attn_bwd(v)");
    ULM_MAP(do128, d_o, do_sb, do_sh, do_ss, BR, "ulm_attn_bwd(do)");
  }
  if (a->mode & 4) {
    ULM_MAP(q64, q, q_sb, q_sh, q_ss, BT, "ulm_attn_bwd(q)");
    ULM_MAP(k128, k, k_sb, k_sh, k_ss, BR, "ulm_attn_bwd(k)");
    ULM_MAP(v128, v, v_sb, v_sh, v_ss, BR, "ulm_attn_bwd(v)");
    ULM_MAP(do64, d_o, do_sb, do_sh, do_ss, BT, "ulm_attn_bwd(do)");
  }
  if ((a->mode & 3) == 3) ULM_MAP(o128, o, o_sb, o_sh, o_ss, BR, "ulm_attn_bwd(o)");   // the dQ kernel computes delta itself
#undef ULM_MAP
  if (a->dtype == ULM_F16) return rope ? dispatch_bwd<__half, true>(a, dev.device, m) : dispatch_bwd<__half, false>(a, dev.device, m);
  return rope ? dispatch_bwd<__nv_bfloat16, true>(a, dev.device, m) : dispatch_bwd<__nv_bfloat16, false>(a, dev.device, m);
}
