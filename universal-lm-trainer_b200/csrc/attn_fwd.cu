// Causal FlashAttention-2 forward for head_dim 64 on sm_100a.
//
// Replaces fa_fwd_kernel of the reference (csrc/flash_attn_v100/
// flash_attn_v100.cu:40-309): same math (online softmax in the log2 domain with
// the scale folded in, fp32 accumulation, undropped softmax denominator, natural
// log LSE), different machine.
//
// One CTA owns 128 query rows of one (batch, head) and walks key tiles of 64 up
// to the diagonal.  Three roles:
//   warp 8 (one lane)  TMA producer: Q once, then K and V tiles of 64 keys into a
//                      4-deep ring (128-byte swizzle, rows past S read as 0).
//   warp 9 (one lane)  tcgen05 issuer: S = Q K^T (128x64x64, both operands in
//                      shared memory) into one of TWO TMEM score buffers, always one
//                      tile ahead of the softmax; then O_a += P_a V[0:32) and
//                      O_b += P_b V[32:64) with P read from TMEM and V as an MN-major
//                      shared operand.
//   warps 0-7          softmax.  Query row r (TMEM lane r) is shared by two threads:
//                      warp r/32 takes keys [0,32) of every tile, warp r/32 + 4 keys
//                      [32,64).  Each runs its OWN online softmax (own running max,
//                      own denominator, own accumulator O_a / O_b), so the two never
//                      exchange anything per tile; the epilogue merges the halves as
//                      O = (O_a 2^(m_a-m) + O_b 2^(m_b-m)) / (l_a 2^(m_a-m) + l_b 2^(m_b-m)).
//                      Exponentials are taken against the running max while the
//                      tile's own max is still being collected and are redone (and
//                      the accumulator rescaled in TMEM) only when a row max grew by
//                      more than 2^8; the final 1/l normalisation makes the result
//                      identical.  P is written back over S as packed 16-bit.
// TMEM: S/P buffers at columns [0,64) and [64,128), O_a at [128,192), O_b at
// [192,256); two CTAs share an SM, which puts four softmax warps on every
// scheduler to keep the SFU (one exp2 per score) busy.
// Fused RoPE (template parameter ROPE): Q arrives unrotated; the softmax warps rotate
// the resident tile in shared memory right after its TMA load (two threads per row,
// the arithmetic of rope_math.cuh, so the bits equal the stand-alone kernel's), make
// the writes visible to the tensor core's shared-memory reads with a proxy fence and
// release the MMA issuer; the rotated tile is also written out for the backward.  A
// Q tile belongs to exactly one CTA, so nothing is rotated twice.  K tiles are read by
// every query tile of their head and therefore come rotated by the stand-alone kernel.
// Every barrier wait is bounded; on expiry the CTA records a status bit, drains
// its loads, frees TMEM and returns.  Waits of the softmax warps are made warp-uniform
// by a vote, because warp-wide instructions (TMEM loads, votes) follow them.
#include "tc.cuh"
#include "rope_math.cuh"

namespace ulm {
namespace {

using namespace tc;

constexpr int BM = 128;            // query rows per CTA
constexpr int BN = 64;             // keys per tile
constexpr int HD = 64;             // head_dim
constexpr int kStages = 4;
constexpr int kThreads = 320;           // 8 softmax warps, producer warp, MMA warp
constexpr uint32_t kQBytes = BM * HD * 2;     // 16 KB
constexpr uint32_t kTileBytes = BN * HD * 2;  //  8 KB (one K or V tile)
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;    // score buffer b at kColS + 64*b; accumulator of key half h at kColO + 64*h
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleGap = 8.0f;   // log2 units a row max may lag before O is rescaled

struct Ctl {
  uint64_t q_full, q_ready, k_full[kStages], v_full[kStages], kv_empty[kStages], s_full[2], p_ready[2], o_done;
  uint32_t tmem_base;
  int abort;
  uint32_t fail_bits;
  float m_half[2][BM], l_half[2][BM];   // the two per-row softmax states, exchanged once before the epilogue
};
constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + kQBytes + (size_t)kTileBytes * 2 * kStages + sizeof(Ctl);

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU;
  x ^= x >> 15; x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}
// keep mask of the reference (fa_common.cuh:30-38): a pure function of
// (seed, query row, key column, batch*head)
__device__ __forceinline__ bool dropout_keep(uint32_t seed_mix, int row, int col, float p) {
  uint32_t h = seed_mix ^ ((uint32_t)(row + 1) * 0x85EBCA6Bu) ^ ((uint32_t)(col + 1) * 0xC2B2AE35u);
  h = hash_u32(h);
  return ((h >> 8) * (1.0f / 16777216.0f)) >= p;
}

// Tables and destination of the fused Q rotation (unused when ROPE is false).
struct RopeQ {
  const float* cos_tab; const float* sin_tab;
  int64_t cos_stride, sin_stride;
  void* q_rot;
  int64_t sb, sh, ss;
};

// All lanes of a warp learn together whether the wait succeeded.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}

template <typename T, bool CAUSAL, bool DROPOUT, bool ROPE>
__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, T* __restrict__ O, float* __restrict__ LSE,
                int64_t o_sb, int64_t o_sh, int64_t o_ss, int S, int H, float scale2,
                float dropout_p, uint32_t seed, uint32_t* status, const RopeQ rq) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sKV = base + kQBytes;                        // [stage][K|V]
  Ctl* ctl = reinterpret_cast<Ctl*>(sKV + (size_t)kTileBytes * 2 * kStages);
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, b = bh / H, h = bh % H;
  const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;   // heaviest (latest) query tiles are scheduled first
  const int m0 = qt * BM;
  const int n_tiles_all = (S + BN - 1) / BN;
  const int n_causal = (m0 + BM) / BN;                   // key tiles that reach this tile's last row
  const int nkv = CAUSAL ? (n_causal < n_tiles_all ? n_causal : n_tiles_all) : n_tiles_all;

  // Fused RoPE: the 256 softmax threads rotate the Q tile with EIGHT threads per row (rope_math.cuh), four
  // rows per thread: task j of thread t is row 32 j + t / 8, column group t % 8.  They fetch their table
  // values first of all, so that the loads' latency runs under the barrier set-up, the TMEM allocation and
  // the Q tile's TMA load.
  [[maybe_unused]] RopeQuad rope_tab[4];
  if constexpr (ROPE) {
    if (warp < 8) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row = m0 + 32 * j + ((int)threadIdx.x >> 3);
        const int srow = row < S ? row : S - 1;          // rows past S are zero-filled by TMA; any table row does
        rope_load_quad(rope_tab[j], rq.cos_tab + (int64_t)srow * rq.cos_stride, rq.sin_tab + (int64_t)srow * rq.sin_stride,
                       (int)threadIdx.x & 7);
      }
    }
  }
  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->q_ready, 256);
    for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->k_full[s], 1); mbar_init(&ctl->v_full[s], 1); mbar_init(&ctl->kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&ctl->s_full[i], 1); mbar_init(&ctl->p_ready[i], 256); }
    mbar_init(&ctl->o_done, 1);
    ctl->abort = 0;
    ctl->fail_bits = 0;
    fence_mbar_init();
  }
  if (warp == 9) { tmem_alloc(&ctl->tmem_base, kTmemCols); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(&ctl->q_full, kQBytes);
      tma_load_4d(sQ, &tmQ, &ctl->q_full, 0, m0, h, b);
      int issued = 0;
      for (int j = 0; j < nkv; ++j) {
        const int s = j % kStages;
        if (j >= kStages && !mbar_wait(&ctl->kv_empty[s], ((j / kStages) - 1) & 1, abort_flag)) {
          atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA);
          break;
        }
        uint8_t* k_dst = sKV + (size_t)s * 2 * kTileBytes;
        mbar_expect_tx(&ctl->k_full[s], kTileBytes);
        tma_load_4d(k_dst, &tmK, &ctl->k_full[s], 0, j * BN, h, b);
        mbar_expect_tx(&ctl->v_full[s], kTileBytes);
        tma_load_4d(k_dst + kTileBytes, &tmV, &ctl->v_full[s], 0, j * BN, h, b);
        issued = j + 1;
      }
      if (*abort_flag) {   // let our own copies land before the CTA's shared memory goes away
        mbar_wait(&ctl->q_full, 0, abort_flag);
        for (int j = issued > kStages ? issued - kStages : 0; j < issued; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!(mbar_try(&ctl->k_full[j % kStages], (j / kStages) & 1) && mbar_try(&ctl->v_full[j % kStages], (j / kStages) & 1)))
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr int fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc(fmt, BM, BN, 0);
      constexpr uint32_t idesc_o = make_idesc(fmt, BM, HD, 1);
      const uint32_t tS = tmem_base + kColS, tO = tmem_base + kColO;
      // with the fused rotation the tile is usable once the softmax warps have rewritten it
      bool ok = ROPE ? mbar_wait(&ctl->q_ready, 0, abort_flag) : mbar_wait(&ctl->q_full, 0, abort_flag);
      if (!ok) atomicOr(&ctl->fail_bits, (uint32_t)(ROPE ? ULM_STATUS_TIMEOUT_SOFTMAX : ULM_STATUS_TIMEOUT_LOAD));
      fence_after_sync();
      const uint64_t dq = make_sdesc_sw128(smem_u32(sQ));
      auto issue_scores = [&](int j) -> bool {             // S_j = Q K_j^T into score buffer j & 1
        const int s = j % kStages;
        if (!mbar_wait(&ctl->k_full[s], (j / kStages) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD); return false; }
        fence_after_sync();
        const uint64_t dk = make_sdesc_sw128(smem_u32(sKV + (size_t)s * 2 * kTileBytes));
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)             // 32 bytes along the row per K=16 step
          mma_ss(tS + (uint32_t)((j & 1) * BN), dq + (uint64_t)(kk * 2), dk + (uint64_t)(kk * 2), idesc_s, kk > 0);
        mma_commit(&ctl->s_full[j & 1]);
        return true;
      };
      if (ok && nkv > 0) ok = issue_scores(0);
      for (int j = 0; ok && j < nkv; ++j) {
        const int s = j % kStages;
        // scores of the next tile first: its buffer last held P_{j-1}, whose P V was issued an
        // iteration ago (tcgen05.mma executes in issue order)
        if (j + 1 < nkv && !issue_scores(j + 1)) break;
        if (!mbar_wait(&ctl->p_ready[j & 1], (j >> 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_SOFTMAX); break; }
        if (!mbar_wait(&ctl->v_full[s], (j / kStages) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD); break; }
        fence_after_sync();
        const uint64_t dv = make_sdesc_sw128(smem_u32(sKV + (size_t)s * 2 * kTileBytes + kTileBytes));
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {           // 16 keys = 2048 bytes of V per step; P: 8 TMEM columns
          const int hf = kk >> 1;                        // keys [0,32) feed O_a, keys [32,64) feed O_b
          mma_ts(tO + (uint32_t)(hf * HD), tS + (uint32_t)((j & 1) * BN + hf * 32 + (kk & 1) * 8),
                 dv + (uint64_t)(kk * (2048 >> 4)), idesc_o, (j > 0 || (kk & 1)) ? 1u : 0u);
        }
        mma_commit(&ctl->kv_empty[s]);
      }
      mma_commit(&ctl->o_done);
    }
  } else {
    // ------------------------------ softmax warps -----------------------------
    const int sw = warp & 3, hf = warp >> 2;             // TMEM sub-partition; key half of every tile
    const int r = sw * 32 + lane;                        // row within the tile == TMEM lane
    const int grow = m0 + r;
    const uint32_t t_row = tmem_base + ((uint32_t)(sw * 32) << 16);
    const uint32_t t_acc = t_row + kColO + (uint32_t)(hf * HD);
    const uint32_t seed_mix = (seed * 0x9E3779B1u) ^ (((uint32_t)bh + 1u) * 0x27D4EB2Fu);
    const float inv_keep = DROPOUT ? 1.f / (1.f - dropout_p) : 1.f;
    const uint64_t sc2 = f2_pack(scale2, scale2);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    if constexpr (ROPE) {
      // Rotate the resident Q tile in place (128-byte-swizzled rows) and write the rotated rows out.
      ok = warp_wait(&ctl->q_full, 0, abort_flag);
      if (!ok && lane == 0) atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD);
      if (ok) {
        const int cg = (int)threadIdx.x & 7;
        T* qr_base = rq.q_rot ? reinterpret_cast<T*>(rq.q_rot) + (int64_t)b * rq.sb + (int64_t)h * rq.sh : nullptr;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = 32 * j + ((int)threadIdx.x >> 3);
          uint2* p_lo = reinterpret_cast<uint2*>(sQ + swz_quad_offset(row, cg));
          uint2* p_hi = reinterpret_cast<uint2*>(sQ + swz_quad_offset(row, cg + 8));
          uint2 olo, ohi;
          rope_apply_quad<T, false>(rope_tab[j], *p_lo, *p_hi, olo, ohi);
          *p_lo = olo;
          *p_hi = ohi;
          if (qr_base && m0 + row < S) {
            T* dst = qr_base + (int64_t)(m0 + row) * rq.ss;
            *reinterpret_cast<uint2*>(dst + 4 * cg) = olo;
            *reinterpret_cast<uint2*>(dst + 32 + 4 * cg) = ohi;
          }
        }
        // generic-proxy writes -> visible to the tensor core's (async proxy) operand reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&ctl->q_ready);
      }
    }
    uint32_t sv[32];
    for (int j = 0; ok && j < nkv; ++j) {
      const uint32_t t_s = t_row + kColS + (uint32_t)((j & 1) * BN + hf * 32);
      if (!warp_wait(&ctl->s_full[j & 1], (j >> 1) & 1, abort_flag)) { if (lane == 0) atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA); ok = false; break; }
      fence_after_sync();
      tmem_ld32(t_s, sv);
      tmem_wait_ld();
      const int c0 = j * BN + hf * 32;                   // first key of this thread's half tile
      if ((CAUSAL && c0 + 31 > m0 + sw * 32) || (c0 + 32 > S)) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int col = c0 + c;
          const bool valid = (col < S) && (!CAUSAL || col <= grow);
          if (!valid) sv[c] = 0xff800000u;               // -inf: comes out of exp2 as an exact zero
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};                   // four chains of two-wide partial sums
      uint32_t pk[16];
      // P = 2^(S*scale - mm) for the half tile, packed to 16 bits (mm = 0 while the half has seen
      // no unmasked key: every score is -inf then and P is all zeros)
      auto exp_pass = [&](const float mm, const bool with_max) {
        const float neg = mm == -INFINITY ? 0.f : -mm;
        const uint64_t nm2 = f2_pack(neg, neg);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float s0 = __uint_as_float(sv[c]), s1 = __uint_as_float(sv[c + 1]);
          if (with_max) mx4[(c >> 1) & 3] = fmax3(mx4[(c >> 1) & 3], s0, s1);
          float x0, x1;
          f2_unpack(f2_fma(f2_pack(s0, s1), sc2, nm2), x0, x1);
          float p0 = ex2(x0), p1 = ex2(x1);
          sum2[(c >> 1) & 3] = f2_add(sum2[(c >> 1) & 3], f2_pack(p0, p1));
          if (DROPOUT) {
            p0 = dropout_keep(seed_mix, grow, c0 + c, dropout_p) ? p0 * inv_keep : 0.f;
            p1 = dropout_keep(seed_mix, grow, c0 + c + 1, dropout_p) ? p1 * inv_keep : 0.f;
          }
          pk[c >> 1] = Cvt<T>::pack2(p0, p1);
        }
      };
      if (j > 0) {
        exp_pass(m, true);                               // optimistic: against the running max
      } else {
#pragma unroll
        for (int c = 0; c < 32; c += 2) mx4[(c >> 1) & 3] = fmaxf(mx4[(c >> 1) & 3], fmaxf(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])));
      }
      const float ms = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale2;
      if (j == 0 || __any_sync(0xffffffffu, ms > m + kRescaleGap)) {
        const float mn = fmaxf(m, ms);
        if (j > 0) {
          const float alpha = mn == -INFINITY ? 1.f : ex2(m - mn);
          l *= alpha;
          // O may only be touched once P_{j-1} V has finished: its completion released stage (j-1)
          if (!warp_wait(&ctl->kv_empty[(j - 1) % kStages], ((j - 1) / kStages) & 1, abort_flag)) {
            if (lane == 0) atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA);
            ok = false; break;
          }
          fence_after_sync();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t ov[16];
            tmem_ld16(t_acc + q4 * 16, ov);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 16; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * alpha);
            st16(t_acc + q4 * 16, ov);
          }
        }
        m = mn;
        sum2[0] = sum2[1] = sum2[2] = sum2[3] = 0ull;
        exp_pass(m, false);
      }
      st16(t_s, pk);
      {
        float a0, a1;
        f2_unpack(f2_add(f2_add(sum2[0], sum2[1]), f2_add(sum2[2], sum2[3])), a0, a1);
        l += a0 + a1;
      }
      tmem_wait_st();
      fence_before_sync();
      mbar_arrive(&ctl->p_ready[j & 1]);
    }
    // epilogue: merge the two key halves, O / l -> 16-bit, LSE
    ctl->m_half[hf][r] = m;
    ctl->l_half[hf][r] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");      // the eight softmax warps only
    if (ok && !warp_wait(&ctl->o_done, 0, abort_flag)) { if (lane == 0) atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA); ok = false; }
    if (ok) {
      fence_after_sync();
      const float m_a = ctl->m_half[0][r], m_b = ctl->m_half[1][r];
      const float m_all = fmaxf(m_a, m_b);                // finite: key 0 is visible to every row
      const float w_a = ex2(m_a - m_all), w_b = ex2(m_b - m_all);   // 2^-inf = 0 for a half that saw no key
      const float l_all = ctl->l_half[0][r] * w_a + ctl->l_half[1][r] * w_b;
      const float inv_l = 1.f / l_all;
      const float f_a = w_a * inv_l, f_b = w_b * inv_l;
      // this thread writes head dims [32 hf, 32 hf + 32) of its row
      T* orow = O + (int64_t)b * o_sb + (int64_t)h * o_sh + (int64_t)grow * o_ss + hf * 32;
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        uint32_t oa[16], ob[16];
        tmem_ld16(t_row + kColO + (uint32_t)(hf * 32 + q2 * 16), oa);
        tmem_ld16(t_row + kColO + (uint32_t)(HD + hf * 32 + q2 * 16), ob);
        tmem_wait_ld();
        if (grow < S) {
          float y[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) y[c] = fmaf(__uint_as_float(oa[c]), f_a, __uint_as_float(ob[c]) * f_b);
#pragma unroll
          for (int v4 = 0; v4 < 2; ++v4) {
            uint4 u;
            u.x = Cvt<T>::pack2(y[v4 * 8 + 0], y[v4 * 8 + 1]);
            u.y = Cvt<T>::pack2(y[v4 * 8 + 2], y[v4 * 8 + 3]);
            u.z = Cvt<T>::pack2(y[v4 * 8 + 4], y[v4 * 8 + 5]);
            u.w = Cvt<T>::pack2(y[v4 * 8 + 6], y[v4 * 8 + 7]);
            *reinterpret_cast<uint4*>(orow + q2 * 16 + v4 * 8) = u;
          }
        }
      }
      if (hf == 0 && grow < S) LSE[(int64_t)bh * S + grow] = (m_all + log2f(l_all)) * kLn2;
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && ctl->fail_bits && status) atomicOr(status, ctl->fail_bits);
}

template <typename T, bool CAUSAL, bool DROPOUT, bool ROPE>
int launch(const ulm_attn_fwd_args* a, int device, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv) {
  static std::atomic<bool> attr_set[kMaxDevices];
  auto kern = attn_fwd_kernel<T, CAUSAL, DROPOUT, ROPE>;
  if (int rc = ensure_smem_attr(kern, kSmemBytes, device, attr_set, "ulm_attn_fwd")) return rc;
  RopeQ rq{};
  if (ROPE) rq = RopeQ{a->cos_tab, a->sin_tab, a->cos_stride, a->sin_stride, a->q_rot, a->qr_sb, a->qr_sh, a->qr_ss};
  dim3 grid((unsigned)(a->B * a->H), (unsigned)((a->S + BM - 1) / BM));
  kern<<<grid, kThreads, kSmemBytes, (cudaStream_t)a->stream>>>(
      mq, mk, mv, (T*)a->o, a->lse, a->o_sb, a->o_sh, a->o_ss, a->S, a->H,
      a->softmax_scale * kLog2e, a->dropout_p, a->seed, a->status_dev, rq);
  return check_launch("ulm_attn_fwd");
}

template <typename T, bool ROPE>
int dispatch(const ulm_attn_fwd_args* a, int device, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv) {
  const bool drop = a->dropout_p > 0.f;
  if (a->causal) return drop ? launch<T, true, true, ROPE>(a, device, mq, mk, mv) : launch<T, true, false, ROPE>(a, device, mq, mk, mv);
  return drop ? launch<T, false, true, ROPE>(a, device, mq, mk, mv) : launch<T, false, false, ROPE>(a, device, mq, mk, mv);
}

}  // namespace
}  // namespace ulm

extern "C" int ulm_attn_fwd(const ulm_attn_fwd_args* a) {
  using namespace ulm;
  if (!a) return fail(ULM_ERR_ARG, "ulm_attn_fwd: null args");
  if (a->dtype != ULM_F16 && a->dtype != ULM_BF16) return fail(ULM_ERR_ARG, "ulm_attn_fwd: dtype must be f16 or bf16");
  if (a->B < 0 || a->H < 0 || a->S < 0) return fail(ULM_ERR_ARG, "ulm_attn_fwd: negative size");
  if (a->B == 0 || a->H == 0 || a->S == 0) return ULM_OK;
  if (!a->q || !a->k || !a->v || !a->o || !a->lse) return fail(ULM_ERR_ARG, "ulm_attn_fwd: null tensor");
  if (!(a->softmax_scale > 0.f)) return fail(ULM_ERR_ARG, "ulm_attn_fwd: softmax_scale must be positive");
  if (a->dropout_p < 0.f || a->dropout_p >= 1.f) return fail(ULM_ERR_ARG, "ulm_attn_fwd: dropout_p must be in [0,1)");
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) || a->o_sb % 8 || a->o_sh % 8 || a->o_ss % 8)
    return fail(ULM_ERR_ARG, "ulm_attn_fwd: o must be 16-byte aligned with strides that are multiples of 8");
  if ((int64_t)a->B * a->H > 0x7fffffffLL || (a->S + BM - 1) / BM > 65535) return fail(ULM_ERR_TOO_LARGE, "ulm_attn_fwd: grid too large");
  const bool rope = a->cos_tab || a->sin_tab;
  if (rope) {
    if (!a->cos_tab || !a->sin_tab) return fail(ULM_ERR_ARG, "ulm_attn_fwd: cos_tab and sin_tab must be given together");
    if ((reinterpret_cast<uintptr_t>(a->cos_tab) & 15) || (reinterpret_cast<uintptr_t>(a->sin_tab) & 15) || a->cos_stride % 4 || a->sin_stride % 4 ||
        a->cos_stride < 64 || a->sin_stride < 64)
      return fail(ULM_ERR_ARG, "ulm_attn_fwd: RoPE tables must be 16-byte aligned with row strides that are multiples of 4 floats, at least 64");
    if (a->q_rot && ((reinterpret_cast<uintptr_t>(a->q_rot) & 15) || a->qr_sb % 8 || a->qr_sh % 8 || a->qr_ss % 8))
      return fail(ULM_ERR_ARG, "ulm_attn_fwd: q_rot must be 16-byte aligned with strides that are multiples of 8");
  }
  tc::DeviceScope dev(a->q, "ulm_attn_fwd");
  if (dev.rc) return dev.rc;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = tc::encode_bhsd_map(&mq, a->q, a->dtype, a->B, a->H, a->S, a->q_sb, a->q_sh, a->q_ss, BM, "ulm_attn_fwd(q)"))) return rc;
  if ((rc = tc::encode_bhsd_map(&mk, a->k, a->dtype, a->B, a->H, a->S, a->k_sb, a->k_sh, a->k_ss, BN, "ulm_attn_fwd(k)"))) return rc;
  if ((rc = tc::encode_bhsd_map(&mv, a->v, a->dtype, a->B, a->H, a->S, a->v_sb, a->v_sh, a->v_ss, BN, "ulm_attn_fwd(v)"))) return rc;
  if (a->dtype == ULM_F16) return rope ? dispatch<__half, true>(a, dev.device, mq, mk, mv) : dispatch<__half, false>(a, dev.device, mq, mk, mv);
  return rope ? dispatch<__nv_bfloat16, true>(a, dev.device, mq, mk, mv) : dispatch<__nv_bfloat16, false>(a, dev.device, mq, mk, mv);
}
