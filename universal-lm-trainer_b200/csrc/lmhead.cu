// lm-head GEMM with the cross-entropy statistics taken in its epilogue, for sm_100a.
//
// Replaces, for the forward of the loss, the pair "fc_out GEMM, then a pass over the logits for
// log-sum-exp" of the reference's chunk loop (train.py:2075-2079: `F.cross_entropy(self.fc_out(h), t)`):
//   logits[r, c] = sum_k H[r, k] W[c, k]          (16-bit operands, fp32 accumulation in TMEM)
//   z            = logits rounded to the 16-bit type (what the reference's autocast linear returns)
//   (m, s)[r, g] = running max and sum of 2^((z - m) log2 e) over the columns of column group g
// and, optionally, z written to global memory for the backward.  A second small kernel merges the
// per-group statistics into lse[r] and loss[r] = lse[r] - z[r, target[r]] (ulm_ce_fwd's outputs).
//
// Machine mapping.  Persistent CTAs (one per SM), 320 threads: warps 0-7 epilogue, warp 8 one-lane TMA
// producer, warp 9 one-lane tcgen05.mma issuer.  Output tile 128 rows x 256 columns: one
// tcgen05.mma.cta_group::1.kind::f16 M128 x N256 x K16 per 16 elements of the inner dimension, operands in
// 128-byte-swizzled shared memory (4 stages of a 128x64 H tile and a 256x64 W tile), two accumulators of 256
// TMEM columns so that the epilogue of one tile runs under the MMAs of the next.  Epilogue: thread = row
// (TMEM lane), two threads per row (128 columns each), in two passes of 64 columns: TMEM -> registers ->
// rounded to 16 bits -> a swizzled 128x64 staging tile -> one TMA store per pass and column half; the
// statistics are taken from the rounded values in registers.  A work item is (128 rows, a group of up to
// 25 column tiles): the running statistics stay in registers across the group's tiles; all CTAs sweep the
// same column group at the same time, so the W tiles are shared through L2.
// All barrier waits are bounded (status bit + clean exit on expiry), like the attention kernels'.
#include "tc.cuh"

namespace ulm {
namespace {

using namespace tc;

constexpr int LM_BM = 128, LM_BN = 256, LM_BK = 64;
constexpr int kLmStages = 4;
constexpr int kLmGroupTiles = 25;                      // column tiles per work item (upper bound)
constexpr uint32_t kLmATile = LM_BM * LM_BK * 2;       // 16 KB
constexpr uint32_t kLmBTile = LM_BN * LM_BK * 2;       // 32 KB
constexpr uint32_t kLmStage = kLmATile + kLmBTile;
constexpr uint32_t kLmStaging = 128 * 64 * 2;          // one 128-row x 64-column block of 16-bit logits
constexpr int kLmEpiWarps = 8;
constexpr int kLmThreads = (kLmEpiWarps + 2) * 32;
constexpr float kLmLog2e = 1.4426950408889634f;
constexpr float kLmLn2 = 0.6931471805599453f;

struct CtlLM {
  uint64_t full[kLmStages], empty[kLmStages], acc_full[2], acc_free[2];
  uint32_t tmem_base;
  int abort;
  uint32_t fail_bits;
};
constexpr size_t kLmCtlBytes = 1024;
static_assert(sizeof(CtlLM) <= kLmCtlBytes, "control block");
constexpr size_t kLmSmem = 1024 + (size_t)kLmStages * kLmStage + 2 * (size_t)kLmStaging + kLmCtlBytes;
static_assert(kLmSmem <= 227 * 1024, "shared memory");

template <typename T> struct LmFmt { static constexpr int v = 0; };
template <> struct LmFmt<__nv_bfloat16> { static constexpr int v = 1; };

// 4-D tiled store shared -> global (the counterpart of tma_load_4d), completion tracked by bulk groups
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Barrier over the 128 threads of one column half (ids 1, 2) whose OR-reduction tells every one of them
// whether any of them (or another role of the CTA) has given up.
__device__ __forceinline__ bool half_sync_any(int half, bool fail) {
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, %2, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(any) : "r"((uint32_t)fail), "r"(half + 1) : "memory");
  return any != 0;
}

struct LmItems {
  int n_rb, n_ct, n_groups, group_tiles;
  __host__ __device__ LmItems(int64_t rows, int V) {
    n_rb = (int)((rows + LM_BM - 1) / LM_BM);
    n_ct = (V + LM_BN - 1) / LM_BN;
    n_groups = (n_ct + kLmGroupTiles - 1) / kLmGroupTiles;
    group_tiles = (n_ct + n_groups - 1) / n_groups;
  }
  __host__ __device__ int n_items() const { return n_rb * n_groups; }
  // all CTAs are on one column group at a time: its W tiles are read from L2 by everyone
  __device__ void decode(int idx, int& rb, int& g, int& ct0, int& nct) const {
    g = idx / n_rb;
    rb = idx - g * n_rb;
    ct0 = g * group_tiles;
    nct = n_ct - ct0 < group_tiles ? n_ct - ct0 : group_tiles;
  }
};

template <typename T, bool KEEP>
__global__ void __launch_bounds__(kLmThreads, 1)
lmhead_lse_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmW,
                  const __grid_constant__ CUtensorMap tmZ, float* __restrict__ part_m, float* __restrict__ part_s,
                  int64_t rows, int V, int n_kb, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = base;                                             // [stage][H tile | W tile]
  uint8_t* staging = base + (size_t)kLmStages * kLmStage;             // [column half] one 128x64 block each
  CtlLM* ctl = reinterpret_cast<CtlLM*>(staging + 2 * (size_t)kLmStaging);
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const LmItems items(rows, V);
  const int n_items = items.n_items();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kLmStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&ctl->acc_full[b], 1); mbar_init(&ctl->acc_free[b], kLmEpiWarps * 32); }
    ctl->abort = 0;
    ctl->fail_bits = 0;
    fence_mbar_init();
  }
  if (warp == kLmEpiWarps + 1) { tmem_alloc(&ctl->tmem_base, 512); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == kLmEpiWarps) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmH); tma_prefetch_desc(&tmW);
      ItemIter it_items(n_items);
      uint32_t it = 0;                                   // k-blocks issued so far, over all tiles
      int idx;
      bool ok = true;
      while (ok && it_items.next(idx)) {
        int rb, g, ct0, nct;
        items.decode(idx, rb, g, ct0, nct);
        for (int t = 0; ok && t < nct; ++t) {
          for (int kb = 0; kb < n_kb; ++kb, ++it) {
            const uint32_t s = it % kLmStages;
            if (it >= (uint32_t)kLmStages && !mbar_wait(&ctl->empty[s], ((it / kLmStages) - 1) & 1, abort_flag)) {
              atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA);
              ok = false;
              break;
            }
            uint8_t* dst = stages + (size_t)s * kLmStage;
            mbar_expect_tx(&ctl->full[s], kLmStage);
            tma_load_4d(dst, &tmH, &ctl->full[s], 0, rb * LM_BM, kb, 0);
            tma_load_4d(dst + kLmATile, &tmW, &ctl->full[s], 0, (ct0 + t) * LM_BN, kb, 0);
          }
        }
      }
      if (*abort_flag) {   // let our own copies land before the CTA's shared memory goes away
        for (uint32_t u = it > (uint32_t)kLmStages ? it - kLmStages : 0; u < it; ++u) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try(&ctl->full[u % kLmStages], (u / kLmStages) & 1))
            if (globaltimer_ns() - t0 > kWaitLimitNs) break;
        }
      }
    }
  } else if (warp == kLmEpiWarps + 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(LmFmt<T>::v, LM_BM, LM_BN, 0);   // 128 x 256, both operands K-major
      ItemIter it_items(n_items);
      uint32_t it = 0, tt = 0;                           // k-blocks / tiles so far
      int idx;
      bool ok = true;
      while (ok && it_items.next(idx)) {
        int rb, g, ct0, nct;
        items.decode(idx, rb, g, ct0, nct);
        for (int t = 0; ok && t < nct; ++t, ++tt) {
          const uint32_t b = tt & 1;
          // the accumulator still holds tile tt-2 until the epilogue warps have read it
          if (tt >= 2 && !mbar_wait(&ctl->acc_free[b], ((tt >> 1) - 1) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_SOFTMAX); ok = false; break; }
          fence_after_sync();
          for (int kb = 0; kb < n_kb; ++kb, ++it) {
            const uint32_t s = it % kLmStages;
            if (!mbar_wait(&ctl->full[s], (it / kLmStages) & 1, abort_flag)) { atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD); ok = false; break; }
            fence_after_sync();
            const uint64_t da = make_sdesc_sw128(smem_u32(stages + (size_t)s * kLmStage));
            const uint64_t db = make_sdesc_sw128(smem_u32(stages + (size_t)s * kLmStage + kLmATile));
#pragma unroll
            for (int kk = 0; kk < LM_BK / 16; ++kk)
              mma_ss(tmem_base + b * LM_BN, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            mma_commit(&ctl->empty[s]);                  // the stage is free once these MMAs have read it
          }
          if (ok) mma_commit(&ctl->acc_full[b]);
        }
      }
    }
  } else {
    // ---------------- epilogue: statistics and (KEEP) the rounded logits ----------------
    const int half = warp >> 2;                          // columns [128 half, 128 half + 128) of the tile
    const int r = ((warp & 3) << 5) | lane;              // row within the tile == TMEM lane
    const int tg = (int)threadIdx.x - half * 128;        // thread within its half (0..127)
    const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    uint8_t* my_staging = staging + (size_t)half * kLmStaging;
    ItemIter it_items(n_items);
    uint32_t tt = 0;
    int idx;
    bool ok = true;
    while (ok && it_items.next(idx)) {
      int rb, g, ct0, nct;
      items.decode(idx, rb, g, ct0, nct);
      float m = -INFINITY, ssum = 0.f;                   // base-2 domain: m = max(z) * log2e
      for (int t = 0; ok && t < nct; ++t, ++tt) {
        const uint32_t b = tt & 1;
        const bool waited = __all_sync(0xffffffffu, mbar_wait(&ctl->acc_full[b], (tt >> 1) & 1, abort_flag));
        if (!waited && lane == 0) atomicOr(&ctl->fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_MMA);
        // every thread of the half learns the same verdict (a barrier follows inside the passes)
        if (half_sync_any(half, !waited || *abort_flag != 0)) { ok = false; break; }
        fence_after_sync();
        const int col_tile = (ct0 + t) * LM_BN;
#pragma unroll 1
        for (int pass = 0; pass < 2; ++pass) {
          const int c_blk = half * 128 + pass * 64;      // first column of this pass within the tile
          uint32_t acc[64];
          tmem_ld32(t_row + b * LM_BN + c_blk, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
          tmem_ld32(t_row + b * LM_BN + c_blk + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
          tmem_wait_ld();
          if (pass == 1) {                               // everything of this tile is in registers: hand the accumulator back
            fence_before_sync();
            mbar_arrive(&ctl->acc_free[b]);
          }
          // round to 16 bits (what the reference's linear returns), keep both forms
          uint32_t pk[32];
          float mx = -INFINITY;
          const int col0 = col_tile + c_blk;
          const bool edge = col0 + 64 > V;
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            pk[c >> 1] = Cvt<T>::pack2(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]));
            float2 z = Cvt<T>::unpack2(pk[c >> 1]);
            if (edge) {
              if (col0 + c >= V) z.x = -INFINITY;
              if (col0 + c + 1 >= V) z.y = -INFINITY;
            }
            acc[c] = __float_as_uint(z.x);
            acc[c + 1] = __float_as_uint(z.y);
            mx = fmaxf(mx, fmaxf(z.x, z.y));
          }
          if (KEEP) {
            // the previous store out of this staging block must have read it
            if (tg == 0) bulk_wait_read0();
            if (half_sync_any(half, *abort_flag != 0)) { ok = false; break; }
            // row r of a 128-byte-swizzled block: 16-byte chunk c sits at chunk position c ^ (r & 7)
            uint8_t* row = my_staging + (size_t)r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            fence_proxy_async_smem();
            if (half_sync_any(half, *abort_flag != 0)) { ok = false; break; }
            if (tg == 0) {
              tma_store_4d(&tmZ, my_staging, 0, rb * LM_BM, (col_tile + c_blk) >> 6, 0);
              bulk_commit();
            }
          }
          // running statistics over the rounded values
          const float m_new = fmaxf(m, mx * kLmLog2e);
          if (m_new > -INFINITY) {
            ssum *= ex2(m - m_new);                      // 2^(-inf) = 0 on the first tile
            const float nm = -m_new;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
              s0 += ex2(fmaf(__uint_as_float(acc[c]), kLmLog2e, nm));
              s1 += ex2(fmaf(__uint_as_float(acc[c + 1]), kLmLog2e, nm));
              s2 += ex2(fmaf(__uint_as_float(acc[c + 2]), kLmLog2e, nm));
              s3 += ex2(fmaf(__uint_as_float(acc[c + 3]), kLmLog2e, nm));
            }
            ssum += (s0 + s1) + (s2 + s3);
            m = m_new;
          }
        }
      }
      if (!ok) break;
      const int64_t grow = (int64_t)rb * LM_BM + r;
      if (grow < rows) {
        // [row][group][half]: the finishing kernel merges 2 * n_groups pairs per row
        const int64_t o = (grow * items.n_groups + g) * 2 + half;
        part_m[o] = m;
        part_s[o] = ssum;
      }
    }
    if (KEEP && tg == 0) bulk_wait0();                   // our stores must be complete before the CTA ends
  }

  fence_before_sync();
  __syncthreads();
  if (warp == kLmEpiWarps + 1) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && ctl->fail_bits && status) atomicOr(status, ctl->fail_bits);
}

// lse[r] = ln sum_c exp(z[r,c]) from the per-group (max, sum) pairs; loss[r] = lse[r] - z[r, target[r]]
// (0 for ignored rows), z read from the stored logits.  One thread per row.
template <typename T>
__global__ void lmhead_finish_kernel(const float* __restrict__ part_m, const float* __restrict__ part_s, int n_parts,
                                     const T* __restrict__ logits, int64_t row_stride, const int64_t* __restrict__ target,
                                     int64_t ignore_index, int V, float* __restrict__ lse, float* __restrict__ loss, int64_t rows) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY;
  for (int i = 0; i < n_parts; ++i) m = fmaxf(m, part_m[r * n_parts + i]);
  float s = 0.f;
  for (int i = 0; i < n_parts; ++i) {
    const float mi = part_m[r * n_parts + i];
    if (mi > -INFINITY) s += part_s[r * n_parts + i] * exp2f(mi - m);
  }
  const float l = (m + log2f(s)) * kLmLn2;
  lse[r] = l;
  if (loss) {
    const int64_t t = target[r];
    loss[r] = (t == ignore_index || t < 0 || t >= V) ? 0.f : l - Cvt<T>::to_f(logits[r * row_stride + t]);
  }
}

template <typename T, bool KEEP>
int launch_lmhead(const ulm_lmhead_lse_args* a, const CUtensorMap& mh, const CUtensorMap& mw, const CUtensorMap& mz, int device) {
  static std::atomic<bool> attr_set[kMaxDevices];
  auto kern = lmhead_lse_kernel<T, KEEP>;
  if (int rc = ensure_smem_attr(kern, kLmSmem, device, attr_set, "ulm_lmhead_lse")) return rc;
  const LmItems items(a->rows, a->V);
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int grid = items.n_items() < sms ? items.n_items() : sms;
  kern<<<grid, kLmThreads, kLmSmem, (cudaStream_t)a->stream>>>(mh, mw, mz, a->part_m, a->part_s, a->rows, a->V, a->d / LM_BK, a->status_dev);
  return ULM_OK;
}

}  // namespace
}  // namespace ulm

extern "C" int64_t ulm_lmhead_lse_parts(int32_t V) {
  const ulm::LmItems items(1, V);
  return 2 * (int64_t)items.n_groups;
}

extern "C" int ulm_lmhead_lse(const ulm_lmhead_lse_args* a) {
  using namespace ulm;
  const char* who = "ulm_lmhead_lse";
  if (!a) return fail(ULM_ERR_ARG, "%s: null args", who);
  if (a->dtype != ULM_F16 && a->dtype != ULM_BF16) return fail(ULM_ERR_ARG, "%s: dtype must be fp16 or bf16", who);
  if (a->rows < 0 || a->V <= 0 || a->d <= 0 || a->d % LM_BK) return fail(ULM_ERR_ARG, "%s: need rows >= 0, V > 0, d a positive multiple of %d", who, LM_BK);
  if (a->rows == 0) return ULM_OK;
  if (!a->h || !a->w || !a->part_m || !a->part_s || !a->lse) return fail(ULM_ERR_ARG, "%s: null tensor", who);
  if (a->h_stride < a->d || a->w_stride < a->d || a->h_stride % 8 || a->w_stride % 8)
    return fail(ULM_ERR_ARG, "%s: row strides must be multiples of 8 elements and at least d", who);
  const bool keep = a->logits != nullptr;
  if (a->loss && (!keep || !a->target)) return fail(ULM_ERR_ARG, "%s: loss needs the logits buffer and the targets", who);
  if (keep && (a->V % 64 || a->z_stride < a->V || a->z_stride % 8))
    return fail(ULM_ERR_ARG, "%s: storing the logits needs V a multiple of 64 and a row stride that is a multiple of 8 and at least V", who);
  tc::DeviceScope scope(a->h, who);
  if (scope.rc) return scope.rc;
  int rc;
  // the matrices as [row][block of 64 columns][64]: the tensor-map encoder's (S, H, 64) with B = 1
  CUtensorMap mh, mw, mz;
  const int n_kb = a->d / LM_BK;
  if ((rc = tc::encode_bhsd_map(&mh, a->h, a->dtype, 1, n_kb, (int)a->rows, 0, 64, a->h_stride, LM_BM, who))) return rc;
  if ((rc = tc::encode_bhsd_map(&mw, a->w, a->dtype, 1, n_kb, a->V, 0, 64, a->w_stride, LM_BN, who))) return rc;
  mz = mh;
  if (keep && (rc = tc::encode_bhsd_map(&mz, a->logits, a->dtype, 1, a->V / 64, (int)a->rows, 0, 64, a->z_stride, 128, who))) return rc;
  if (a->dtype == ULM_BF16) rc = keep ? launch_lmhead<__nv_bfloat16, true>(a, mh, mw, mz, scope.device) : launch_lmhead<__nv_bfloat16, false>(a, mh, mw, mz, scope.device);
  else rc = keep ? launch_lmhead<__half, true>(a, mh, mw, mz, scope.device) : launch_lmhead<__half, false>(a, mh, mw, mz, scope.device);
  if (rc) return rc;
  if ((rc = check_launch(who))) return rc;
  const int n_parts = (int)ulm_lmhead_lse_parts(a->V);
  const int threads = 128;
  const unsigned blocks = (unsigned)((a->rows + threads - 1) / threads);
  if (a->dtype == ULM_BF16)
    lmhead_finish_kernel<__nv_bfloat16><<<blocks, threads, 0, (cudaStream_t)a->stream>>>(
        a->part_m, a->part_s, n_parts, static_cast<const __nv_bfloat16*>(a->logits), a->z_stride, a->target, a->ignore_index, a->V, a->lse, a->loss, a->rows);
  else
    lmhead_finish_kernel<__half><<<blocks, threads, 0, (cudaStream_t)a->stream>>>(
        a->part_m, a->part_s, n_parts, static_cast<const __half*>(a->logits), a->z_stride, a->target, a->ignore_index, a->V, a->lse, a->loss, a->rows);
  return check_launch(who);
}
