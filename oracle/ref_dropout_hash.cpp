// Host-callable handle on the reference's own dropout hash.
//
// The keep-mask of the reference's attention kernels is a pure integer function that
// lives in a CUDA header of the reference (csrc/flash_attn_v100/fa_common.cuh:21-38:
// hash_u32, dropout_keep).  The header is plain C++ apart from the __device__
// qualifier, which a host compiler ignores, so this file includes it where it lies
// and exports the two functions with C linkage.  Test infrastructure only: the
// resulting library pins oracle/ops.py's numpy restatement (and, through the committed
// fixture made from it, the CUDA kernels' masks).  No reference source is copied here.
#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include "fa_common.cuh"   // found through -I <reference>/csrc/flash_attn_v100

extern "C" unsigned int ref_hash_u32(unsigned int x) { return fav100::hash_u32(x); }

extern "C" int ref_dropout_keep(unsigned int seed, int row, int col, unsigned int bh, float p) {
  return fav100::dropout_keep(seed, row, col, bh, p) ? 1 : 0;
}

// keep[r * ncols + c] for rows [row0, row0 + nrows) x cols [col0, col0 + ncols)
extern "C" void ref_dropout_keep_block(unsigned int seed, unsigned int bh, float p, int row0, int nrows,
                                       int col0, int ncols, unsigned char* keep) {
  for (int r = 0; r < nrows; ++r)
    for (int c = 0; c < ncols; ++c)
      keep[(long)r * ncols + c] = fav100::dropout_keep(seed, row0 + r, col0 + c, bh, p) ? 1 : 0;
}
