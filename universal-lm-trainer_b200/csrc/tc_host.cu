// Host side of the TMA plumbing: fetches cuTensorMapEncodeTiled from the driver
// at run time and encodes maps for (B,H,S,64) 16-bit tensors.
#include "tc.cuh"

#include <cudaTypedefs.h>
#include <mutex>

namespace ulm {
namespace tc {
namespace {

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_once;
cudaError_t g_once_err = cudaSuccess;

void fetch_entry_point() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  g_once_err = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &q);
  if (g_once_err == cudaSuccess && q == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

}  // namespace

int bind_device_of(const void* dev_ptr, const char* what) {
  cudaPointerAttributes at;
  cudaError_t e = cudaPointerGetAttributes(&at, dev_ptr);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(ULM_ERR_CUDA, "%s: cudaPointerGetAttributes: %s", what, cudaGetErrorString(e)); }
  if (at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged)
    return fail(ULM_ERR_ARG, "%s: tensor is not in device memory", what);
  e = cudaSetDevice(at.device);
  if (e != cudaSuccess) return fail(ULM_ERR_CUDA, "%s: cudaSetDevice(%d): %s", what, at.device, cudaGetErrorString(e));
  return ULM_OK;
}

int encode_bhsd_map(CUtensorMap* out, const void* base, int dtype, int B, int H, int S,
                    int64_t sb, int64_t sh, int64_t ss, int box_rows, const char* what) {
  std::call_once(g_once, fetch_entry_point);
  if (!g_encode) return fail(ULM_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available (%s)", what, cudaGetErrorString(g_once_err));
  if (reinterpret_cast<uintptr_t>(base) & 15) return fail(ULM_ERR_ARG, "%s: base pointer must be 16-byte aligned", what);
  // A dimension of extent 1 never advances, so its stride only has to be legal.
  const int64_t dense_s = 64;
  if (S == 1) ss = dense_s;
  if (H == 1) sh = (int64_t)S * ss;
  if (B == 1) sb = (int64_t)H * (sh > (int64_t)S * ss ? sh : (int64_t)S * ss);
  if (ss < 64 || sh <= 0 || sb <= 0 || ss % 8 || sh % 8 || sb % 8)
    return fail(ULM_ERR_ARG, "%s: strides (%lld,%lld,%lld) must be positive multiples of 8 elements, rows at least 64 apart",
                what, (long long)sb, (long long)sh, (long long)ss);
  const cuuint64_t dims[4] = {64, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == ULM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ULM_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return ULM_OK;
}

}  // namespace tc
}  // namespace ulm
