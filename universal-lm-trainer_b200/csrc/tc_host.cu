// Host side of the TMA plumbing: fetches cuTensorMapEncodeTiled from the driver
// at run time, encodes maps for (B,H,S,64) 16-bit tensors and caches them.
#include "tc.cuh"

#include <cudaTypedefs.h>
#include <cstring>
#include <mutex>
#include <unordered_map>

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

// ---- cache of encoded maps --------------------------------------------------
struct MapKey {
  const void* base;
  int64_t sb, sh, ss;
  int32_t dtype, B, H, S, box_rows, pad;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    uint64_t h = 0x9E3779B97F4A7C15ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) { h ^= w[i]; h *= 0xBF58476D1CE4E5B9ull; h ^= h >> 29; }
    return (size_t)h;
  }
};
static_assert(sizeof(MapKey) % 8 == 0, "hashed as 64-bit words");
constexpr size_t kCacheMax = 8192;       // 8192 x ~200 B; cleared wholesale when full
std::mutex g_cache_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash>& cache() {
  static auto* m = new std::unordered_map<MapKey, CUtensorMap, MapKeyHash>();   // never destroyed: no exit-order hazards
  return *m;
}
std::atomic<uint64_t> g_cache_hits{0}, g_cache_misses{0};

}  // namespace

DeviceScope::DeviceScope(const void* dev_ptr, const char* what) : rc(ULM_OK), device(-1), previous(-1) {
  cudaPointerAttributes at;
  cudaError_t e = cudaPointerGetAttributes(&at, dev_ptr);
  if (e != cudaSuccess) { cudaGetLastError(); rc = fail(ULM_ERR_CUDA, "%s: cudaPointerGetAttributes: %s", what, cudaGetErrorString(e)); return; }
  if (at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged) { rc = fail(ULM_ERR_ARG, "%s: tensor is not in device memory", what); return; }
  device = at.device;
  int cur = -1;
  e = cudaGetDevice(&cur);
  if (e != cudaSuccess) { rc = fail(ULM_ERR_CUDA, "%s: cudaGetDevice: %s", what, cudaGetErrorString(e)); return; }
  // Also when the device already is the current one: cudaSetDevice binds its primary context to the calling
  // thread, and a thread that has made no runtime call of its own yet (an autograd worker whose first node is
  // one of ours, its outputs coming from cached allocator blocks) has none -- the tensor-map encoder is a driver
  // call and fails with "invalid context" there.
  e = cudaSetDevice(device);
  if (e != cudaSuccess) { rc = fail(ULM_ERR_CUDA, "%s: cudaSetDevice(%d): %s", what, device, cudaGetErrorString(e)); return; }
  if (cur != device) previous = cur;
}

DeviceScope::~DeviceScope() {
  if (previous >= 0) cudaSetDevice(previous);
}

void map_cache_stats(uint64_t* hits, uint64_t* misses) {
  *hits = g_cache_hits.load(std::memory_order_relaxed);
  *misses = g_cache_misses.load(std::memory_order_relaxed);
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
  // a tensor map's strides must stay below 2^40 bytes; the stride of an extent-1 dimension is never applied
  if (B == 1 && sb * 2 >= (int64_t)1 << 40) sb = ss;
  if (H == 1 && sh * 2 >= (int64_t)1 << 40) sh = ss;
  if (ss < 64 || sh <= 0 || sb <= 0 || ss % 8 || sh % 8 || sb % 8)
    return fail(ULM_ERR_ARG, "%s: strides (%lld,%lld,%lld) must be positive multiples of 8 elements, rows at least 64 apart",
                what, (long long)sb, (long long)sh, (long long)ss);
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base; key.sb = sb; key.sh = sh; key.ss = ss;
  key.dtype = dtype; key.B = B; key.H = H; key.S = S; key.box_rows = box_rows;
  {
    std::lock_guard<std::mutex> lock(g_cache_mu);
    auto it = cache().find(key);
    if (it != cache().end()) {
      *out = it->second;
      g_cache_hits.fetch_add(1, std::memory_order_relaxed);
      return ULM_OK;
    }
  }
  const cuuint64_t dims[4] = {64, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == ULM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ULM_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  g_cache_misses.fetch_add(1, std::memory_order_relaxed);
  {
    std::lock_guard<std::mutex> lock(g_cache_mu);
    if (cache().size() >= kCacheMax) cache().clear();
    cache().emplace(key, *out);
  }
  return ULM_OK;
}

}  // namespace tc
}  // namespace ulm

// Hits and misses of the tensor-map cache since the library was loaded (diagnostics).
extern "C" void ulm_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses) {
  uint64_t h = 0, m = 0;
  ulm::tc::map_cache_stats(&h, &m);
  if (hits) *hits = h;
  if (misses) *misses = m;
}
