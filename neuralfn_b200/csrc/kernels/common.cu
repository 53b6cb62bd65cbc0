// Library-wide host helpers: per-device status word, error strings, device facts,
// and the TMA tensor-map encoder (resolved from the driver at run time so the
// library links without libcuda).
#include "common.h"

#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>
#include <cstring>
#include <cstdio>

namespace nfn {

static __device__ int g_status_word[8];

static thread_local std::string g_last_error;
static std::atomic<long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

void set_last_error(const char* msg) { g_last_error = msg; }

int fail(int code, const char* msg) {
  g_last_error = msg;
  return code;
}

struct DeviceFacts {
  bool ready = false;
  int* status = nullptr;
  int sm_count = 0;
  int max_smem_optin = 0;
};
static DeviceFacts g_facts[64];
static std::mutex g_facts_mu;

static DeviceFacts& facts() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(g_facts_mu);
  DeviceFacts& f = g_facts[dev & 63];
  if (!f.ready) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) == cudaSuccess) f.status = static_cast<int*>(p);
    cudaDeviceGetAttribute(&f.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&f.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    f.ready = true;
  }
  return f;
}

int* status_ptr() { return facts().status; }
int sm_count() { return facts().sm_count; }
int max_smem_optin() { return facts().max_smem_optin; }

// ------------------------------------------------------------ tensor maps ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t d0, d1, d2, s1, s2;
  uint32_t b0, b1, b2, rank, esize, swz;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
static std::mutex g_maps_mu;

static bool encode_cached(CUtensorMap* out, const MapKey& key) {
  {
    std::lock_guard<std::mutex> lk(g_maps_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[3] = {key.d0, key.d1, key.d2};
  cuuint64_t strides[2] = {key.s1, key.s2};
  cuuint32_t box[3] = {key.b0, key.b1, key.b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = key.esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : key.esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUtensorMapSwizzle sw = key.swz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : key.swz == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : key.swz == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                          : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, key.rank, const_cast<void*>(key.ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof buf,
             "cuTensorMapEncodeTiled failed (%d): ptr=%p rank=%u dims=(%llu,%llu,%llu) "
             "strides=(%llu,%llu) box=(%u,%u,%u)",
             (int)r, key.ptr, key.rank, (unsigned long long)key.d0, (unsigned long long)key.d1,
             (unsigned long long)key.d2, (unsigned long long)key.s1, (unsigned long long)key.s2,
             key.b0, key.b1, key.b2);
    set_last_error(buf);
    return false;
  }
  std::lock_guard<std::mutex> lk(g_maps_mu);
  if (g_maps.size() > 8192) g_maps.clear();
  g_maps.emplace(key, *out);
  return true;
}

bool make_tmap_2d(CUtensorMap* out, const void* ptr, int elem_size, uint64_t inner,
                  uint64_t outer, uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer,
                  int swizzle_bytes) {
  MapKey key;
  std::memset(&key, 0, sizeof key);
  key.ptr = ptr;
  key.d0 = inner; key.d1 = outer; key.d2 = 1;
  key.s1 = ld_elems * (uint64_t)elem_size; key.s2 = 0;
  key.b0 = box_inner; key.b1 = box_outer; key.b2 = 1;
  key.rank = 2; key.esize = (uint32_t)elem_size; key.swz = (uint32_t)swizzle_bytes;
  return encode_cached(out, key);
}

bool make_tmap_3d(CUtensorMap* out, const void* ptr, int elem_size, uint64_t d0, uint64_t d1,
                  uint64_t d2, uint64_t stride1_elems, uint64_t stride2_elems, uint32_t b0,
                  uint32_t b1, uint32_t b2, int swizzle_bytes) {
  MapKey key;
  std::memset(&key, 0, sizeof key);
  key.ptr = ptr;
  key.d0 = d0; key.d1 = d1; key.d2 = d2;
  key.s1 = stride1_elems * (uint64_t)elem_size; key.s2 = stride2_elems * (uint64_t)elem_size;
  key.b0 = b0; key.b1 = b1; key.b2 = b2;
  key.rank = 3; key.esize = (uint32_t)elem_size; key.swz = (uint32_t)swizzle_bytes;
  return encode_cached(out, key);
}

}  // namespace nfn

extern "C" {

int nfn_abi_version(void) { return 1; }

int nfn_status_read_reset(void) {
  int* p = nfn::status_ptr();
  if (!p) return -1;
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

int nfn_status_peek(void) {
  int* p = nfn::status_ptr();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  return v;
}

// Test hook: overwrite the status word of the current device from the host (what a kernel's
// timed-out wait would have left there), so error handling can be exercised without a device fault.
int nfn_status_set(int code) {
  int* p = nfn::status_ptr();
  if (!p) return -1;
  return cudaMemcpy(p, &code, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -2;
}

const char* nfn_last_error(void) { return nfn::g_last_error.c_str(); }

long long nfn_launch_count(void) { return nfn::launches(); }

}  // extern "C"
