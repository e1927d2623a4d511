// Host-side plumbing shared by the kernels: error strings, the device status word,
// tensor-map (TMA descriptor) encoding with a small cache, device properties.
#include <atomic>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace b200 {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  uint64_t words[16];
  bool operator==(const MapKey& o) const { return std::memcmp(words, o.words, sizeof(words)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t w : k.words) {
      h ^= w;
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};

std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> g_maps;
constexpr size_t kMaxCachedMaps = 16384;  // 2 MiB of descriptors at most
constexpr unsigned kScratchMaps = 8;

}  // namespace

bool encode_tensor_map(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                       CUtensorMapL2promotion l2, CUtensorMapDataType dtype) {
  if (rank < 1 || rank > 4 || out == nullptr) return false;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdims[4];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[4];
  cuuint32_t estrides[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    if (i + 1 < rank) gstrides[i] = strides_bytes[i];
  }
  return fn(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims,
            gstrides, gbox, estrides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, l2,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

const CUtensorMap* get_tensor_map(const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                                  const uint32_t* box, CUtensorMapSwizzle swizzle, CUtensorMapL2promotion l2,
                                  CUtensorMapDataType dtype) {
  if (rank < 1 || rank > 4) return nullptr;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  int dev = 0;
  cudaGetDevice(&dev);
  key.words[0] = reinterpret_cast<uint64_t>(base);
  key.words[1] = (static_cast<uint64_t>(rank) << 32) | (static_cast<uint64_t>(swizzle) << 16) |
                 (static_cast<uint64_t>(l2) << 8) | static_cast<uint64_t>(dev) | (static_cast<uint64_t>(dtype) << 40);
  for (int i = 0; i < rank; ++i) {
    key.words[2 + i] = dims[i];
    key.words[6 + i] = i + 1 < rank ? strides_bytes[i] : 0;
    key.words[10 + i] = box[i];
  }
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) return it->second;
  if (g_maps.size() >= kMaxCachedMaps) {
    // The cache is keyed by base address, and eager steps hand in fresh activation addresses all the time: once it
    // is full, further descriptors are encoded into a small per-thread ring instead of being kept (a launch copies
    // the descriptor into its kernel parameters, and no launch uses more than kScratchMaps of them).
    alignas(64) static thread_local CUtensorMap scratch[kScratchMaps];
    static thread_local unsigned next = 0;
    CUtensorMap* m = &scratch[next++ % kScratchMaps];
    return encode_tensor_map(m, base, rank, dims, strides_bytes, box, swizzle, l2, dtype) ? m : nullptr;
  }
  // The descriptor is a 128-byte host object passed to kernels by value; cached ones are kept for the process lifetime.
  CUtensorMap* m = static_cast<CUtensorMap*>(aligned_alloc(64, sizeof(CUtensorMap)));
  if (!m) return nullptr;
  if (!encode_tensor_map(m, base, rank, dims, strides_bytes, box, swizzle, l2, dtype)) {
    free(m);
    return nullptr;
  }
  g_maps.emplace(key, m);
  return m;
}

int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
  const bool slot = dev >= 0 && dev < 64;
  int n = slot ? cached[dev].load(std::memory_order_relaxed) : 0;
  if (n == 0) {
    if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (slot) cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace b200

extern "C" {

int b200_version(void) { return 1000; }

const char* b200_error_string(int code) {
  switch (code) {
    case B200_OK: return "ok";
    case B200_ERR_INVALID_ARGUMENT: return "invalid argument";
    case B200_ERR_ALIGNMENT: return "pointer or leading dimension not 16-byte aligned";
    case B200_ERR_WORKSPACE: return "workspace too small";
    case B200_ERR_LAUNCH: return "kernel launch failed";
    case B200_ERR_DRIVER: return "tensor map could not be encoded";
    case B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case B200_ERR_SCRATCH_LIMIT: return "the problem needs more scratch than the library's built-in array holds";
    default: return "unknown error";
  }
}

int b200_device_status(int reset, int* status_out) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, b200::g_device_status, sizeof(int)) != cudaSuccess) return B200_ERR_LAUNCH;
  if (status_out) *status_out = v;
  if (reset) {
    int z = 0;
    if (cudaMemcpyToSymbol(b200::g_device_status, &z, sizeof(int)) != cudaSuccess) return B200_ERR_LAUNCH;
  }
  return B200_OK;
}

int b200_set_wait_limit_ns(uint64_t limit_ns) {
  if (limit_ns == 0) return B200_ERR_INVALID_ARGUMENT;
  const unsigned long long v = limit_ns;
  if (cudaMemcpyToSymbol(b200::g_wait_limit_ns, &v, sizeof(v)) != cudaSuccess) {
    (void)cudaGetLastError();
    return B200_ERR_LAUNCH;
  }
  return B200_OK;
}

int b200_copy_rows_h2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                       b200_stream_t stream) {
  if (!dst || !src || width_bytes == 0 || rows == 0 || dst_pitch < width_bytes || src_pitch < width_bytes)
    return B200_ERR_INVALID_ARGUMENT;
  if (cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyHostToDevice,
                        reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
    (void)cudaGetLastError();
    return B200_ERR_DRIVER;
  }
  return B200_OK;
}

}  // extern "C"
