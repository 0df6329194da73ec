// Host-side runtime of the native library: tensor-map (TMA descriptor) cache, the status-word
// registry and small device queries.  No kernel lives here.
#include <mutex>
#include <unordered_map>
#include <vector>
#include <string.h>
#include <stdio.h>

#include "common.cuh"
#include "yafsdp_b200.h"

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    // resolved through the runtime so the library carries no link-time dependency on libcuda
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  uint64_t v[12];
  bool operator==(const MapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 12; ++i) {
      h ^= k.v[i];
      h *= 1099511628211ull;
    }
    return (size_t)h;
  }
};

std::mutex g_map_mu;
// values are heap blocks that are never moved or freed: kernels receive them by value, callers by pointer
std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> g_maps;

const CUtensorMap* encode(int rank, const void* base, const uint64_t* dims, const uint64_t* pitch_elems,
                          const uint32_t* box, int elem_bytes, int swizzle128) {
  MapKey key;
  memset(&key, 0, sizeof(key));
  int dev = 0;
  cudaGetDevice(&dev);
  key.v[0] = reinterpret_cast<uint64_t>(base);
  key.v[1] = ((uint64_t)rank << 48) | ((uint64_t)elem_bytes << 40) | ((uint64_t)swizzle128 << 32) | (uint64_t)dev;
  for (int i = 0; i < rank; ++i) {
    key.v[2 + i] = dims[i];
    key.v[5 + i] = (i > 0) ? pitch_elems[i - 1] : 0;
    key.v[8 + i] = box[i];
  }
  std::lock_guard<std::mutex> lk(g_map_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) return it->second;
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return nullptr;
  cuuint64_t gdim[3];
  cuuint64_t gstride[2];
  cuuint32_t gbox[3];
  cuuint32_t estr[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    if (i > 0) gstride[i - 1] = pitch_elems[i - 1] * (uint64_t)elem_bytes;
  }
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  CUtensorMap* m = new CUtensorMap;
  CUresult r = fn(m, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[yafsdp_b200] cuTensorMapEncodeTiled failed: %d (base %p rank %d)\n", (int)r, base, rank);
    delete m;
    return nullptr;
  }
  if (g_maps.size() > 65536) g_maps.clear();  // descriptors of long-dead buffers; blocks stay allocated on purpose
  g_maps.emplace(key, m);
  return m;
}

}  // namespace

const CUtensorMap* yf_tensor_map_2d(const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_elems,
                                    uint32_t box_inner, uint32_t box_outer, int elem_bytes, int swizzle128) {
  uint64_t dims[2] = {inner, outer};
  uint64_t pitch[1] = {pitch_elems};
  uint32_t box[2] = {box_inner, box_outer};
  return encode(2, base, dims, pitch, box, elem_bytes, swizzle128);
}

const CUtensorMap* yf_tensor_map_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1_elems,
                                    uint64_t pitch2_elems, uint32_t b0, uint32_t b1, uint32_t b2, int elem_bytes,
                                    int swizzle128) {
  uint64_t dims[3] = {d0, d1, d2};
  uint64_t pitch[2] = {pitch1_elems, pitch2_elems};
  uint32_t box[3] = {b0, b1, b2};
  return encode(3, base, dims, pitch, box, elem_bytes, swizzle128);
}

int yf_tensor_map_3d_encode(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1_elems,
                            uint64_t pitch2_elems, uint32_t b0, uint32_t b1, uint32_t b2, int elem_bytes, int swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -2;
  cuuint64_t gdim[3] = {d0, d1, d2};
  cuuint64_t gstride[2] = {pitch1_elems * (uint64_t)elem_bytes, pitch2_elems * (uint64_t)elem_bytes};
  cuuint32_t gbox[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), gdim, gstride, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

int yf_num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

// The status word: a page of this library's own static storage, pinned and mapped into every GPU's address space on first
// use (cudaHostRegister: nothing is allocated, so entry points that promise not to allocate may bind it too).
int* yf_status_word() {
  alignas(4096) static int storage[1024];
  static int* word = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    memset(storage, 0, sizeof(storage));
    if (cudaHostRegister(storage, sizeof(storage), cudaHostRegisterMapped | cudaHostRegisterPortable) == cudaSuccess) word = storage;
  });
  return word;
}

extern "C" int yf_status_read(int* code, int* site, int clear) {
  volatile int* w = yf_status_word();
  if (w == nullptr) return -1;
  const int c = w[0], s = w[1], aborted = w[2];
  if (code) *code = (c == 0 && aborted != 0) ? YF_ERR_FLAG_TIMEOUT : c;
  if (site) *site = s;
  if (clear && (c != 0 || aborted != 0)) {
    w[0] = 0;
    w[1] = 0;
    w[2] = 0;
  }
  return 0;
}

// Plain device-to-device copy on a stream (the copy engines do the work; used for peer-to-peer transport so that
// bulk NVLink traffic takes no SM away from the GEMMs).
extern "C" int yf_memcpy_async(void* dst, const void* src, long long nbytes, void* stream) {
  if (nbytes <= 0) return 0;
  return -(int)cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int yf_version() { return 1; }
extern "C" int yf_sm_count() { return yf_num_sms(); }
