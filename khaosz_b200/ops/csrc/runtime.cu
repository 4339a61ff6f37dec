// Host-side runtime shared by all kernels of the library: the per-device error word that
// bounded waits report into, and tensor-map (TMA descriptor) encoding through the driver
// entry point so the library needs no link-time dependency on libcuda.
#include <mutex>

#include "common.cuh"
#include "kb_api.h"

namespace kb {

namespace {
constexpr int kMaxDevices = 64;
int* g_err_words[kMaxDevices] = {nullptr};
std::mutex g_mutex;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
int g_last_tmap_error = 0;

// The driver call needs the primary context bound to the calling thread; worker threads
// (e.g. an autograd thread) may not have touched the runtime yet.
void bind_context_once() {
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(0);
    bound = true;
  }
}

EncodeTiledFn get_encode() {
  bind_context_once();
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess) return nullptr;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}

CUtensorMapDataType dtype_of(int elem_bytes) {
  switch (elem_bytes) {
    case 1: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case 2: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}
}  // namespace

int tmap_error_code() { return g_last_tmap_error; }

int* error_word(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  if (g_err_words[device]) return g_err_words[device];
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_err_words[device]) return g_err_words[device];
  int* p = nullptr;
  if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, 64);
  g_err_words[device] = p;
  return p;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_last_tmap_error = (int)r;
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims_in[3],
                 const uint64_t strides_bytes[2], const uint32_t box_in[3], bool swizzle128) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[3] = {dims_in[0], dims_in[1], dims_in[2]};
  cuuint64_t strides[2] = {strides_bytes[0], strides_bytes[1]};
  cuuint32_t box[3] = {box_in[0], box_in[1], box_in[2]};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_last_tmap_error = (int)r;
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims_in[4],
                 const uint64_t strides_bytes[3], const uint32_t box_in[4], bool swizzle128) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[4] = {dims_in[0], dims_in[1], dims_in[2], dims_in[3]};
  cuuint64_t strides[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t box[4] = {box_in[0], box_in[1], box_in[2], box_in[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_last_tmap_error = (int)r;
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace kb

extern "C" {

// Reads the current device's error word (synchronises the device) and clears it.
int kb_last_error(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  int* p = kb::error_word(dev);
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

// Enqueues a copy of the current device's error word into `pinned_host` (4 bytes of page-locked
// host memory) on `stream`; the caller records an event behind it and reads the value once the
// event has completed, so nobody waits for the device.
int kb_error_probe(int* pinned_host, void* stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || pinned_host == nullptr) return KB_STATUS_BAD_ARG;
  int* p = kb::error_word(dev);
  if (!p) return KB_STATUS_CUDA_ERROR;
  return cudaMemcpyAsync(pinned_host, p, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)) ==
                 cudaSuccess
             ? KB_STATUS_OK
             : KB_STATUS_CUDA_ERROR;
}

namespace {
__global__ void store_f32x2_kernel(float* dst, float a, float b) {
  dst[0] = a;
  dst[1] = b;
}
}  // namespace

// dst[0] = a, dst[1] = b on `stream`: host scalars that kernels read from device memory (learning
// rate and step of the optimizer kernels) travel as launch arguments, not through a staging buffer
// that a later step could overwrite before the copy ran.
int kb_store_f32x2(float* dst, float a, float b, void* stream) {
  if (dst == nullptr) return KB_STATUS_BAD_ARG;
  store_f32x2_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(dst, a, b);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// One asynchronous device-to-device copy on `stream` (copy engine; the source may be a peer's memory that
// is mapped into this process).  One call per copy.
int kb_copy_async(void* dst, const void* src, long long bytes, void* stream) {
  if (dst == nullptr || src == nullptr || bytes < 0) return KB_STATUS_BAD_ARG;
  if (bytes == 0) return KB_STATUS_OK;
  return cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? KB_STATUS_OK
             : KB_STATUS_CUDA_ERROR;
}

int kb_sm_count(void) {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

int kb_last_tmap_error(void) { return kb::tmap_error_code(); }

const char* kb_version(void) { return "khaosz_b200 kernels (sm_100a)"; }
}
