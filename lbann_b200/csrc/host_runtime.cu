// Host-side services shared by all kernels: per-device status word, tensor-map
// encoding through the driver entry point, device properties.
#include "common.cuh"
#include <cstdio>
#include <mutex>

namespace lbhost {

namespace {
constexpr int kMaxDevices = 16;
int* g_status[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};
std::mutex g_mutex;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
    fprintf(stderr, "[lbann_b200] cuTensorMapEncodeTiled is not available: %s\n",
            cudaGetErrorString(e));
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

int* status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_status[dev]) {
    cudaMalloc(&g_status[dev], 64);
    cudaMemset(g_status[dev], 0, 64);
  }
  return g_status[dev];
}

int consume_status(cudaStream_t stream) {
  int* w = status_word();
  int host = 0;
  cudaMemcpyAsync(&host, w, sizeof(int), cudaMemcpyDeviceToHost, stream);
  cudaStreamSynchronize(stream);
  if (host != 0) cudaMemsetAsync(w, 0, sizeof(int), stream);
  return host;
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (!g_sm_count[dev]) {
    cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sm_count[dev];
}

static thread_local SplitKOffer g_splitk_offer;

SplitKOffer take_splitk_offer() {
  SplitKOffer o = g_splitk_offer;
  g_splitk_offer = SplitKOffer();
  return o;
}

int plan_splitk(const SplitKOffer& o, int num_tiles, int k_iters, int bn) {
  if (!o.ws || num_tiles <= 0) return 1;
  const int sms = sm_count();
  if (num_tiles * 2 > sms || k_iters < 8) return 1;
  int splits = sms / num_tiles;
  if (splits > k_iters / 4) splits = k_iters / 4;     // at least four pipeline stages per item
  if (splits > 32) splits = 32;
  const long long tile_bytes = 128ll * bn * 4;
  while (splits > 1 && (long long)num_tiles * splits * tile_bytes > o.ws_bytes) --splits;
  return splits < 1 ? 1 : splits;
}

bool encode_tmap(CUtensorMap* out, int dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, const uint32_t* elem_strides,
                 int swizzle_bytes) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return false;
  {
    // The driver call needs a current context.  A host thread that has made no runtime call
    // yet (an autograd worker thread entering a backward function) has none bound: selecting
    // the device it already uses binds the primary context.
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
  }
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (dtype == lb::kF16) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (dtype == lb::kF32) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (dtype == lb::kI64) dt = CU_TENSOR_MAP_DATA_TYPE_INT64;
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                  reinterpret_cast<const cuuint64_t*>(dims),
                  reinterpret_cast<const cuuint64_t*>(strides_bytes),
                  reinterpret_cast<const cuuint32_t*>(box),
                  elem_strides ? reinterpret_cast<const cuuint32_t*>(elem_strides) : ones,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[lbann_b200] cuTensorMapEncodeTiled failed (%d): rank=%d base=%p dims=[%llu,%llu,%llu] "
            "box=[%u,%u,%u] stride1=%llu\n",
            (int)r, rank, base, (unsigned long long)dims[0],
            (unsigned long long)(rank > 1 ? dims[1] : 0),
            (unsigned long long)(rank > 2 ? dims[2] : 0), box[0], rank > 1 ? box[1] : 0,
            rank > 2 ? box[2] : 0, (unsigned long long)(rank > 1 ? strides_bytes[0] : 0));
    return false;
  }
  return true;
}

}  // namespace lbhost

extern "C" {

// Returns the first error recorded by a kernel since the last call (0 = none) and clears it.
int lb_consume_status(void* stream) {
  return lbhost::consume_status(reinterpret_cast<cudaStream_t>(stream));
}

// Budget, in nanoseconds, of every device-side wait on another rank (0 = the built-in 2 s).
// Stored next to the status word on the current device; takes effect for kernels launched
// after the call.
int lb_set_wait_budget_ns(unsigned long long ns) {
  int* w = lbhost::status_word();
  return (int)cudaMemcpy(reinterpret_cast<char*>(w) + 8, &ns, sizeof(ns), cudaMemcpyHostToDevice);
}

// Device pointer of the status word (for kernels launched from other libraries/tests).
void* lb_status_ptr() { return lbhost::status_word(); }

int lb_sm_count() { return lbhost::sm_count(); }

// Lends scratch to the next GEMM / convolution launch of the calling thread (see
// lbhost::SplitKOffer).  `ws` must be 16-byte aligned.
int lb_splitk_offer(void* ws, long long ws_bytes) {
  if ((reinterpret_cast<uintptr_t>(ws) & 15) || ws_bytes < 0) return -1;
  lbhost::g_splitk_offer.ws = reinterpret_cast<float*>(ws);
  lbhost::g_splitk_offer.ws_bytes = ws_bytes;
  return 0;
}

int lb_abi_version() { return 1; }

}  // extern "C"
