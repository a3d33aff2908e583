// Host-side helpers shared by the launchers: TMA descriptor encoding through the driver entry
// point (no link-time dependency on libcuda), the host-mapped status word, launch error checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>

namespace mbh {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The encode call is a driver-API call: it needs a context current on the calling thread.  A thread whose first
// CUDA work is one of our launchers (an autograd worker whose first backward node is a GEMM) may have none yet.
// cudaSetDevice on the current device binds the primary context (CUDA 12 initialises it there); only if the
// driver still reports no current context does the classic cudaFree(nullptr), which releases nothing, run.
inline void bind_context_to_thread() {
  static thread_local bool bound = false;
  if (bound) return;
  bound = true;
  typedef CUresult (*CtxGetCurrentFn)(CUcontext*);
  static CtxGetCurrentFn get_current = nullptr;
  if (!get_current) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      get_current = reinterpret_cast<CtxGetCurrentFn>(p);
  }
  CUcontext ctx = nullptr;
  if (get_current && get_current(&ctx) == CUDA_SUCCESS && ctx) return;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);
  ctx = nullptr;
  if (get_current && get_current(&ctx) == CUDA_SUCCESS && ctx) return;
  cudaFree(nullptr);
}

inline EncodeTiledFn encode_fn() {
  bind_context_to_thread();
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
      fprintf(stderr, "maester_b200: cuTensorMapEncodeTiled unavailable (%d)\n", (int)e);
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch `ld` elements,
// box = box_inner x box_outer, 128-byte swizzle (box_inner must be 64 bf16 = 128 B).
inline int make_tmap_bf16_2d(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                             uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "maester_b200: cuTensorMapEncodeTiled failed (%d) base=%p inner=%llu outer=%llu ld=%llu\n",
            (int)r, base, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld);
    return -2;
  }
  return 0;
}

// General N-d bf16 tensor map with explicit element strides (dims[0] is contiguous).
inline int make_tmap_bf16_nd(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                             const uint64_t* strides_elems /* rank-1 entries, for dims[1..] */,
                             const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i < rank - 1; ++i) s[i] = strides_elems[i] * 2;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), d, s, b, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "maester_b200: cuTensorMapEncodeTiled(nd) failed (%d)\n", (int)r);
    return -2;
  }
  return 0;
}

// One host-mapped status word per process.  Kernels record the first non-zero error code there;
// the host reads it after a synchronisation point (mb_status()).
struct Status {
  int* host = nullptr;
  int* dev = nullptr;
};
inline Status& status() {
  static Status s;
  if (!s.host) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&s.host), 64, cudaHostAllocMapped | cudaHostAllocPortable) ==
        cudaSuccess) {
      for (int i = 0; i < 16; ++i) s.host[i] = 0;
      cudaHostGetDevicePointer(reinterpret_cast<void**>(&s.dev), s.host, 0);
    }
  }
  return s;
}

// Per-device caches: a process may drive several GPUs, and function attributes and SM counts belong to the
// device that is current at the launch.
constexpr int MAX_DEVICES = 64;
inline int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev < 0 || dev >= MAX_DEVICES) ? 0 : dev;
}

inline int sm_count() {
  static std::atomic<int> n[MAX_DEVICES];
  const int dev = current_device();
  int v = n[dev].load(std::memory_order_relaxed);
  if (!v) {
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    n[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

// Raises a kernel's dynamic shared-memory limit once per device (one bit per device in a per-call-site mask).
#define MB_SET_MAX_SMEM_ONCE(kernel, bytes)                                                                  \
  do {                                                                                                       \
    static std::atomic<unsigned long long> mb_done_{0};                                                      \
    const unsigned long long mb_bit_ = 1ull << mbh::current_device();                                        \
    if (!(mb_done_.load(std::memory_order_acquire) & mb_bit_)) {                                             \
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);                      \
      mb_done_.fetch_or(mb_bit_, std::memory_order_release);                                                 \
    }                                                                                                        \
  } while (0)

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "maester_b200: launch of %s failed: %s\n", what, cudaGetErrorString(e));
    return -100 - (int)e;
  }
  return 0;
}

}  // namespace mbh
