// mmb200_scaled_mm_static: the scratch-memory GEMM path for hosts that cannot give it any memory.
//
// Some hosts of this library own nothing on the device except the operand and result buffers they were handed: a
// plugin called from inside another framework's executor, a binding from a language runtime that exposes no device
// allocator, or a serving loop that must not touch the allocator because cudaMalloc and cudaFree may synchronise the
// whole device and take an unbounded time. The fastest path of this library (operands decoded once, then streamed)
// needs scratch memory, which mmb200_scaled_mm_ws expects from its caller. This entry point takes the scratch from a
// fixed array that is part of the library's device image instead, so the call allocates nothing: no cudaMalloc, no
// cudaFree, no stream-ordered allocation, no torch allocation.
//
// The price: the array has a fixed size (MMB200_STATIC_SCRATCH_BYTES, 64 MiB), every GPU that loads the library
// holds it until the process exits, and all calls on a device share it. The array keeps whatever the previous call
// left in it; the parts that must start at zero (per-row non-finite flags, status word) are cleared on the stream at
// the start of every call, everything else is fully rewritten before it is read. Two calls that overlap on the same
// GPU (different streams, or the same stream from two host threads without ordering) race on the array and give
// garbage; order them on one stream.
//
// Set-up: the device address of the array is looked up once per device, by the first call made with that device
// current, and cached. That first call should be made before any stream capture begins on the device.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t SCRATCH_BYTES = MMB200_STATIC_SCRATCH_BYTES;
constexpr int MAX_DEVICES = 64;

// Device scratch. In host code this name is only a handle for cudaGetSymbolAddress, never an address to pass on.
static __device__ __align__(256) unsigned char g_static_scratch[SCRATCH_BYTES];

std::mutex g_mutex;
void* g_scratch_ptr[MAX_DEVICES] = {};

// The array's address on the current device (looked up on first use there), or nullptr with `status` set.
void* scratch_on_current_device(int* status) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) {
    *status = mmb::record_cuda_error(err);
    return nullptr;
  }
  if (dev < 0 || dev >= MAX_DEVICES) {
    *status = MMB200_ERR_UNSUPPORTED;          // device ordinal beyond the address cache
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || !ptr) {
      *status = mmb::record_cuda_error(err != cudaSuccess ? err : cudaErrorInvalidSymbol);
      return nullptr;
    }
    g_scratch_ptr[dev] = ptr;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" int mmb200_scaled_mm_static(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b,
                                       void* D, int64_t ldd, int out_dtype, int M, int N, int K, int nfma, int fast,
                                       const float* scale_a, const float* scale_b, const float* scale_result,
                                       void* stream) {
  if (M < 0 || N < 0 || K < 0) return MMB200_ERR_BAD_ARG;
  if ((fmt_a != MMB200_FMT_E4M3 && fmt_a != MMB200_FMT_E5M2) || (fmt_b != MMB200_FMT_E4M3 && fmt_b != MMB200_FMT_E5M2))
    return MMB200_ERR_BAD_ARG;
  if (out_dtype < MMB200_OUT_F32 || out_dtype > MMB200_OUT_E5M2 || !scale_a || !scale_b) return MMB200_ERR_BAD_ARG;
  if (nfma != 16 && nfma != 32) return MMB200_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return MMB200_OK;
  // only requests the scratch-memory kernel serves: unsplit plan, K % 16 == 0, 16-byte aligned operands
  if (K == 0 || mmb200_kernel_for(A, lda, B, ldb, K, nfma, 1) != MMB200_KERNEL_FAST) return MMB200_ERR_UNSUPPORTED;
  if (mmb200_workspace_bytes(M, N, K) > SCRATCH_BYTES) return MMB200_ERR_TOO_LARGE;
  int status = MMB200_OK;
  void* scratch = scratch_on_current_device(&status);
  if (!scratch) return status;
  return mmb200_scaled_mm_ws(A, lda, fmt_a, B, ldb, fmt_b, D, ldd, out_dtype, M, N, K, nfma, fast, 1, MMB200_SCHEME_NONE,
                             scale_a, scale_b, scale_result, MMB200_KERNEL_FAST, scratch, SCRATCH_BYTES, stream);
}

extern "C" int mmb200_scaled_mm_static_status(int M, int N, int K, void* stream) {
  if (M < 0 || N < 0 || K < 0) return MMB200_ERR_BAD_ARG;
  if (M == 0 || N == 0 || K == 0) return MMB200_OK;
  int status = MMB200_OK;
  void* scratch = scratch_on_current_device(&status);
  if (!scratch) return status;
  return mmb200_workspace_status(scratch, M, N, K, 1, stream);
}
