// Host side of the C ABI (include/mmaemu_b200.h): argument checks, kernel choice, launches. No allocation except in
// mmb200_scaled_mm_host, which stages host operands through the stream-ordered allocator.
#include <atomic>
#include <mutex>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace {

thread_local char g_cuda_error[256] = "";
std::atomic<long long> g_launches{0};

int cuda_fail(cudaError_t err) {
  const char* s = cudaGetErrorString(err);
  std::strncpy(g_cuda_error, s ? s : "unknown CUDA error", sizeof(g_cuda_error) - 1);
  g_cuda_error[sizeof(g_cuda_error) - 1] = 0;
  return MMB200_ERR_LAUNCH;
}

// Status word of a staged launch, read after the stream has drained.
int read_status(const void* workspace, int M, int N, int K, int S, cudaStream_t st) {
  if (!workspace || M <= 0 || N <= 0 || K <= 0) return MMB200_OK;
  int word = 0;
  cudaError_t err = cudaMemcpyAsync(&word, static_cast<const unsigned char*>(workspace) + mmb::staged_status_offset(M, N, K, S),
                                    sizeof(int), cudaMemcpyDeviceToHost, st);
  if (err == cudaSuccess) err = cudaStreamSynchronize(st);
  if (err != cudaSuccess) return cuda_fail(err);
  return word ? MMB200_ERR_TIMEOUT : MMB200_OK;
}

bool fmt_ok(int f) { return f == MMB200_FMT_E4M3 || f == MMB200_FMT_E5M2; }

int current_device_ok() {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return cuda_fail(err);
  return mmb200_device_supported(dev);
}

// Shared argument validation and dispatch of the three device-pointer entry points.
int run(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, void* D, int64_t ldd,
        int out_dtype, int M, int N, int K, int nfma, int fast, int S, int scheme, const float* sa, const float* sb,
        const float* sr, int epilogue, int patch, int kernel, void* stream, void* workspace = nullptr,
        size_t workspace_bytes = 0, const void* a_hp = nullptr, int64_t ld_hp = 0, int hp_dtype = 0,
        const float* quant_scale = nullptr, void* const* peer_D = nullptr, int n_peers = 0,
        unsigned char* shared_b = nullptr) {
  if (n_peers < 0 || n_peers > MMB200_MAX_PEERS || (n_peers > 0 && !peer_D)) return MMB200_ERR_BAD_ARG;
  for (int q = 0; q < n_peers; ++q)
    if (!peer_D[q]) return MMB200_ERR_BAD_ARG;
  if (M < 0 || N < 0 || K < 0) return MMB200_ERR_BAD_ARG;
  if (!fmt_ok(fmt_a) || !fmt_ok(fmt_b)) return MMB200_ERR_BAD_ARG;
  if (out_dtype < MMB200_OUT_F32 || out_dtype > MMB200_OUT_E5M2) return MMB200_ERR_BAD_ARG;
  if (nfma != MMB200_PRESET_ADA && nfma != MMB200_PRESET_HOPPER && nfma != MMB200_PRESET_B200_MMA_SYNC)
    return MMB200_ERR_UNSUPPORTED;
  // no GEMM level is characterised for the late-accumulator preset: unsplit fast accumulation only
  if (nfma == MMB200_PRESET_B200_MMA_SYNC && (!fast || S != 1)) return MMB200_ERR_UNSUPPORTED;
  if (S < 1 || scheme < MMB200_SCHEME_NONE || scheme > MMB200_SCHEME_CONTIGUOUS) return MMB200_ERR_BAD_ARG;
  if (S > 1 && scheme == MMB200_SCHEME_NONE) return MMB200_ERR_BAD_ARG;
  if (S > MMB200_MAX_SPLITS) return MMB200_ERR_TOO_LARGE;
  if (kernel < MMB200_KERNEL_AUTO || kernel > MMB200_KERNEL_FAST) return MMB200_ERR_BAD_ARG;
  if (a_hp) {                                   // quantise prologue: E4M3 codes of A are produced by the call
    if (hp_dtype != MMB200_HP_F32 && hp_dtype != MMB200_HP_BF16) return MMB200_ERR_BAD_ARG;
    if (fmt_a != MMB200_FMT_E4M3 || !quant_scale || ld_hp < K) return MMB200_ERR_BAD_ARG;
  }
  if (M == 0 || N == 0) return MMB200_OK;
  if (!D || ldd < N) return MMB200_ERR_BAD_ARG;
  if (K > 0 && (!A || !B || lda < K || ldb < K)) return MMB200_ERR_BAD_ARG;
  if (K >= (1 << 24)) return MMB200_ERR_TOO_LARGE;   // fp32 holds the non-finite term counts and block exponents
  int rc = current_device_ok();
  if (rc != MMB200_OK) return rc;

  mmb::Params p;
  std::memset(&p, 0, sizeof(p));
  p.A = static_cast<const uint8_t*>(A);
  p.B = static_cast<const uint8_t*>(B);
  p.D = D;
  p.scale_a = sa;
  p.scale_b = sb;
  p.scale_result = sr;
  p.lda = lda; p.ldb = ldb; p.ldd = ldd;
  p.M = M; p.N = N; p.K = K;
  p.fmt_a = fmt_a; p.fmt_b = fmt_b; p.out_dtype = out_dtype;
  p.fast = fast ? 1 : 0;
  p.S = S;
  p.scheme = S > 1 ? scheme : MMB200_SCHEME_NONE;
  p.epilogue = epilogue;
  p.patch_nonfinite = patch;
  p.n_peers = n_peers;
  for (int q = 0; q < n_peers; ++q) p.peer_D[q] = peer_D[q];
  p.shared_b = shared_b;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t err;
  int launches = 1;
  if (a_hp) {
    p.a_hp = a_hp;
    p.ld_hp = ld_hp;
    p.a_hp_dtype = hp_dtype;
    p.a_quant_scale = quant_scale;
    p.a_codes = static_cast<uint8_t*>(const_cast<void*>(A));
    const int per16 = hp_dtype == MMB200_HP_F32 ? 4 : 8;      // elements per 16 bytes
    if ((reinterpret_cast<uintptr_t>(a_hp) & 15) || (ld_hp % per16) != 0) return MMB200_ERR_UNSUPPORTED;
  }
  // fast kernels: every plan with enough scratch memory (staged), unsplit plans without; else the integer kernel
  const bool direct_ok = mmb::fast_supports(p, nfma);
  const bool staged_ok = mmb::staged_supports(p, nfma) && workspace &&
                         workspace_bytes >= mmb::staged_workspace_bytes(M, N, K, S, false, shared_b != nullptr) &&
                         !(reinterpret_cast<uintptr_t>(workspace) & 127);
  if (shared_b && !staged_ok) return MMB200_ERR_UNSUPPORTED;      // only the staged kernels read a shared B area
  if (kernel == MMB200_KERNEL_FAST && !direct_ok && !staged_ok) return MMB200_ERR_UNSUPPORTED;
  if (a_hp && (!staged_ok || kernel == MMB200_KERNEL_INTEGER)) return MMB200_ERR_UNSUPPORTED;   // only the pre-decode pass quantises
  if (kernel != MMB200_KERNEL_INTEGER && staged_ok) {
    launches = 0;
    err = mmb::launch_staged(p, nfma, workspace, workspace_bytes, st, &launches);
  } else if (kernel != MMB200_KERNEL_INTEGER && direct_ok) {
    err = mmb::launch_fast(p, nfma, st);
  } else {
    err = mmb::launch_integer(p, nfma, st);
  }
  if (err != cudaSuccess) return cuda_fail(err);
  g_launches.fetch_add(launches, std::memory_order_relaxed);
  return MMB200_OK;
}

// Staging memory of the host-buffer entry point: a memory pool of this library per device that keeps what it has
// allocated (release threshold at its maximum), so that repeated calls do not return the memory to the driver at
// every synchronisation and map it again.
cudaError_t staging_pool(cudaMemPool_t* pool) {
  static std::mutex mu;
  static cudaMemPool_t pools[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!pools[dev]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    err = cudaMemPoolCreate(&pools[dev], &props);
    if (err != cudaSuccess) { pools[dev] = nullptr; return err; }
    unsigned long long keep = ~0ull;
    err = cudaMemPoolSetAttribute(pools[dev], cudaMemPoolAttrReleaseThreshold, &keep);
    if (err != cudaSuccess) return err;
  }
  *pool = pools[dev];
  return cudaSuccess;
}

// Internal streams and events of the host-buffer entry point (one set per device, created on first use; a call holds
// the mutex while it uses them).
struct HostPipeline {
  static constexpr int STREAMS = 8;                     // one per slab: no slab waits behind another one
  std::mutex mu;
  cudaStream_t s[STREAMS] = {};
  cudaEvent_t start = nullptr, b_ready = nullptr, done[STREAMS] = {};
  bool ready = false;
};
constexpr size_t PIPELINE_MIN_BYTES = (size_t)8 << 20;   // operands + output below this: one slab, the caller's stream
constexpr int PIPELINE_SLAB_TILES = 128;                // output tiles of 128 x 128 per slab: at least this many (a slab of
                                                        // at most one wave of CTAs lets the next slab's CTAs fill its tail)
constexpr int PIPELINE_MAX_SLABS = HostPipeline::STREAMS;

// MMAEMU_B200_HOST_PIPELINE: "0" = copy, compute, copy back on one stream; a number from 2 to 8 = that many slabs
// whatever the size of the call (tests and tuning); anything else = the automatic choice. Returns 0, the number, or -1.
int host_pipeline_setting() {
  const char* env = std::getenv("MMAEMU_B200_HOST_PIPELINE");
  if (!env || !env[0]) return -1;
  const int v = std::atoi(env);
  if (v == 0 && env[0] == '0') return 0;
  return (v >= 2 && v <= PIPELINE_MAX_SLABS) ? v : -1;
}

cudaError_t host_pipeline(HostPipeline** out) {
  static std::mutex mu;
  static HostPipeline pipes[64];
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  HostPipeline& hp = pipes[dev];
  if (!hp.ready) {
    for (int q = 0; q < HostPipeline::STREAMS; ++q) {
      if (!hp.s[q] && (err = cudaStreamCreateWithFlags(&hp.s[q], cudaStreamNonBlocking)) != cudaSuccess) return err;
      if (!hp.done[q] && (err = cudaEventCreateWithFlags(&hp.done[q], cudaEventDisableTiming)) != cudaSuccess) return err;
    }
    if (!hp.start && (err = cudaEventCreateWithFlags(&hp.start, cudaEventDisableTiming)) != cudaSuccess) return err;
    if (!hp.b_ready && (err = cudaEventCreateWithFlags(&hp.b_ready, cudaEventDisableTiming)) != cudaSuccess) return err;
    hp.ready = true;
  }
  *out = &hp;
  return cudaSuccess;
}

size_t out_size(int out_dtype) {
  return out_dtype == MMB200_OUT_F32 ? 4 : (out_dtype <= MMB200_OUT_F16 ? 2 : 1);
}

// Issue-rate probe: every thread runs `iters` rounds of 32 independent dependent-chain steps of one instruction kind
// (0: fma.rz.f32, 1: a three-input integer add and a three-input logic operation alternating), so that a launch with
// enough warps per SM is bound by the issue rate of that instruction's pipe. The result is stored so that nothing is
// optimised away.
template <int KIND>
__global__ void __launch_bounds__(256) probe_kernel(int iters, float* sink) {
  float f[32];
  uint32_t u[32];
#pragma unroll
  for (int q = 0; q < 32; ++q) {
    f[q] = 1.0f + (float)(threadIdx.x + q) * 1e-3f;
    u[q] = threadIdx.x * 2654435761u + q;
  }
  const float m = 1.0f + 1e-7f * (float)blockIdx.x, c = 1e-9f;
  const uint32_t k1 = blockIdx.x | 1u, k2 = threadIdx.x;
#pragma unroll 1
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      if (KIND == 0) f[q] = __fmaf_rz(f[q], m, c);
      else u[q] = (q & 1) ? (u[q] + k1 + k2) : ((u[q] & k1) ^ k2);
    }
  }
  float acc = 0.0f;
#pragma unroll
  for (int q = 0; q < 32; ++q) acc += KIND == 0 ? f[q] : (float)u[q];
  sink[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = acc;
}

}  // namespace

int mmb::record_cuda_error(cudaError_t err) { return cuda_fail(err); }

extern "C" {

int mmb200_abi_version(void) { return MMB200_ABI_VERSION; }

const char* mmb200_status_string(int status) {
  switch (status) {
    case MMB200_OK: return "ok";
    case MMB200_ERR_BAD_ARG: return "bad argument";
    case MMB200_ERR_UNSUPPORTED: return "unsupported request";
    case MMB200_ERR_ARCH: return "the device is not sm_100 (this library holds sm_100a kernels only)";
    case MMB200_ERR_LAUNCH: return "CUDA runtime error (see mmb200_last_cuda_error)";
    case MMB200_ERR_TOO_LARGE: return "size beyond a documented limit";
    case MMB200_ERR_TIMEOUT: return "a bounded wait inside a kernel ran out; the output was not written";
    default: return "unknown status";
  }
}

const char* mmb200_last_cuda_error(void) { return g_cuda_error; }

int mmb200_device_supported(int device) {
  int major = 0;
  cudaError_t err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (err != cudaSuccess) return cuda_fail(err);
  int minor = 0;
  err = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
  if (err != cudaSuccess) return cuda_fail(err);
  return (major == 10 && minor == 0) ? MMB200_OK : MMB200_ERR_ARCH;
}

int mmb200_chain(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, float* C, int64_t ldc,
                 int M, int N, int K, int nfma, int kernel, void* stream) {
  return run(A, lda, fmt_a, B, ldb, fmt_b, C, ldc, MMB200_OUT_F32, M, N, K, nfma, 1, 1, MMB200_SCHEME_NONE, nullptr,
             nullptr, nullptr, 0, 0, kernel, stream);
}

int mmb200_accumulate(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, float* C,
                      int64_t ldc, int M, int N, int K, int nfma, int fast, int S, int scheme, int kernel,
                      void* stream) {
  return run(A, lda, fmt_a, B, ldb, fmt_b, C, ldc, MMB200_OUT_F32, M, N, K, nfma, fast, S, scheme, nullptr, nullptr,
             nullptr, 0, 1, kernel, stream);
}

int mmb200_scaled_mm(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, void* D,
                     int64_t ldd, int out_dtype, int M, int N, int K, int nfma, int fast, int S, int scheme,
                     const float* scale_a, const float* scale_b, const float* scale_result, int kernel,
                     void* stream) {
  if (!scale_a || !scale_b) return MMB200_ERR_BAD_ARG;
  return run(A, lda, fmt_a, B, ldb, fmt_b, D, ldd, out_dtype, M, N, K, nfma, fast, S, scheme, scale_a, scale_b,
             scale_result, 1, 1, kernel, stream);
}

size_t mmb200_workspace_status_offset(int M, int N, int K, int S) { return mmb::staged_status_offset(M, N, K, S); }

int mmb200_workspace_status(const void* workspace, int M, int N, int K, int S, void* stream) {
  if (M < 0 || N < 0 || K < 0 || S < 1) return MMB200_ERR_BAD_ARG;
  return read_status(workspace, M, N, K, S, static_cast<cudaStream_t>(stream));
}

int mmb200_probe_issue_rate(int kind, int ctas, int iters, float* sink, void* stream) {
  if ((kind != 0 && kind != 1) || ctas <= 0 || iters <= 0 || !sink) return MMB200_ERR_BAD_ARG;
  int rc = current_device_ok();
  if (rc != MMB200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kind == 0) probe_kernel<0><<<ctas, 256, 0, st>>>(iters, sink);
  else probe_kernel<1><<<ctas, 256, 0, st>>>(iters, sink);
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? MMB200_OK : cuda_fail(err);
}

void mmb200_test_hooks(int wait_polls, int announce_extra_bytes) { mmb::staged_test_hooks(wait_polls, announce_extra_bytes); }

size_t mmb200_workspace_bytes(int M, int N, int K) { return mmb::staged_workspace_bytes(M, N, K, 1, false); }
size_t mmb200_workspace_bytes_split(int M, int N, int K, int S) { return mmb::staged_workspace_bytes(M, N, K, S, true); }

int mmb200_scaled_mm_ws(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, void* D,
                        int64_t ldd, int out_dtype, int M, int N, int K, int nfma, int fast, int S, int scheme,
                        const float* scale_a, const float* scale_b, const float* scale_result, int kernel,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (!scale_a || !scale_b) return MMB200_ERR_BAD_ARG;
  return run(A, lda, fmt_a, B, ldb, fmt_b, D, ldd, out_dtype, M, N, K, nfma, fast, S, scheme, scale_a, scale_b,
             scale_result, 1, 1, kernel, stream, workspace, workspace_bytes);
}

int mmb200_scaled_mm_peers(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, void* D,
                           int64_t ldd, int out_dtype, int M, int N, int K, int nfma, int fast, int S, int scheme,
                           const float* scale_a, const float* scale_b, const float* scale_result, int kernel,
                           void* workspace, size_t workspace_bytes, void* const* peer_D, int n_peers, void* stream) {
  if (!scale_a || !scale_b) return MMB200_ERR_BAD_ARG;
  return run(A, lda, fmt_a, B, ldb, fmt_b, D, ldd, out_dtype, M, N, K, nfma, fast, S, scheme, scale_a, scale_b,
             scale_result, 1, 1, kernel, stream, workspace, workspace_bytes, nullptr, 0, 0, nullptr, peer_D, n_peers);
}

int mmb200_quantize_scaled_mm_ws(const void* X, int64_t ldx, int x_dtype, const float* quant_scale, void* A_codes,
                                 int64_t lda, const void* B, int64_t ldb, int fmt_b, void* D, int64_t ldd, int out_dtype,
                                 int M, int N, int K, int nfma, int fast, int S, int scheme, const float* scale_a,
                                 const float* scale_b, const float* scale_result, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  if (!scale_a || !scale_b || !X || !A_codes) return MMB200_ERR_BAD_ARG;
  return run(A_codes, lda, MMB200_FMT_E4M3, B, ldb, fmt_b, D, ldd, out_dtype, M, N, K, nfma, fast, S, scheme, scale_a,
             scale_b, scale_result, 1, 1, MMB200_KERNEL_AUTO, stream, workspace, workspace_bytes, X, ldx, x_dtype,
             quant_scale);
}

int mmb200_accumulate_ws(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, float* C,
                         int64_t ldc, int M, int N, int K, int nfma, int fast, int S, int scheme, int kernel,
                         void* workspace, size_t workspace_bytes, void* stream) {
  return run(A, lda, fmt_a, B, ldb, fmt_b, C, ldc, MMB200_OUT_F32, M, N, K, nfma, fast, S, scheme, nullptr, nullptr,
             nullptr, 0, 1, kernel, stream, workspace, workspace_bytes);
}

int mmb200_scaled_mm_host(const void* A, int64_t lda, int fmt_a, const void* B, int64_t ldb, int fmt_b, void* D,
                          int64_t ldd, int out_dtype, int M, int N, int K, int nfma, int fast, int S, int scheme,
                          float scale_a, float scale_b, const float* scale_result, int kernel, void* stream) {
  if (M < 0 || N < 0 || K < 0) return MMB200_ERR_BAD_ARG;
  if (out_dtype < MMB200_OUT_F32 || out_dtype > MMB200_OUT_E5M2) return MMB200_ERR_BAD_ARG;
  if (M == 0 || N == 0) return MMB200_OK;
  if (!D || ldd < N || (K > 0 && (!A || !B || lda < K || ldb < K))) return MMB200_ERR_BAD_ARG;
  if (!fmt_ok(fmt_a) || !fmt_ok(fmt_b)) return MMB200_ERR_BAD_ARG;
  {
    const int rc_dev = current_device_ok();
    if (rc_dev != MMB200_OK) return rc_dev;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t es = out_size(out_dtype);
  const size_t kpad = ((size_t)K + 15) / 16 * 16;       // dense device copies with a 16-byte aligned row stride
  const size_t a_bytes = (size_t)M * kpad, b_bytes = (size_t)N * kpad, d_bytes = (size_t)M * N * es;
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  const bool staged = K > 0 && K % 16 == 0 && S >= 1 && S <= MMB200_MAX_SPLITS && kernel != MMB200_KERNEL_INTEGER &&
                      (nfma == MMB200_PRESET_ADA || nfma == MMB200_PRESET_HOPPER);
  // Row slabs: with enough work the rows of A are cut into slabs, each on an internal stream of its own (copy of its
  // rows, its kernels, copy-back of its outputs), so that the copies of some slabs overlap the kernels of others and the
  // GPU always has a slab whose rows have arrived (rows are independent of one another; B is copied and decoded once,
  // into a shared area). A slab on a stream of its own never waits behind another slab: with fewer streams than slabs
  // the slab queued behind the one the GPU happened to run last ran alone at the end.
  HostPipeline* pipe = nullptr;
  int slab_rows = M, n_slabs = 1;
  const int setting = host_pipeline_setting();
  if (staged && setting != 0 && (setting > 0 || a_bytes + b_bytes + d_bytes >= PIPELINE_MIN_BYTES)) {
    const int tiles_n = (N + 127) / 128, tiles_m = (M + 127) / 128;
    int tile_rows = (PIPELINE_SLAB_TILES + tiles_n - 1) / tiles_n;
    if (setting > 0) tile_rows = (tiles_m + setting - 1) / setting;
    int slabs = (tiles_m + tile_rows - 1) / tile_rows;
    if (slabs > PIPELINE_MAX_SLABS) {
      tile_rows = ((M + 127) / 128 + PIPELINE_MAX_SLABS - 1) / PIPELINE_MAX_SLABS;
      slabs = ((M + 127) / 128 + tile_rows - 1) / tile_rows;
    }
    if (slabs >= 2) {
      cudaError_t perr = host_pipeline(&pipe);
      if (perr != cudaSuccess) return cuda_fail(perr);
      slab_rows = tile_rows * 128;
      n_slabs = slabs;
    }
  }
  // device staging: A, B, D, the three scales, then scratch memory of the staged kernels (one per slab, B shared)
  const size_t a_off = 0, b_off = up(a_bytes), d_off = b_off + up(b_bytes), s_off = d_off + up(d_bytes);
  const size_t sb_off = s_off + 256;
  const size_t sb_bytes = pipe ? up(mmb::staged_shared_b_bytes(N, K)) : 0;
  const size_t w_off = sb_off + sb_bytes;
  const size_t w_each = staged ? up(mmb::staged_workspace_bytes(slab_rows, N, K, S, true, pipe != nullptr)) : 0;
  const size_t total = w_off + w_each * (size_t)n_slabs;
  uint8_t* buf = nullptr;
  cudaMemPool_t pool = nullptr;
  cudaError_t err = staging_pool(&pool);
  if (err != cudaSuccess) return cuda_fail(err);
  std::unique_lock<std::mutex> lock;
  if (pipe) lock = std::unique_lock<std::mutex>(pipe->mu);   // the internal streams and events serve one call at a time
  err = cudaMallocFromPoolAsync(reinterpret_cast<void**>(&buf), total, pool, st);
  if (err != cudaSuccess) return cuda_fail(err);
  int rc = MMB200_OK;
  float scales[3] = {scale_a, scale_b, scale_result ? *scale_result : 1.0f};
  int words[PIPELINE_MAX_SLABS] = {};
  const float* sdev = reinterpret_cast<const float*>(buf + s_off);
  do {
    if (K > 0 && kpad != (size_t)K) {
      err = cudaMemsetAsync(buf, 0, b_off + b_bytes, st);
      if (err != cudaSuccess) break;
    }
    if (!pipe) {
      if (K > 0) {
        err = cudaMemcpy2DAsync(buf + a_off, kpad, A, (size_t)lda, (size_t)K, (size_t)M, cudaMemcpyHostToDevice, st);
        if (err != cudaSuccess) break;
        err = cudaMemcpy2DAsync(buf + b_off, kpad, B, (size_t)ldb, (size_t)K, (size_t)N, cudaMemcpyHostToDevice, st);
        if (err != cudaSuccess) break;
      }
      err = cudaMemcpyAsync(buf + s_off, scales, sizeof(scales), cudaMemcpyHostToDevice, st);
      if (err != cudaSuccess) break;
      rc = mmb200_scaled_mm_ws(buf + a_off, (int64_t)kpad, fmt_a, buf + b_off, (int64_t)kpad, fmt_b, buf + d_off, N,
                               out_dtype, M, N, K, nfma, fast, S, scheme, sdev, sdev + 1,
                               scale_result ? sdev + 2 : nullptr, kernel, w_each ? buf + w_off : nullptr, w_each, stream);
      if (rc != MMB200_OK) break;
      if (w_each) {                       // the staged kernels report a wait that ran out; D is then not copied back
        rc = read_status(buf + w_off, M, N, K, S, st);
        if (rc != MMB200_OK) break;
      }
      err = cudaMemcpy2DAsync(D, (size_t)ldd * es, buf + d_off, (size_t)N * es, (size_t)N * es, (size_t)M,
                              cudaMemcpyDeviceToHost, st);
      break;
    }
    // ---- row slabs on the internal streams
    err = cudaEventRecord(pipe->start, st);                 // the allocation and earlier work of the caller's stream
    if (err != cudaSuccess) break;
    for (int q = 0; q < HostPipeline::STREAMS && err == cudaSuccess; ++q) err = cudaStreamWaitEvent(pipe->s[q], pipe->start, 0);
    if (err != cudaSuccess) break;
    cudaStream_t s0 = pipe->s[0];
    err = cudaMemcpy2DAsync(buf + b_off, kpad, B, (size_t)ldb, (size_t)K, (size_t)N, cudaMemcpyHostToDevice, s0);
    if (err != cudaSuccess) break;
    err = cudaMemcpyAsync(buf + s_off, scales, sizeof(scales), cudaMemcpyHostToDevice, s0);
    if (err != cudaSuccess) break;
    {
      mmb::Params pb;
      std::memset(&pb, 0, sizeof(pb));
      pb.B = buf + b_off; pb.ldb = (long long)kpad; pb.N = N; pb.K = K; pb.fmt_a = fmt_a; pb.fmt_b = fmt_b;
      pb.shared_b = buf + sb_off;
      int launches = 0;
      err = mmb::launch_predecode_b(pb, nfma, s0, &launches);
      if (err != cudaSuccess) break;
      g_launches.fetch_add(launches, std::memory_order_relaxed);
    }
    err = cudaEventRecord(pipe->b_ready, s0);
    if (err != cudaSuccess) break;
    for (int i = 0; i < n_slabs && rc == MMB200_OK; ++i) {
      cudaStream_t sq = pipe->s[i];
      const int m0 = i * slab_rows, rows = (M - m0 < slab_rows) ? M - m0 : slab_rows;
      uint8_t* a_dev = buf + a_off + (size_t)m0 * kpad;
      uint8_t* d_dev = buf + d_off + (size_t)m0 * N * es;
      uint8_t* ws = buf + w_off + (size_t)i * w_each;
      err = cudaMemcpy2DAsync(a_dev, kpad, static_cast<const uint8_t*>(A) + (size_t)m0 * (size_t)lda, (size_t)lda,
                              (size_t)K, (size_t)rows, cudaMemcpyHostToDevice, sq);
      if (err != cudaSuccess) break;
      err = cudaStreamWaitEvent(sq, pipe->b_ready, 0);
      if (err != cudaSuccess) break;
      rc = run(a_dev, (int64_t)kpad, fmt_a, buf + b_off, (int64_t)kpad, fmt_b, d_dev, N, out_dtype, rows, N, K, nfma,
               fast, S, scheme, sdev, sdev + 1, scale_result ? sdev + 2 : nullptr, 1, 1, kernel, sq, ws, w_each, nullptr,
               0, 0, nullptr, nullptr, 0, buf + sb_off);
      if (rc != MMB200_OK) break;
      err = cudaMemcpy2DAsync(static_cast<uint8_t*>(D) + (size_t)m0 * (size_t)ldd * es, (size_t)ldd * es, d_dev,
                              (size_t)N * es, (size_t)N * es, (size_t)rows, cudaMemcpyDeviceToHost, sq);
      if (err != cudaSuccess) break;
    }
  } while (0);
  if (pipe) {
    // back to the caller's stream: it continues when every internal stream is done -- also after an error above, so
    // that the staging memory is not freed under work that was already enqueued
    for (int q = 0; q < HostPipeline::STREAMS; ++q) {
      cudaError_t e2 = cudaEventRecord(pipe->done[q], pipe->s[q]);
      if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(st, pipe->done[q], 0);
      if (e2 != cudaSuccess && err == cudaSuccess) err = e2;
    }
    for (int i = 0; i < n_slabs && err == cudaSuccess && rc == MMB200_OK; ++i) {   // status words of the slabs' bounded waits
      const int m0 = i * slab_rows, rows = (M - m0 < slab_rows) ? M - m0 : slab_rows;
      err = cudaMemcpyAsync(&words[i], buf + w_off + (size_t)i * w_each + mmb::staged_status_offset(rows, N, K, S, true),
                            sizeof(int), cudaMemcpyDeviceToHost, st);
    }
  }
  cudaError_t ferr = cudaFreeAsync(buf, st);
  cudaError_t serr = cudaStreamSynchronize(st);   // the scales array and the caller's buffers must outlive the copies
  if (rc != MMB200_OK) return rc;
  if (err != cudaSuccess) return cuda_fail(err);
  if (ferr != cudaSuccess) return cuda_fail(ferr);
  if (serr != cudaSuccess) return cuda_fail(serr);
  for (int i = 0; i < n_slabs; ++i)
    if (words[i] != 0) return MMB200_ERR_TIMEOUT;   // slabs are copied back as they finish: D is unspecified then
  return MMB200_OK;
}

int mmb200_kernel_for(const void* A, int64_t lda, const void* B, int64_t ldb, int K, int nfma, int S) {
  mmb::Params p;
  std::memset(&p, 0, sizeof(p));
  p.A = static_cast<const uint8_t*>(A);
  p.B = static_cast<const uint8_t*>(B);
  p.lda = lda; p.ldb = ldb; p.K = K; p.S = S;
  return mmb::fast_supports(p, nfma) ? MMB200_KERNEL_FAST : MMB200_KERNEL_INTEGER;
}

int64_t mmb200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
