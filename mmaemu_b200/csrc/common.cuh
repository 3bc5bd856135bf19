// Shared device/host definitions of the mmaemu_b200 kernels: enums, the per-launch parameter block, FP8 decode,
// the plan walker (which k-tiles form which chain, and how chains and split partials are combined), the IEEE class of
// non-finite outputs and the fused epilogue.
//
// Reference behaviour restated here (astding/mmaemu): mmaemu/formats.py:14-62 (formats), mmaemu/model/plan.py:62-156
// (split layouts, slow-accumulation chunks, reduction orders), mmaemu/model/specials.py:25-80 (non-finite inputs),
// mmaemu/model/epilogue.py:34-78 (alpha, output conversion, canonical NaN).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <type_traits>

#include "../../include/mmaemu_b200.h"
#include "plan.cuh"

namespace mmb {

constexpr int PRESET_B200_MMA_SYNC = MMB200_PRESET_B200_MMA_SYNC;   // late-accumulator preset: integer kernel only
constexpr uint32_t CANON_NAN32 = 0x7FFFFFFFu;
#define MMB200_MAX_SLICES 32

// Everything a kernel needs; passed by value (__grid_constant__).
struct Params {
  const uint8_t* A;   // [M, K] codes, row stride lda
  const uint8_t* B;   // [N, K] codes, row stride ldb
  void* D;            // [M, N] of out_dtype, row stride ldd (elements)
  const float* scale_a;       // device scalars; nullptr = 1.0 (accumulate / chain entry points)
  const float* scale_b;
  const float* scale_result;  // nullable
  long long lda, ldb, ldd;
  int M, N, K;
  int fmt_a, fmt_b, out_dtype;
  int fast, S, scheme;
  int epilogue;       // 0: store the fp32 accumulator (no alpha); 1: full epilogue
  int patch_nonfinite;  // 0: non-finite codes are plain +0 (chain entry point); 1: IEEE patch
  int tiles_m, tiles_n;
  // scratch memory of the staged fast kernel (null otherwise): decoded tiles, per-row non-finite flags, status word
  unsigned char* ws_a;
  unsigned char* ws_b;
  int* ws_flag_a;
  int* ws_flag_b;
  int* status;
  int k_tiles;
  // B decoded by an earlier launch (the host-buffer entry point decodes B once and runs the rows of A slab by slab):
  // shared_b holds B's tile images followed by its column flags (staged_shared_b_bytes); the launch then neither
  // decodes B nor clears its flags. only_b: decode B into shared_b and launch nothing else.
  unsigned char* shared_b;
  int only_b;
  int few_rows;          // the staged launch uses the kernels that work on 16 rows per CTA and decode both operands
                         // themselves (set by the launcher: calls with at most 16 rows, and calls whose 128 x 128 output
                         // tiles and chains would leave most SMs idle)
  int row_groups;        // 16-row groups per 128-row tile in that case (grid z): 1 or 8
  int no_tensor_epass;   // 1: the staged kernels keep the exponent pass on the CUDA cores (packed integers) for every pair
  // multi-GPU assembly: the same output element is also stored at the same index of every peer_D[i] (device pointers
  // into other GPUs' memory, mapped into this process), so that every GPU ends up with the whole result
  void* peer_D[MMB200_MAX_PEERS];
  int n_peers;
  int wait_polls;        // bound of every wait on an mbarrier in the staged kernels, in polls of up to ~1 us each
  int test_announce_extra;  // test hook: bytes the issuing thread announces beyond what it copies (the wait then runs out)
  // quantise prologue (staged kernels, operand A in E4M3 only): when a_hp is set, the pre-decode pass reads M x K
  // activations of a_hp_dtype (MMB200_HP_F32 / MMB200_HP_BF16, row stride ld_hp elements), forms the E4M3 codes of
  // clamp(x * *a_quant_scale, +-448), writes them to a_codes (row stride lda; A must point there too) and decodes them
  const void* a_hp;
  long long ld_hp;
  int a_hp_dtype;
  const float* a_quant_scale;
  uint8_t* a_codes;
  // split plans on the staged kernels: the order of the 32-element k-tiles (plan_sequence) and, per output tile, the
  // running total and the pair slot of the split reduction (scratch memory)
  const uint32_t* ws_seq;
  int seq_len;
  const uint32_t* ws_events;   // K slices: the sequence entries after which a chain or a split is complete, in order
  int n_events;
  float* ws_tot;
  float* ws_slot;
  // K-sliced execution of plans with few output tiles (chains are independent of one another): slice y of the grid
  // walks the sequence entries [slice_start[y], slice_start[y + 1]) and stores its chain results, chain_base[y] onward,
  // into ws_chains [tile][chain][output of the thread][thread]; a second kernel adds them in the plan's order
  int slices;
  int n_chains;
  int plan_group;
  int slice_start[MMB200_MAX_SLICES + 1];
  int chain_base[MMB200_MAX_SLICES + 1];
  float* ws_chains;
};

// ---------------------------------------------------------------------------------------------------------------
// FP8 decode of one code byte into (magnitude significand, clamped exponent, sign, class).
// E4M3: s eeee mmm, bias 7, emin -6, NaN = x1111111, no Inf. E5M2: s eeeee mm, bias 15, emin -14, Inf = x1111100,
// NaN = x11111{01,10,11}. Subnormals keep a denormalised significand at emin. Zero and non-finite codes have
// significand 0 (a zero product never takes part in the block maximum and adds nothing).
struct Dec {
  int mag;   // integer significand: E4M3 in units of 2^-3 (<= 15), E5M2 in units of 2^-2 (<= 7)
  int exp;   // clamped exponent; meaningless when mag == 0
  int neg;   // sign bit
  int cls;   // 0 finite, 1 NaN, 2 +-Inf
};

__host__ __device__ __forceinline__ Dec decode_fp8(uint32_t code, int fmt) {
  Dec d;
  d.neg = (code >> 7) & 1;
  const uint32_t x = code & 0x7Fu;
  if (fmt == MMB200_FMT_E4M3) {
    const int e = x >> 3, m = x & 7;
    d.cls = (x == 0x7F) ? 1 : 0;
    d.mag = d.cls ? 0 : (e ? (8 | m) : m);
    d.exp = e ? e - 7 : -6;
  } else {
    const int e = x >> 2, m = x & 3;
    d.cls = (e == 31) ? (m ? 1 : 2) : 0;
    d.mag = d.cls ? 0 : (e ? (4 | m) : m);
    d.exp = e ? e - 15 : -14;
  }
  return d;
}

__host__ __device__ __forceinline__ int fmt_frac_bits(int fmt) { return fmt == MMB200_FMT_E4M3 ? 3 : 2; }

// ---------------------------------------------------------------------------------------------------------------
// IEEE class of sum_k a[k] * b[k] over the original codes when it is not finite: NaN for any NaN operand, Inf * 0, or
// +Inf and -Inf terms together, else +-Inf. Returns false when the sum is finite.
__device__ inline bool nonfinite_value(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, int K, int fmt_a,
                                       int fmt_b, uint32_t& bits) {
  bool nan = false, pos = false, neg = false;
  for (int k = 0; k < K; ++k) {
    const Dec da = decode_fp8(a[k], fmt_a), db = decode_fp8(b[k], fmt_b);
    if ((da.cls | db.cls) == 0) continue;
    if (da.cls == 1 || db.cls == 1) { nan = true; continue; }
    const bool a_zero = da.cls == 0 && da.mag == 0, b_zero = db.cls == 0 && db.mag == 0;
    if (a_zero || b_zero) { nan = true; continue; }
    if (da.neg ^ db.neg) neg = true; else pos = true;
  }
  if (nan || (pos && neg)) { bits = CANON_NAN32; return true; }
  if (pos) { bits = 0x7F800000u; return true; }
  if (neg) { bits = 0xFF800000u; return true; }
  return false;
}

// The same from the class flags of the output's row and column (bit 0: a NaN code was seen, bit 1: an infinity): a NaN
// code anywhere in the row or the column makes the sum NaN whatever it is multiplied with, so only outputs whose row or
// column holds infinities and no NaN need the walk over K. Returns false when the sum is finite.
__device__ __forceinline__ bool nonfinite_patch(int flags, const uint8_t* __restrict__ a, const uint8_t* __restrict__ b,
                                                int K, int fmt_a, int fmt_b, uint32_t& bits) {
  if (flags & 1) { bits = CANON_NAN32; return true; }
  if (flags & 2) return nonfinite_value(a, b, K, fmt_a, fmt_b, bits);
  return false;
}

// ---------------------------------------------------------------------------------------------------------------
// Epilogue: y = RN32(fma(acc, alpha, +0)) with alpha = RN32(scale_a * scale_b); conversion to the output dtype with
// a second rounding; fp8 outputs: optional RN32(y * scale_result), saturation to +-448 / +-57344 (Inf included, NaN
// passes), round to nearest even; canonical NaN (fp32 0x7FFFFFFF, bf16 / fp16 0x7FFF, fp8 0x7F).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
  uint16_t h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));   // IEEE round to nearest even; overflow gives Inf
  return h;
}

__device__ __forceinline__ uint8_t f32_to_fp8_bits(float f, int fmt) {
  const uint32_t u = __float_as_uint(f);
  const uint32_t sign = (u >> 24) & 0x80u, x = u & 0x7FFFFFFFu;
  if (x > 0x7F800000u) return 0x7F;
  const int mbits = fmt == MMB200_FMT_E4M3 ? 3 : 2, bias = fmt == MMB200_FMT_E4M3 ? 7 : 15;
  const uint32_t maxcode = fmt == MMB200_FMT_E4M3 ? 0x7Eu : 0x7Bu;
  const uint32_t maxbits = fmt == MMB200_FMT_E4M3 ? 0x43E00000u : 0x47600000u;   // 448.0f, 57344.0f
  if (x >= maxbits) return (uint8_t)(sign | maxcode);
  if (x < 0x00800000u) return (uint8_t)sign;
  const int e = (int)(x >> 23) - 127, emin = 1 - bias;
  const uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
  int sh = 23 - mbits;
  int eb = e + bias;
  if (e < emin) { sh += emin - e; eb = 0; }
  if (sh > 31) return (uint8_t)sign;
  uint32_t q = m >> sh;
  const uint32_t rem = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  uint32_t code = eb > 0 ? (((uint32_t)(eb - 1) << mbits) + q) : q;
  if (code > maxcode) code = maxcode;
  return (uint8_t)(sign | code);
}

struct Epilogue {
  float alpha, scale_result;
  int has_scale_result, out_dtype, enabled, n_peers;
  void* const* peers;
  __device__ __forceinline__ void init(const Params& p) {
    enabled = p.epilogue;
    out_dtype = p.out_dtype;
    const float sa = p.scale_a ? *p.scale_a : 1.0f, sb = p.scale_b ? *p.scale_b : 1.0f;
    alpha = __fmul_rn(sa, sb);
    has_scale_result = p.scale_result != nullptr;
    scale_result = has_scale_result ? *p.scale_result : 1.0f;
    n_peers = p.n_peers;
    peers = p.peer_D;
  }
  __device__ __forceinline__ int elem_size() const {
    return (!enabled || out_dtype == MMB200_OUT_F32) ? 4 : (out_dtype <= MMB200_OUT_F16 ? 2 : 1);
  }
  // Bit pattern of one output element (in the low bits of the result) for an accumulator value.
  __device__ __forceinline__ uint32_t bits_of(float acc) const {
    if (!enabled) {
      const uint32_t u = __float_as_uint(acc);
      return (u & 0x7FFFFFFFu) > 0x7F800000u ? CANON_NAN32 : u;
    }
    float y = __fmaf_rn(acc, alpha, 0.0f);
    switch (out_dtype) {
      case MMB200_OUT_F32: {
        const uint32_t u = __float_as_uint(y);
        return (u & 0x7FFFFFFFu) > 0x7F800000u ? CANON_NAN32 : u;
      }
      case MMB200_OUT_BF16: return f32_to_bf16_bits(y);
      case MMB200_OUT_F16: return f32_to_f16_bits(y);
      default:
        if (has_scale_result) y = __fmul_rn(y, scale_result);
        return f32_to_fp8_bits(y, out_dtype == MMB200_OUT_E4M3 ? MMB200_FMT_E4M3 : MMB200_FMT_E5M2);
    }
  }
  // One element at index idx of D and of every peer's buffer (plain stores; the peers' copies become visible to their
  // GPUs with the synchronisation that follows the kernel).
  __device__ __forceinline__ void store(void* D, long long idx, float acc) const {
    const uint32_t b = bits_of(acc);
    const int es = elem_size();
    for (int q = -1; q < n_peers; ++q) {
      void* dst = q < 0 ? D : peers[q];
      if (es == 4) reinterpret_cast<uint32_t*>(dst)[idx] = b;
      else if (es == 2) reinterpret_cast<uint16_t*>(dst)[idx] = (uint16_t)b;
      else reinterpret_cast<uint8_t*>(dst)[idx] = (uint8_t)b;
    }
  }
  // Tile-wise output for the 128 x 128 kernels: every thread parks the elements it owns in a shared-memory image of the
  // CTA's output tile (rows of 128 elements, 16 bytes of padding per row), then the whole CTA writes the image out in
  // 16-byte pieces of whole rows -- to D and to every peer's buffer -- so that the stores are full 32-byte sectors
  // locally and large packets over NVLink instead of 2-byte scattered ones.
  static constexpr int TILE_DIM = 128;
  __device__ __forceinline__ int tile_pitch() const { return TILE_DIM * elem_size() + 16; }
  __device__ __forceinline__ void park(unsigned char* tile, int lr, int lc, float acc) const {
    const uint32_t b = bits_of(acc);
    const int es = elem_size();
    unsigned char* dst = tile + lr * tile_pitch() + lc * es;
    if (es == 4) *reinterpret_cast<uint32_t*>(dst) = b;
    else if (es == 2) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)b;
    else *dst = (uint8_t)b;
  }
  // `rows`: how many rows of the image (from its first) were parked
  __device__ __forceinline__ void flush(const Params& p, const unsigned char* tile, int m0, int n0, int tid,
                                        int nthreads, int rows = TILE_DIM) const {
    const int es = elem_size(), pitch = tile_pitch(), per_row = TILE_DIM * es / 16, per_piece = 16 / es;
    bool vec = (reinterpret_cast<uintptr_t>(p.D) % 16 == 0) && ((p.ldd * es) % 16 == 0);
    for (int q = 0; q < n_peers; ++q) vec = vec && (reinterpret_cast<uintptr_t>(peers[q]) % 16 == 0);
    for (int idx = tid; idx < rows * per_row; idx += nthreads) {
      const int row = idx / per_row, piece = idx % per_row, gm = m0 + row, gn = n0 + piece * per_piece;
      if (gm >= p.M || gn >= p.N) continue;
      const unsigned char* src = tile + row * pitch + piece * 16;
      const long long off = ((long long)gm * p.ldd + gn) * es;
      if (vec && gn + per_piece <= p.N) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        for (int q = -1; q < n_peers; ++q)
          *reinterpret_cast<uint4*>(static_cast<unsigned char*>(q < 0 ? p.D : peers[q]) + off) = v;
      } else {
        const int bytes = min(per_piece, p.N - gn) * es;
        for (int q = -1; q < n_peers; ++q) {
          unsigned char* dst = static_cast<unsigned char*>(q < 0 ? p.D : peers[q]) + off;
          for (int e = 0; e < bytes; ++e) dst[e] = src[e];
        }
      }
    }
  }
};

// Launchers implemented by the kernel translation units; each returns a cudaError_t.
cudaError_t launch_integer(const Params& p, int nfma, cudaStream_t stream);
cudaError_t launch_fast(const Params& p, int nfma, cudaStream_t stream);
bool fast_supports(const Params& p, int nfma);
// Staged fast kernel: scratch bytes it needs for a shape, and the launch (pre-decode of both operands, then the GEMM).
// `launches` is increased by the number of kernels launched.
bool staged_supports(const Params& p, int nfma);            // like fast_supports, any plan
size_t staged_workspace_bytes(int M, int N, int K, int S, bool with_slices, bool shared_b = false);
// Bytes of a shared B area (tile images of every 128-column group, then one int per column), and the launch that fills
// it (p.B, p.ldb, p.N, p.K, the formats; p.shared_b = the area, 128-byte aligned).
size_t staged_shared_b_bytes(int N, int K);
cudaError_t launch_predecode_b(const Params& p, int nfma, cudaStream_t stream, int* launches);
cudaError_t launch_staged(const Params& p, int nfma, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                          int* launches);
// Byte offset, inside the scratch memory of a staged launch, of the int32 status word (0, or 1 when a bounded wait ran
// out and the output was not written); the same with and without K slices.
size_t staged_status_offset(int M, int N, int K, int S, bool shared_b = false);
// Test hooks of the bounded waits (process-wide; wait_polls <= 0 and announce_extra <= 0 restore the defaults).
void staged_test_hooks(int wait_polls, int announce_extra);
// Text of the last CUDA runtime error seen by this thread inside the library; returns MMB200_ERR_LAUNCH.
int record_cuda_error(cudaError_t err);

}  // namespace mmb
