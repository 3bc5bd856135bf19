// Scalar building blocks of the fast kernel's arithmetic, written so that the very same code compiles for the device
// and for the host (tests/test_fast_math_host.py builds them with g++ and checks them against the oracle's block
// model; on the host the directed-rounding instructions are emulated with the floating-point environment).
//
// Notation: E is the block's alignment exponent, u = 2^(E-13) the grid, "field" the biased fp32 exponent field.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define MMB_HD __host__ __device__ __forceinline__
#else
#define MMB_HD static inline
#endif

#if !defined(__CUDA_ARCH__)
#include <cfenv>
#include <cmath>
#include <cstring>
#endif

namespace mmb {
namespace fm {

#if defined(__CUDA_ARCH__)
MMB_HD uint32_t f2u(float f) { return __float_as_uint(f); }
MMB_HD float u2f(uint32_t u) { return __uint_as_float(u); }
MMB_HD float fma_rz(float a, float b, float c) { return __fmaf_rz(a, b, c); }
MMB_HD float add_rz(float a, float b) { return __fadd_rz(a, b); }
MMB_HD float add_rn(float a, float b) { return __fadd_rn(a, b); }
MMB_HD float sub_rn(float a, float b) { return __fsub_rn(a, b); }
MMB_HD float max_abs(float v, float p) { return fmaxf(fabsf(v), p); }
MMB_HD int addmin_relu(int a, int b, int c) { return __viaddmin_s32_relu(a, b, c); }
MMB_HD int addmax(int a, int b, int c) { return __viaddmax_s32(a, b, c); }
MMB_HD uint32_t addmax16x2(uint32_t a, uint32_t b, uint32_t c) { return __viaddmax_s16x2(a, b, c); }
MMB_HD uint32_t dot4(uint32_t a, uint32_t b, uint32_t c) { return __dp4a(a, b, c); }
MMB_HD int round_to_int(float x) { return __float2int_rn(x); }
MMB_HD uint32_t replicate_byte(uint32_t x) { return __byte_perm(x, 0u, 0u); }   // x < 256 in all four bytes
#else
MMB_HD uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
MMB_HD float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
MMB_HD float fma_rz(float a, float b, float c) {
  const int old = std::fegetround();
  std::fesetround(FE_TOWARDZERO);
  volatile float r = std::fmaf(a, b, c);
  std::fesetround(old);
  return r;
}
MMB_HD float add_rz(float a, float b) {
  const int old = std::fegetround();
  std::fesetround(FE_TOWARDZERO);
  volatile float va = a, vb = b;
  volatile float r = va + vb;
  std::fesetround(old);
  return r;
}
MMB_HD float add_rn(float a, float b) { volatile float r = a + b; return r; }
MMB_HD float sub_rn(float a, float b) { volatile float r = a - b; return r; }
MMB_HD float max_abs(float v, float p) { return std::fmax(std::fabs(v), p); }
MMB_HD int addmin_relu(int a, int b, int c) { int s = a + b; s = s < c ? s : c; return s > 0 ? s : 0; }
MMB_HD int addmax(int a, int b, int c) { const int s = a + b; return s > c ? s : c; }
MMB_HD int round_to_int(float x) { return (int)std::lrintf(x); }          // nearest even in the default rounding mode
MMB_HD uint32_t replicate_byte(uint32_t x) { return (x & 0xFFu) * 0x01010101u; }
MMB_HD uint32_t addmax16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r = 0;
  for (int h = 0; h < 2; ++h) {
    const int s = (int16_t)(a >> (16 * h)) + (int16_t)(b >> (16 * h)), m = (int16_t)(c >> (16 * h));
    r |= (uint32_t)(uint16_t)(int16_t)(s > m ? s : m) << (16 * h);
  }
  return r;
}
MMB_HD uint32_t dot4(uint32_t a, uint32_t b, uint32_t c) {
  for (int q = 0; q < 4; ++q) c += ((a >> (8 * q)) & 0xFFu) * ((b >> (8 * q)) & 0xFFu);
  return c;
}
#endif

constexpr int FMT_E4M3 = 0, FMT_E5M2 = 1;

template <int FMT> struct F8;
template <> struct F8<FMT_E4M3> {
  static constexpr int TMAX = 17;      // largest low-bit code: (8 + 6) + 3 trailing zeros
  static constexpr int TOFF = 9;       // low-bit code = (position of the lowest set bit of the value) + 9
  static constexpr int EOFF = 6;       // clamped exponent + 6 >= 0
};
template <> struct F8<FMT_E5M2> {
  static constexpr int TMAX = 31;      // (15 + 14) + 2
  static constexpr int TOFF = 16;
  static constexpr int EOFF = 14;
};
constexpr int XBIAS_A = 64, XBIAS_B = 63;   // E-pass exponent biases; their sum is the fp32 exponent bias

// Constants of a format pair. A product of nonzero codes is a multiple of u iff Ta + Tb >= Th with
// Th = E - 13 + TOFF_A + TOFF_B. The byte sum  Ta + (Tb + 127 - TSUM) + clamp(TSUM + 1 - Th, 0, TSUM + 1)  has bit 7
// set exactly then; zero operands (codes TSUM + 1 and 128) always set it; the largest sum, 130 + 2 * TSUM, fits a byte.
template <int FA, int FB> struct Pair {
  static constexpr int TSUM = F8<FA>::TMAX + F8<FB>::TMAX;
  static constexpr uint32_t TADD_A = 0, TADD_B = 127 - TSUM;
  static constexpr uint32_t TZERO_A = TSUM + 1, TZERO_B = 128;
  static constexpr int KTH = TSUM + 1 + 127 + 13 - F8<FA>::TOFF - F8<FB>::TOFF;   // threshold = clamp(KTH - field)
};

// Byte-parallel decode of 4 codes (one 32-bit word) into: the sanitised codes `ws` (non-finite codes become +0), the
// E-pass exponent bytes `xb` (clamped exponent + xbias, 0 for zero codes), the low-bit codes `tcode` (`tzero` for zero
// codes), the sign bits and the non-finite classes seen (bit 0 NaN, bit 1 Inf). No operation carries from one byte
// into the next.
template <int FMT, int POWMUL = 8>
MMB_HD void decode_bits(uint32_t w, int xbias, uint32_t tadd, uint32_t tzero, uint32_t& ws, uint32_t& xb,
                        uint32_t& tcode, uint32_t& sign, uint32_t& cls, uint32_t* pow256 = nullptr,
                        uint32_t pow_bias = 0) {
  sign = w & 0x80808080u;
  uint32_t m7 = w & 0x7F7F7F7Fu;
  uint32_t e, tz, nf;
  if (FMT == FMT_E4M3) {
    nf = (m7 + 0x01010101u) & 0x80808080u;                      // 0x7F: NaN
    cls = nf ? 1u : 0u;
  } else {
    nf = (m7 + 0x04040404u) & 0x80808080u;                      // >= 0x7C: Inf or NaN
    const uint32_t frac = ((m7 & 0x03030303u) + 0x7F7F7F7Fu) & 0x80808080u;   // 0x80 where the fraction is nonzero
    cls = ((nf & frac) ? 1u : 0u) | ((nf & ~frac) ? 2u : 0u);
  }
  m7 &= ~((nf >> 7) * 0xFFu);                                   // non-finite codes count as +0
  const uint32_t nzm = (((m7 + 0x7F7F7F7Fu) & 0x80808080u) >> 7) * 0xFFu;   // 0xFF per nonzero byte
  if (FMT == FMT_E4M3) {
    e = (m7 >> 3) & 0x0F0F0F0Fu;
    const uint32_t y = (m7 & 0x07070707u) | 0x08080808u;
    const uint32_t lsb = y & ((~y & 0x0F0F0F0Fu) + 0x01010101u);  // lowest set bit of (8 | m): 1, 2, 4 or 8
    tz = ((lsb >> 1) & 0x07070707u) - ((lsb >> 3) & 0x01010101u); // its position: 0..3
  } else {
    e = (m7 >> 2) & 0x1F1F1F1Fu;
    const uint32_t y = (m7 & 0x03030303u) | 0x04040404u;
    const uint32_t lsb = y & ((~y & 0x07070707u) + 0x01010101u);  // 1, 2 or 4
    tz = (lsb >> 1) & 0x03030303u;                                // 0..2
  }
  const uint32_t ec = e - (((e + 0x7F7F7F7Fu) >> 7) & 0x01010101u);   // clamped exponent + EOFF: max(e, 1) - 1
  tcode = ((ec + tz + tadd * 0x01010101u) & nzm) | ((tzero * 0x01010101u) & ~nzm);
  xb = (ec + (uint32_t)(xbias - F8<FMT>::EOFF) * 0x01010101u) & nzm;
  ws = sign | m7;
  // Per byte the fp32 / bf16 exponent field of a power 2^(POWMUL ea + const), i.e. pow_bias + POWMUL (ea + EOFF); 0 for
  // zero codes (the tensor-core exponent pass sums products of these powers, see block_exponent_pow and
  // block_exponent_pow5). POWMUL 8 serves E4M3 x E4M3, POWMUL 5 the mixed pairs; ec <= 29, so 5 ec fits a byte.
  if (pow256) {
    const uint32_t scaled = POWMUL == 8 ? (ec << 3) : ((ec << 2) + ec);
    *pow256 = (POWMUL == 8 && FMT != FMT_E4M3) ? 0u : ((scaled + pow_bias * 0x01010101u) & nzm);
  }
}

// Tensor-core exponent pass (E4M3 x E4M3): the (max, +) product is read off an ordinary product of powers. The
// operands are 2^(8 ea - 7) and 2^(8 eb) (exponent fields POW_BIAS_A + 8 (ea + 6) and POW_BIAS_B + 8 (eb + 6), exact in
// bf16), so a nonzero product contributes 2^(8 (ea + eb) - 7) = 2^(8 e - 7) with fp32 exponent field 120 + 8 e, a
// multiple of 8. The sum S of a block's at most 32 such terms -- in any order and with any rounding or truncation of
// the small addends -- is at least its largest term 2^(8 E - 7) and below 33 * (1 + 2^-8)^33 times it, which is
// less than 2^8 times it: field(S) >> 3 = 15 + E exactly. e lies in [-12, 16], so every term is a normal number and the
// sum stays below 2^126.
constexpr uint32_t POW_BIAS_A = 72, POW_BIAS_B = 79;

// The exponent field of 2^E, E = max(E_prod, exponent(acc)), from such a sum. f2u(S) >> 3 holds 15 + E_prod in the
// exponent position (and bits of no consequence below it: the maximum with |acc| is only used for its exponent field).
// A block without nonzero products has S = 0 and yields max(2^-15, |acc|): below every product exponent (>= -12), and
// every accumulator is a multiple of 2^(-12 - 13), so it is a multiple of the unit 2^(-15 - 13) and passes unchanged.
MMB_HD uint32_t block_exponent_pow_raw(float acc, float S) {
  // a floating-point maximum with |acc| (the absolute value is an operand modifier, not an instruction); both
  // arguments are positive normal numbers or zero. Raw: the field sits in bits 23..30, bit 31 is zero, the bits below
  // the field are of no consequence (block_start_at reads the field alone).
  return f2u(max_abs(acc, u2f((f2u(S) >> 3) + (112u << 23))));
}
MMB_HD uint32_t block_exponent_pow(float acc, float S) { return block_exponent_pow_raw(acc, S) & 0x7F800000u; }

// Tensor-core exponent pass of the mixed pairs (E5M2 x E4M3 and E4M3 x E5M2). The product exponents span 44 values,
// too many for powers of 256 in fp32's 254 binades, so the powers are 2^(5 (ea + EOFF) + 66 - 127) and
// 2^(5 (eb + EOFF) + 66 - 127) (exponent fields POW5_BIAS + 5 ec, exact in bf16, between 66 and 211): a nonzero
// product has the field 5 + 5 s with s = eca + ecb in [0, 43]. A sum of at most 16 such terms -- what one
// mma.sync.m16n8k16 adds -- lies in [2^(5 S), 2^(5 S) * 16 * (1 + 2^-8)^16), S the largest s, whatever the order and
// rounding of the additions: below 2^(5 S + 4.1), so floor(field / 5) = 1 + S exactly and the mantissa of a sum whose
// field is 5 S + 9 stays below 1.07. A block of 32 products takes the larger of its two 16-term sums (max and floor
// commute). The division by 5 is a multiplication of the float's bit pattern x = field * 2^23 + mantissa:
// floor(x / (5 * 2^23)) = (x * 1639) >> 36, exact here because 1639 / 2^36 exceeds 1 / (5 * 2^23) by a factor
// 1 + 3.7e-4, which moves a quotient below 51.1 by less than 0.02, and the fractional part of the exact quotient never
// exceeds (4 + 0.07) / 5.
constexpr uint32_t POW5_BIAS = 66;
MMB_HD uint32_t mulhi_u32(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return (uint32_t)(((uint64_t)a * b) >> 32);
#endif
}
// Raw exponent field (see block_exponent_pow_raw) of 2^E, E = max(E_prod, exponent(acc)), from the larger 16-term sum.
// A block without nonzero products has P = 0 and yields max(2^(-1 - EOFF_A - EOFF_B), |acc|): below every product
// exponent, and every accumulator is a multiple of that value's unit.
template <int FA, int FB>
MMB_HD uint32_t block_exponent_pow5_raw(float acc, float P) {
  const uint32_t q = mulhi_u32(f2u(P), 1639u) >> 4;                       // floor(field / 5) = 1 + eca + ecb, or 0
  const uint32_t field = q + (uint32_t)(126 - F8<FA>::EOFF - F8<FB>::EOFF);
  return f2u(max_abs(acc, u2f(field << 23)));
}

// The same from the packed-integer E-pass: `esum_shifted` is the maximum of (xa + xb) for this output (the exponent
// field of 2^E_prod, or a value below every real field when the block has no nonzero product), already shifted to bits
// 23..30; other bits: any.
MMB_HD uint32_t block_exponent(float acc, uint32_t esum_shifted) {
  return f2u(max_abs(acc, u2f(esum_shifted & 0x7FFFFFFFu)));      // raw: see block_exponent_pow_raw
}

// Block start, given the exponent field of 2^E in bits 23..30 of `eb` (bit 31 zero, lower bits any): returns
// R = 1.5 * 2^(E+10) + trunc(acc), the threshold byte replicated four times, and the offset 1.5 * 2^(E+10) itself, which
// the block end subtracts again.
template <int FA, int FB>
MMB_HD float block_start_at(float acc, uint32_t eb, uint32_t& tt, float& offset) {
  const uint32_t field = eb >> 23;
  const uint32_t c0bits = field * 0x00800000u + 0x05400000u;      // 1.5 * 2^(E+10), from the field alone
  const float mc = u2f((f2u(acc) & 0x80000000u) | c0bits);        // same sign as acc
  const float ct = sub_rn(add_rz(acc, mc), mc);                   // acc truncated toward zero to multiples of u
  tt = replicate_byte((uint32_t)addmin_relu(Pair<FA, FB>::KTH, -(int)field, Pair<FA, FB>::TSUM + 1));
  offset = u2f(c0bits);
  return add_rn(ct, offset);
}
template <int FA, int FB>
MMB_HD float block_start(float acc, uint32_t esum_shifted, uint32_t& tt, float& offset) {
  return block_start_at<FA, FB>(acc, block_exponent(acc, esum_shifted), tt, offset);
}

// One product: R + floor(a * b / u) * u.
MMB_HD float product(float a, float b, float R) { return fma_rz(a, b, R); }

// Four products of one output (codes of 4 consecutive k): count those that are negative and not a multiple of u.
// The count is kept apart from R and scaled by 128 (the flag stays in bit 7 of its byte), so a group costs one
// three-input add, one three-input logic operation and one dot4; apply_count adds one ulp per counted product, once per
// block. R is positive (its offset 1.5 * 2^(E+10) exceeds the truncated accumulator), so adding to its bits adds ulps.
MMB_HD uint32_t count_group(uint32_t n128, uint32_t ta, uint32_t sa, uint32_t tb, uint32_t sb, uint32_t tt) {
  const uint32_t v = ta + tb + tt;                                // bit 7 of a byte: multiple of u
  return dot4(~v & (sa ^ sb), 0x01010101u, n128);
}
MMB_HD float apply_count(float R, uint32_t n128) { return u2f(f2u(R) + (n128 >> 7)); }

// Block end: acc = R - 1.5 * 2^(E+10) (exact; R never leaves the binade of its offset). The offset is the one block_start_at
// returned, or -- where keeping it in a register costs more than one logic operation -- rebuilt from R's exponent field.
MMB_HD float block_end(float R, float offset) { return sub_rn(R, offset); }
MMB_HD float block_end(float R) { return sub_rn(R, u2f((f2u(R) & 0xFF800000u) | 0x00400000u)); }

// Quantise prologue: E4M3 code of a value that was already multiplied by the quantisation scale: clamp to +-448
// (infinities too), round to nearest even into the normal or subnormal grid, the sign kept on zeros; NaN gives 0x7F
// with the value's sign bit -- the result of torch's  v.clamp(-448, 448).to(torch.float8_e4m3fn).
MMB_HD uint32_t quantise_e4m3(float v) {
  uint32_t bits = f2u(v);
  const uint32_t sign = (bits >> 24) & 0x80u;
  bits &= 0x7FFFFFFFu;
  if (bits > 0x7F800000u) return sign | 0x7Fu;                    // NaN
  if (bits > 0x43E00000u) bits = 0x43E00000u;                     // 448
  if (bits < (121u << 23))                                        // below 2^-6: multiples of 2^-9, ties to even
    return sign | (uint32_t)round_to_int(u2f(bits) * 512.0f);
  bits += ((uint32_t)(7 - 127) << 23) + 0x7FFFFu + ((bits >> 20) & 1u);
  return sign | (bits >> 20);
}

// Chain end: cut to 14 significant bits, toward zero. +0 stays +0.
MMB_HD float chain_cut(float acc) {
  const float m2 = u2f((f2u(acc) & 0xFF800000u) + (10u << 23));
  return sub_rn(add_rz(acc, m2), m2);
}

}  // namespace fm
}  // namespace mmb
