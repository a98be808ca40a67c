// Device helpers shared by the block-quantize kernels: bf16 unpacking, packed abs-max,
// the fixed 16-point Hadamard transform, the scale arithmetic of both formats and the
// tile-edge store helpers.
#pragma once

#include <cuda_fp8.h>
#include <float.h>

#include "mt_common.cuh"

namespace mt {

constexpr int QT_ROWS = 128;     // tile rows (tokens)
constexpr int QT_COLS = 128;     // tile columns (features)
constexpr int Q_THREADS = 256;   // 8 warps

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Packed bf16x2 running abs-max: |result| = max(|a|, |b|) per half (the sign bit of the result
// is the xor of the input signs and is stripped at the end with absmax_finish*).
__device__ __forceinline__ uint32_t absmax2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Larger of the two |bf16| halves of an absmax2 accumulator, as fp32.
__device__ __forceinline__ float absmax2_to_float(uint32_t m) {
  m &= 0x7FFF7FFFu;
  return fmaxf(bf16_lo(m), bf16_hi(m));
}
__device__ __forceinline__ float absmax2_lo(uint32_t m) { return bf16_lo(m & 0x7FFF7FFFu); }
__device__ __forceinline__ float absmax2_hi(uint32_t m) { return bf16_hi(m & 0x7FFF7FFFu); }

// ---- two fp32 values in one 64-bit register (Blackwell packed fp32 arithmetic) ----
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pack2(float lo, float hi) {
  f32x2_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2_t mul2(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2_t add2(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c) {
  f32x2_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2_t sub2(f32x2_t a, f32x2_t b) {
  f32x2_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// Packed bf16x2 word -> (low half, high half) as packed fp32.
__device__ __forceinline__ f32x2_t bf16x2_to_f32x2(uint32_t w) { return pack2(bf16_lo(w), bf16_hi(w)); }
// Packed fp32 pair -> packed bf16x2 word (round to nearest even), low element in the low half.
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(f32x2_t v) {
  float lo, hi;
  unpack2(v, lo, hi);
  uint32_t w;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
  return w;
}

__device__ __forceinline__ float round_to_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// 16-point randomized Hadamard transform of two adjacent columns at once.
// w[j] holds rows j = 0..15 of the two columns as packed bf16x2; on return w[j] holds
// y_j = bf16( (1/4) * sum_i s_i * x_i * (-1)^popcount(i & j) ) for both columns.
// Sign vector s = (+,+,+,-,+,-,-,-,-,-,-,+,-,+,-,-). The butterfly runs in packed fp32.
// The signs cost no instruction: a butterfly on (s_a * A, s_b * B) equals s_a * (A +- B) with
// add and subtract exchanged when s_a != s_b, so each block of 2h values carries the sign of
// its first element as a common factor, and the whole vector ends with the factor s_0 = +1.
// Negation commutes with rounding, so every value equals the one computed with the signs
// applied up front, except that a zero may come out with the other sign; zeros of either
// sign quantize to code 0 and do not move an abs-max.
__device__ __forceinline__ void rht16_x2(uint32_t (&w)[16]) {
  constexpr uint32_t kNegRows = (1u << 3) | (1u << 5) | (1u << 6) | (1u << 7) | (1u << 8) | (1u << 9) | (1u << 10) |
                                (1u << 12) | (1u << 14) | (1u << 15);
  f32x2_t v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = bf16x2_to_f32x2(w[i]);
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        const int first = i & ~(h - 1);   // first element of this value's block of h
        const bool exchange = ((kNegRows >> first) & 1u) != ((kNegRows >> (first + h)) & 1u);
        const f32x2_t a = v[i], b = v[i + h];
        v[i] = exchange ? sub2(a, b) : add2(a, b);
        v[i + h] = exchange ? add2(a, b) : sub2(a, b);
      }
    }
  }
  const f32x2_t quarter = pack2(0.25f, 0.25f);
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = f32x2_to_bf16x2(mul2(v[i], quarter));
}

// ---- NVFP4 scale arithmetic (same operation order as the PyTorch emulation) ----
struct Nvfp4Global {
  float ges;  // global encode scale = min(448*6/amax, FLT_MAX), 0 -> 1
  float gds;  // 1 / ges
};
__device__ __forceinline__ Nvfp4Global nvfp4_global(float amax) {
  Nvfp4Global g;
  g.ges = fminf(__fdiv_rn(2688.0f, amax), FLT_MAX);
  if (g.ges == 0.0f) g.ges = 1.0f;
  g.gds = __fdiv_rn(1.0f, g.ges);
  return g;
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// Block abs-max -> E4M3 scale byte and the fp32 factor applied to the elements (reference
// form: every step spelled out; used to fill the lookup table below).
__device__ __forceinline__ void nvfp4_block_scale(float vmax, const Nvfp4Global& g, uint8_t& sbyte, float& encode) {
  float d = __fdiv_rn(vmax, 6.0f);
  d = fminf(__fmul_rn(d, g.ges), FLT_MAX);
  d = fminf(d, 448.0f);
  sbyte = __nv_cvt_float_to_fp8(d, __NV_SATFINITE, __NV_E4M3);
  float sdec = e4m3_to_float(sbyte);
  encode = fminf(__fdiv_rn(1.0f, __fmul_rn(sdec, g.gds)), FLT_MAX);
}
// The element factor depends only on the scale byte (127 non-negative E4M3 values) and the
// per-tensor scale: table[b] = min(1 / (e4m3(b) * gds), FLT_MAX).
__device__ __forceinline__ float nvfp4_encode_for_byte(uint32_t b, const Nvfp4Global& g) {
  return fminf(__fdiv_rn(1.0f, __fmul_rn(e4m3_to_float(static_cast<uint8_t>(b)), g.gds)), FLT_MAX);
}
// v / 6 correctly rounded for any non-negative bf16-representable v: one multiply by
// RN(1/6) plus one FMA correction step (checked exhaustively against IEEE division for all
// bf16 inputs); infinity passes through.
__device__ __forceinline__ float div6_bf16(float v) {
  const float c = 0x1.555556p-3f;
  float q = __fmul_rn(v, c);
  const float r = __fmaf_rn(-6.0f, q, v);
  q = __fmaf_rn(r, c, q);
  return (v == INFINITY) ? v : q;
}
// Fast form of nvfp4_block_scale: same scale byte, element factor from the table in shared memory.
__device__ __forceinline__ void nvfp4_block_scale_lut(float vmax, float ges, const float* __restrict__ lut,
                                                      uint32_t& sbyte, float& encode) {
  const float d = fminf(__fmul_rn(div6_bf16(vmax), ges), 448.0f);
  sbyte = __nv_cvt_float_to_fp8(d, __NV_SATFINITE, __NV_E4M3);
  encode = lut[sbyte & 0x7Fu];
}
// x * enc with the emulation's treatment of negative zero: the emulation rounds the product to
// fp32 and maps -0.0 to code 0. `fused` (per tensor, see nvfp4_can_fuse_scaling) selects one
// FMA x*enc + (+0.0), which turns an exact -0 product (x = -0) into +0 and equals the rounded
// product otherwise unless a non-zero product underflows to -0; tensors where that could
// happen take the two-step form (round the product, then add +0.0).
__device__ __forceinline__ f32x2_t scale2(f32x2_t x, f32x2_t enc2, bool fused) {
  const f32x2_t z2 = pack2(0.0f, 0.0f);
  return fused ? fma2(x, enc2, z2) : add2(mul2(x, enc2), z2);
}
// Every element factor is at least 6 / amax and every non-zero bf16 magnitude at least 2^-133,
// so no non-zero product can underflow to zero in fp32 while 6 / amax * 2^-133 >= 2^-149.
__device__ __forceinline__ bool nvfp4_can_fuse_scaling(float amax) { return amax <= 6.0f * 65536.0f; }
// Two scaled fp32 pairs -> one byte each holding two E2M1 nibbles.
__device__ __forceinline__ uint32_t e2m1_byte(float lo, float hi) {
  uint32_t out;
  asm("{\n\t.reg .b8 b0;\n\tcvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\tcvt.u32.u8 %0, b0;\n\t}"
      : "=r"(out) : "f"(lo), "f"(hi));
  return out;
}
// Eight E2M1 codes from four packed bf16x2 words (elements in memory order), one factor for all.
__device__ __forceinline__ uint32_t e2m1x8_from_words(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, float enc,
                                                  bool fused) {
  const f32x2_t e2 = pack2(enc, enc);
  float a0, a1, b0, b1, c0, c1, d0, d1;
  unpack2(scale2(bf16x2_to_f32x2(w0), e2, fused), a0, a1);
  unpack2(scale2(bf16x2_to_f32x2(w1), e2, fused), b0, b1);
  unpack2(scale2(bf16x2_to_f32x2(w2), e2, fused), c0, c1);
  unpack2(scale2(bf16x2_to_f32x2(w3), e2, fused), d0, d1);
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1), "f"(d0), "f"(d1));
  return out;
}
// Column form: 8 consecutive rows of two adjacent columns (packed per row), factors (enc_lo,
// enc_hi) per column -> 8 codes of the low column and 8 codes of the high column.
__device__ __forceinline__ void e2m1x8_two_columns(const uint32_t* w, f32x2_t enc2, bool fused, uint32_t& codes_lo,
                                                   uint32_t& codes_hi) {
  float lo[8], hi[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) unpack2(scale2(bf16x2_to_f32x2(w[j]), enc2, fused), lo[j], hi[j]);
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(codes_lo)
      : "f"(lo[0]), "f"(lo[1]), "f"(lo[2]), "f"(lo[3]), "f"(lo[4]), "f"(lo[5]), "f"(lo[6]), "f"(lo[7]));
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(codes_hi)
      : "f"(hi[0]), "f"(hi[1]), "f"(hi[2]), "f"(hi[3]), "f"(hi[4]), "f"(hi[5]), "f"(hi[6]), "f"(hi[7]));
}

// ---- stochastic rounding (gradient codes) ----
// 32 random bits for one group of four elements: a counter-based hash of (seed, group index), so
// that a launch is reproducible from its seed and independent of the grid.
__device__ __forceinline__ uint32_t sr_bits(uint64_t seed, uint64_t group) {
  uint64_t z = (group + seed) * 0x9E3779B97F4A7C15ull;
  z ^= z >> 32;
  uint32_t x = static_cast<uint32_t>(z) ^ static_cast<uint32_t>(seed >> 32);
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}
// Four scaled fp32 values -> four E2M1 nibbles (x0 in the lowest), each rounded to one of its
// two neighbouring codes with probability proportional to its distance from the other
// (cvt.rs: stochastic rounding with the given random bits).
__device__ __forceinline__ uint32_t e2m1x4_sr(float x0, float x1, float x2, float x3, uint32_t rbits) {
  uint16_t out;
  asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(out) : "f"(x3), "f"(x2), "f"(x1), "f"(x0), "r"(rbits));
  return out;
}
// Stochastic-rounding forms of e2m1x8_from_words / e2m1x8_two_columns.
__device__ __forceinline__ uint32_t e2m1x8_from_words_sr(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, float enc,
                                                         bool fused, uint32_t rb0, uint32_t rb1) {
  const f32x2_t e2 = pack2(enc, enc);
  float a0, a1, b0, b1, c0, c1, d0, d1;
  unpack2(scale2(bf16x2_to_f32x2(w0), e2, fused), a0, a1);
  unpack2(scale2(bf16x2_to_f32x2(w1), e2, fused), b0, b1);
  unpack2(scale2(bf16x2_to_f32x2(w2), e2, fused), c0, c1);
  unpack2(scale2(bf16x2_to_f32x2(w3), e2, fused), d0, d1);
  return e2m1x4_sr(a0, a1, b0, b1, rb0) | (e2m1x4_sr(c0, c1, d0, d1, rb1) << 16);
}
__device__ __forceinline__ void e2m1x8_two_columns_sr(const uint32_t* w, f32x2_t enc2, bool fused, uint32_t& codes_lo,
                                                      uint32_t& codes_hi, uint32_t rb0, uint32_t rb1) {
  float lo[8], hi[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) unpack2(scale2(bf16x2_to_f32x2(w[j]), enc2, fused), lo[j], hi[j]);
  codes_lo = e2m1x4_sr(lo[0], lo[1], lo[2], lo[3], rb0) | (e2m1x4_sr(lo[4], lo[5], lo[6], lo[7], rb1) << 16);
  // the neighbouring column gets its own bits (a rotation keeps them decorrelated enough for rounding)
  const uint32_t r2 = __funnelshift_l(rb0, rb1, 13), r3 = __funnelshift_l(rb1, rb0, 7);
  codes_hi = e2m1x4_sr(hi[0], hi[1], hi[2], hi[3], r2) | (e2m1x4_sr(hi[4], hi[5], hi[6], hi[7], r3) << 16);
}

// ---- MXFP8 scale arithmetic ----
// ceil(log2(amax/448)) clamped to [-127, 127], from the bits of the fp32 quotient.
__device__ __forceinline__ int e8m0_exponent(float amax) {
  float v = __fdiv_rn(amax, 448.0f);
  uint32_t b = __float_as_uint(v);
  int E = static_cast<int>(b >> 23) & 0xFF;
  uint32_t M = b & 0x7FFFFFu;
  int e;
  if (E == 0) e = (M > 0x400000u) ? -126 : -127;  // subnormal quotient: only (2^-127, 2^-126) rounds up
  else e = E - 127 + (M != 0 ? 1 : 0);
  return max(-127, min(127, e));
}
// 2^-e as fp32 (e in [-127, 127]; 2^-127 is subnormal).
__device__ __forceinline__ float exp2_neg(int e) {
  return (e == 127) ? __uint_as_float(0x00200000u) : __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
}
// Four scaled fp32 values -> four E4M3 bytes (round to nearest even, saturating at 448).
__device__ __forceinline__ uint32_t e4m3x4_from_words(uint32_t w0, uint32_t w1, f32x2_t enc2) {
  float t0, t1, t2, t3;
  unpack2(mul2(bf16x2_to_f32x2(w0), enc2), t0, t1);
  unpack2(mul2(bf16x2_to_f32x2(w1), enc2), t2, t3);
  uint32_t out;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(out)
      : "f"(t0), "f"(t1), "f"(t2), "f"(t3));
  return out;
}
// Column form: 4 consecutive rows of two adjacent columns -> 4 E4M3 bytes per column.
__device__ __forceinline__ void e4m3x4_two_columns(const uint32_t* w, f32x2_t enc2, uint32_t& out_lo, uint32_t& out_hi) {
  float lo[4], hi[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) unpack2(mul2(bf16x2_to_f32x2(w[j]), enc2), lo[j], hi[j]);
  asm("{\n\t.reg .b16 a, b;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 a, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 b, %4, %3;\n\t"
      "mov.b32 %0, {a, b};\n\t}"
      : "=r"(out_lo) : "f"(lo[0]), "f"(lo[1]), "f"(lo[2]), "f"(lo[3]));
  asm("{\n\t.reg .b16 a, b;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 a, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 b, %4, %3;\n\t"
      "mov.b32 %0, {a, b};\n\t}"
      : "=r"(out_hi) : "f"(hi[0]), "f"(hi[1]), "f"(hi[2]), "f"(hi[3]));
}
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d, float encode) {
  uint32_t out;
  float t0 = __fmul_rn(a, encode), t1 = __fmul_rn(b, encode), t2 = __fmul_rn(c, encode), t3 = __fmul_rn(d, encode);
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(out)
      : "f"(t0), "f"(t1), "f"(t2), "f"(t3));
  return out;
}

// Position of scale (row r, block kb) inside its 512-byte chunk of the GEMM-ready layout.
__device__ __forceinline__ int sf_chunk_offset(int r, int kb) { return (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3); }

// Copies n (<= 16) bytes from shared to global, using one 16-byte store when possible.
__device__ __forceinline__ void store_bytes(uint8_t* dst, const uint8_t* src, int n) {
  if (n <= 0) return;
  if (n == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  } else if (n == 8 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
  } else {
    for (int i = 0; i < n; ++i) dst[i] = src[i];
  }
}

}  // namespace mt
