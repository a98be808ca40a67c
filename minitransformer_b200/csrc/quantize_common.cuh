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

// max(|a|, |b|) on two packed bf16 lanes.
__device__ __forceinline__ uint32_t absmax2(uint32_t a, uint32_t b) {
  __nv_bfloat162 x = __habs2(*reinterpret_cast<__nv_bfloat162*>(&a));
  __nv_bfloat162 y = __habs2(*reinterpret_cast<__nv_bfloat162*>(&b));
  __nv_bfloat162 m = __hmax2(x, y);
  return *reinterpret_cast<uint32_t*>(&m);
}
// Larger of the two |bf16| halves of a word that already holds absolute values, as fp32.
__device__ __forceinline__ float absmax2_to_float(uint32_t m) { return fmaxf(bf16_lo(m), bf16_hi(m)); }

__device__ __forceinline__ float round_to_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// 16-point randomized Hadamard transform of one group, in place:
// y_j = (1/4) * sum_i s_i * x_i * (-1)^popcount(i & j), each y_j rounded to bf16.
// Sign vector s = (+,+,+,-,+,-,-,-,-,-,-,+,-,+,-,-).
__device__ __forceinline__ void rht16(float (&v)[16]) {
  v[3] = -v[3];   v[5] = -v[5];   v[6] = -v[6];   v[7] = -v[7];
  v[8] = -v[8];   v[9] = -v[9];   v[10] = -v[10]; v[12] = -v[12];
  v[14] = -v[14]; v[15] = -v[15];
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        float a = v[i], b = v[i + h];
        v[i] = __fadd_rn(a, b);
        v[i + h] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = round_to_bf16(__fmul_rn(v[i], 0.25f));
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
// Block abs-max -> E4M3 scale byte and the fp32 factor applied to the elements.
__device__ __forceinline__ void nvfp4_block_scale(float vmax, const Nvfp4Global& g, uint8_t& sbyte, float& encode) {
  float d = __fdiv_rn(vmax, 6.0f);
  d = fminf(__fmul_rn(d, g.ges), FLT_MAX);
  d = fminf(d, 448.0f);
  sbyte = __nv_cvt_float_to_fp8(d, __NV_SATFINITE, __NV_E4M3);
  float sdec = e4m3_to_float(sbyte);
  encode = fminf(__fdiv_rn(1.0f, __fmul_rn(sdec, g.gds)), FLT_MAX);
}
// Eight scaled fp32 values -> eight E2M1 nibbles, element 0 in the lowest nibble.
// +0.0 is added first so that a negative zero encodes as code 0, like the emulation.
__device__ __forceinline__ uint32_t e2m1x8(const float* v, float encode) {
  float t[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) t[i] = __fadd_rn(__fmul_rn(v[i], encode), 0.0f);
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(t[0]), "f"(t[1]), "f"(t[2]), "f"(t[3]), "f"(t[4]), "f"(t[5]), "f"(t[6]), "f"(t[7]));
  return out;
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
