// CUDA-core block-scaled GEMM used only to check the tensor-core kernels on the device at
// sizes where a CPU check would take minutes. It follows the emulation's structure:
// for every K block, an fp32 dot product of the decoded elements, multiplied by the two
// block scales, accumulated in fp32; NVFP4 results are then multiplied by
// alpha = amax_a * amax_b / (6*6*448*448).
#include <cuda_fp8.h>

#include "mt_common.cuh"
#include "../../include/mt_b200_test.h"

namespace mt {

constexpr int CK_TILE = 64;    // output tile edge
constexpr int CK_KSLAB = 64;   // K elements staged per step

__device__ __forceinline__ float e2m1_value(uint32_t nib) {
  // 0, 0.5, 1, 1.5, 2, 3, 4, 6 with sign bit 3
  const uint32_t mag = nib & 7u;
  float v = (mag < 2) ? 0.5f * mag : (mag < 4 ? 0.5f * mag : (mag == 4 ? 2.0f : (mag == 5 ? 3.0f : (mag == 6 ? 4.0f : 6.0f))));
  return (nib & 8u) ? -v : v;
}
__device__ __forceinline__ float e4m3_value(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ float e8m0_value(uint8_t b) {
  return (b == 0) ? __uint_as_float(0x00400000u) : __uint_as_float(static_cast<uint32_t>(b) << 23);
}

// 256 threads, each computes a 4x4 patch of a 64x64 output tile.
template <bool kFp4>
__global__ void __launch_bounds__(256) gemm_check_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ sa,
                                                         int64_t sa_stride, const uint8_t* __restrict__ b,
                                                         const uint8_t* __restrict__ sb, int64_t sb_stride,
                                                         const float* amax_a, const float* amax_b, int64_t M, int64_t N,
                                                         int64_t K, void* d, int d_dtype, int64_t ldd, int accumulate) {
  constexpr int BLK = kFp4 ? 16 : 32;
  __shared__ float As[CK_KSLAB][CK_TILE + 1];
  __shared__ float Bs[CK_KSLAB][CK_TILE + 1];
  __shared__ float SAs[CK_KSLAB / BLK][CK_TILE];
  __shared__ float SBs[CK_KSLAB / BLK][CK_TILE];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * CK_TILE, n0 = (int64_t)blockIdx.x * CK_TILE;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += CK_KSLAB) {
    for (int i = threadIdx.x; i < CK_TILE * CK_KSLAB; i += 256) {
      const int r = i / CK_KSLAB, k = i % CK_KSLAB;
      const int64_t gk = k0 + k;
      float va = 0.f, vb = 0.f;
      if (gk < K) {
        if (m0 + r < M) {
          if (kFp4) { uint8_t byte = a[(m0 + r) * (K / 2) + gk / 2]; va = e2m1_value((gk & 1) ? (byte >> 4) : (byte & 15)); }
          else va = e4m3_value(a[(m0 + r) * K + gk]);
        }
        if (n0 + r < N) {
          if (kFp4) { uint8_t byte = b[(n0 + r) * (K / 2) + gk / 2]; vb = e2m1_value((gk & 1) ? (byte >> 4) : (byte & 15)); }
          else vb = e4m3_value(b[(n0 + r) * K + gk]);
        }
      }
      As[k][r] = va;
      Bs[k][r] = vb;
    }
    for (int i = threadIdx.x; i < CK_TILE * (CK_KSLAB / BLK); i += 256) {
      const int r = i / (CK_KSLAB / BLK), kb = i % (CK_KSLAB / BLK);
      const int64_t gkb = k0 / BLK + kb;
      float fa = 0.f, fb = 0.f;
      if (gkb * BLK < K) {
        if (m0 + r < M) fa = kFp4 ? e4m3_value(sa[(m0 + r) * sa_stride + gkb]) : e8m0_value(sa[(m0 + r) * sa_stride + gkb]);
        if (n0 + r < N) fb = kFp4 ? e4m3_value(sb[(n0 + r) * sb_stride + gkb]) : e8m0_value(sb[(n0 + r) * sb_stride + gkb]);
      }
      SAs[kb][r] = fa;
      SBs[kb][r] = fb;
    }
    __syncthreads();
    for (int kb = 0; kb < CK_KSLAB / BLK; ++kb) {
      float part[4][4] = {};
      for (int k = 0; k < BLK; ++k) {
        float av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { av[i] = As[kb * BLK + k][ty * 4 + i]; bv[i] = Bs[kb * BLK + k][tx * 4 + i]; }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) part[i][j] = fmaf(av[i], bv[j], part[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(__fmul_rn(SAs[kb][ty * 4 + i], SBs[kb][tx * 4 + j]), part[i][j]));
    }
    __syncthreads();
  }
  float alpha = 1.0f;
  if (kFp4) alpha = __fdiv_rn(__fmul_rn(*amax_a, *amax_b), 6.0f * 6.0f * 448.0f * 448.0f);
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const int64_t r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
      if (r >= M || c >= N) continue;
      float v = (kFp4 && K > 0) ? __fmul_rn(alpha, acc[i][j]) : acc[i][j];
      if (d_dtype == MT_F32) {
        float* p = static_cast<float*>(d) + r * ldd + c;
        *p = accumulate ? *p + v : v;
      } else {
        __nv_bfloat16* p = static_cast<__nv_bfloat16*>(d) + r * ldd + c;
        *p = __float2bfloat16_rn(accumulate ? __bfloat162float(*p) + v : v);
      }
    }
}

static int check_common(bool fp4, const uint8_t* a, const uint8_t* sa, int64_t sa_stride, const float* amax_a,
                        const uint8_t* b, const uint8_t* sb, int64_t sb_stride, const float* amax_b, int64_t M,
                        int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd, int accumulate, cudaStream_t st) {
  MT_REQUIRE(a && sa && b && sb && d, "gemm check: null pointer");
  MT_REQUIRE(M >= 0 && N >= 0 && K >= 0 && K % (fp4 ? 16 : 32) == 0, "gemm check: bad shape");
  MT_REQUIRE(!fp4 || (amax_a && amax_b), "gemm check: abs-max pointers required");
  MT_REQUIRE(d_dtype == MT_BF16 || d_dtype == MT_F32, "gemm check: bad output dtype");
  if (M == 0 || N == 0) return MT_OK;
  dim3 grid((unsigned)((N + CK_TILE - 1) / CK_TILE), (unsigned)((M + CK_TILE - 1) / CK_TILE));
  if (fp4)
    gemm_check_kernel<true><<<grid, 256, 0, st>>>(a, sa, sa_stride, b, sb, sb_stride, amax_a, amax_b, M, N, K, d, d_dtype, ldd, accumulate);
  else
    gemm_check_kernel<false><<<grid, 256, 0, st>>>(a, sa, sa_stride, b, sb, sb_stride, amax_a, amax_b, M, N, K, d, d_dtype, ldd, accumulate);
  MT_CUDA(cudaGetLastError());
  return MT_OK;
}

}  // namespace mt

extern "C" {

int mt_gemm_nvfp4_check(const uint8_t* a, const uint8_t* sa, int64_t sa_stride, const float* amax_a, const uint8_t* b,
                        const uint8_t* sb, int64_t sb_stride, const float* amax_b, int64_t M, int64_t N, int64_t K,
                        void* d, int d_dtype, int64_t ldd, int accumulate, mt_stream_t stream) {
  return mt::check_common(true, a, sa, sa_stride, amax_a, b, sb, sb_stride, amax_b, M, N, K, d, d_dtype, ldd,
                          accumulate, static_cast<cudaStream_t>(stream));
}

int mt_gemm_mxfp8_check(const uint8_t* a, const uint8_t* sa, int64_t sa_stride, const uint8_t* b, const uint8_t* sb,
                        int64_t sb_stride, int64_t M, int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd,
                        int accumulate, mt_stream_t stream) {
  return mt::check_common(false, a, sa, sa_stride, nullptr, b, sb, sb_stride, nullptr, M, N, K, d, d_dtype, ldd,
                          accumulate, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
