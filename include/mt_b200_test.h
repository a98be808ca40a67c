/*
 * Test-only entry points of libmt_b200.so: device-side checkers that the parity tests call.
 * They are not product paths and a caller of the library never needs them.
 */
#ifndef MT_B200_TEST_H_
#define MT_B200_TEST_H_

#include "mt_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The contracts of mt_gemm_nvfp4 / mt_gemm_mxfp8, computed by a plain CUDA-core kernel that
 * follows the emulation's summation structure (per-block fp32 dot, scaled, fp32 accumulate;
 * miniTransformer/ops/nvfp4_quantize_op_ref.py:534-551). Scales are given in the row-major
 * layout. It exists so the tensor-core kernels can be checked on the device at sizes where a
 * CPU check would take minutes. */
int mt_gemm_nvfp4_check(const uint8_t* a, const uint8_t* sa, int64_t sa_stride, const float* amax_a,
                        const uint8_t* b, const uint8_t* sb, int64_t sb_stride, const float* amax_b,
                        int64_t M, int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd,
                        int accumulate, mt_stream_t stream);
int mt_gemm_mxfp8_check(const uint8_t* a, const uint8_t* sa, int64_t sa_stride,
                        const uint8_t* b, const uint8_t* sb, int64_t sb_stride,
                        int64_t M, int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd,
                        int accumulate, mt_stream_t stream);

/* Launches one CTA whose single thread waits, with the library's bounded mbarrier wait and the
 * given limit, on a barrier that nothing ever signals. The wait gives up by construction: the
 * kernel raises the "TMA wait" bit in the device status word (mt_read_device_status) and
 * returns. Checks the give-up path of every kernel's waits without any kernel having to hang. */
int mt_test_bounded_wait(int64_t timeout_ns, mt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MT_B200_TEST_H_ */
