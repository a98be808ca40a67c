/*
 * C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * Every entry point takes raw device pointers, 64-bit sizes and a CUDA stream, launches
 * asynchronously on that stream, allocates nothing, never synchronises the device
 * (mt_read_device_status excepted) and returns 0 on success or a negative mt_status on failure (mt_last_error_string() then
 * describes it for the calling thread). Pointers must be 16-byte aligned unless stated.
 *
 * Reference interfaces these replace are cited per function as file:line inside
 * fy1214/miniTransformer.
 */
#ifndef MT_B200_H_
#define MT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* mt_stream_t; /* cudaStream_t */

enum mt_status {
  MT_OK = 0,
  MT_ERR_INVALID_ARG = -1,   /* null pointer, bad shape, bad alignment, bad flag */
  MT_ERR_UNSUPPORTED = -2,   /* valid request this build does not implement */
  MT_ERR_CUDA = -3,          /* a CUDA runtime / driver call failed */
  MT_ERR_DEVICE_TIMEOUT = -4 /* a bounded device-side wait expired (see mt_read_device_status) */
};

/* Output element types of the GEMM entry points. */
enum mt_dtype { MT_BF16 = 0, MT_F32 = 1 };

/* Flags of mt_quantize_nvfp4 / mt_amax_bf16. */
enum mt_quantize_flags {
  MT_Q_2D = 1,       /* one scale per 16x16 block, shared by both copies */
  MT_Q_RHT = 2,      /* 16-point randomized Hadamard transform on the transposed copy */
  MT_Q_ROWPAD16 = 4, /* scale tensors have their row count padded to a multiple of 16 */
  MT_Q_AMAX_ZEROED = 8 /* mt_amax_bf16: the caller has set amax_row / amax_col to 0 (ordered before this call on
                        * the stream); no memset is issued, so the call is one kernel launch */
};

int mt_version(void);
const char* mt_last_error_string(void);

/* Launch overlap (process-wide switch, on by default). When on, the quantize, pair-GEMM and peer
 * exchange / gather / reduce kernels are launched programmatically dependent on the kernel
 * before them in the stream: they may become resident on the SMs which that kernel's last
 * blocks leave, wait there for it to complete, and start without a launch gap; results and the
 * order of completion along a stream are the same either way. A caller that runs other kernels
 * on side streams beside these and has sized their grids to share the SMs should switch it off:
 * blocks that are resident early hold SM resources which the side stream's kernels then find
 * taken. Returns the previous setting. */
int mt_set_launch_overlap(int enabled);

/* Number of bytes of the GEMM-ready ("swizzled") scale-factor tensor for an operand with
 * `rows` rows and `k_blocks` scale factors per row: ceil(rows/128) x ceil(k_blocks/4)
 * chunks of 512 bytes, chunk (rb, kc) holding rows rb*128.. and blocks kc*4.., byte
 * (r%32)*16 + (r/32)*4 + (kb%4); the K-chunk count is rounded up to a multiple of 4.
 * This is the layout the reference anticipates for its cuBLASLt call
 * (miniTransformer/csrc/util/common.h:29-33, csrc/ops/fp4/gemm/gemm_cublas.cu:275-277). */
int64_t mt_swizzled_scale_bytes(int64_t rows, int64_t k_blocks);

/* Per-tensor abs-max of a bf16 matrix x[rows, cols] (row stride = cols).
 * amax_row <- max|x|. If amax_col is non-null: with MT_Q_RHT it receives the abs-max of the
 * Hadamard-transformed transpose (groups of 16 consecutive rows of one column, fixed sign
 * vector, scale 1/4, rounded to bf16), otherwise a copy of amax_row. Both are device fp32
 * scalars and are overwritten (with MT_Q_AMAX_ZEROED they must hold 0 on entry).
 * rows % 16 == 0 is required with MT_Q_RHT; cols % 8 == 0 always.
 * Replaces the two torch.max(torch.abs(.)) reductions of
 * miniTransformer/ops/nvfp4_quantize_op_ref.py:357-369. */
int mt_amax_bf16(const void* x, int64_t rows, int64_t cols, int flags,
                 float* amax_row, float* amax_col, mt_stream_t stream);

/* mt_amax_bf16 that also returns the column sums of x in col_sum[cols] (fp32, overwritten;
 * rows % 16 == 0): the bias gradient b_grad = sum over tokens of dy, taken from the pass over dy
 * that its quantization needs anyway instead of a pass of its own
 * (miniTransformer/module/linear.py:352). Summation order varies with scheduling (fp32 atomics). */
int mt_amax_colsum_bf16(const void* x, int64_t rows, int64_t cols, int flags,
                        float* amax_row, float* amax_col, float* col_sum, mt_stream_t stream);

/* NVFP4 cast (+ transpose): E2M1 codes packed two per byte (even column in the low
 * nibble), one E4M3 scale per 1x16 block (or per 16x16 block with MT_Q_2D), using the
 * per-tensor abs-max values already on the device (mt_amax_bf16, optionally max-reduced
 * across ranks by the caller).
 *   x        bf16 [rows, cols], cols % 16 == 0 (rows % 2 == 0 when q_t is requested)
 *   q        u8 [rows, cols/2]
 *   s        u8 (E4M3) [rows_s, cols/16], row stride s_stride bytes; rows_s = rows, or rows
 *            rounded up to 16 with MT_Q_ROWPAD16 / MT_Q_2D (padded rows are written as 0)
 *   s_swz    optional GEMM-ready copy of s (mt_swizzled_scale_bytes(rows, cols/16) bytes)
 *   q_t      optional u8 [cols, rows/2]: codes of x^T (after the transform with MT_Q_RHT)
 *   s_t      u8 [cols_s, ceil(rows/16)], row stride s_t_stride; required iff q_t
 *   s_t_swz  optional GEMM-ready copy of s_t
 * Replaces fp4_gemm.quantize_transpose_nvfp4 (miniTransformer/csrc/ops.h:7-15,
 * csrc/ops/fp4/quantization/quantize_transpose_nvfp4.cu:1136-1228) with the arithmetic of
 * Nvfp4TiledQuantizeRefOp._quantize (miniTransformer/ops/nvfp4_quantize_op_ref.py:258-417). */
int mt_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int flags,
                      const float* amax_row, const float* amax_col,
                      uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz,
                      uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                      mt_stream_t stream);

/* The same cast with stochastic rounding of the codes: every element becomes one of its two
 * neighbouring E2M1 values, the nearer one more often, so that the expectation of the dequantized
 * value equals the input (for gradients; scales and abs-max handling are unchanged, 1x16 blocks
 * only). `seed` makes a launch reproducible; use a fresh one per call. The reference carries this
 * path compiled out (miniTransformer/csrc/util/ptx.cuh:222-260, 319-352;
 * csrc/ops/fp4/quantization/quantize_transpose_nvfp4.cu:1145 use_stochastic_rounding = false). */
int mt_quantize_nvfp4_sr(const void* x, int64_t rows, int64_t cols, int flags,
                         const float* amax_row, const float* amax_col,
                         uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz,
                         uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                         uint64_t seed, mt_stream_t stream);

/* MXFP8 cast (+ transpose): E4M3 elements, one E8M0 scale byte (exponent + 127) per 1x32
 * block. Scale rule: 2^ceil(log2(amax/448)) clamped to 2^+-127 (cast_to_e8,
 * miniTransformer/ops/nvfp4_quantize_op_ref.py:12-21).
 *   x bf16 [rows, cols], cols % 32 == 0; q u8 [rows, cols]; s u8 [rows, cols/32];
 *   q_t optional u8 [cols, rows] (x^T, blocks along rows; a ragged row count is padded
 *   with zeros to 32 for the scale); s_t u8 [cols, ceil(rows/32)]; *_swz as above. */
int mt_quantize_mxfp8(const void* x, int64_t rows, int64_t cols,
                      uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz,
                      uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                      mt_stream_t stream);

/* Row-major scale bytes s[rows, k_blocks] (row stride s_stride) -> GEMM-ready layout.
 * Rows / blocks beyond the source extent are written as 0. */
int mt_swizzle_scales(const uint8_t* s, int64_t rows, int64_t k_blocks, int64_t s_stride,
                      uint8_t* s_swz, mt_stream_t stream);

/* Optional per-call settings of the GEMM entry points (a null pointer = all defaults).
 *   sm_margin  SMs this launch leaves idle. The GEMM kernels are persistent, one CTA per SM; a
 *              collective launched beside such a grid gets no SM until GEMM CTAs retire. A
 *              caller that overlaps a reduce-scatter with the wgrad GEMM gives that GEMM a
 *              margin (the role of the sm_margin of the userbuffer overlap flags the
 *              reference's Linear carries, miniTransformer/module/linear.py:649-671).
 *   d_amax     optional device fp32 scalar: the kernel raises it (atomic max) to the largest
 *              |value| it stores in d, after rounding to d's type. Zero it before the launch.
 *              The next layer's NVFP4 quantize can take it as its per-tensor abs-max instead
 *              of re-reading d (the QuantizeInputMetaBase.amax hook,
 *              miniTransformer/ops/quantization.py:90-94). Not available with accumulate.
 *   n_dest, my_rank, dest, dest_rows   (n_dest > 1) scatter of the output rows over the ranks of a
 *              tensor-parallel group, the first half of a reduce-scatter done by the GEMM
 *              itself: output rows [r * dest_rows, (r + 1) * dest_rows) are not written to d but
 *              stored over NVLink into rank r's staging buffer dest[r] (a mapped peer address,
 *              see mt_ipc_import; dest[my_rank] is local), a bf16 matrix
 *              [n_dest * dest_rows, N] with row pitch N, at rows my_rank * dest_rows + (row
 *              inside the slice). After a peer barrier every rank sums the n_dest slices of its
 *              own staging buffer with mt_peer_reduce_bf16. Needs bf16 output without
 *              accumulate or bias, M == n_dest * dest_rows, dest_rows % 256 == 0, N % 8 == 0;
 *              d may be null. Replaces the reduce-scatter of bf16 partial sums after a
 *              row-parallel GEMM (miniTransformer/module/linear.py:322-328, 404-410) with
 *              stores that travel while later tiles are still being computed. */
#define MT_MAX_PEERS 8
typedef struct mt_gemm_opts {
  int sm_margin;
  float* d_amax;
  int n_dest;
  int my_rank;
  void* dest[MT_MAX_PEERS];
  int64_t dest_rows;
} mt_gemm_opts;

/* Block-scaled GEMM  D[M,N] = alpha * (A . B^T) (+ bias[N]) (+ D when accumulate), both
 * operands K-major, fp32 accumulation in tensor memory (tcgen05.mma, block_scale).
 *   NVFP4: a u8 [M, K/2], b u8 [N, K/2], K % 32 == 0, scales E4M3 per 16, swizzled layout;
 *          alpha = amax_a[0] * amax_b[0] / (6*6*448*448) read on the device.
 *   MXFP8: a u8 [M, K],   b u8 [N, K],   K % 16 == 0, scales E8M0 per 32; alpha = 1.
 *   d: bf16 or fp32 [M, N] with row stride ldd elements; bias: optional fp32/bf16 per
 *   bias_dtype; accumulate != 0 adds the previous contents of d (fp32 add, then rounding).
 * Replaces QuantizeOpBase.qgemm (miniTransformer/ops/quantization.py:121-160), i.e. the
 * emulation Nvfp4TiledQuantizeRefOp._ref_qgemm (ops/nvfp4_quantize_op_ref.py:449-560) and
 * the cuBLASLt call the reference intended (csrc/ops/fp4/gemm/gemm_cublas.cu:75-255). */
int mt_gemm_nvfp4(const uint8_t* a, const uint8_t* sa_swz, const float* amax_a,
                  const uint8_t* b, const uint8_t* sb_swz, const float* amax_b,
                  int64_t M, int64_t N, int64_t K,
                  void* d, int d_dtype, int64_t ldd,
                  const void* bias, int bias_dtype, int accumulate,
                  const mt_gemm_opts* opts, mt_stream_t stream);

int mt_gemm_mxfp8(const uint8_t* a, const uint8_t* sa_swz,
                  const uint8_t* b, const uint8_t* sb_swz,
                  int64_t M, int64_t N, int64_t K,
                  void* d, int d_dtype, int64_t ldd,
                  const void* bias, int bias_dtype, int accumulate,
                  const mt_gemm_opts* opts, mt_stream_t stream);

/* The same GEMMs for operands whose contraction dimension is split into slabs stored one
 * after another: a is a_slabs matrices [M, K / a_slabs] (bytes as above) back to back, and
 * sa_swz is the a_slabs GEMM-layout scale buffers of those matrices back to back (each
 * mt_swizzled_scale_bytes(M, K / a_slabs / block) bytes); likewise b with b_slabs. This is
 * the layout an all-gather of per-rank transposed shards produces (rank r holds the tokens
 * [r T/n, (r+1) T/n) of x^T), so the wgrad GEMM of a sequence-parallel layer reads the
 * gathered buffer as it arrives, with no re-interleaving copy. Slab count 1 = plain layout.
 * Needs M > 128, N > 128 and K / slabs a multiple of 256 (NVFP4) or 128 (MXFP8) elements.
 * No counterpart in the reference, whose gather helpers move high-precision tensors
 * (miniTransformer/distributed/distributed.py:68-121). */
int mt_gemm_nvfp4_kslab(const uint8_t* a, const uint8_t* sa_swz, const float* amax_a, int64_t a_slabs,
                        const uint8_t* b, const uint8_t* sb_swz, const float* amax_b, int64_t b_slabs,
                        int64_t M, int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd,
                        const void* bias, int bias_dtype, int accumulate,
                        const mt_gemm_opts* opts, mt_stream_t stream);

int mt_gemm_mxfp8_kslab(const uint8_t* a, const uint8_t* sa_swz, int64_t a_slabs,
                        const uint8_t* b, const uint8_t* sb_swz, int64_t b_slabs,
                        int64_t M, int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd,
                        const void* bias, int bias_dtype, int accumulate,
                        const mt_gemm_opts* opts, mt_stream_t stream);

/* ---- Grouped (per-expert) MXFP8 path behind GroupedLinear ----
 * Rows of the activation matrix are split into G consecutive groups by m_offsets[G+1], an array
 * in DEVICE memory (m_offsets[0] = 0, m_offsets[G] = rows, non-decreasing; empty groups
 * allowed); group g multiplies with its own weight. Replaces the calls the reference's
 * GroupedLinear makes into modules that do not exist in its tree: grouped_qgemm
 * (miniTransformer/module/group_linear.py:108-119, 198-209), grouped_transpose_quantize
 * (:231-236) and cutlass_grouped_gemm_1d1d (:238-243).
 *
 * A plan is built once per distinct m_offsets by mt_grouped_plan_build (one small kernel, no
 * host copy) into caller-owned device memory of mt_grouped_plan_bytes(rows, G) bytes and is
 * then shared by every grouped call of the step (fc1 / fc2, forward and backward): it holds the
 * offsets, the offsets after padding every group to 128 tokens and the tile tables. The
 * grouped entry points read it on the device; none of them touches host memory or
 * synchronises. Offsets that are not a valid partition of [0, rows) leave an empty plan (the
 * grouped calls then compute nothing) and raise bit 32 of the device status word
 * (mt_read_device_status). `padded_rows` below is the padded token total, which the caller
 * knows from its split sizes: sum over groups of ceil(m_g / 128) * 128. */
int64_t mt_grouped_plan_bytes(int64_t rows, int64_t groups);
int mt_grouped_plan_build(const int64_t* m_offsets, int64_t groups, int64_t rows,
                          void* plan, int64_t plan_bytes, mt_stream_t stream);

/* Transposed MXFP8 quantization with per-group blocks: q_t[cols, padded_rows] holds x^T with
 * group g's tokens at columns pad_offset[g].., zero-padded to 128; 1x32 blocks start at each
 * group's first token, so no block mixes two groups. s_t (optional, row-major
 * [cols, padded_rows/32], stride s_t_stride) and s_t_swz (GEMM layout,
 * mt_swizzled_scale_bytes(cols, padded_rows/32) bytes). */
int mt_grouped_transpose_quantize_mxfp8(const void* x, int64_t rows, int64_t cols,
                                        const void* plan, int64_t G, int64_t padded_rows,
                                        uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                                        mt_stream_t stream);

/* The same transposed copy plus, from the same read of x, the plain row-wise copy that
 * mt_quantize_mxfp8 would produce: q [rows, cols], s (optional, row-major [rows, cols/32], stride
 * s_stride) and s_swz (GEMM layout, mt_swizzled_scale_bytes(rows, cols/32) bytes; bytes of rows
 * beyond `rows` in the last 128-row chunk are not written: zero the buffer once if a defined
 * value is wanted there). One pass over x serves the dgrad operand (row-wise dy) and the wgrad
 * operand (dy^T per group); the reference's GroupedLinear quantizes and transposes in separate
 * steps (miniTransformer/module/group_linear.py:87-108, 231-238). */
int mt_grouped_quantize_mxfp8(const void* x, int64_t rows, int64_t cols,
                              const void* plan, int64_t G, int64_t padded_rows,
                              uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz,
                              uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                              mt_stream_t stream);

/* D[rows of g, 0:N] = A[rows of g, 0:K] . B_g^T for every group g. A, D and sa_swz use the
 * plain (unpadded) row numbering. B is one matrix of b_rows rows of ldb bytes; group g uses
 * its rows [g*b_group_rows, +N) and contraction bytes [g*b_group_k, +K):
 *   forward: B = stacked weights [G*N, K]          -> b_group_rows = N, b_group_k = 0
 *   dgrad:   B = transposed stacked weights [N, G*K] -> b_group_rows = 0, b_group_k = K
 * N and K must be multiples of 128. */
int mt_grouped_gemm_mxfp8(const uint8_t* a, const uint8_t* sa_swz, const uint8_t* b, const uint8_t* sb_swz,
                          int64_t b_rows, int64_t ldb, const void* plan, int64_t G, int64_t rows,
                          int64_t N, int64_t K, int64_t b_group_rows, int64_t b_group_k,
                          void* d, int d_dtype, int64_t ldd, mt_stream_t stream);

/* mt_grouped_gemm_mxfp8 without a caller-provided plan buffer. No counterpart in the reference.
 *
 * Some callers have no way to hand over device memory for the plan: every free byte of the
 * GPU already belongs to someone else's allocator (a training framework's caching pool, an
 * inference server with a fixed memory plan), or they sit in a latency-critical loop where a
 * cudaMalloc / cudaFree would synchronise the whole device. For them the plan lives in a fixed
 * array inside the library image: about 0.3 MB of device memory on every GPU that loads the
 * library, held until the process exits. The call takes the device offsets array directly,
 * builds the plan into that array and runs the GEMM; it allocates nothing, neither on the
 * device nor through any library.
 *
 * Limits: at most MT_STATIC_MAX_GROUPS groups and MT_STATIC_MAX_ROWS rows; larger problems
 * are rejected with MT_ERR_INVALID_ARG and a message naming the limit.
 * All calls on one GPU share the one array. Each call rebuilds the plan before it uses it, so
 * nothing needs clearing between calls, but two calls whose kernels can overlap on the GPU
 * (different streams) race on it: serialise them.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress);
 * make that first call before starting any stream capture.
 * Other arguments, results and tolerances are those of mt_grouped_gemm_mxfp8. */
#define MT_STATIC_MAX_GROUPS 1024
#define MT_STATIC_MAX_ROWS 1048576
int mt_grouped_gemm_mxfp8_static(const uint8_t* a, const uint8_t* sa_swz, const uint8_t* b, const uint8_t* sb_swz,
                                 int64_t b_rows, int64_t ldb, const int64_t* m_offsets, int64_t G, int64_t rows,
                                 int64_t N, int64_t K, int64_t b_group_rows, int64_t b_group_k,
                                 void* d, int d_dtype, int64_t ldd, mt_stream_t stream);

/* Per-group weight gradients: D_g[N_out, K_out] (+)= A_t[:, cols_g] . B_t[:, cols_g]^T with
 * cols_g = [pad_offset[g], pad_offset[g+1]) of the padded token axis (outputs of
 * mt_grouped_transpose_quantize_mxfp8 on dy and x with the same plan). The G outputs are
 * stored back to back; an empty group yields zeros. */
int mt_grouped_wgrad_mxfp8(const uint8_t* a_t, const uint8_t* sa_t_swz, const uint8_t* b_t, const uint8_t* sb_t_swz,
                           const void* plan, int64_t G, int64_t rows, int64_t padded_rows,
                           int64_t N_out, int64_t K_out, void* d, int d_dtype, int accumulate,
                           mt_stream_t stream);

/* ---- Tensor-parallel exchange over NVLink peer memory (ranks of one node, one GPU per process) ----
 * These replace the NCCL collectives of the sequence-parallel Linear on one NVSwitch node
 * (miniTransformer/distributed/distributed.py:43-121 as used by module/linear.py:231-240,
 * 322-328, 356-365, 404-410) with kernels of this library that read and write the peers' memory
 * directly. Every rank allocates its buffers itself (any cudaMalloc'ed memory), exports them with
 * mt_ipc_export, exchanges the handles through its own channel (a process group, a file), and
 * maps the peers' buffers with mt_ipc_import. The entry points take tables of n addresses
 * indexed by rank; entry `me` is the rank's own buffer. All waits on peers are bounded (2 s);
 * on expiry bit 64 of the device status word is raised (mt_read_device_status).
 *
 * Control block: MT_PEER_CTRL_BYTES bytes per rank, zeroed once before every rank's first call
 * (with a host-side barrier between the zeroing and the first use). `channel` (0..7) separates
 * call sequences that may overlap in time (different streams); on one channel every rank must
 * issue the same sequence of exchanges, one at a time. The exchanges number themselves with a
 * counter in the control block, so a stream capture that contains them can be replayed. */
#define MT_PEER_CTRL_BYTES 4096
#define MT_MAX_GATHER_SEGS 8
#define MT_IPC_HANDLE_BYTES 64
int mt_ipc_export(const void* ptr, uint8_t* handle_out /* MT_IPC_HANDLE_BYTES */, int64_t* offset_out);
int mt_ipc_import(const uint8_t* handle, int64_t offset, void** ptr_out);
int mt_ipc_close(void* ptr, int64_t offset);

/* All ranks' work enqueued before the barrier on `stream` (on each rank's own stream) is complete
 * and visible to every rank's work enqueued after it. One 32-thread kernel. */
int mt_peer_barrier(const void* const* ctrl, int n, int me, int channel, mt_stream_t stream);

/* vals[0..nvals) (device fp32, nvals <= 4, non-negative values) <- element-wise maximum over all
 * ranks; also a barrier. The per-tensor abs-max of a token-sharded activation before its shards
 * are quantized (the MAX all-reduce of miniTransformer/ops/quantization.py:100-119 `reduce_amax`). */
int mt_peer_allreduce_max(const void* const* ctrl, int n, int me, int channel,
                          float* vals, int nvals, mt_stream_t stream);

/* All-gather by pulling: for every segment s < nseg and every rank r < n, copies shard_bytes[s]
 * bytes from shared[r] + src_offsets[s] to dsts[s] + r * shard_bytes[s]. The quantize kernels
 * write a rank's shard (codes, scales, transposed codes, transposed scales) straight into its
 * shared buffer; after a peer barrier this one launch assembles the gathered tensors in the
 * layout the GEMMs read. `ctas` is the grid size. whole_sms = 0: CTAs of 128 threads, for a copy
 * that has the GPU to itself (two per SM saturate NVLink). whole_sms = 1: CTAs of 1024 threads that
 * each occupy one SM, for a copy that runs beside a GEMM launched with mt_gemm_opts.sm_margin =
 * ctas (a GEMM CTA fills its SM's register file, so the two kernels cannot share SMs).
 * Sizes, offsets and addresses are multiples of 16 bytes. The caller keeps a shard unchanged
 * until a later barrier shows that every rank has pulled it. */
int mt_peer_gather(const void* const* shared, int n, int me, const int64_t* src_offsets, void* const* dsts,
                   const int64_t* shard_bytes, int nseg, int ctas, int whole_sms, mt_stream_t stream);

/* out[rows, cols] (bf16) = sum over s < n of stage[s][rows, cols] (bf16, fp32 accumulation in rank
 * order, one rounding): the second half of the reduce-scatter started by a GEMM with
 * mt_gemm_opts.n_dest, run after a peer barrier. amax_out (optional, zeroed by the caller) is
 * raised to max |out|. */
int mt_peer_reduce_bf16(const void* stage, int n, int64_t rows, int64_t cols, void* out, float* amax_out,
                        mt_stream_t stream);

/* Reads and clears the device-side status word the kernels raise when a bounded wait
 * expires (0 = clean). Synchronises the given stream. */
int mt_read_device_status(int* status_out, mt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MT_B200_H_ */
