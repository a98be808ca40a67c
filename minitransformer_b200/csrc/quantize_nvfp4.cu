// NVFP4 block quantize for sm_100a: per-tensor abs-max, then cast (+ transpose) of a bf16
// matrix to packed E2M1 codes with one E4M3 scale per 1x16 (or 16x16) block.
//
// One CTA handles one 128x128 tile. The tile arrives in shared memory through a single TMA
// load (out-of-range rows/columns are zero-filled, which is exactly the zero padding the
// emulation applies to ragged shapes). A row pass quantizes 1x16 blocks straight from
// shared memory to global memory; a column pass reads 16-row strips, optionally applies
// the 16-point Hadamard transform, and stages the transposed codes in shared memory so the
// global stores are 16-byte and row-contiguous. All scale bytes are staged and written
// twice: row-major (the tensor the operator API returns) and in the 128x4-chunk layout the
// tensor-core GEMM copies into tensor memory.
#include "quantize_common.cuh"

namespace mt {

struct __align__(128) Nvfp4Smem {
  uint16_t in[QT_ROWS][QT_COLS];         // 32 KiB, TMA destination
  uint8_t out_t[QT_COLS][QT_ROWS / 2];   // 8 KiB, transposed codes (8-byte slots XOR-swizzled)
  uint8_t s_lin[QT_ROWS][8];             // row-wise scales, row-major
  uint8_t s_swz[2][512];                 // row-wise scales, chunk layout
  uint8_t st_blk[8][QT_COLS];            // column-wise scales as produced: [token block][feature]
  float blk_amax[8][8];                  // 16x16 block abs-max (2-D mode)
  float lut_row[128];                    // element factor per scale byte, row-wise copy
  float lut_col[128];                    // same for the transposed copy (its own per-tensor scale)
  uint64_t bar;
  int abort_flag;
};

// ------------------------------------------------------------------------------------------
// abs-max
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) amax_plain_kernel(const uint4* __restrict__ x, int64_t n_vec,
                                                         float* __restrict__ amax_row) {
  pdl_trigger();   // the kernel that reads the result may take its place on the SMs this one leaves
  pdl_wait();
  uint32_t m = 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v = __ldg(x + i);
    m = absmax2(m, absmax2(absmax2(v.x, v.y), absmax2(v.z, v.w)));
  }
  float f = absmax2_to_float(m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) f = fmaxf(f, __shfl_xor_sync(0xffffffffu, f, o));
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = f;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) f = fmaxf(f, red[i]);
    atomicMax(reinterpret_cast<unsigned int*>(amax_row), __float_as_uint(f));
  }
}

// Row abs-max and abs-max of the Hadamard-transformed transpose in one read of x.
// Lane <-> 4 adjacent columns, warp <-> 16 consecutive rows, CTA <-> 128x128 tile.
// kColSum: the same read also accumulates the column sums of x (fp32 atomics into col_sum[cols]):
// the bias gradient of a linear layer, taken from the pass over dy that its quantization needs anyway.
template <bool kRHT, bool kColSum>
__global__ void __launch_bounds__(256) amax_tiled_kernel(const uint16_t* __restrict__ x, int64_t rows, int64_t cols,
                                                         float* __restrict__ amax_row, float* __restrict__ amax_col,
                                                         float* __restrict__ col_sum) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c0 = (int64_t)blockIdx.x * QT_COLS + lane * 4;
  const int64_t r0 = (int64_t)blockIdx.y * QT_ROWS + warp * 16;
  float frow = 0.f, fcol = 0.f;
  pdl_trigger();
  pdl_wait();
  float cs[4] = {0.f, 0.f, 0.f, 0.f};
  if (c0 < cols && r0 < rows) {  // rows % 16 == 0, cols % 4 == 0: the strip is all-in or all-out
    uint32_t wa[16], wb[16];   // columns (c0, c0+1) and (c0+2, c0+3), one packed word per row
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint2 t = __ldg(reinterpret_cast<const uint2*>(x + (r0 + j) * cols + c0));
      wa[j] = t.x;
      wb[j] = t.y;
    }
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) m = absmax2(absmax2(m, wa[j]), wb[j]);
    frow = absmax2_to_float(m);
    if (kColSum) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        cs[0] += bf16_lo(wa[j]); cs[1] += bf16_hi(wa[j]);
        cs[2] += bf16_lo(wb[j]); cs[3] += bf16_hi(wb[j]);
      }
    }
    if (kRHT) {
      rht16_x2(wa);
      rht16_x2(wb);
      m = 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) m = absmax2(absmax2(m, wa[j]), wb[j]);
      fcol = absmax2_to_float(m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    frow = fmaxf(frow, __shfl_xor_sync(0xffffffffu, frow, o));
    if (kRHT) fcol = fmaxf(fcol, __shfl_xor_sync(0xffffffffu, fcol, o));
  }
  __shared__ float red[2][8];
  __shared__ float csum[8][QT_COLS];
  if (lane == 0) { red[0][warp] = frow; red[1][warp] = fcol; }
  if (kColSum) *reinterpret_cast<float4*>(&csum[warp][lane * 4]) = make_float4(cs[0], cs[1], cs[2], cs[3]);
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) { frow = fmaxf(frow, red[0][i]); fcol = fmaxf(fcol, red[1][i]); }
    atomicMax(reinterpret_cast<unsigned int*>(amax_row), __float_as_uint(frow));
    if (amax_col != nullptr) atomicMax(reinterpret_cast<unsigned int*>(amax_col), __float_as_uint(kRHT ? fcol : frow));
  }
  if (kColSum && threadIdx.x < QT_COLS) {
    const int64_t c = (int64_t)blockIdx.x * QT_COLS + threadIdx.x;
    if (c < cols) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += csum[w][threadIdx.x];
      atomicAdd(col_sum + c, t);
    }
  }
}

__global__ void copy_scalar_kernel(const float* src, float* dst) {
  pdl_trigger();
  pdl_wait();
  *dst = *src;
}

// ------------------------------------------------------------------------------------------
// cast + transpose
// ------------------------------------------------------------------------------------------
struct Nvfp4Args {
  int64_t rows, cols;
  int64_t rows_s;       // rows of the row-major scale tensor s (>= rows)
  int64_t cols_s;       // rows of the row-major scale tensor s_t (>= cols)
  int64_t s_stride, s_t_stride;
  int64_t kc_row;       // K-chunks per row block in s_swz   (multiple of 4)
  int64_t kc_col;       // K-chunks per row block in s_t_swz (multiple of 4)
  const float* amax_row;
  const float* amax_col;
  uint8_t *q, *s, *s_swz, *q_t, *s_t, *s_t_swz;
  int* status;
  uint64_t seed;        // stochastic rounding only
};

// kSR: codes are rounded stochastically (cvt.rs) instead of to nearest-even; scales are unchanged.
template <bool kTranspose, bool k2D, bool kRHT, bool kSR = false>
__global__ void __launch_bounds__(Q_THREADS) quantize_nvfp4_kernel(const __grid_constant__ CUtensorMap in_map,
                                                                   const Nvfp4Args a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Nvfp4Smem& sm = *reinterpret_cast<Nvfp4Smem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t k0 = (int64_t)blockIdx.x * QT_COLS;
  const int64_t m0 = (int64_t)blockIdx.y * QT_ROWS;

  pdl_trigger();
  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.bar, 1);
    mbar_fence_init();
  }
  pdl_wait();   // the tensor and its abs-max come from the kernels before this one
  __syncthreads();
  if (tid == 0) {
    mbar_expect_tx(&sm.bar, QT_ROWS * QT_COLS * 2);
    tma_load_2d(&sm.in[0][0], &in_map, &sm.bar, (int32_t)k0, (int32_t)m0);
  }
  const Nvfp4Global g_row = nvfp4_global(*a.amax_row);
  const Nvfp4Global g_col = kTranspose ? nvfp4_global(*a.amax_col) : g_row;
  const bool fuse_row = nvfp4_can_fuse_scaling(*a.amax_row);
  const bool fuse_col = kTranspose ? nvfp4_can_fuse_scaling(*a.amax_col) : fuse_row;
  // element-factor tables (one entry per non-negative E4M3 scale byte), filled while the tile loads
  if (tid < 128) sm.lut_row[tid] = nvfp4_encode_for_byte(tid, g_row);
  else if (kTranspose) sm.lut_col[tid - 128] = nvfp4_encode_for_byte(tid - 128, g_col);
  __syncthreads();

  const bool ok = mbar_wait_bounded(&sm.bar, 0, &sm.abort_flag, a.status, DS_QUANT_WAIT);
  if (!ok) return;  // no copy of ours can still be in flight only if it never started; status is raised

  // ---- 2-D mode: abs-max of every 16x16 block, shared by both passes ----
  if (k2D) {
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint2 w = *reinterpret_cast<const uint2*>(&sm.in[warp * 16 + j][lane * 4]);
      m = absmax2(m, absmax2(w.x, w.y));
    }
    float f = absmax2_to_float(m);
    f = fmaxf(f, __shfl_xor_sync(0xffffffffu, f, 1));
    f = fmaxf(f, __shfl_xor_sync(0xffffffffu, f, 2));
    // All four lanes of a block hold the same value and all store it. (Guarding the store
    // with lane % 4 == 0 made nvcc 12.9 reuse the guarded address, byte offset = lane, for
    // the unguarded loads below: a misaligned fp32 load.)
    sm.blk_amax[warp][lane >> 2] = f;
    __syncthreads();
  }

  // ---- row pass: thread <-> (row, 1x16 block) ----
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int r = it * 32 + (tid >> 3);
    const int b = tid & 7;
    const uint4 w0 = *reinterpret_cast<const uint4*>(&sm.in[r][b * 16]);
    const uint4 w1 = *reinterpret_cast<const uint4*>(&sm.in[r][b * 16 + 8]);
    float vmax;
    if (k2D) {
      vmax = sm.blk_amax[r >> 4][b];
    } else {
      const uint32_t m = absmax2(absmax2(absmax2(w0.x, w0.y), absmax2(w0.z, w0.w)),
                                 absmax2(absmax2(w1.x, w1.y), absmax2(w1.z, w1.w)));
      vmax = absmax2_to_float(m);
    }
    uint32_t sbyte;
    float enc;
    nvfp4_block_scale_lut(vmax, g_row.ges, sm.lut_row, sbyte, enc);
    uint2 codes;
    const int64_t gr = m0 + r, gc = k0 + b * 16;
    if (kSR) {
      const uint64_t grp = (uint64_t)(gr * a.cols + gc) >> 2;     // groups of four consecutive elements
      codes.x = e2m1x8_from_words_sr(w0.x, w0.y, w0.z, w0.w, enc, fuse_row, sr_bits(a.seed, grp), sr_bits(a.seed, grp + 1));
      codes.y = e2m1x8_from_words_sr(w1.x, w1.y, w1.z, w1.w, enc, fuse_row, sr_bits(a.seed, grp + 2), sr_bits(a.seed, grp + 3));
    } else {
      codes.x = e2m1x8_from_words(w0.x, w0.y, w0.z, w0.w, enc, fuse_row);
      codes.y = e2m1x8_from_words(w1.x, w1.y, w1.z, w1.w, enc, fuse_row);
    }
    if (gr < a.rows && gc < a.cols)
      *reinterpret_cast<uint2*>(a.q + gr * (a.cols >> 1) + (gc >> 1)) = codes;
    sm.s_lin[r][b] = static_cast<uint8_t>(sbyte);
    sm.s_swz[b >> 2][sf_chunk_offset(r, b)] = static_cast<uint8_t>(sbyte);
  }

  // ---- column pass: lane <-> 4 adjacent columns, warp <-> 16 rows ----
  if (kTranspose) {
    uint32_t sb_word = 0;  // scale bytes of this lane's 4 columns (block = this warp's 16 rows)
    uint32_t wp[2][16];   // wp[p][j]: row j of column pair p (columns 4*lane + 2p, + 2p + 1)
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint2 t = *reinterpret_cast<const uint2*>(&sm.in[warp * 16 + j][lane * 4]);
      wp[0][j] = t.x;
      wp[1][j] = t.y;
    }
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      if (kRHT) rht16_x2(wp[p]);
      float vmax_lo, vmax_hi;
      if (k2D) {
        vmax_lo = vmax_hi = sm.blk_amax[warp][lane >> 2];
      } else {
        uint32_t m = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) m = absmax2(m, wp[p][j]);
        vmax_lo = absmax2_lo(m);
        vmax_hi = absmax2_hi(m);
      }
      uint32_t sb_lo, sb_hi;
      float enc_lo, enc_hi;
      nvfp4_block_scale_lut(vmax_lo, g_col.ges, sm.lut_col, sb_lo, enc_lo);
      nvfp4_block_scale_lut(vmax_hi, g_col.ges, sm.lut_col, sb_hi, enc_hi);
      const f32x2_t enc2 = pack2(enc_lo, enc_hi);
      uint2 c_lo, c_hi;
      const int col = lane * 4 + 2 * p;
      if (kSR) {
        // the transposed copy draws from its own part of the counter space
        const uint64_t grp = (((uint64_t)(k0 + col) * (uint64_t)a.rows + (uint64_t)(m0 + warp * 16)) >> 2) + (1ull << 40);
        e2m1x8_two_columns_sr(&wp[p][0], enc2, fuse_col, c_lo.x, c_hi.x, sr_bits(a.seed, grp), sr_bits(a.seed, grp + 1));
        e2m1x8_two_columns_sr(&wp[p][8], enc2, fuse_col, c_lo.y, c_hi.y, sr_bits(a.seed, grp + 2), sr_bits(a.seed, grp + 3));
      } else {
        e2m1x8_two_columns(&wp[p][0], enc2, fuse_col, c_lo.x, c_hi.x);
        e2m1x8_two_columns(&wp[p][8], enc2, fuse_col, c_lo.y, c_hi.y);
      }
      const int slot = warp ^ (lane & 7);
      *reinterpret_cast<uint2*>(&sm.out_t[col][slot * 8]) = c_lo;
      *reinterpret_cast<uint2*>(&sm.out_t[col + 1][slot * 8]) = c_hi;
      sb_word |= ((sb_lo & 0xFFu) | ((sb_hi & 0xFFu) << 8)) << (16 * p);
    }
    // one conflict-free 4-byte store per lane; the row-major and GEMM layouts are assembled
    // from this array when the tile is written out
    *reinterpret_cast<uint32_t*>(&sm.st_blk[warp][lane * 4]) = sb_word;
  }
  __syncthreads();

  // ---- cooperative, row-contiguous global stores of the staged outputs ----
  // Row-wise scales, row-major: 128 rows x 8 bytes.
  if (tid < QT_ROWS) {
    const int64_t gr = m0 + tid;
    const int64_t kb0 = k0 >> 4;
    const int nvalid = (int)min((int64_t)8, (a.cols >> 4) - kb0);
    if (gr < a.rows_s) store_bytes(a.s + gr * a.s_stride + kb0, sm.s_lin[tid], nvalid);
  }
  // Row-wise scales, chunk layout: two 512-byte chunks (+ zero chunks up to the padded count
  // when this is the last tile along K).
  if (a.s_swz != nullptr) {
    uint8_t* base = a.s_swz + ((m0 >> 7) * a.kc_row + (k0 >> 6)) * 512;
    if (tid < 64) *reinterpret_cast<uint4*>(base + tid * 16) = *reinterpret_cast<const uint4*>(&sm.s_swz[0][0] + tid * 16);
    if (k0 + QT_COLS >= a.cols) {
      const int64_t extra = a.kc_row - ((k0 >> 6) + 2);
      for (int64_t i = tid; i < extra * 32; i += Q_THREADS)
        *reinterpret_cast<uint4*>(base + 1024 + i * 16) = make_uint4(0, 0, 0, 0);
    }
  }
  if (kTranspose) {
    // Transposed codes: 128 feature rows x 64 bytes (128 tokens).
    const int64_t row_bytes = a.rows >> 1;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int row = it * 64 + (tid >> 2);
      const int ch = tid & 3;
      const int64_t gk = k0 + row;
      const int swz = (row >> 2) & 7;
      // the two 8-byte slots 2ch, 2ch+1 sit in one 16-byte chunk, possibly swapped
      const int p0 = (2 * ch) ^ swz;
      uint4 val = *reinterpret_cast<const uint4*>(&sm.out_t[row][(p0 & ~1) * 8]);
      if (p0 & 1) val = make_uint4(val.z, val.w, val.x, val.y);
      const int64_t byte0 = (m0 >> 1) + ch * 16;
      const int n = (int)max((int64_t)0, min((int64_t)16, row_bytes - byte0));
      if (gk < a.cols && n > 0) {
        uint8_t* dst = a.q_t + gk * row_bytes + byte0;
        if (n == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
          *reinterpret_cast<uint4*>(dst) = val;
        } else {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(&val);
          for (int i = 0; i < n; ++i) dst[i] = src[i];
        }
      }
    }
    if (tid < QT_COLS) {
      // feature tid: its 8 token-block scales, gathered from the 8 rows of the staging array
      const int64_t gk = k0 + tid;
      const int64_t mb0 = m0 >> 4;
      const int nvalid = (int)min((int64_t)8, ((a.rows + 15) >> 4) - mb0);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        lo |= static_cast<uint32_t>(sm.st_blk[w][tid]) << (8 * w);
        hi |= static_cast<uint32_t>(sm.st_blk[w + 4][tid]) << (8 * w);
      }
      if (gk < a.cols_s && nvalid > 0) {
        uint8_t* dst = a.s_t + gk * a.s_t_stride + mb0;
        if (nvalid == 8 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
        } else {
          for (int i = 0; i < nvalid; ++i) dst[i] = static_cast<uint8_t>((i < 4 ? lo >> (8 * i) : hi >> (8 * (i - 4))) & 0xFFu);
        }
      }
    }
    if (a.s_t_swz != nullptr) {
      uint8_t* base = a.s_t_swz + ((k0 >> 7) * a.kc_col + (m0 >> 6)) * 512;
      if (tid >= 128 && tid < 192) {
        // 16-byte cell (chunk c, lane row r5): byte q * 4 + kb = scale of feature q * 32 + r5, block 4c + kb
        const int c = (tid - 128) >> 5, r5 = tid & 31;
        uint32_t cell[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t v = 0;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) v |= static_cast<uint32_t>(sm.st_blk[c * 4 + kb][q * 32 + r5]) << (8 * kb);
          cell[q] = v;
        }
        *reinterpret_cast<uint4*>(base + c * 512 + r5 * 16) = make_uint4(cell[0], cell[1], cell[2], cell[3]);
      }
      if (m0 + QT_ROWS >= a.rows) {
        const int64_t extra = a.kc_col - ((m0 >> 6) + 2);
        for (int64_t i = tid; i < extra * 32; i += Q_THREADS)
          *reinterpret_cast<uint4*>(base + 1024 + i * 16) = make_uint4(0, 0, 0, 0);
      }
    }
  }
}

// Row-major scale bytes -> chunk layout (for callers that only hold the row-major tensor).
__global__ void swizzle_scales_kernel(const uint8_t* __restrict__ s, int64_t rows, int64_t k_blocks, int64_t s_stride,
                                      uint8_t* __restrict__ out, int64_t kc_pad) {
  // one CTA per (row block, chunk): 128 threads <-> 128 rows, 4 bytes each
  const int64_t rb = blockIdx.y, kc = blockIdx.x;
  const int r = threadIdx.x;
  const int64_t gr = rb * 128 + r;
  uint32_t word = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t kb = kc * 4 + i;
    uint32_t b = (gr < rows && kb < k_blocks) ? s[gr * s_stride + kb] : 0u;
    word |= b << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(out + (rb * kc_pad + kc) * 512 + (r & 31) * 16 + (r >> 5) * 4) = word;
}

static int64_t padded_chunks(int64_t k_blocks) { return ((k_blocks + 3) / 4 + 3) / 4 * 4; }

template <bool T, bool D2, bool R, bool SR = false>
static int launch_nvfp4(const CUtensorMap& map, const Nvfp4Args& args, dim3 grid, cudaStream_t st) {
  static bool attr_set[MT_MAX_DEVICES] = {};
  const int slot = current_device_slot();
  auto kern = quantize_nvfp4_kernel<T, D2, R, SR>;
  const int smem = (int)sizeof(Nvfp4Smem) + 128;
  if (!attr_set[slot]) {
    MT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[slot] = true;
  }
  MT_CUDA(launch_pdl(kern, grid, dim3(Q_THREADS), (size_t)smem, st, map, args));
  return MT_OK;
}

}  // namespace mt

static int amax_impl(const void* x, int64_t rows, int64_t cols, int flags, float* amax_row, float* amax_col,
                     float* col_sum, mt_stream_t stream) {
  using namespace mt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MT_REQUIRE(amax_row != nullptr, "mt_amax_bf16: null amax_row");
  MT_REQUIRE(rows >= 0 && cols >= 0 && cols % 8 == 0, "mt_amax_bf16: cols (%lld) must be a multiple of 8", (long long)cols);
  if (rows == 0 || cols == 0) {  // an empty tensor has abs-max 0 and may come with a null pointer
    MT_CUDA(cudaMemsetAsync(amax_row, 0, sizeof(float), st));
    if (amax_col) MT_CUDA(cudaMemsetAsync(amax_col, 0, sizeof(float), st));
    if (col_sum && cols > 0) MT_CUDA(cudaMemsetAsync(col_sum, 0, sizeof(float) * cols, st));
    return MT_OK;
  }
  MT_REQUIRE(x != nullptr, "mt_amax_bf16: null x");
  MT_REQUIRE(col_sum == nullptr || rows % 16 == 0, "mt_amax_colsum_bf16: column sums need rows %% 16 == 0 (rows=%lld)",
             (long long)rows);
  MT_REQUIRE(aligned16(x), "mt_amax_bf16: x must be 16-byte aligned");
  const bool rht = (flags & MT_Q_RHT) && amax_col != nullptr;
  MT_REQUIRE(!rht || rows % 16 == 0, "mt_amax_bf16: the Hadamard transform needs rows %% 16 == 0 (rows=%lld)", (long long)rows);
  // one memset node when the two scalars are neighbours in one buffer (how the Python front end allocates them)
  const bool zero_col = rht || (col_sum && amax_col);
  if (flags & MT_Q_AMAX_ZEROED) {
    // the caller's scalars are zero already: nothing between the previous kernel and this one
  } else if (zero_col && amax_col == amax_row + 1) {
    MT_CUDA(cudaMemsetAsync(amax_row, 0, 2 * sizeof(float), st));
  } else {
    MT_CUDA(cudaMemsetAsync(amax_row, 0, sizeof(float), st));
    if (zero_col) MT_CUDA(cudaMemsetAsync(amax_col, 0, sizeof(float), st));
  }
  if (col_sum) MT_CUDA(cudaMemsetAsync(col_sum, 0, sizeof(float) * cols, st));
  if (rht || col_sum) {
    dim3 grid((unsigned)((cols + QT_COLS - 1) / QT_COLS), (unsigned)((rows + QT_ROWS - 1) / QT_ROWS));
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    if (rht && col_sum) amax_tiled_kernel<true, true><<<grid, 256, 0, st>>>(xp, rows, cols, amax_row, amax_col, col_sum);
    else if (rht) amax_tiled_kernel<true, false><<<grid, 256, 0, st>>>(xp, rows, cols, amax_row, amax_col, nullptr);
    else amax_tiled_kernel<false, true><<<grid, 256, 0, st>>>(xp, rows, cols, amax_row, amax_col, col_sum);
  } else {
    const int64_t n_vec = rows * cols / 8;
    int blocks = (int)std::min<int64_t>((n_vec + 255) / 256, 148 * 8);
    amax_plain_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint4*>(x), n_vec, amax_row);
    // without the transform both copies share one abs-max: a caller that passes the same scalar twice needs no copy
    if (amax_col && amax_col != amax_row)
      MT_CUDA(launch_pdl(copy_scalar_kernel, dim3(1), dim3(1), 0, st, (const float*)amax_row, amax_col));
  }
  MT_CUDA(cudaGetLastError());
  return MT_OK;
}

static int quantize_nvfp4_impl(const void* x, int64_t rows, int64_t cols, int flags, const float* amax_row,
                               const float* amax_col, uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz,
                               uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz, bool sr, uint64_t seed,
                               mt_stream_t stream) {
  using namespace mt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MT_REQUIRE(rows >= 0 && cols >= 0, "mt_quantize_nvfp4: negative shape");
  if (rows == 0 || cols == 0) return MT_OK;  // nothing to write; pointers may be null
  MT_REQUIRE(x && q && s && amax_row, "mt_quantize_nvfp4: null x/q/s/amax_row");
  MT_REQUIRE(cols % 16 == 0, "mt_quantize_nvfp4: cols (%lld) must be a multiple of 16", (long long)cols);
  MT_REQUIRE(aligned16(x) && aligned16(q), "mt_quantize_nvfp4: x and q must be 16-byte aligned");
  const bool transpose = q_t != nullptr;
  const bool d2 = (flags & MT_Q_2D) != 0, rht = (flags & MT_Q_RHT) != 0;
  const bool pad16 = d2 || (flags & MT_Q_ROWPAD16);
  MT_REQUIRE(!transpose || (s_t && amax_col), "mt_quantize_nvfp4: q_t given without s_t / amax_col");
  MT_REQUIRE(!transpose || rows % 2 == 0, "mt_quantize_nvfp4: the transposed copy needs an even row count (rows=%lld)", (long long)rows);
  MT_REQUIRE(!(d2 && rht), "mt_quantize_nvfp4: 2-D scaling together with the Hadamard transform is not supported");
  MT_REQUIRE(!(sr && d2), "mt_quantize_nvfp4_sr: stochastic rounding is offered for 1x16 blocks only");
  MT_REQUIRE(!rht || rows % 16 == 0, "mt_quantize_nvfp4: the Hadamard transform needs rows %% 16 == 0");
  MT_REQUIRE(s_stride >= cols / 16 && (!transpose || s_t_stride >= (rows + 15) / 16), "mt_quantize_nvfp4: scale stride too small");
  MT_REQUIRE((!s_swz || aligned16(s_swz)) && (!s_t_swz || aligned16(s_t_swz)), "mt_quantize_nvfp4: swizzled scale buffers must be 16-byte aligned");
  if (rows == 0 || cols == 0) return MT_OK;

  Nvfp4Args args;
  args.rows = rows; args.cols = cols;
  args.rows_s = pad16 ? (rows + 15) / 16 * 16 : rows;
  args.cols_s = pad16 ? (cols + 15) / 16 * 16 : cols;
  args.s_stride = s_stride; args.s_t_stride = s_t_stride;
  args.kc_row = padded_chunks(cols / 16);
  args.kc_col = padded_chunks((rows + 15) / 16);
  args.amax_row = amax_row; args.amax_col = transpose ? amax_col : amax_row;
  args.q = q; args.s = s; args.s_swz = s_swz; args.q_t = q_t; args.s_t = s_t; args.s_t_swz = s_t_swz;
  args.status = device_status_ptr();
  if (!args.status) return fail(MT_ERR_CUDA, "device status word not reachable");
  args.seed = seed;

  CUtensorMap map;
  int rc = make_tensor_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)cols, (uint64_t)rows,
                              (uint64_t)cols * 2, QT_COLS, QT_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MT_OK) return rc;
  dim3 grid((unsigned)((cols + QT_COLS - 1) / QT_COLS), (unsigned)((rows + QT_ROWS - 1) / QT_ROWS));
  if (sr) {
    if (!transpose) return launch_nvfp4<false, false, false, true>(map, args, grid, st);
    return rht ? launch_nvfp4<true, false, true, true>(map, args, grid, st)
               : launch_nvfp4<true, false, false, true>(map, args, grid, st);
  }
  if (!transpose) {
    return d2 ? launch_nvfp4<false, true, false>(map, args, grid, st) : launch_nvfp4<false, false, false>(map, args, grid, st);
  }
  if (d2) return launch_nvfp4<true, true, false>(map, args, grid, st);
  if (rht) return launch_nvfp4<true, false, true>(map, args, grid, st);
  return launch_nvfp4<true, false, false>(map, args, grid, st);
}

extern "C" {

int mt_amax_bf16(const void* x, int64_t rows, int64_t cols, int flags, float* amax_row, float* amax_col,
                 mt_stream_t stream) {
  return amax_impl(x, rows, cols, flags, amax_row, amax_col, nullptr, stream);
}

int mt_amax_colsum_bf16(const void* x, int64_t rows, int64_t cols, int flags, float* amax_row, float* amax_col,
                        float* col_sum, mt_stream_t stream) {
  MT_REQUIRE(col_sum != nullptr, "mt_amax_colsum_bf16: null col_sum");
  return amax_impl(x, rows, cols, flags, amax_row, amax_col, col_sum, stream);
}

int mt_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int flags, const float* amax_row,
                      const float* amax_col, uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz, uint8_t* q_t,
                      uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz, mt_stream_t stream) {
  return quantize_nvfp4_impl(x, rows, cols, flags, amax_row, amax_col, q, s, s_stride, s_swz, q_t, s_t, s_t_stride,
                             s_t_swz, false, 0, stream);
}

int mt_quantize_nvfp4_sr(const void* x, int64_t rows, int64_t cols, int flags, const float* amax_row,
                         const float* amax_col, uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz, uint8_t* q_t,
                         uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz, uint64_t seed, mt_stream_t stream) {
  return quantize_nvfp4_impl(x, rows, cols, flags, amax_row, amax_col, q, s, s_stride, s_swz, q_t, s_t, s_t_stride,
                             s_t_swz, true, seed, stream);
}

int mt_swizzle_scales(const uint8_t* s, int64_t rows, int64_t k_blocks, int64_t s_stride, uint8_t* s_swz,
                      mt_stream_t stream) {
  using namespace mt;
  MT_REQUIRE(s && s_swz, "mt_swizzle_scales: null pointer");
  MT_REQUIRE(rows >= 0 && k_blocks >= 0 && s_stride >= k_blocks, "mt_swizzle_scales: bad shape");
  MT_REQUIRE(aligned16(s_swz), "mt_swizzle_scales: output must be 16-byte aligned");
  if (rows == 0 || k_blocks == 0) return MT_OK;
  const int64_t kc = padded_chunks(k_blocks);
  dim3 grid((unsigned)kc, (unsigned)((rows + 127) / 128));
  swizzle_scales_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(s, rows, k_blocks, s_stride, s_swz, kc);
  MT_CUDA(cudaGetLastError());
  return MT_OK;
}

}  // extern "C"
