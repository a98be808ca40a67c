// MXFP8 block quantize for sm_100a: bf16 -> E4M3 elements with one E8M0 (power-of-two)
// scale byte per 1x32 block, row-wise copy plus an optional transposed copy whose blocks
// run along the original rows.
//
// Same tiling as the NVFP4 kernel: one CTA per 128x128 tile, one TMA load (zero fill
// outside the tensor), a row pass from shared memory straight to global memory and a
// column pass staged through shared memory so that global stores stay 16-byte and
// row-contiguous. There is no per-tensor scale in this format, hence no abs-max pre-pass.
#include <algorithm>

#include "grouped_plan.cuh"
#include "quantize_common.cuh"

namespace mt {

struct __align__(128) Mxfp8Smem {
  uint16_t in[QT_ROWS][QT_COLS];      // 32 KiB, TMA destination
  uint8_t out_t[QT_COLS][QT_ROWS];    // 16 KiB, transposed codes (16-byte chunks XOR-swizzled)
  uint8_t s_lin[QT_ROWS][4];
  uint8_t s_swz[512];
  uint8_t st_lin[QT_COLS][4];
  uint8_t st_swz[512];
  uint64_t bar;
  int abort_flag;
};

struct Mxfp8Args {
  int64_t rows, cols;
  int64_t s_stride, s_t_stride;
  int64_t kc_row, kc_col;
  uint8_t *q, *s, *s_swz, *q_t, *s_t, *s_t_swz;
  int* status;
  // grouped transposed mode: tile t covers input rows [tiles[t].row_start, +rows_valid) of one
  // group and writes 128 zero-padded token columns starting at tiles[t].out_col
  const int4* tiles;   // {row_start, rows_valid, out_col, last_tile}
  const int32_t* num_tiles_dev;   // device count of valid entries of `tiles`
  int64_t out_cols;    // padded token count (row length of q_t)
};

// kGroupedRow (grouped mode only): also emit the plain row-wise copy of the tile's rows (codes,
// row-major scales, GEMM-layout scales by global row index), so that one read of the tensor
// serves both the dgrad operand and the wgrad operand.
template <bool kTranspose, bool kGrouped = false, bool kGroupedRow = false>
__global__ void __launch_bounds__(Q_THREADS) quantize_mxfp8_kernel(const __grid_constant__ CUtensorMap in_map,
                                                                   const Mxfp8Args a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Mxfp8Smem& sm = *reinterpret_cast<Mxfp8Smem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t k0 = (int64_t)blockIdx.x * QT_COLS;
  int64_t m0 = (int64_t)blockIdx.y * QT_ROWS;
  int4 gt = make_int4(0, QT_ROWS, 0, 0);
  pdl_trigger();
  pdl_wait();   // before the plan, the tensor or anything else in global memory is read
  if (kGrouped) {
    if ((int)blockIdx.y >= *a.num_tiles_dev) return;   // uniform for the CTA: the plan holds fewer tiles
    gt = a.tiles[blockIdx.y];
    if ((int64_t)gt.z + QT_ROWS > a.out_cols) return;   // the caller's padded count disagrees with the plan
    m0 = gt.x;
  }

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0) {
    mbar_expect_tx(&sm.bar, QT_ROWS * QT_COLS * 2);
    tma_load_2d(&sm.in[0][0], &in_map, &sm.bar, (int32_t)k0, (int32_t)m0);
  }
  if (!mbar_wait_bounded(&sm.bar, 0, &sm.abort_flag, a.status, DS_QUANT_WAIT)) return;
  if (kGrouped) {
    // rows past the end of this group belong to the next one: they contribute zeros here
    const int r = tid >> 1, h = tid & 1;
    if (r >= gt.y) {
      uint4* p = reinterpret_cast<uint4*>(&sm.in[r][h * 64]);
#pragma unroll
      for (int i = 0; i < 8; ++i) p[i] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
  }

  // ---- row pass: thread <-> (row, 1x32 block); 4 blocks per tile row ----
#pragma unroll
  for (int it = 0; it < ((kGrouped && !kGroupedRow) ? 0 : 2); ++it) {
    const int r = it * 64 + (tid >> 2);
    const int b = tid & 3;
    uint4 w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = *reinterpret_cast<const uint4*>(&sm.in[r][b * 32 + i * 8]);
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) m = absmax2(m, absmax2(absmax2(w[i].x, w[i].y), absmax2(w[i].z, w[i].w)));
    const int e = e8m0_exponent(absmax2_to_float(m));
    const float enc = exp2_neg(e);
    uint4 out[2];
    uint32_t* o = reinterpret_cast<uint32_t*>(out);
    const f32x2_t enc2 = pack2(enc, enc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = e4m3x4_from_words(w[i].x, w[i].y, enc2);
      o[2 * i + 1] = e4m3x4_from_words(w[i].z, w[i].w, enc2);
    }
    const int64_t gr = m0 + r, gc = k0 + b * 32;
    if (gr < a.rows && gc < a.cols && (!kGrouped || r < gt.y)) {
      uint4* dst = reinterpret_cast<uint4*>(a.q + gr * a.cols + gc);
      dst[0] = out[0];
      dst[1] = out[1];
    }
    const uint8_t sbyte = static_cast<uint8_t>(e + 127);
    sm.s_lin[r][b] = sbyte;
    sm.s_swz[sf_chunk_offset(r, b)] = sbyte;
  }

  // ---- column pass: lane <-> 2 adjacent columns, warp <-> (32-row group, column half) ----
  if (kTranspose) {
    const int grp = warp & 3, half = warp >> 2;
    const int cbase = half * 64 + lane * 2;
    uint32_t w[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = *reinterpret_cast<const uint32_t*>(&sm.in[grp * 32 + j][cbase]);
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) m = absmax2(m, w[j]);
    // the two halves of the accumulator are the two columns' abs-max
    const int e0 = e8m0_exponent(absmax2_lo(m)), e1 = e8m0_exponent(absmax2_hi(m));
    const f32x2_t enc2 = pack2(exp2_neg(e0), exp2_neg(e1));
    uint4 out_lo[2], out_hi[2];
    uint32_t* ol = reinterpret_cast<uint32_t*>(out_lo);
    uint32_t* oh = reinterpret_cast<uint32_t*>(out_hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) e4m3x4_two_columns(&w[4 * i], enc2, ol[i], oh[i]);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int col = cbase + c;
      const int swz = (col >> 1) & 7;
      *reinterpret_cast<uint4*>(&sm.out_t[col][((2 * grp) ^ swz) * 16]) = c ? out_hi[0] : out_lo[0];
      *reinterpret_cast<uint4*>(&sm.out_t[col][((2 * grp + 1) ^ swz) * 16]) = c ? out_hi[1] : out_lo[1];
      const uint8_t sbyte = static_cast<uint8_t>((c ? e1 : e0) + 127);
      sm.st_lin[col][grp] = sbyte;
      sm.st_swz[sf_chunk_offset(col, grp)] = sbyte;
    }
  }
  __syncthreads();

  if (kGrouped) {
    // transposed codes: 128 feature rows x 128 token bytes at the group's padded position
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int row = it * 32 + (tid >> 3);
      const int ch = tid & 7;
      const int64_t gk = k0 + row;
      const int swz = (row >> 1) & 7;
      if (gk < a.cols)
        *reinterpret_cast<uint4*>(a.q_t + gk * a.out_cols + gt.z + ch * 16) =
            *reinterpret_cast<const uint4*>(&sm.out_t[row][(ch ^ swz) * 16]);
    }
    if (a.s_t != nullptr && tid < QT_COLS && k0 + tid < a.cols)
      *reinterpret_cast<uint32_t*>(a.s_t + (k0 + tid) * a.s_t_stride + (gt.z >> 5)) =
          *reinterpret_cast<const uint32_t*>(sm.st_lin[tid]);
    uint8_t* base = a.s_t_swz + ((k0 >> 7) * a.kc_col + (gt.z >> 7)) * 512;
    if (tid < 32) *reinterpret_cast<uint4*>(base + tid * 16) = *reinterpret_cast<const uint4*>(sm.st_swz + tid * 16);
    if (gt.w) {  // last tile along the token axis: zero the chunks up to the padded count
      const int64_t extra = a.kc_col - ((gt.z >> 7) + 1);
      for (int64_t i = tid; i < extra * 32; i += Q_THREADS)
        *reinterpret_cast<uint4*>(base + 512 + i * 16) = make_uint4(0, 0, 0, 0);
    }
    if (kGroupedRow && tid < gt.y) {
      // row-wise scales of this tile's rows: the tile starts anywhere inside a 128-row chunk of
      // the GEMM layout, so every row stores its own 4 bytes (one 16-byte cell quarter)
      const int64_t gr = m0 + tid;
      const int64_t kb0 = k0 >> 5;
      const int nvalid = (int)min((int64_t)4, (a.cols >> 5) - kb0);
      uint32_t word = *reinterpret_cast<const uint32_t*>(sm.s_lin[tid]);
      if (nvalid < 4) word &= (1u << (8 * nvalid)) - 1u;   // blocks beyond the tensor read as scale byte 0
      if (a.s != nullptr) {
        uint8_t* dst = a.s + gr * a.s_stride + kb0;
        if (nvalid == 4 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = word;
        else for (int i = 0; i < nvalid; ++i) dst[i] = sm.s_lin[tid][i];
      }
      uint8_t* cell = a.s_swz + ((gr >> 7) * a.kc_row + (k0 >> 7)) * 512 + (gr & 31) * 16 + ((gr >> 5) & 3) * 4;
      *reinterpret_cast<uint32_t*>(cell) = word;
      if (k0 + QT_COLS >= a.cols) {  // chunks up to the padded count along K
        const int64_t extra = a.kc_row - ((k0 >> 7) + 1);
        for (int64_t i = 1; i <= extra; ++i) *reinterpret_cast<uint32_t*>(cell + i * 512) = 0u;
      }
    }
    return;
  }
  if (tid < QT_ROWS) {
    const int64_t gr = m0 + tid;
    const int64_t kb0 = k0 >> 5;
    const int nvalid = (int)min((int64_t)4, (a.cols >> 5) - kb0);
    if (gr < a.rows) {
      uint8_t* dst = a.s + gr * a.s_stride + kb0;
      if (nvalid == 4 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0)
        *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(sm.s_lin[tid]);
      else
        for (int i = 0; i < nvalid; ++i) dst[i] = sm.s_lin[tid][i];
    }
  }
  if (a.s_swz != nullptr) {
    uint8_t* base = a.s_swz + ((m0 >> 7) * a.kc_row + (k0 >> 7)) * 512;
    if (tid < 32) *reinterpret_cast<uint4*>(base + tid * 16) = *reinterpret_cast<const uint4*>(sm.s_swz + tid * 16);
    if (k0 + QT_COLS >= a.cols) {
      const int64_t extra = a.kc_row - ((k0 >> 7) + 1);
      for (int64_t i = tid; i < extra * 32; i += Q_THREADS)
        *reinterpret_cast<uint4*>(base + 512 + i * 16) = make_uint4(0, 0, 0, 0);
    }
  }
  if (kTranspose) {
    // Transposed codes: 128 feature rows x 128 bytes (128 tokens), 8 chunks of 16 bytes.
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int row = it * 32 + (tid >> 3);
      const int ch = tid & 7;
      const int64_t gk = k0 + row;
      const int swz = (row >> 1) & 7;
      const uint4 val = *reinterpret_cast<const uint4*>(&sm.out_t[row][(ch ^ swz) * 16]);
      const int64_t byte0 = m0 + ch * 16;
      const int n = (int)max((int64_t)0, min((int64_t)16, a.rows - byte0));
      if (gk < a.cols && n > 0) {
        uint8_t* dst = a.q_t + gk * a.rows + byte0;
        if (n == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
          *reinterpret_cast<uint4*>(dst) = val;
        } else {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(&val);
          for (int i = 0; i < n; ++i) dst[i] = src[i];
        }
      }
    }
    if (tid < QT_COLS) {
      const int64_t gk = k0 + tid;
      const int64_t mb0 = m0 >> 5;
      const int nvalid = (int)min((int64_t)4, ((a.rows + 31) >> 5) - mb0);
      if (gk < a.cols) {
        uint8_t* dst = a.s_t + gk * a.s_t_stride + mb0;
        if (nvalid == 4 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0)
          *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(sm.st_lin[tid]);
        else
          for (int i = 0; i < nvalid; ++i) dst[i] = sm.st_lin[tid][i];
      }
    }
    if (a.s_t_swz != nullptr) {
      uint8_t* base = a.s_t_swz + ((k0 >> 7) * a.kc_col + (m0 >> 7)) * 512;
      if (tid < 32) *reinterpret_cast<uint4*>(base + tid * 16) = *reinterpret_cast<const uint4*>(sm.st_swz + tid * 16);
      if (m0 + QT_ROWS >= a.rows) {
        const int64_t extra = a.kc_col - ((m0 >> 7) + 1);
        for (int64_t i = tid; i < extra * 32; i += Q_THREADS)
          *reinterpret_cast<uint4*>(base + 512 + i * 16) = make_uint4(0, 0, 0, 0);
      }
    }
  }
}

static int64_t padded_chunks(int64_t k_blocks) { return ((k_blocks + 3) / 4 + 3) / 4 * 4; }

template <bool T, bool GRP = false, bool GRPROW = false>
static int launch_mxfp8(const CUtensorMap& map, const Mxfp8Args& args, dim3 grid, cudaStream_t st) {
  static bool attr_set[MT_MAX_DEVICES] = {};
  const int slot = current_device_slot();
  auto kern = quantize_mxfp8_kernel<T, GRP, GRPROW>;
  const int smem = (int)sizeof(Mxfp8Smem) + 128;
  if (!attr_set[slot]) {
    MT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[slot] = true;
  }
  MT_CUDA(launch_pdl(kern, grid, dim3(Q_THREADS), (size_t)smem, st, map, args));
  return MT_OK;
}

}  // namespace mt

extern "C" int mt_quantize_mxfp8(const void* x, int64_t rows, int64_t cols, uint8_t* q, uint8_t* s, int64_t s_stride,
                                 uint8_t* s_swz, uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                                 mt_stream_t stream) {
  using namespace mt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MT_REQUIRE(rows >= 0 && cols >= 0, "mt_quantize_mxfp8: negative shape");
  if (rows == 0 || cols == 0) return MT_OK;  // nothing to write; pointers may be null
  MT_REQUIRE(x && q && s, "mt_quantize_mxfp8: null x/q/s");
  MT_REQUIRE(cols % 32 == 0, "mt_quantize_mxfp8: cols (%lld) must be a multiple of 32", (long long)cols);
  MT_REQUIRE(aligned16(x) && aligned16(q), "mt_quantize_mxfp8: x and q must be 16-byte aligned");
  const bool transpose = q_t != nullptr;
  MT_REQUIRE(!transpose || s_t, "mt_quantize_mxfp8: q_t given without s_t");
  MT_REQUIRE(s_stride >= cols / 32 && (!transpose || s_t_stride >= (rows + 31) / 32), "mt_quantize_mxfp8: scale stride too small");
  MT_REQUIRE((!s_swz || aligned16(s_swz)) && (!s_t_swz || aligned16(s_t_swz)), "mt_quantize_mxfp8: swizzled scale buffers must be 16-byte aligned");
  if (rows == 0 || cols == 0) return MT_OK;

  Mxfp8Args args;
  args.rows = rows; args.cols = cols;
  args.s_stride = s_stride; args.s_t_stride = s_t_stride;
  args.kc_row = padded_chunks(cols / 32);
  args.kc_col = padded_chunks((rows + 31) / 32);
  args.q = q; args.s = s; args.s_swz = s_swz; args.q_t = q_t; args.s_t = s_t; args.s_t_swz = s_t_swz;
  args.status = device_status_ptr();
  if (!args.status) return fail(MT_ERR_CUDA, "device status word not reachable");
  CUtensorMap map;
  int rc = make_tensor_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)cols, (uint64_t)rows,
                              (uint64_t)cols * 2, QT_COLS, QT_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MT_OK) return rc;
  dim3 grid((unsigned)((cols + QT_COLS - 1) / QT_COLS), (unsigned)((rows + QT_ROWS - 1) / QT_ROWS));
  return transpose ? launch_mxfp8<true>(map, args, grid, st) : launch_mxfp8<false>(map, args, grid, st);
}


namespace mt {
// `plan` is the device buffer build_grouped_plan wrote for (rows, G); `padded_rows` is the padded
// token count the caller sized q_t with (every group rounded up to 128 tokens).
static int grouped_quantize_mxfp8(const char* name, const void* x, int64_t rows, int64_t cols, const void* plan,
                                  int64_t G, int64_t padded_rows, uint8_t* q, uint8_t* s, int64_t s_stride,
                                  uint8_t* s_swz, uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                                  cudaStream_t st) {
  MT_REQUIRE(G > 0 && G <= PLAN_MAX_GROUPS && rows >= 0 && rows <= PLAN_MAX_ROWS, "%s: bad group description", name);
  MT_REQUIRE(cols > 0 && cols % 32 == 0, "%s: cols (%lld) must be a positive multiple of 32", name, (long long)cols);
  MT_REQUIRE(padded_rows >= 0 && padded_rows % 128 == 0 && padded_rows <= rows + 127 * G,
             "%s: padded row count %lld is not a multiple of 128 within [0, rows + 127 G]", name, (long long)padded_rows);
  if (rows == 0 || padded_rows == 0) return MT_OK;
  const int64_t out_col = padded_rows;
  MT_REQUIRE(x && q_t && s_t_swz && plan, "%s: null pointer", name);
  MT_REQUIRE(aligned16(x) && aligned16(q_t) && aligned16(s_t_swz) && aligned16(plan), "%s: pointers must be 16-byte aligned", name);
  MT_REQUIRE(!s_t || (s_t_stride >= out_col / 32 && s_t_stride % 4 == 0), "%s: bad s_t stride", name);
  const PlanView pv = plan_view(const_cast<void*>(plan), rows, G);

  Mxfp8Args args{};
  args.rows = rows; args.cols = cols;
  args.s_t_stride = s_t_stride;
  args.kc_col = padded_chunks(out_col / 32);
  args.q_t = q_t; args.s_t = s_t; args.s_t_swz = s_t_swz;
  const bool row_too = q != nullptr;
  if (row_too) {
    MT_REQUIRE(s_swz && aligned16(q) && aligned16(s_swz), "%s: row-wise outputs need q and s_swz, 16-byte aligned", name);
    MT_REQUIRE(!s || s_stride >= cols / 32, "%s: bad s stride", name);
    args.q = q; args.s = s; args.s_swz = s_swz; args.s_stride = s_stride;
    args.kc_row = padded_chunks(cols / 32);
  }
  args.status = device_status_ptr();
  if (!args.status) return fail(MT_ERR_CUDA, "device status word not reachable");
  args.tiles = pv.qtiles;
  args.num_tiles_dev = &pv.header->n_qtiles;
  args.out_cols = out_col;
  CUtensorMap map;
  int rc = make_tensor_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)cols, (uint64_t)rows,
                              (uint64_t)cols * 2, QT_COLS, QT_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MT_OK) return rc;
  // one grid row per 128-token tile: the padded count bounds the number of tiles; rows of the grid
  // beyond the plan's tile count return at once
  dim3 grid((unsigned)((cols + QT_COLS - 1) / QT_COLS), (unsigned)(out_col / 128));
  return row_too ? launch_mxfp8<true, true, true>(map, args, grid, st) : launch_mxfp8<true, true>(map, args, grid, st);
}
}  // namespace mt

extern "C" int mt_grouped_transpose_quantize_mxfp8(const void* x, int64_t rows, int64_t cols, const void* plan, int64_t G,
                                                   int64_t padded_rows, uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride,
                                                   uint8_t* s_t_swz, mt_stream_t stream) {
  return mt::grouped_quantize_mxfp8("mt_grouped_transpose_quantize_mxfp8", x, rows, cols, plan, G, padded_rows, nullptr,
                                    nullptr, 0, nullptr, q_t, s_t, s_t_stride, s_t_swz,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int mt_grouped_quantize_mxfp8(const void* x, int64_t rows, int64_t cols, const void* plan, int64_t G,
                                         int64_t padded_rows, uint8_t* q, uint8_t* s, int64_t s_stride, uint8_t* s_swz,
                                         uint8_t* q_t, uint8_t* s_t, int64_t s_t_stride, uint8_t* s_t_swz,
                                         mt_stream_t stream) {
  MT_REQUIRE(q != nullptr, "mt_grouped_quantize_mxfp8: null q");
  return mt::grouped_quantize_mxfp8("mt_grouped_quantize_mxfp8", x, rows, cols, plan, G, padded_rows, q, s, s_stride,
                                    s_swz, q_t, s_t, s_t_stride, s_t_swz, static_cast<cudaStream_t>(stream));
}
