// Block-scaled GEMM for sm_100a: D[M,N] = alpha * (A . B^T) with FP4 (E2M1, E4M3 scale per
// 16) or FP8 (E4M3, E8M0 scale per 32) operands, both K-major, fp32 accumulation in tensor
// memory.
//
// Two persistent, warp-specialised kernels share the tile descriptions and the epilogue helpers:
//
// gemm_blockscaled_pair_kernel (the one that runs whenever M > 128 and N > 128): a cluster of
// two CTAs (cta_group::2, 320 threads each) per 256 x 256 output tile, described in the comment
// above it. It serves the dense GEMM, the grouped GEMMs (rows grouped by expert; per-expert
// contraction ranges for wgrad) and operands whose contraction dimension is split into slabs
// (the raw result of an all-gather of per-rank transposed shards).
//
// gemm_blockscaled_kernel (small shapes): one CTA per SM, 192 threads:
//   warp 0     TMA producer: per K step one 2-D tiled load each for the A and B tiles
//              (128-byte rows, 128-byte swizzle) and 1-D bulk copies of the scale-factor
//              chunks, all completing on the stage's "full" mbarrier;
//   warp 1     allocates tensor memory; one elected lane copies the scale factors
//              shared -> tensor memory (tcgen05.cp) and issues tcgen05.mma ... block_scale,
//              releasing each shared-memory stage with tcgen05.commit;
//   warps 2-5  epilogue: tcgen05.ld of the 128 x BLOCK_N fp32 accumulator (one 32-lane
//              quarter per warp), alpha / bias / accumulate, conversion, global stores.
// Every wait on an mbarrier is bounded; on expiry the CTA raises a bit in the device status
// word, abandons its remaining tiles, frees its tensor memory and exits.
//
// Grouped modes: a tile is described by (group, row block, column block) and the operand /
// output bases are looked up per group (TileCoord / PairTile).
#include <algorithm>
#include <climits>

#include "grouped_plan.cuh"
#include "mt_common.cuh"

namespace mt {

constexpr int G_BLOCK_M = 128;
constexpr int G_BLOCK_KB = 128;  // bytes of K per row per stage (256 FP4 or 128 FP8 elements)
constexpr int G_THREADS = 192;
constexpr int G_TMEM_COLS = 512;

enum GemmFormat : int { FMT_NVFP4 = 0, FMT_MXFP8 = 1 };
enum GemmMode : int { MODE_DENSE = 0, MODE_GROUPED_ROWS = 1, MODE_GROUPED_K = 2 };

struct GemmArgs {
  // operands
  const uint8_t* sa;   // A scale factors, chunk layout
  const uint8_t* sb;   // B scale factors, chunk layout
  int64_t kc_a, kc_b;  // chunks per 128-row block in sa / sb
  int64_t rb_a, rb_b;  // number of 128-row blocks available in sa / sb
  int64_t M, N, K_bytes;
  // output
  void* d;
  int64_t ldd;
  int d_dtype;
  const void* bias;
  int bias_dtype;
  int accumulate;
  const float* amax_a;
  const float* amax_b;
  int* status;
  // tiling
  int tiles_m, tiles_n, num_tiles;
  const int32_t* entries_dev;    // MODE_GROUPED_ROWS: device count of (row block, group) entries; the tile
                                 // count is *entries_dev * tiles_n (num_tiles is only its upper bound)
  // grouping
  int mode;
  int num_groups;
  const int64_t* group_offsets;  // device int64[G+1]: row offsets (MODE_GROUPED_ROWS, any values) or
                                 // contraction-element offsets (MODE_GROUPED_K, multiples of 128)
  const int32_t* tile_rb;        // MODE_GROUPED_ROWS: 128-row block of A / D handled by entry i
  const int32_t* tile_group;     // MODE_GROUPED_ROWS: group of entry i
  int64_t b_group_rows;          // MODE_GROUPED_ROWS: rows of B to skip per group
  int64_t b_group_k_bytes;       // MODE_GROUPED_ROWS: contraction bytes of B to skip per group
  int64_t d_group_stride;        // MODE_GROUPED_K: elements between consecutive group outputs
  int k_elems_per_byte_x2;       // 4 for FP4 (2 elements per byte), 2 for FP8
  int tma_store;                 // pair kernel: output goes through shared memory and TMA stores
  int direct_store;              // pair kernel: plain output rows go from registers to global memory in 32-byte pieces
  int64_t map_rows;              // rows of the output tensor map (all groups' matrices when stacked)
  float* d_amax;                 // optional: atomic max of |stored value| (pair kernel, no accumulation)
  int n_dest, my_rank;           // n_dest > 1 (pair kernel, dense, staged stores): output rows are scattered over
  int64_t dest_rows;             // the ranks' staging buffers, dest_rows rows each (PeerMaps), instead of d
#ifdef MT_TIMING_KNOBS
  int knobs;                     // builds with -DMT_TIMING_KNOBS only (results are wrong when set): bit 0 the
                                 // epilogue drains tensor memory but writes nothing, bit 1 scale factors are
                                 // copied for the first K step only, bit 2 B tiles are not loaded, bit 3 the
                                 // epilogue stages the output in shared memory but issues no TMA store,
                                 // bit 6 the accumulator is handed back unread
#endif
  int sm_margin;                 // host only: SMs the persistent grid leaves idle (room for a collective's
                                 // kernel that should run beside the GEMM instead of behind it)
  int band;                      // pair kernel: tile rows per band of the tile order (0 = row index fastest over all rows)
  // Pair kernel, operands split along K into slabs stored one after another (what an all-gather
  // of per-rank transposed shards produces): K step k of A lies in slab k / a_slab_steps, whose
  // rows start a_slab_rows further down the tensor map and whose scale chunks start
  // a_slab_chunks further down the chunk list. One slab spanning all K steps = plain layout.
  int a_slab_steps, b_slab_steps;
  int64_t a_slab_rows, b_slab_rows;
  int64_t a_slab_chunks, b_slab_chunks;
};

// Timing experiments exist only in builds with -DMT_TIMING_KNOBS (a separate library used for
// A/B measurements); the shipped library reads no tuning variable from the environment.
#ifdef MT_TIMING_KNOBS
// Phase timestamps of one epilogue warp (CTA 0, first epilogue warp), summed over its tiles:
// [0] tiles, [1] wait for the accumulator, [2] tensor-memory loads, [3] staging + stores, [4] whole tile.
__device__ unsigned long long g_epi_prof[8];
#define MT_PROF_T(var) const uint64_t var = global_timer_ns()
#define MT_PROF_C(var) const long long var = clock64()
#define MT_PROF_ADD(i, v) do { if (blockIdx.x == 0 && (threadIdx.x >> 5) == 2 && lane == 0) atomicAdd(&g_epi_prof[i], (unsigned long long)(v)); } while (0)
#define MT_KNOB(args, bit) (((args).knobs & (bit)) != 0)
static int env_knob(const char* name, int dflt) { const char* e = getenv(name); return e ? atoi(e) : dflt; }
#else
#define MT_PROF_T(var)
#define MT_PROF_C(var)
#define MT_PROF_ADD(i, v)
#define MT_KNOB(args, bit) false
static int env_knob(const char*, int dflt) { return dflt; }
#endif

template <int kFormat, int BLOCK_N, int STAGES, int ACC_STAGES>
struct GemmCfg {
  static constexpr int CH = (kFormat == FMT_NVFP4) ? 4 : 1;   // SF chunks per stage per 128 rows
  static constexpr int NH = BLOCK_N / 128;                    // 128-row halves of the B tile
  static constexpr int A_BYTES = G_BLOCK_M * G_BLOCK_KB;
  static constexpr int B_BYTES = BLOCK_N * G_BLOCK_KB;
  static constexpr int SFA_BYTES = CH * 512;
  static constexpr int SFB_BYTES = NH * CH * 512;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = STAGES * A_BYTES;
  static constexpr int OFF_SFA = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_SFB = OFF_SFA + STAGES * SFA_BYTES;
  static constexpr int OFF_BAR = OFF_SFB + STAGES * SFB_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 2 * ACC_STAGES;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 16;
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;  // slack for manual 1024-byte alignment
  static constexpr int TMEM_ACC = 0;
  static constexpr int TMEM_SFA = ACC_STAGES * BLOCK_N;
  static constexpr int TMEM_SFB = TMEM_SFA + 4 * CH;
  static_assert(TMEM_SFB + 4 * CH * NH <= G_TMEM_COLS, "tensor memory over-subscribed");
  static_assert(SMEM_ALLOC <= 227 * 1024, "shared memory over-subscribed");
};

__device__ __forceinline__ uint32_t make_idesc(int format, int block_n, int sf_id) {
  uint32_t d = 0;
  if (format == FMT_NVFP4) {
    d |= 1u << 7;   // A: E2M1
    d |= 1u << 10;  // B: E2M1
    // scale format UE4M3 = 0 at bit 23
  } else {
    // A, B: E4M3 = 0
    d |= 1u << 23;                             // scale format UE8M0
    d |= static_cast<uint32_t>(sf_id) << 4;    // B scale-factor byte inside the 32-bit column
    d |= static_cast<uint32_t>(sf_id) << 29;   // A scale-factor byte
  }
  d |= static_cast<uint32_t>(block_n >> 3) << 17;
  d |= static_cast<uint32_t>(G_BLOCK_M >> 4) << 24;
  return d;
}

template <int kFormat>
__device__ __forceinline__ void issue_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if (kFormat == FMT_NVFP4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

// Running abs-max of what a thread stores: bf16 outputs are tracked two per word with the packed
// bf16 instruction (sign bits are garbage until amax_finish strips them), fp32 outputs as fp32.
struct AmaxAcc {
  uint32_t packed = 0;
  float f = 0.0f;
};
__device__ __forceinline__ void amax_bf16x2(AmaxAcc& m, uint32_t w) {
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(m.packed) : "r"(m.packed), "r"(w));
}
__device__ __forceinline__ float amax_finish(const AmaxAcc& m) {
  const uint32_t p = m.packed & 0x7FFF7FFFu;
  return fmaxf(m.f, fmaxf(__uint_as_float(p << 16), __uint_as_float(p & 0xFFFF0000u)));
}
// Warp-wide maximum of the threads' abs-max values -> one atomic max on the fp32 scalar (values
// are non-negative, so their bit patterns order like unsigned integers).
__device__ __forceinline__ void amax_publish(float* d_amax, const AmaxAcc& m, int lane) {
  const uint32_t bits = __reduce_max_sync(0xffffffffu, __float_as_uint(amax_finish(m)));
  if (lane == 0 && bits != 0) atomicMax(reinterpret_cast<unsigned int*>(d_amax), bits);
}

__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// One thread's 32 consecutive fp32 accumulators of one output row -> alpha / bias /
// accumulate -> global memory (bf16 or fp32): whole 32-byte sectors per store when the row is
// 32-byte aligned, 16-byte stores when 16-byte aligned, scalar stores at ragged edges.
__device__ __forceinline__ void store_row_chunk(const GemmArgs& a, const uint32_t (&r)[32], float alpha, bool has_k,
                                                int64_t off, int64_t col0, AmaxAcc& am) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = has_k ? __fmul_rn(alpha, __uint_as_float(r[i])) : 0.0f;
  const int nvalid = (int)min((int64_t)32, a.N - col0);
  if (a.bias != nullptr) {
    for (int i = 0; i < nvalid; ++i)
      v[i] += (a.bias_dtype == MT_F32) ? static_cast<const float*>(a.bias)[col0 + i]
                                       : __bfloat162float(static_cast<const __nv_bfloat16*>(a.bias)[col0 + i]);
  }
  const bool track = a.d_amax != nullptr;
  if (a.d_dtype == MT_F32) {
    float* dst = static_cast<float*>(a.d) + off;
    if (track)
      for (int i = 0; i < nvalid; ++i) am.f = fmaxf(am.f, fabsf(v[i]));
    if (nvalid == 32 && !a.accumulate && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = __float_as_uint(v[8 * i + j]);
        st_global_v8(dst + 8 * i, w);
      }
    } else if (nvalid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        if (a.accumulate) { float4 p = d4[i]; o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w; }
        d4[i] = o;
      }
    } else {
      for (int i = 0; i < nvalid; ++i) dst[i] = a.accumulate ? dst[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.d) + off;
    if (nvalid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      const uint4* s4 = reinterpret_cast<const uint4*>(dst);
      uint32_t ow[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (a.accumulate) {
          uint4 p = s4[i];
          const uint32_t pw[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[8 * i + 2 * j] += __uint_as_float(pw[j] << 16);
            v[8 * i + 2 * j + 1] += __uint_as_float(pw[j] & 0xFFFF0000u);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
          ow[4 * i + j] = *reinterpret_cast<uint32_t*>(&h);
          if (track) amax_bf16x2(am, ow[4 * i + j]);
        }
      }
      if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t w[8] = {ow[8 * i], ow[8 * i + 1], ow[8 * i + 2], ow[8 * i + 3],
                                 ow[8 * i + 4], ow[8 * i + 5], ow[8 * i + 6], ow[8 * i + 7]};
          st_global_v8(dst + 16 * i, w);
        }
      } else {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int i = 0; i < 4; ++i) d4[i] = make_uint4(ow[4 * i], ow[4 * i + 1], ow[4 * i + 2], ow[4 * i + 3]);
      }
    } else {
      for (int i = 0; i < nvalid; ++i) {
        float o = a.accumulate ? __bfloat162float(dst[i]) + v[i] : v[i];
        const __nv_bfloat16 h = __float2bfloat16_rn(o);
        if (track) am.f = fmaxf(am.f, fabsf(__bfloat162float(h)));
        dst[i] = h;
      }
    }
  }
}

__device__ __forceinline__ float bias_at(const GemmArgs& a, int64_t col) {
  return (a.bias_dtype == MT_F32) ? static_cast<const float*>(a.bias)[col]
                                  : __bfloat162float(static_cast<const __nv_bfloat16*>(a.bias)[col]);
}

// One warp's 32 rows x `ncols` (<= 128) accumulator block, already in registers (acc[c][i] =
// column 32c + i of this lane's row), -> alpha / bias -> bf16 or fp32 -> shared memory -> TMA
// store (or TMA add-reduction for fp32 accumulation). The warp's 4 KiB buffer is used as two
// 2 KiB halves of 32 rows x 64 bytes (64-byte swizzle) in alternation: filling one half overlaps
// the TMA engine reading the other. 32 (bf16) or 16 (fp32) columns per store. `row0` / `colw`
// are the block's first row / column in the tensor map's coordinates; rows and columns beyond
// the map's bounds are clipped by the hardware.
__device__ __forceinline__ void store_block_staged(const GemmArgs& a, const CUtensorMap* map_d,
                                                        const uint32_t (&acc)[4][32], int ncols, uint8_t* stage,
                                                        int lane, int64_t row0, int64_t map_rows, int64_t colw,
                                                        float alpha, bool has_k, AmaxAcc& am) {
  const bool track = a.d_amax != nullptr;
  const uint32_t swz = (lane >> 1) & 3;
  const bool f32 = a.d_dtype == MT_F32;
  const int cols_per = f32 ? 16 : 32;
  const int nchunks = ncols / cols_per;
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    if (ch >= nchunks) break;
    uint8_t* buf = stage + (ch & 1) * 2048;
    if (lane == 0) bulk_wait_read_all_but_one();   // the store issued two chunks ago has drained this half
    __syncwarp();
    if (!f32) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {               // 16-byte piece j = columns 8j .. 8j+7 of the chunk
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int col = (ch & 3) * 32 + j * 8 + t * 2;
          float v0 = has_k ? __fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31])) : 0.0f;
          float v1 = has_k ? __fmul_rn(alpha, __uint_as_float(acc[(col + 1) >> 5][(col + 1) & 31])) : 0.0f;
          if (a.bias != nullptr) {
            const int64_t gc = colw + col;
            if (gc < a.N) v0 += bias_at(a, gc);
            if (gc + 1 < a.N) v1 += bias_at(a, gc + 1);
          }
          __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
          w[t] = *reinterpret_cast<uint32_t*>(&h);
          if (track) amax_bf16x2(am, w[t]);
        }
        *reinterpret_cast<uint4*>(buf + lane * 64 + ((j ^ swz) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {               // 16-byte piece j = columns 4j .. 4j+3 of the chunk
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int col = ch * 16 + j * 4 + t;
          v[t] = has_k ? __fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31])) : 0.0f;
          if (a.bias != nullptr) {
            const int64_t gc = colw + col;
            if (gc < a.N) v[t] += bias_at(a, gc);
          }
          if (track) am.f = fmaxf(am.f, fabsf(v[t]));
        }
        *reinterpret_cast<float4*>(buf + lane * 64 + ((j ^ swz) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    const int64_t c0 = colw + (int64_t)ch * cols_per;
    if (lane == 0) {
      if (row0 < map_rows && c0 < a.N && !MT_KNOB(a, 8)) {
        if (f32 && a.accumulate) tma_reduce_add_2d(map_d, buf, (int32_t)c0, (int32_t)row0);
        else tma_store_2d(map_d, buf, (int32_t)c0, (int32_t)row0);
      }
      // one group per chunk, empty when the chunk lies outside the output: the "all but one"
      // wait above counts groups, so the two halves must keep alternating group by group
      bulk_commit_group();
    }
  }
}

// The same with 128-byte rows: 32 rows x 128 bytes per store (64 bf16 or 32 fp32 columns, 128-byte
// swizzle, the warp's whole 4 KiB buffer). Whole 128-byte lines per row measured 2 - 3 % faster
// than the 64-byte halves for local outputs and are what stores across NVLink need; the buffer is
// refilled once the previous store has read it. Used for every staged output (local or a peer's
// staging buffer); fp32 accumulation goes through the TMA add-reduction.
__device__ __forceinline__ void store_block_staged_wide(const GemmArgs& a, const CUtensorMap* map_d,
                                                        const uint32_t (&acc)[4][32], int ncols, uint8_t* stage,
                                                        int lane, int64_t row0, int64_t map_rows, int64_t colw,
                                                        float alpha, bool has_k, AmaxAcc& am) {
  const uint32_t swz = lane & 7;
  const bool f32 = a.d_dtype == MT_F32;
  const bool track = a.d_amax != nullptr;
  const bool plain = has_k && a.bias == nullptr && !track;
  const int cols_per = f32 ? 32 : 64;
  const int nchunks = ncols / cols_per;
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    if (ch >= nchunks) break;
    MT_PROF_C(pc0);
    if (lane == 0) bulk_wait_read_all();
    __syncwarp();
    MT_PROF_C(pc1);
    if (plain && !f32) {
      // the common case (no bias, no abs-max, K > 0) free of per-element branches: two multiplies
      // and one packing conversion per pair of columns
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int col = (ch & 1) * 64 + j * 8 + t * 2;
          const __nv_bfloat162 h = __floats2bfloat162_rn(__fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31])),
                                                         __fmul_rn(alpha, __uint_as_float(acc[(col + 1) >> 5][(col + 1) & 31])));
          w[t] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ swz) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else if (plain) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int col = ch * 32 + j * 4 + t;
          v[t] = __fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31]));
        }
        *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ swz) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
      }
    } else if (!f32) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {               // 16-byte piece j = columns 8j .. 8j+7 of the chunk
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int col = (ch & 1) * 64 + j * 8 + t * 2;
          float v0 = has_k ? __fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31])) : 0.0f;
          float v1 = has_k ? __fmul_rn(alpha, __uint_as_float(acc[(col + 1) >> 5][(col + 1) & 31])) : 0.0f;
          if (a.bias != nullptr) {
            const int64_t gc = colw + col;
            if (gc < a.N) v0 += bias_at(a, gc);
            if (gc + 1 < a.N) v1 += bias_at(a, gc + 1);
          }
          __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
          w[t] = *reinterpret_cast<uint32_t*>(&h);
          if (track) amax_bf16x2(am, w[t]);
        }
        *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ swz) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {               // 16-byte piece j = columns 4j .. 4j+3 of the chunk
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int col = ch * 32 + j * 4 + t;
          v[t] = has_k ? __fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31])) : 0.0f;
          if (a.bias != nullptr) {
            const int64_t gc = colw + col;
            if (gc < a.N) v[t] += bias_at(a, gc);
          }
          if (track) am.f = fmaxf(am.f, fabsf(v[t]));
        }
        *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ swz) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    MT_PROF_C(pc2);
    fence_proxy_async_smem();
    __syncwarp();
    const int64_t c0 = colw + (int64_t)ch * cols_per;
    if (lane == 0) {
      if (row0 < map_rows && c0 < a.N && !MT_KNOB(a, 8)) {
        if (f32 && a.accumulate) tma_reduce_add_2d(map_d, stage, (int32_t)c0, (int32_t)row0);
        else tma_store_2d(map_d, stage, (int32_t)c0, (int32_t)row0);
      }
      bulk_commit_group();
    }
    MT_PROF_C(pc3);
    MT_PROF_ADD(5, pc1 - pc0); MT_PROF_ADD(6, pc2 - pc1); MT_PROF_ADD(7, pc3 - pc2);
  }
}

struct TileCoord {
  int64_t a_row0;      // first row of the A tile (TMA y coordinate)
  int64_t b_row0;      // first row of the B tile
  int64_t a_k_byte0;   // first contraction byte (TMA x coordinate) in A
  int64_t b_k_byte0;   // first contraction byte in B
  int num_k;           // K steps of 128 bytes
  int64_t sfa_rb;      // 128-row block index into sa
  int64_t sfb_rb;      // 128-row block index into sb (first half)
  int64_t sfa_kc0;     // first chunk index along K in sa
  int64_t sfb_kc0;     // first chunk index along K in sb
  int64_t d_row0;      // output row of accumulator row 0
  int64_t d_row_lo;    // rows outside [d_row_lo, d_row_hi) are not stored
  int64_t d_row_hi;
  int64_t d_col0;      // first output column
  int64_t d_base;      // element offset of the group's output matrix
};

template <int kFormat, int BLOCK_N>
__device__ __forceinline__ TileCoord tile_coord(const GemmArgs& a, int tile) {
  constexpr int CH = (kFormat == FMT_NVFP4) ? 4 : 1;
  TileCoord t;
  t.a_k_byte0 = t.b_k_byte0 = 0;
  t.num_k = (int)((a.K_bytes + G_BLOCK_KB - 1) / G_BLOCK_KB);
  t.sfa_kc0 = t.sfb_kc0 = 0;
  t.d_base = 0;
  if (a.mode == MODE_DENSE) {
    const int nb = tile / a.tiles_m, mb = tile - nb * a.tiles_m;
    t.a_row0 = (int64_t)mb * G_BLOCK_M;
    t.b_row0 = (int64_t)nb * BLOCK_N;
    t.d_row0 = t.a_row0;
    t.d_row_lo = 0;
    t.d_row_hi = a.M;
    t.d_col0 = t.b_row0;
  } else if (a.mode == MODE_GROUPED_ROWS) {
    // entries (row block, group) for every group that owns rows of the block; column block fastest
    const int e = tile / a.tiles_n, nb = tile - e * a.tiles_n;
    const int g = a.tile_group[e];
    t.a_row0 = (int64_t)a.tile_rb[e] * G_BLOCK_M;
    t.b_row0 = (int64_t)g * a.b_group_rows + (int64_t)nb * BLOCK_N;
    t.b_k_byte0 = (int64_t)g * a.b_group_k_bytes;
    t.sfb_kc0 = t.b_k_byte0 / G_BLOCK_KB * CH;
    t.d_row0 = t.a_row0;
    t.d_row_lo = a.group_offsets[g];
    t.d_row_hi = a.group_offsets[g + 1];
    t.d_col0 = (int64_t)nb * BLOCK_N;
  } else {
    // MODE_GROUPED_K: tile = (g * tiles_n + nb) * tiles_m + mb; group g contracts over its own
    // (padded) range of the shared contraction dimension and writes its own output matrix
    const int per_group = a.tiles_m * a.tiles_n;
    const int g = tile / per_group;
    const int r = tile - g * per_group;
    const int nb = r / a.tiles_m, mb = r - nb * a.tiles_m;
    const int64_t e0 = a.group_offsets[g], e1 = a.group_offsets[g + 1];
    t.a_row0 = (int64_t)mb * G_BLOCK_M;
    t.b_row0 = (int64_t)nb * BLOCK_N;
    t.a_k_byte0 = t.b_k_byte0 = e0 * 2 / a.k_elems_per_byte_x2;
    t.num_k = (int)(((e1 - e0) * 2 / a.k_elems_per_byte_x2 + G_BLOCK_KB - 1) / G_BLOCK_KB);
    t.sfa_kc0 = t.sfb_kc0 = t.a_k_byte0 / G_BLOCK_KB * CH;
    t.d_row0 = t.a_row0;
    t.d_row_lo = 0;
    t.d_row_hi = a.M;
    t.d_col0 = t.b_row0;
    t.d_base = (int64_t)g * a.d_group_stride;
  }
  t.sfa_rb = t.a_row0 / 128;
  t.sfb_rb = t.b_row0 / 128;
  return t;
}

template <int kFormat, int BLOCK_N, int STAGES, int ACC_STAGES>
__global__ void __launch_bounds__(G_THREADS, 1) gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                        const __grid_constant__ CUtensorMap map_b,
                                                                        const GemmArgs a) {
  using Cfg = GemmCfg<kFormat, BLOCK_N, STAGES, ACC_STAGES>;
  constexpr int CH = Cfg::CH, NH = Cfg::NH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = a.entries_dev ? min(a.num_tiles, *a.entries_dev * a.tiles_n) : a.num_tiles;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < ACC_STAGES; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, G_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ================= TMA producer =================
    if (elect_one()) {
      uint32_t it = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        const TileCoord t = tile_coord<kFormat, BLOCK_N>(a, tile);
        for (int k = 0; k < t.num_k; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag, a.status, DS_EMPTY_WAIT)) { alive = false; break; }
          uint32_t bytes = Cfg::A_BYTES + Cfg::B_BYTES + Cfg::SFA_BYTES;
          int nh_valid = 0;
#pragma unroll
          for (int h = 0; h < NH; ++h) nh_valid += (t.sfb_rb + h < a.rb_b) ? 1 : 0;
          bytes += nh_valid * CH * 512;
          mbar_expect_tx(&full_bar[s], bytes);
          tma_load_2d(smem + Cfg::OFF_A + s * Cfg::A_BYTES, &map_a, &full_bar[s],
                      (int32_t)(t.a_k_byte0 + (int64_t)k * G_BLOCK_KB), (int32_t)t.a_row0);
          tma_load_2d(smem + Cfg::OFF_B + s * Cfg::B_BYTES, &map_b, &full_bar[s],
                      (int32_t)(t.b_k_byte0 + (int64_t)k * G_BLOCK_KB), (int32_t)t.b_row0);
          bulk_load_1d(smem + Cfg::OFF_SFA + s * Cfg::SFA_BYTES,
                       a.sa + (t.sfa_rb * a.kc_a + t.sfa_kc0 + (int64_t)k * CH) * 512, CH * 512, &full_bar[s]);
          const int64_t kc = t.sfb_kc0 + (int64_t)k * CH;
#pragma unroll
          for (int h = 0; h < NH; ++h) {
            if (t.sfb_rb + h < a.rb_b)
              bulk_load_1d(smem + Cfg::OFF_SFB + s * Cfg::SFB_BYTES + h * CH * 512,
                           a.sb + ((t.sfb_rb + h) * a.kc_b + kc) * 512, CH * 512, &full_bar[s]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool alive = true;
      const uint32_t a_base = smem_u32(smem + Cfg::OFF_A), b_base = smem_u32(smem + Cfg::OFF_B);
      const uint32_t sfa_base = smem_u32(smem + Cfg::OFF_SFA), sfb_base = smem_u32(smem + Cfg::OFF_SFB);
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++tile_it) {
        const TileCoord t = tile_coord<kFormat, BLOCK_N>(a, tile);
        const int as = tile_it % ACC_STAGES;
        const uint32_t aph = (tile_it / ACC_STAGES) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aph ^ 1, abort_flag, a.status, DS_ACC_EMPTY_WAIT)) { alive = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + Cfg::TMEM_ACC + as * BLOCK_N;
        for (int k = 0; k < t.num_k; ++k, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, a.status, DS_TMA_WAIT)) { alive = false; break; }
          tc_fence_after();
          // scale factors: shared -> tensor memory
#pragma unroll
          for (int c = 0; c < CH; ++c)
            tc_copy_sf(tmem_base + Cfg::TMEM_SFA + 4 * c, umma_desc_sf(sfa_base + s * Cfg::SFA_BYTES + c * 512));
#pragma unroll
          for (int h = 0; h < NH; ++h)
#pragma unroll
            for (int c = 0; c < CH; ++c)
              tc_copy_sf(tmem_base + Cfg::TMEM_SFB + 4 * (c * NH + h),
                         umma_desc_sf(sfb_base + s * Cfg::SFB_BYTES + (h * CH + c) * 512));
          const uint64_t adesc = umma_desc_sw128(a_base + s * Cfg::A_BYTES);
          const uint64_t bdesc = umma_desc_sw128(b_base + s * Cfg::B_BYTES);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t idesc = make_idesc(kFormat, BLOCK_N, j);
            const uint32_t sfa_t = tmem_base + Cfg::TMEM_SFA + (kFormat == FMT_NVFP4 ? 4 * j : 0);
            const uint32_t sfb_t = tmem_base + Cfg::TMEM_SFB + (kFormat == FMT_NVFP4 ? 4 * NH * j : 0);
            issue_mma<kFormat>(tmem_d, adesc + 2 * j, bdesc + 2 * j, idesc, sfa_t, sfb_t, (k > 0 || j > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);
        }
        if (alive) tc_commit(&acc_full[as]);
      }
    }
    __syncwarp();
  } else {
    // ================= epilogue =================
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    float alpha = 1.0f;
    if (a.amax_a != nullptr && a.amax_b != nullptr)
      alpha = __fdiv_rn(__fmul_rn(*a.amax_a, *a.amax_b), 6.0f * 6.0f * 448.0f * 448.0f);
    uint32_t tile_it = 0;
    bool alive = true;
    AmaxAcc am;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++tile_it) {
      const TileCoord t = tile_coord<kFormat, BLOCK_N>(a, tile);
      const int as = tile_it % ACC_STAGES;
      const uint32_t aph = (tile_it / ACC_STAGES) & 1;
      if (!mbar_wait_bounded(&acc_full[as], aph, abort_flag, a.status, DS_ACC_FULL_WAIT)) { alive = false; break; }
      tc_fence_after();
      const int64_t row = t.d_row0 + q * 32 + lane;
      const bool row_ok = row >= t.d_row_lo && row < t.d_row_hi;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        tc_ld_32x32(tmem_base + Cfg::TMEM_ACC + as * BLOCK_N + (static_cast<uint32_t>(q * 32) << 16) + c * 32, r);
        tc_wait_ld();
        const int64_t col0 = t.d_col0 + c * 32;
        if (row_ok && col0 < a.N) store_row_chunk(a, r, alpha, t.num_k > 0, t.d_base + row * a.ldd + col0, col0, am);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
    }
    if (a.d_amax != nullptr) amax_publish(a.d_amax, am, lane);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, G_TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------
// CTA-pair kernel (cta_group::2): a cluster of two CTAs computes a 256 x BN output tile,
// BN = 256 (one accumulator) or 192 (two accumulators: the epilogue of a tile overlaps the
// MMAs of the next one; 2 * 192 accumulator columns + 48 scale-factor columns fit the 512
// columns of tensor memory).
// CTA r of the pair owns rows [128 r, 128 r + 128) of the tile (its A rows, its half of the
// accumulator in its own tensor memory) and loads rows [r * BN/2, +BN/2) of the B tile; the
// tensor cores of both SMs read both halves of B, so each byte of B is fetched from L2 and
// written to shared memory once per pair. Scale factors: each CTA loads the A scales of its
// own rows and the B scales of the two 128-row chunks the tile's columns touch (a 192-wide
// tile starts 0 or 64 rows into a chunk: the MMA is pointed 0 or 2 tensor-memory columns
// into the copied chunks). The leader (rank 0) waits on one "full" barrier that both CTAs' TMA
// loads signal, copies scale factors and issues the MMAs for both SMs; tcgen05.commit signals
// the "empty" and "accumulator full" barriers in both CTAs. No load is multicast.
// ------------------------------------------------------------------------------------------
constexpr int P_EPI_WARPS = 8;                       // two warps per tensor-memory lane quarter
constexpr int P_THREADS = 64 + 32 * P_EPI_WARPS;     // producer warp + MMA warp + epilogue warps

template <int kFormat, int BN, int STAGES>
struct PairCfg {
  static_assert(BN == 256 || BN == 192, "pair tile width");
  static constexpr int CH = (kFormat == FMT_NVFP4) ? 4 : 1;
  static constexpr int ACC = (BN == 256) ? 1 : 2;              // accumulator buffers
  static constexpr int NSB = 2;                                // 128-row B scale chunks per tile
  static constexpr int A_BYTES = G_BLOCK_M * G_BLOCK_KB;       // 128 rows of A
  static constexpr int B_BYTES = (BN / 2) * G_BLOCK_KB;        // this CTA's rows of B
  static constexpr int SFA_BYTES = CH * 512;
  static constexpr int SFB_BYTES = NSB * CH * 512;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = STAGES * A_BYTES;
  static constexpr int OFF_SFA = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_SFB = OFF_SFA + STAGES * SFA_BYTES;
  // one 4 KiB output staging buffer per epilogue warp: 32 rows x 128 bytes (a second buffer per
  // warp would cost a pipeline stage, which measured slower); 1024-byte aligned so the swizzle
  // pattern of the TMA store lines up with the row index used when filling it
  static constexpr int OFF_EPI = (OFF_SFB + STAGES * SFB_BYTES + 1023) / 1024 * 1024;
  static constexpr int EPI_BYTES = P_EPI_WARPS * 4096;
  static constexpr int OFF_BAR = OFF_EPI + EPI_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 2 * ACC;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 16;
  static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
  static constexpr int TMEM_ACC = 0;
  static constexpr int TMEM_SFA = ACC * BN;
  static constexpr int TMEM_SFB = TMEM_SFA + 4 * CH;
  static_assert(B_BYTES % 1024 == 0, "B stage must keep the 1024-byte swizzle alignment");
  static_assert(TMEM_SFB + 4 * NSB * CH <= G_TMEM_COLS, "tensor memory over-subscribed");
  static_assert(SMEM_ALLOC <= 227 * 1024, "shared memory over-subscribed");
};

template <int kFormat>
__device__ __forceinline__ void issue_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  if (kFormat == FMT_NVFP4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

__device__ __forceinline__ uint32_t make_idesc_pair(int format, int block_n, int sf_id) {
  uint32_t d = 0;
  if (format == FMT_NVFP4) {
    d |= 1u << 7;
    d |= 1u << 10;
  } else {
    d |= 1u << 23;
    d |= static_cast<uint32_t>(sf_id) << 4;
    d |= static_cast<uint32_t>(sf_id) << 29;
  }
  d |= static_cast<uint32_t>(block_n >> 3) << 17;
  d |= static_cast<uint32_t>(256 >> 4) << 24;  // M = 256 across the pair
  return d;
}

// Tile order of the pair kernel. band < 0: column index fastest (CTAs that run together share
// the A tile and sweep B); band == 0: row index fastest; band > 0: bands of `band` tile rows,
// row index fastest inside a band.
__device__ __forceinline__ void pair_tile_coord(const GemmArgs& a, int tile, int& mb, int& nb) {
  if (a.band == 0) {
    nb = tile / a.tiles_m;
    mb = tile - nb * a.tiles_m;
    return;
  }
  if (a.band < 0) {
    mb = tile / a.tiles_n;
    nb = tile - mb * a.tiles_n;
    return;
  }
  const int per_band = a.band * a.tiles_n;
  const int b = tile / per_band;
  const int r = tile - b * per_band;
  const int rows = min(a.band, a.tiles_m - b * a.band);
  nb = r / rows;
  mb = b * a.band + (r - nb * rows);
}

// Tile of the pair kernel in every mode: the TileCoord fields (a_row0 = first of the tile's 256
// rows) plus the row of accumulator row 0 in the output tensor map (grouped-K outputs are one
// map over all groups' matrices stacked along rows) and whether d_row_hi coincides with the
// map's last row, so that the map's own clipping may stand in for the row-range test.
struct PairTile : TileCoord {
  int64_t d_map_row0;
  bool hi_is_end;
};

template <int kFormat, int BN>
__device__ __forceinline__ PairTile pair_tile(const GemmArgs& a, int tile) {
  constexpr int CH = (kFormat == FMT_NVFP4) ? 4 : 1;
  PairTile t;
  t.a_k_byte0 = t.b_k_byte0 = 0;
  t.num_k = (int)((a.K_bytes + G_BLOCK_KB - 1) / G_BLOCK_KB);
  t.sfa_kc0 = t.sfb_kc0 = 0;
  t.d_base = 0;
  if (a.mode == MODE_DENSE) {
    int mb, nb;
    pair_tile_coord(a, tile, mb, nb);
    // Scattered output: consecutive row blocks go to different destinations, starting with the
    // rank after this one and ending with its own, so that a rank's stores are spread evenly over
    // its links for the whole run of the kernel and no destination is written by every rank at
    // once (all ranks walking the rows in the same order would do exactly that).
    if (a.n_dest > 1) {
      const int per_dest = a.tiles_m / a.n_dest;
      const int dest = (a.my_rank + 1 + mb % a.n_dest) % a.n_dest;
      mb = dest * per_dest + mb / a.n_dest;
    }
    t.a_row0 = (int64_t)mb * 256;
    t.b_row0 = (int64_t)nb * BN;
    t.d_row_lo = 0;
    t.d_row_hi = a.M;
    t.d_map_row0 = t.a_row0;
    t.hi_is_end = true;
  } else if (a.mode == MODE_GROUPED_ROWS) {
    // entries (256-row block, group), column block fastest: pairs that run together share A
    const int e = tile / a.tiles_n, nb = tile - e * a.tiles_n;
    const int g = a.tile_group[e];
    t.a_row0 = (int64_t)a.tile_rb[e] * 256;
    t.b_row0 = (int64_t)g * a.b_group_rows + (int64_t)nb * BN;
    t.b_k_byte0 = (int64_t)g * a.b_group_k_bytes;
    t.sfb_kc0 = t.b_k_byte0 / G_BLOCK_KB * CH;
    t.d_row_lo = a.group_offsets[g];
    t.d_row_hi = a.group_offsets[g + 1];
    t.d_col0 = (int64_t)nb * BN;
    t.d_map_row0 = t.a_row0;
    t.hi_is_end = t.d_row_hi == a.M;
  } else {
    const int per_group = a.tiles_m * a.tiles_n;
    const int g = tile / per_group;
    const int r = tile - g * per_group;
    const int mb = r / a.tiles_n, nb = r - mb * a.tiles_n;
    const int64_t e0 = a.group_offsets[g], e1 = a.group_offsets[g + 1];
    t.a_row0 = (int64_t)mb * 256;
    t.b_row0 = (int64_t)nb * BN;
    t.a_k_byte0 = t.b_k_byte0 = e0 * 2 / a.k_elems_per_byte_x2;
    t.num_k = (int)(((e1 - e0) * 2 / a.k_elems_per_byte_x2 + G_BLOCK_KB - 1) / G_BLOCK_KB);
    t.sfa_kc0 = t.sfb_kc0 = t.a_k_byte0 / G_BLOCK_KB * CH;
    t.d_row_lo = 0;
    t.d_row_hi = a.M;
    t.d_base = (int64_t)g * a.d_group_stride;
    t.d_map_row0 = (int64_t)g * a.M + t.a_row0;
    t.hi_is_end = g == a.num_groups - 1;
  }
  if (a.mode != MODE_GROUPED_ROWS) t.d_col0 = t.b_row0;
  t.d_row0 = t.a_row0;
  t.sfa_rb = t.a_row0 / 128;
  t.sfb_rb = t.b_row0 / 128;
  return t;
}

// Output tensor maps of a scattering GEMM: one per destination rank, identical geometry
// ([n_dest * dest_rows, N] bf16), different base address.
struct alignas(64) PeerMaps {
  CUtensorMap m[MT_MAX_PEERS];
};

template <int kFormat, int BN, int STAGES>
// Register budget: 10 warps land 3 + 3 + 2 + 2 on the four SM sub-partitions of 16384 registers
// each, so 168 per thread is the most that launches (more fails with "too many resources").
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
    gemm_blockscaled_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                 const __grid_constant__ CUtensorMap map_sfa,
                                 const __grid_constant__ CUtensorMap map_sfb,
                                 const __grid_constant__ CUtensorMap map_d, const __grid_constant__ PeerMaps maps_peer,
                                 const GemmArgs a) {
  using Cfg = PairCfg<kFormat, BN, STAGES>;
  constexpr int CH = Cfg::CH, ACC = Cfg::ACC, NSB = Cfg::NSB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* full_bar = bars;                        // used in the leader only (both CTAs' loads signal it)
  uint64_t* empty_bar = bars + STAGES;              // one set per CTA, signalled by the leader's commit
  uint64_t* acc_full = bars + 2 * STAGES;           // per CTA and accumulator, signalled by the leader's commit
  uint64_t* acc_empty = bars + 2 * STAGES + ACC;    // leader only: 2 x P_EPI_WARPS arrivals each
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  // Everything up to pdl_wait() touches shared memory, tensor memory and kernel parameters only:
  // it may run while the kernel before this one in the stream is finishing.
  pdl_trigger();
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < ACC; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 2 * P_EPI_WARPS); }
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_sfa);
    prefetch_tensormap(&map_sfb);
    if (a.tma_store) prefetch_tensormap(&map_d);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, G_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers must exist before either CTA signals the other
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  const int num_tiles = a.entries_dev ? min(a.num_tiles, *a.entries_dev * a.tiles_n) : a.num_tiles;

  if (warp == 0) {
    // ================= TMA producer (one per CTA) =================
    if (elect_one()) {
      uint32_t it = 0, ph = 0;
      int s = 0;
      bool alive = true;
      for (int tile = pair; tile < num_tiles && alive; tile += num_pairs) {
        const PairTile t = pair_tile<kFormat, BN>(a, tile);
        const int32_t a_row = (int32_t)t.a_row0 + (int)rank * 128;
        const int32_t b_row = (int32_t)t.b_row0 + (int)rank * (BN / 2);
        const int32_t sfa_chunk0 = (int32_t)((t.sfa_rb + (int)rank) * a.kc_a + t.sfa_kc0);
        const int64_t sfb_rb0 = t.sfb_rb;   // first 128-row chunk of B scales the tile touches
        const int32_t sfb_kc0 = (int32_t)t.sfb_kc0;
        const int32_t a_kx0 = (int32_t)t.a_k_byte0, b_kx0 = (int32_t)t.b_k_byte0;
        const int num_k = t.num_k;
        // slab of each operand the K step falls in and the step inside the slab, kept as counters
        // (this single thread issues every load of the CTA: no divisions in its loop)
        int sl_a = 0, ka = 0, sl_b = 0, kb = 0;
        for (int k = 0; k < num_k; ++k, ++it) {
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag, a.status, DS_EMPTY_WAIT)) { alive = false; break; }
          const bool skip_b = MT_KNOB(a, 4);
          if (leader) mbar_expect_tx(&full_bar[s], 2 * (Cfg::STAGE_BYTES - (skip_b ? Cfg::B_BYTES : 0)));
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
          tma_load_2d_pair(smem + Cfg::OFF_A + s * Cfg::A_BYTES, &map_a, bar, a_kx0 + ka * G_BLOCK_KB,
                           a_row + (int32_t)(sl_a * a.a_slab_rows));
          if (!skip_b)
            tma_load_2d_pair(smem + Cfg::OFF_B + s * Cfg::B_BYTES, &map_b, bar, b_kx0 + kb * G_BLOCK_KB,
                             b_row + (int32_t)(sl_b * a.b_slab_rows));
          tma_load_2d_pair(smem + Cfg::OFF_SFA + s * Cfg::SFA_BYTES, &map_sfa, bar, 0,
                           sfa_chunk0 + (int32_t)(sl_a * a.a_slab_chunks) + ka * CH);
#pragma unroll
          for (int h = 0; h < NSB; ++h)
            tma_load_2d_pair(smem + Cfg::OFF_SFB + s * Cfg::SFB_BYTES + h * CH * 512, &map_sfb, bar, 0,
                             (int32_t)((sfb_rb0 + h) * a.kc_b + sl_b * a.b_slab_chunks) + sfb_kc0 + kb * CH);
          if (++ka == a.a_slab_steps) { ka = 0; ++sl_a; }
          if (++kb == a.b_slab_steps) { kb = 0; ++sl_b; }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer (leader CTA only) =================
    if (leader && elect_one()) {
      uint32_t it = 0, tile_it = 0, ph = 0;
      int s = 0;
      bool alive = true;
      const int dense_num_k = (int)((a.K_bytes + G_BLOCK_KB - 1) / G_BLOCK_KB);
      const uint32_t a_base = smem_u32(smem + Cfg::OFF_A), b_base = smem_u32(smem + Cfg::OFF_B);
      const uint32_t sfa_base = smem_u32(smem + Cfg::OFF_SFA), sfb_base = smem_u32(smem + Cfg::OFF_SFB);
      for (int tile = pair; tile < num_tiles && alive; tile += num_pairs, ++tile_it) {
        // The issuing thread needs the tile's K steps and where the tile starts inside its first
        // 128-row chunk of B scales (in columns); with 256-wide tiles the latter is always 0 (the
        // per-group row offset of B is a multiple of 128) and only grouped-K tiles differ in K, so
        // the index arithmetic and table reads of the full tile description stay off this thread.
        int num_k = dense_num_k;
        uint32_t sfb_col_off = 0;
        if (BN != 256 || (a.mode != MODE_DENSE && a.mode != MODE_GROUPED_ROWS)) {
          const PairTile t = pair_tile<kFormat, BN>(a, tile);
          num_k = t.num_k;
          sfb_col_off = ((uint32_t)t.b_row0 & 127u) >> 5;
        }
        const int as = tile_it % ACC;
        const uint32_t aph = (tile_it / ACC) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aph ^ 1, abort_flag, a.status, DS_ACC_EMPTY_WAIT)) { alive = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + Cfg::TMEM_ACC + as * BN;
        for (int k = 0; k < num_k; ++k, ++it) {
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, a.status, DS_TMA_WAIT)) { alive = false; break; }
          tc_fence_after();
          if (!MT_KNOB(a, 2) || k == 0) {
#pragma unroll
          for (int c = 0; c < CH; ++c)
            tc_copy_sf_pair(tmem_base + Cfg::TMEM_SFA + 4 * c, umma_desc_sf(sfa_base + s * Cfg::SFA_BYTES + c * 512));
#pragma unroll
          for (int h = 0; h < NSB; ++h)
#pragma unroll
            for (int c = 0; c < CH; ++c)
              tc_copy_sf_pair(tmem_base + Cfg::TMEM_SFB + 4 * (c * NSB + h),
                              umma_desc_sf(sfb_base + s * Cfg::SFB_BYTES + (h * CH + c) * 512));
          }
          const uint64_t adesc = umma_desc_sw128(a_base + s * Cfg::A_BYTES);
          const uint64_t bdesc = umma_desc_sw128(b_base + s * Cfg::B_BYTES);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t idesc = make_idesc_pair(kFormat, BN, j);
            const uint32_t sfa_t = tmem_base + Cfg::TMEM_SFA + (kFormat == FMT_NVFP4 ? 4 * j : 0);
            const uint32_t sfb_t = tmem_base + Cfg::TMEM_SFB + (kFormat == FMT_NVFP4 ? 4 * NSB * j : 0) + sfb_col_off;
            issue_mma_pair<kFormat>(tmem_d, adesc + 2 * j, bdesc + 2 * j, idesc, sfa_t, sfb_t, (k > 0 || j > 0) ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[s], 3);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (alive) tc_commit_pair(&acc_full[as], 3);
      }
    }
    __syncwarp();
  } else {
    // ======== epilogue (both CTAs): warp e reads lane quarter e % 4; columns [0,128) or [128,BN) ========
    const int e = warp - 2;
    const int q = warp & 3;          // hardware rule: a warp reads the lane quarter warp_id % 4
    const int half = (e >> 2) & 1;   // with 8 warps, quarters repeat after 4 warps
    const int ncols = half ? BN - 128 : 128;   // 128, or 64 for the second half of a 192-wide tile
    float alpha = 1.0f;
    if (a.amax_a != nullptr && a.amax_b != nullptr)
      alpha = __fdiv_rn(__fmul_rn(*a.amax_a, *a.amax_b), 6.0f * 6.0f * 448.0f * 448.0f);
    uint32_t tile_it = 0;
    bool alive = true;
    AmaxAcc am;
    for (int tile = pair; tile < num_tiles && alive; tile += num_pairs, ++tile_it) {
      const PairTile t = pair_tile<kFormat, BN>(a, tile);
      const int num_k = t.num_k;
      const int as = tile_it % ACC;
      const uint32_t aph = (tile_it / ACC) & 1;
      const uint32_t acc_empty_leader = map_to_cta(smem_u32(&acc_empty[as]), 0);
      MT_PROF_T(pt0);
      if (!mbar_wait_bounded(&acc_full[as], aph, abort_flag, a.status, DS_ACC_FULL_WAIT)) { alive = false; break; }
      tc_fence_after();
      MT_PROF_T(pt1);
      const int64_t row0 = t.d_row0 + rank * 128 + q * 32;   // first of this warp's 32 rows
      const int64_t row = row0 + lane;
      const bool row_ok = row >= t.d_row_lo && row < t.d_row_hi;
      const int64_t colw = t.d_col0 + half * 128;            // first of this warp's columns
      const uint32_t tmem_w = tmem_base + Cfg::TMEM_ACC + as * BN + (static_cast<uint32_t>(q * 32) << 16) + half * 128;
      // Pull this warp's accumulator block into registers and hand tensor memory back to the
      // MMA issuer at once; conversion and stores overlap the MMAs that follow.
      uint32_t acc[4][32];
#ifdef MT_TIMING_KNOBS
      if (MT_KNOB(a, 64)) {   // bit 6: the accumulator is handed back unread
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        continue;
      }
#endif
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (BN == 256 || c < 2 || half == 0) tc_ld_32x32(tmem_w + c * 32, acc[c]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      MT_PROF_T(pt2);
      MT_PROF_ADD(0, 1); MT_PROF_ADD(1, pt1 - pt0); MT_PROF_ADD(2, pt2 - pt1);
      if (MT_KNOB(a, 1)) continue;
      if (a.direct_store && num_k > 0) {
        // Plain output (no bias, abs-max, accumulation or peer destination; 32-byte aligned rows):
        // each lane converts its row and writes it as whole 32-byte sectors, masked by row, so
        // blocks that straddle a group boundary need no special case. No shared-memory traffic,
        // which the main loop saturates; measured 2 - 4 % faster than the staged stores at
        // K >= 4096 (bf16 and fp32) and equal at short K.
        if (a.d_dtype == MT_BF16) {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.d) + t.d_base + row * a.ldd + colw;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int col = 16 * i + 2 * j;
              const __nv_bfloat162 h = __floats2bfloat162_rn(__fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31])),
                                                             __fmul_rn(alpha, __uint_as_float(acc[(col + 1) >> 5][(col + 1) & 31])));
              w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            if (16 * i < ncols && row_ok && colw + 16 * i + 16 <= a.N) st_global_v8(dst + 16 * i, w);
          }
        } else {
          float* dst = static_cast<float*>(a.d) + t.d_base + row * a.ldd + colw;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int col = 8 * i + j;
              w[j] = __float_as_uint(__fmul_rn(alpha, __uint_as_float(acc[col >> 5][col & 31])));
            }
            if (8 * i < ncols && row_ok && colw + 8 * i + 8 <= a.N) st_global_v8(dst + 8 * i, w);
          }
        }
        MT_PROF_T(pt3d);
        MT_PROF_ADD(3, pt3d - pt2); MT_PROF_ADD(4, pt3d - pt0);
        continue;
      }
      // The staged path stores whole 32-row blocks; the tensor map clips at its own last row only,
      // so a block that straddles a group boundary takes the direct, row-masked path (as do
      // unaligned outputs and bf16 accumulation).
      const bool staged = a.tma_store >= 1 && row0 >= t.d_row_lo && (row0 + 32 <= t.d_row_hi || t.hi_is_end);
      if (!staged) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int64_t col0 = colw + c * 32;
          if (c * 32 < ncols && row_ok && col0 < a.N)
            store_row_chunk(a, acc[c], alpha, num_k > 0, t.d_base + row * a.ldd + col0, col0, am);
        }
        continue;
      }
      const CUtensorMap* out_map = &map_d;
      int64_t out_row = t.d_map_row0 + rank * 128 + q * 32;
      if (a.n_dest > 1) {
        // this warp's 32 rows belong to one destination rank (dest_rows is a multiple of 256):
        // they go to that rank's staging buffer, into the slice reserved for this rank
        const int dest = (int)(row0 / a.dest_rows);
        out_map = &maps_peer.m[dest];
        out_row = (int64_t)a.my_rank * a.dest_rows + (row0 - (int64_t)dest * a.dest_rows);
      }
#ifdef MT_TIMING_KNOBS
      if (a.tma_store == 2 && a.n_dest <= 1) {   // the 64-byte-wide variant, kept for comparison
        store_block_staged(a, &map_d, acc, ncols, smem + Cfg::OFF_EPI + e * 4096, lane,
                           out_row, a.map_rows, colw, alpha, num_k > 0, am);
        continue;
      }
#endif
      store_block_staged_wide(a, out_map, acc, ncols, smem + Cfg::OFF_EPI + e * 4096, lane, out_row, a.map_rows,
                              colw, alpha, num_k > 0, am);
      MT_PROF_T(pt3);
      MT_PROF_ADD(3, pt3 - pt2); MT_PROF_ADD(4, pt3 - pt0);
    }
    if (a.d_amax != nullptr) amax_publish(a.d_amax, am, lane);
  }

  if (warp >= 2 && lane == 0) bulk_wait_all();  // output stores issued by this lane are complete
  tc_fence_before();
  __syncthreads();
  // neither CTA may exit (or free tensor memory) while its peer can still touch it
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, G_TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int kFormat, int BLOCK_N, int STAGES, int ACC_STAGES>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, cudaStream_t st) {
  using Cfg = GemmCfg<kFormat, BLOCK_N, STAGES, ACC_STAGES>;
  auto kern = gemm_blockscaled_kernel<kFormat, BLOCK_N, STAGES, ACC_STAGES>;
  static bool attr_set[MT_MAX_DEVICES] = {};
  const int slot = current_device_slot();
  if (!attr_set[slot]) {
    MT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_ALLOC));
    attr_set[slot] = true;
  }
  const int grid = std::min(args.num_tiles, std::max(1, sm_count() - args.sm_margin));
  kern<<<grid, G_THREADS, Cfg::SMEM_ALLOC, st>>>(ma, mb, args);
  MT_CUDA(cudaGetLastError());
  return MT_OK;
}

static int64_t padded_chunks(int64_t k_blocks) { return ((k_blocks + 3) / 4 + 3) / 4 * 4; }

template <int kFormat, int BN, int STAGES>
static int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& msa,
                            const CUtensorMap& msb, const CUtensorMap& md, const PeerMaps& mp, const GemmArgs& args,
                            cudaStream_t st) {
  using Cfg = PairCfg<kFormat, BN, STAGES>;
  auto kern = gemm_blockscaled_pair_kernel<kFormat, BN, STAGES>;
  static int max_pairs_dev[MT_MAX_DEVICES] = {};   // 0 = not yet queried on that device
  int& max_pairs = max_pairs_dev[current_device_slot()];
  if (max_pairs <= 0) {
    MT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_ALLOC));
    // how many 2-CTA clusters can be resident at once (SMs pair up inside a GPC)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(P_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_ALLOC;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sm_count() / 2; }
    max_pairs = n;
  }
  const int pairs = std::min(args.num_tiles, std::max(1, max_pairs - (args.sm_margin + 1) / 2));
  MT_CUDA(launch_pdl(kern, dim3(2 * pairs), dim3(P_THREADS), (size_t)Cfg::SMEM_ALLOC, st, ma, mb, msa, msb, md, mp, args));
  return MT_OK;
}

// Timing-knob builds only: MT_GEMM_PAIR=0 forces the single-CTA kernel everywhere.
static bool pair_enabled() {
  static int use_pair = -1;
  if (use_pair < 0) use_pair = env_knob("MT_GEMM_PAIR", 1);
  return use_pair != 0;
}

// Timing-knob builds only: MT_GEMM_PAIR_N = 192 or 256 overrides the pair kernel's tile width.
static int forced_pair_n() {
  static int forced_bn = -1;
  if (forced_bn < 0) forced_bn = env_knob("MT_GEMM_PAIR_N", 0);
  return (forced_bn == 192 || forced_bn == 256) ? forced_bn : 0;
}

// Builds the five tensor maps of the pair kernel and launches it. A is [a_rows, a_ld_bytes]
// bytes, B is [b_rows, b_ld_bytes]; the output map covers [d_rows, d_cols] elements with row
// pitch ldd. args carries everything else (mode, tile counts, scale-factor geometry).
static int launch_pair_any(int format, int pbn, const uint8_t* a, int64_t a_rows, int64_t a_ld_bytes, const uint8_t* b,
                           int64_t b_rows, int64_t b_ld_bytes, void* d, int d_dtype, int64_t d_rows, int64_t d_cols,
                           int64_t ldd, int accumulate, GemmArgs& args, cudaStream_t st, int64_t a_slabs = 1,
                           int64_t b_slabs = 1, void* const* dest = nullptr) {
  static int band = -2;
  if (band == -2) band = env_knob("MT_GEMM_BAND", -1);
  args.band = band;
#ifdef MT_TIMING_KNOBS
  { static int knobs = -1; if (knobs < 0) knobs = env_knob("MT_GEMM_KNOBS", 0); args.knobs = knobs; }
#endif
  // a_slabs / b_slabs > 1: the operand is `slabs` matrices [rows, ld_bytes / slabs] stored one
  // after another, each with its own scale-chunk list (args.kc_* counts chunks per slab)
  const int64_t steps_total = (args.K_bytes + G_BLOCK_KB - 1) / G_BLOCK_KB;
  args.a_slab_steps = (int)std::max<int64_t>(1, steps_total / a_slabs);
  args.b_slab_steps = (int)std::max<int64_t>(1, steps_total / b_slabs);
  args.a_slab_rows = a_rows; args.b_slab_rows = b_rows;
  args.a_slab_chunks = args.rb_a * args.kc_a; args.b_slab_chunks = args.rb_b * args.kc_b;
  CUtensorMap ma, mb, msa, msb;
  int rc = make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)(a_ld_bytes / a_slabs),
                              (uint64_t)(a_rows * a_slabs), (uint64_t)(a_ld_bytes / a_slabs), G_BLOCK_KB, 128,
                              CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  rc = make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)(b_ld_bytes / b_slabs),
                          (uint64_t)(b_rows * b_slabs), (uint64_t)(b_ld_bytes / b_slabs), G_BLOCK_KB, (uint32_t)(pbn / 2),
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  const uint32_t ch = format == FMT_NVFP4 ? 4 : 1;
  rc = make_tensor_map_2d(&msa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, args.sa, 128, (uint64_t)(args.a_slab_chunks * a_slabs), 512,
                          128, ch, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MT_OK) return rc;
  rc = make_tensor_map_2d(&msb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, args.sb, 128, (uint64_t)(args.b_slab_chunks * b_slabs), 512,
                          128, ch, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MT_OK) return rc;
  // Output through shared memory + TMA stores when the output rows are 16-byte aligned;
  // fp32 accumulation uses the TMA add-reduction, bf16 accumulation the direct path.
  const size_t es = d_dtype == MT_F32 ? 4 : 2;
  static int allow_tma_store = -1;  // timing-knob builds only: MT_GEMM_TMA_STORE=0 forces the direct path
  if (allow_tma_store < 0) allow_tma_store = env_knob("MT_GEMM_TMA_STORE", 1);
  CUtensorMap md = ma;
  PeerMaps scatter_maps;
  const PeerMaps* peer_maps = nullptr;
  if (args.n_dest > 1) {
    // scattered output: one map per destination staging buffer, [d_rows, d_cols] bf16 with pitch d_cols
    for (int r = 0; r < args.n_dest; ++r) {
      rc = make_tensor_map_2d(&scatter_maps.m[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dest[r], (uint64_t)d_cols,
                              (uint64_t)d_rows, (uint64_t)d_cols * 2, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != MT_OK) return rc;
    }
    for (int r = args.n_dest; r < MT_MAX_PEERS; ++r) scatter_maps.m[r] = scatter_maps.m[0];
    peer_maps = &scatter_maps;
    d = dest[args.my_rank];
    ldd = d_cols;
  }
  args.tma_store = (allow_tma_store && aligned16(d) && ((size_t)ldd * es) % 16 == 0 && !(accumulate && d_dtype == MT_BF16)) ? allow_tma_store : 0;
  args.map_rows = d_rows;
  static int allow_direct = -1;     // timing-knob builds only: MT_GEMM_DIRECT=0 keeps plain outputs on the staged path
  if (allow_direct < 0) allow_direct = env_knob("MT_GEMM_DIRECT", 1);
  const int per_sector = d_dtype == MT_F32 ? 8 : 16;   // elements per 32-byte sector
  args.direct_store = allow_direct && !accumulate && args.bias == nullptr && args.d_amax == nullptr && args.n_dest <= 1 &&
                      (args.mode == MODE_DENSE || args.mode == MODE_GROUPED_ROWS) &&
                      (reinterpret_cast<uintptr_t>(d) & 31) == 0 && ldd % per_sector == 0 && d_cols % per_sector == 0;
  if (args.n_dest > 1 && args.tma_store != 1) return fail(MT_ERR_INVALID_ARG, "scattered output needs the staged store path");
  static int narrow_store = -1;   // timing-knob builds only: MT_GEMM_NARROW_STORE=1 selects the 64-byte-wide variant
  if (narrow_store < 0) narrow_store = env_knob("MT_GEMM_NARROW_STORE", 0);
  if (args.tma_store) {
    const CUtensorMapDataType dt = d_dtype == MT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (narrow_store && args.n_dest <= 1) {
      // box: 32 rows x 64 bytes (half of a warp's staging buffer), 64-byte swizzle
      rc = make_tensor_map_2d(&md, dt, (int)es, d, (uint64_t)d_cols, (uint64_t)d_rows, (uint64_t)ldd * es,
                              d_dtype == MT_F32 ? 16 : 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
      args.tma_store = 2;
    } else {
      // box: 32 rows x 128 bytes (a warp's whole staging buffer), 128-byte swizzle
      rc = make_tensor_map_2d(&md, dt, (int)es, d, (uint64_t)d_cols, (uint64_t)d_rows, (uint64_t)ldd * es,
                              d_dtype == MT_F32 ? 32 : 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc != MT_OK) return rc;
  }
  static PeerMaps no_peers{};
  const PeerMaps& mp = peer_maps ? *peer_maps : no_peers;
  if (format == FMT_NVFP4)
    return pbn == 192 ? launch_gemm_pair<FMT_NVFP4, 192, 5>(ma, mb, msa, msb, md, mp, args, st)
                      : launch_gemm_pair<FMT_NVFP4, 256, 5>(ma, mb, msa, msb, md, mp, args, st);
  return pbn == 192 ? launch_gemm_pair<FMT_MXFP8, 192, 5>(ma, mb, msa, msb, md, mp, args, st)
                    : launch_gemm_pair<FMT_MXFP8, 256, 5>(ma, mb, msa, msb, md, mp, args, st);
}

// Timing-knob builds only: MT_GEMM_BLOCK_N = 128 or 256 overrides the single-CTA tile width.
static int pick_block_n(int64_t N) {
  static int forced = -1;
  if (forced < 0) forced = env_knob("MT_GEMM_BLOCK_N", 0);
  if (forced == 128 || forced == 256) return forced;
  return N > 128 ? 256 : 128;
}

static int gemm_common(int format, const uint8_t* a, const uint8_t* sa, const float* amax_a, const uint8_t* b,
                       const uint8_t* sb, const float* amax_b, int64_t M, int64_t N, int64_t K, void* d, int d_dtype,
                       int64_t ldd, const void* bias, int bias_dtype, int accumulate, const mt_gemm_opts* opts,
                       cudaStream_t st, int64_t a_slabs = 1, int64_t b_slabs = 1) {
  const char* name = format == FMT_NVFP4 ? "mt_gemm_nvfp4" : "mt_gemm_mxfp8";
  const int sm_margin = opts ? opts->sm_margin : 0;
  float* d_amax = opts ? opts->d_amax : nullptr;
  MT_REQUIRE(sm_margin >= 0 && sm_margin < 128, "%s: sm_margin %d is not a valid SM count", name, sm_margin);
  MT_REQUIRE(!(d_amax && accumulate), "%s: d_amax is not available together with accumulate", name);
  const int n_dest = opts ? opts->n_dest : 0;
  if (n_dest > 1) {
    MT_REQUIRE(n_dest <= MT_MAX_PEERS && opts->my_rank >= 0 && opts->my_rank < n_dest,
               "%s: scatter over %d ranks from rank %d is out of range", name, n_dest, opts->my_rank);
    MT_REQUIRE(d_dtype == MT_BF16 && !accumulate && bias == nullptr && d_amax == nullptr,
               "%s: a scattered output is bf16, without accumulate, bias or d_amax", name);
    MT_REQUIRE(opts->dest_rows > 0 && opts->dest_rows % 256 == 0 && M == n_dest * opts->dest_rows && N % 8 == 0 && K > 0,
               "%s: a scattered output needs M == n_dest * dest_rows, dest_rows %% 256 == 0, N %% 8 == 0 (M=%lld, N=%lld, "
               "dest_rows=%lld)", name, (long long)M, (long long)N, (long long)opts->dest_rows);
    MT_REQUIRE(pair_enabled() && M > G_BLOCK_M && N > 128, "%s: a scattered output needs N > 128", name);
    for (int r = 0; r < n_dest; ++r)
      MT_REQUIRE(opts->dest[r] != nullptr && aligned16(opts->dest[r]), "%s: destination %d is null or misaligned", name, r);
    d = opts->dest[opts->my_rank];
    ldd = N;
  }
  MT_REQUIRE(a_slabs >= 1 && b_slabs >= 1, "%s: slab counts must be positive", name);
  MT_REQUIRE(d != nullptr, "%s: null output pointer", name);
  MT_REQUIRE(M >= 0 && N >= 0 && K >= 0, "%s: negative shape", name);
  if (K == 0) {
    // empty contraction: the product is all zeros (bias and previous contents are kept out of
    // this corner: the emulation returns plain zeros for it as well)
    if (M > 0 && N > 0 && !accumulate) {
      const size_t es = d_dtype == MT_F32 ? 4 : 2;
      MT_CUDA(cudaMemset2DAsync(d, (size_t)ldd * es, 0, (size_t)N * es, (size_t)M, st));
    }
    return MT_OK;
  }
  MT_REQUIRE(a && sa && b && sb, "%s: null pointer", name);
  MT_REQUIRE(d_dtype == MT_BF16 || d_dtype == MT_F32, "%s: output dtype %d not supported", name, d_dtype);
  MT_REQUIRE(bias == nullptr || bias_dtype == MT_BF16 || bias_dtype == MT_F32, "%s: bias dtype %d not supported", name, bias_dtype);
  MT_REQUIRE(ldd >= N, "%s: ldd (%lld) smaller than N (%lld)", name, (long long)ldd, (long long)N);
  const int64_t kmult = format == FMT_NVFP4 ? 32 : 16;
  MT_REQUIRE(K % kmult == 0, "%s: K (%lld) must be a multiple of %lld", name, (long long)K, (long long)kmult);
  MT_REQUIRE(aligned16(a) && aligned16(b) && aligned16(sa) && aligned16(sb), "%s: operands must be 16-byte aligned", name);
  if (format == FMT_NVFP4) MT_REQUIRE(amax_a && amax_b, "%s: per-tensor abs-max pointers are required", name);
  if (M == 0 || N == 0) return MT_OK;
  const int64_t K_bytes = format == FMT_NVFP4 ? K / 2 : K;
  const int64_t block = format == FMT_NVFP4 ? 16 : 32;

  GemmArgs args{};
  args.sa = sa; args.sb = sb;
  const bool slabbed = a_slabs > 1 || b_slabs > 1;
  if (slabbed) {
    // every slab must hold whole K steps, so that no load straddles two slabs
    MT_REQUIRE(K_bytes % (a_slabs * G_BLOCK_KB) == 0 && K_bytes % (b_slabs * G_BLOCK_KB) == 0,
               "%s: each K slab must be a multiple of %d bytes (K_bytes=%lld, slabs %lld / %lld)", name, G_BLOCK_KB,
               (long long)K_bytes, (long long)a_slabs, (long long)b_slabs);
    MT_REQUIRE(pair_enabled() && M > G_BLOCK_M && N > 128,
               "%s: K-slab operands need M > 128 and N > 128 (M=%lld, N=%lld)", name, (long long)M, (long long)N);
  }
  args.kc_a = padded_chunks(K / a_slabs / block);
  args.kc_b = padded_chunks(K / b_slabs / block);
  args.rb_a = (M + 127) / 128; args.rb_b = (N + 127) / 128;
  args.M = M; args.N = N; args.K_bytes = K_bytes;
  args.d = d; args.ldd = ldd; args.d_dtype = d_dtype;
  args.bias = bias; args.bias_dtype = bias_dtype; args.accumulate = accumulate;
  args.amax_a = format == FMT_NVFP4 ? amax_a : nullptr;
  args.amax_b = format == FMT_NVFP4 ? amax_b : nullptr;
  args.status = device_status_ptr();
  if (!args.status) return fail(MT_ERR_CUDA, "device status word not reachable");
  args.mode = MODE_DENSE;
  args.sm_margin = sm_margin;
  args.d_amax = d_amax;
  if (n_dest > 1) {
    args.n_dest = n_dest; args.my_rank = opts->my_rank; args.dest_rows = opts->dest_rows;
  }
  args.k_elems_per_byte_x2 = format == FMT_NVFP4 ? 4 : 2;
  // K == 0 never reaches this point; tensor maps below need K_bytes >= 16
  if (pair_enabled() && M > G_BLOCK_M && N > 128) {
    // Tile width: 256 by default. The 192-wide variant (two accumulators, epilogue overlapped
    // with the next tile's MMAs) measured no faster on the benchmark shapes because the main
    // loop is bound by shared-memory bandwidth either way; MT_GEMM_PAIR_N=192 selects it.
    const int pbn = forced_pair_n() ? forced_pair_n() : 256;
    args.tiles_m = (int)((M + 255) / 256);
    args.tiles_n = (int)((N + pbn - 1) / pbn);
    args.num_tiles = args.tiles_m * args.tiles_n;
    return launch_pair_any(format, pbn, a, M, K_bytes, b, N, K_bytes, d, d_dtype, M, N, ldd, accumulate, args, st, a_slabs,
                           b_slabs, n_dest > 1 ? opts->dest : nullptr);
  }
  const int bn = pick_block_n(N);
  args.tiles_m = (int)((M + G_BLOCK_M - 1) / G_BLOCK_M);
  args.tiles_n = (int)((N + bn - 1) / bn);
  args.num_tiles = args.tiles_m * args.tiles_n;

  CUtensorMap ma, mb;
  // K == 0: no loads are issued, but the maps must still be well-formed
  const uint64_t kb = (uint64_t)std::max<int64_t>(K_bytes, 16);
  int rc = make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, kb, (uint64_t)M, kb, G_BLOCK_KB, G_BLOCK_M,
                              CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  rc = make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, kb, (uint64_t)N, kb, G_BLOCK_KB, (uint32_t)bn,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  if (format == FMT_NVFP4) {
    return bn == 256 ? launch_gemm<FMT_NVFP4, 256, 4, 1>(ma, mb, args, st) : launch_gemm<FMT_NVFP4, 128, 6, 2>(ma, mb, args, st);
  }
  return bn == 256 ? launch_gemm<FMT_MXFP8, 256, 4, 1>(ma, mb, args, st) : launch_gemm<FMT_MXFP8, 128, 6, 2>(ma, mb, args, st);
}


// ------------------------------------------------------------------------------------------
// grouped GEMMs (per-expert weights), MXFP8
// ------------------------------------------------------------------------------------------
// `plan` is a device buffer written by build_grouped_plan for (rows, G): the tile entries, their
// count and the group offsets are read from it by the kernel; the host only knows upper bounds.
static int grouped_rows_gemm(const char* name, const uint8_t* a, const uint8_t* sa, const uint8_t* b, const uint8_t* sb,
                             int64_t b_rows, int64_t ldb_bytes, const void* plan, int64_t G, int64_t R, int64_t N_out,
                             int64_t Kc, int64_t b_group_rows, int64_t b_group_k, void* d, int d_dtype, int64_t ldd,
                             cudaStream_t st) {
  MT_REQUIRE(G > 0 && G <= PLAN_MAX_GROUPS && R >= 0 && R <= PLAN_MAX_ROWS, "%s: bad group description", name);
  MT_REQUIRE(d_dtype == MT_BF16 || d_dtype == MT_F32, "%s: output dtype %d not supported", name, d_dtype);
  MT_REQUIRE(N_out > 0 && N_out % 128 == 0, "%s: N (%lld) must be a positive multiple of 128", name, (long long)N_out);
  MT_REQUIRE(Kc > 0 && Kc % 128 == 0, "%s: K (%lld) must be a positive multiple of 128", name, (long long)Kc);
  MT_REQUIRE(ldd >= N_out, "%s: ldd smaller than N", name);
  MT_REQUIRE(b_group_rows >= 0 && b_group_rows % 128 == 0, "%s: rows of B per group (%lld) must be a multiple of 128", name,
             (long long)b_group_rows);
  if (R == 0) return MT_OK;
  MT_REQUIRE(a && sa && b && sb && d && plan, "%s: null pointer", name);
  MT_REQUIRE(aligned16(a) && aligned16(b) && aligned16(sa) && aligned16(sb) && aligned16(plan),
             "%s: operands must be 16-byte aligned", name);
  const PlanView pv = plan_view(const_cast<void*>(plan), R, G);
  const int64_t max_entries = plan_entries_upper_bound(R, G);

  GemmArgs args{};
  args.sa = sa; args.sb = sb;
  args.kc_a = padded_chunks(Kc / 32);
  args.kc_b = padded_chunks(ldb_bytes / 32);
  args.rb_a = (R + 127) / 128; args.rb_b = (b_rows + 127) / 128;
  args.M = R; args.N = N_out; args.K_bytes = Kc;
  args.d = d; args.ldd = ldd; args.d_dtype = d_dtype;
  args.status = device_status_ptr();
  if (!args.status) return fail(MT_ERR_CUDA, "device status word not reachable");
  args.mode = MODE_GROUPED_ROWS;
  args.num_groups = (int)G;
  args.group_offsets = pv.offsets;
  args.b_group_rows = b_group_rows;
  args.b_group_k_bytes = b_group_k;
  args.k_elems_per_byte_x2 = 2;
  // entries: for every row block (256 rows for the pair kernel, else 128), every group owning
  // at least one of its rows
  const bool pair = pair_enabled() && N_out >= 256 && R > 128;
  if (pair) {
    const int pbn = forced_pair_n() ? forced_pair_n() : 256;
    args.tile_rb = pv.e256_rb; args.tile_group = pv.e256_group;
    args.entries_dev = &pv.header->n_entries256;
    args.tiles_m = (int)max_entries;
    args.tiles_n = (int)((N_out + pbn - 1) / pbn);
    args.num_tiles = (int)std::min<int64_t>(max_entries * args.tiles_n, INT32_MAX);
    return launch_pair_any(FMT_MXFP8, pbn, a, R, Kc, b, b_rows, ldb_bytes, d, d_dtype, R, N_out, ldd, 0, args, st);
  }
  const int bn = N_out % 256 == 0 ? 256 : 128;
  args.tile_rb = pv.e128_rb; args.tile_group = pv.e128_group;
  args.entries_dev = &pv.header->n_entries128;
  args.tiles_m = (int)max_entries;
  args.tiles_n = (int)(N_out / bn);
  args.num_tiles = (int)std::min<int64_t>(max_entries * args.tiles_n, INT32_MAX);
  CUtensorMap ma, mb;
  int rc = make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)Kc, (uint64_t)R, (uint64_t)Kc, G_BLOCK_KB,
                              G_BLOCK_M, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  rc = make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)ldb_bytes, (uint64_t)b_rows, (uint64_t)ldb_bytes,
                          G_BLOCK_KB, (uint32_t)bn, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  return bn == 256 ? launch_gemm<FMT_MXFP8, 256, 4, 1>(ma, mb, args, st) : launch_gemm<FMT_MXFP8, 128, 6, 2>(ma, mb, args, st);
}

}  // namespace mt

extern "C" {

#ifdef MT_TIMING_KNOBS
// knob builds only: reads and clears the epilogue phase sums
int mt_debug_epilogue_profile(unsigned long long* out8) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out8, mt::g_epi_prof, 64);
  unsigned long long z[8] = {};
  cudaMemcpyToSymbol(mt::g_epi_prof, z, 64);
  return 0;
}
#endif

int mt_grouped_gemm_mxfp8(const uint8_t* a, const uint8_t* sa_swz, const uint8_t* b, const uint8_t* sb_swz,
                          int64_t b_rows, int64_t ldb, const void* plan, int64_t G, int64_t rows, int64_t N, int64_t K,
                          int64_t b_group_rows, int64_t b_group_k, void* d, int d_dtype, int64_t ldd,
                          mt_stream_t stream) {
  return mt::grouped_rows_gemm("mt_grouped_gemm_mxfp8", a, sa_swz, b, sb_swz, b_rows, ldb, plan, G, rows, N, K,
                               b_group_rows, b_group_k, d, d_dtype, ldd, static_cast<cudaStream_t>(stream));
}

// ---- the same grouped GEMM for callers that cannot allocate device memory ----
// Its plan lives in this fixed array inside the library image (one copy per GPU that loads the
// library, held until the process exits) instead of a caller-provided buffer.
#define MT_STATIC_PLAN_ENTRIES ((MT_STATIC_MAX_ROWS + 127) / 128 + MT_STATIC_MAX_GROUPS)
#define MT_STATIC_PLAN_R16(n) (((n) + 15) / 16 * 16)
#define MT_STATIC_PLAN_BYTES                                                                       \
  ((64 + 2 * MT_STATIC_PLAN_R16(8 * (MT_STATIC_MAX_GROUPS + 1)) + 4 * MT_STATIC_PLAN_R16(4 * MT_STATIC_PLAN_ENTRIES) + \
    16 * MT_STATIC_PLAN_ENTRIES + 255) / 256 * 256)
static __device__ __align__(256) unsigned char g_grouped_static_plan[MT_STATIC_PLAN_BYTES];

int mt_grouped_gemm_mxfp8_static(const uint8_t* a, const uint8_t* sa_swz, const uint8_t* b, const uint8_t* sb_swz,
                                 int64_t b_rows, int64_t ldb, const int64_t* m_offsets, int64_t G, int64_t rows,
                                 int64_t N, int64_t K, int64_t b_group_rows, int64_t b_group_k, void* d, int d_dtype,
                                 int64_t ldd, mt_stream_t stream) {
  const char* name = "mt_grouped_gemm_mxfp8_static";
  MT_REQUIRE(m_offsets && G > 0 && rows >= 0, "%s: bad group description", name);
  MT_REQUIRE(G <= MT_STATIC_MAX_GROUPS, "%s: %lld groups exceed the built-in limit of %d; use mt_grouped_gemm_mxfp8 "
             "with a caller-provided plan", name, (long long)G, MT_STATIC_MAX_GROUPS);
  MT_REQUIRE(rows <= MT_STATIC_MAX_ROWS, "%s: %lld rows exceed the built-in limit of %d; use mt_grouped_gemm_mxfp8 "
             "with a caller-provided plan", name, (long long)rows, MT_STATIC_MAX_ROWS);
  static_assert(MT_STATIC_PLAN_BYTES >= 0, "static plan size");
  if (mt::plan_bytes(rows, G) > (int64_t)MT_STATIC_PLAN_BYTES)
    return mt::fail(MT_ERR_INVALID_ARG, "%s: plan does not fit the built-in array", name);
  // The array's name is only a host-side handle; the kernels need its device address, which is
  // looked up once per device (with that device current) and remembered.
  static void* dev_ptr[64] = {};
  int dev = -1;
  MT_CUDA(cudaGetDevice(&dev));
  MT_REQUIRE(dev >= 0 && dev < 64, "%s: device ordinal %d not supported", name, dev);
  if (dev_ptr[dev] == nullptr) {
    void* p = nullptr;
    MT_CUDA(cudaGetSymbolAddress(&p, g_grouped_static_plan));
    dev_ptr[dev] = p;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the plan is rebuilt by every call (a tiny kernel ahead of the GEMM on the same stream), so
  // nothing of an earlier call's contents is relied on
  int rc = mt::build_grouped_plan(m_offsets, G, rows, dev_ptr[dev], st);
  if (rc != MT_OK) return rc;
  return mt::grouped_rows_gemm(name, a, sa_swz, b, sb_swz, b_rows, ldb, dev_ptr[dev], G, rows, N, K, b_group_rows,
                               b_group_k, d, d_dtype, ldd, st);
}

int mt_grouped_wgrad_mxfp8(const uint8_t* a_t, const uint8_t* sa_t_swz, const uint8_t* b_t, const uint8_t* sb_t_swz,
                           const void* plan, int64_t G, int64_t rows, int64_t padded_rows, int64_t N_out,
                           int64_t K_out, void* d, int d_dtype, int accumulate, mt_stream_t stream) {
  using namespace mt;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const char* name = "mt_grouped_wgrad_mxfp8";
  MT_REQUIRE(G > 0 && G <= PLAN_MAX_GROUPS && rows >= 0 && rows <= PLAN_MAX_ROWS, "%s: bad group description", name);
  MT_REQUIRE(padded_rows >= 0 && padded_rows % 128 == 0 && padded_rows <= rows + 127 * G,
             "%s: padded row count %lld is not a multiple of 128 within [0, rows + 127 G]", name, (long long)padded_rows);
  MT_REQUIRE(d_dtype == MT_BF16 || d_dtype == MT_F32, "%s: output dtype %d not supported", name, d_dtype);
  MT_REQUIRE(N_out > 0 && K_out > 0, "%s: empty output", name);
  MT_REQUIRE(d != nullptr, "%s: null output", name);
  const int64_t Rp = padded_rows;
  if (Rp == 0) {
    if (!accumulate) {
      const size_t es = d_dtype == MT_F32 ? 4 : 2;
      MT_CUDA(cudaMemsetAsync(d, 0, (size_t)G * N_out * K_out * es, st));
    }
    return MT_OK;
  }
  MT_REQUIRE(a_t && sa_t_swz && b_t && sb_t_swz && plan, "%s: null pointer", name);
  MT_REQUIRE(aligned16(a_t) && aligned16(b_t) && aligned16(sa_t_swz) && aligned16(sb_t_swz) && aligned16(plan),
             "%s: operands must be 16-byte aligned", name);
  const PlanView pv = plan_view(const_cast<void*>(plan), rows, G);

  GemmArgs args{};
  args.sa = sa_t_swz; args.sb = sb_t_swz;
  args.kc_a = args.kc_b = padded_chunks(Rp / 32);
  args.rb_a = (N_out + 127) / 128; args.rb_b = (K_out + 127) / 128;
  args.M = N_out; args.N = K_out; args.K_bytes = Rp;
  args.d = d; args.ldd = K_out; args.d_dtype = d_dtype; args.accumulate = accumulate;
  args.status = device_status_ptr();
  if (!args.status) return fail(MT_ERR_CUDA, "device status word not reachable");
  args.mode = MODE_GROUPED_K;
  args.num_groups = (int)G;
  args.group_offsets = pv.pad_offsets;
  args.d_group_stride = N_out * K_out;
  args.k_elems_per_byte_x2 = 2;
  if (pair_enabled() && N_out > 128 && K_out > 128) {
    const int pbn = forced_pair_n() ? forced_pair_n() : 256;
    args.tiles_m = (int)((N_out + 255) / 256);
    args.tiles_n = (int)((K_out + pbn - 1) / pbn);
    args.num_tiles = (int)(G * args.tiles_m * args.tiles_n);
    return launch_pair_any(FMT_MXFP8, pbn, a_t, N_out, Rp, b_t, K_out, Rp, d, d_dtype, G * N_out, K_out, K_out, accumulate,
                           args, st);
  }
  const int bn = K_out > 128 ? 256 : 128;
  args.tiles_m = (int)((N_out + G_BLOCK_M - 1) / G_BLOCK_M);
  args.tiles_n = (int)((K_out + bn - 1) / bn);
  args.num_tiles = (int)(G * args.tiles_m * args.tiles_n);
  CUtensorMap ma, mb;
  int rc = make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_t, (uint64_t)Rp, (uint64_t)N_out, (uint64_t)Rp, G_BLOCK_KB,
                              G_BLOCK_M, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  rc = make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_t, (uint64_t)Rp, (uint64_t)K_out, (uint64_t)Rp, G_BLOCK_KB,
                          (uint32_t)bn, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MT_OK) return rc;
  return bn == 256 ? launch_gemm<FMT_MXFP8, 256, 4, 1>(ma, mb, args, st) : launch_gemm<FMT_MXFP8, 128, 6, 2>(ma, mb, args, st);
}

int mt_gemm_nvfp4(const uint8_t* a, const uint8_t* sa_swz, const float* amax_a, const uint8_t* b,
                  const uint8_t* sb_swz, const float* amax_b, int64_t M, int64_t N, int64_t K, void* d, int d_dtype,
                  int64_t ldd, const void* bias, int bias_dtype, int accumulate, const mt_gemm_opts* opts,
                  mt_stream_t stream) {
  return mt::gemm_common(mt::FMT_NVFP4, a, sa_swz, amax_a, b, sb_swz, amax_b, M, N, K, d, d_dtype, ldd, bias,
                         bias_dtype, accumulate, opts, static_cast<cudaStream_t>(stream));
}

int mt_gemm_nvfp4_kslab(const uint8_t* a, const uint8_t* sa_swz, const float* amax_a, int64_t a_slabs, const uint8_t* b,
                        const uint8_t* sb_swz, const float* amax_b, int64_t b_slabs, int64_t M, int64_t N, int64_t K,
                        void* d, int d_dtype, int64_t ldd, const void* bias, int bias_dtype, int accumulate,
                        const mt_gemm_opts* opts, mt_stream_t stream) {
  return mt::gemm_common(mt::FMT_NVFP4, a, sa_swz, amax_a, b, sb_swz, amax_b, M, N, K, d, d_dtype, ldd, bias,
                         bias_dtype, accumulate, opts, static_cast<cudaStream_t>(stream), a_slabs, b_slabs);
}

int mt_gemm_mxfp8_kslab(const uint8_t* a, const uint8_t* sa_swz, int64_t a_slabs, const uint8_t* b, const uint8_t* sb_swz,
                        int64_t b_slabs, int64_t M, int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd,
                        const void* bias, int bias_dtype, int accumulate, const mt_gemm_opts* opts, mt_stream_t stream) {
  return mt::gemm_common(mt::FMT_MXFP8, a, sa_swz, nullptr, b, sb_swz, nullptr, M, N, K, d, d_dtype, ldd, bias,
                         bias_dtype, accumulate, opts, static_cast<cudaStream_t>(stream), a_slabs, b_slabs);
}

int mt_gemm_mxfp8(const uint8_t* a, const uint8_t* sa_swz, const uint8_t* b, const uint8_t* sb_swz, int64_t M,
                  int64_t N, int64_t K, void* d, int d_dtype, int64_t ldd, const void* bias, int bias_dtype,
                  int accumulate, const mt_gemm_opts* opts, mt_stream_t stream) {
  return mt::gemm_common(mt::FMT_MXFP8, a, sa_swz, nullptr, b, sb_swz, nullptr, M, N, K, d, d_dtype, ldd, bias,
                         bias_dtype, accumulate, opts, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
