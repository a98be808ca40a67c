// Layout of the grouped-call plan: the tile tables every grouped entry point (GEMMs, wgrad,
// transposed quantize) reads, built on the device from the group offsets by one small kernel
// (grouped_plan.cu) so that no grouped call touches host memory.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

constexpr int32_t PLAN_MAGIC = 0x6d74706c;  // "mtpl"

struct PlanHeader {        // 64 bytes
  int32_t magic;
  int32_t groups;
  int32_t n_entries256;    // (256-row block, group) entries of the CTA-pair grouped GEMM
  int32_t n_entries128;    // (128-row block, group) entries of the single-CTA grouped GEMM
  int32_t n_qtiles;        // 128-token tiles of the grouped transposed quantize
  int32_t error;           // non-zero: the offsets were not a valid partition of [0, rows)
  int64_t rows;
  int64_t padded_rows;     // every group rounded up to 128 tokens
  int32_t reserved[6];
};
static_assert(sizeof(PlanHeader) == 64, "plan header layout");

struct PlanView {
  PlanHeader* header;
  int64_t* offsets;        // [G + 1] row offset of each group
  int64_t* pad_offsets;    // [G + 1] token offset of each group after padding to 128
  int32_t* e256_rb;        // [E] row block of entry i
  int32_t* e256_group;     // [E]
  int32_t* e128_rb;        // [E]
  int32_t* e128_group;     // [E]
  int4* qtiles;            // [E] {first row, valid rows, output column, last tile}
};

// Entries are (row block, group) pairs with at least one row in common: at most one per row
// block plus one per group boundary.
__host__ __device__ inline int64_t plan_entries_upper_bound(int64_t rows, int64_t groups) {
  return (rows + 127) / 128 + groups;
}
__host__ __device__ inline int64_t plan_round16(int64_t n) { return (n + 15) / 16 * 16; }

__host__ __device__ inline int64_t plan_bytes(int64_t rows, int64_t groups) {
  const int64_t e = plan_entries_upper_bound(rows, groups);
  const int64_t n = 64 + 2 * plan_round16(8 * (groups + 1)) + 4 * plan_round16(4 * e) + 16 * e;
  return (n + 255) / 256 * 256;
}

__host__ __device__ inline PlanView plan_view(void* base, int64_t rows, int64_t groups) {
  const int64_t e = plan_entries_upper_bound(rows, groups);
  uint8_t* p = static_cast<uint8_t*>(base);
  PlanView v;
  v.header = reinterpret_cast<PlanHeader*>(p); p += 64;
  v.offsets = reinterpret_cast<int64_t*>(p); p += plan_round16(8 * (groups + 1));
  v.pad_offsets = reinterpret_cast<int64_t*>(p); p += plan_round16(8 * (groups + 1));
  v.e256_rb = reinterpret_cast<int32_t*>(p); p += plan_round16(4 * e);
  v.e256_group = reinterpret_cast<int32_t*>(p); p += plan_round16(4 * e);
  v.e128_rb = reinterpret_cast<int32_t*>(p); p += plan_round16(4 * e);
  v.e128_group = reinterpret_cast<int32_t*>(p); p += plan_round16(4 * e);
  v.qtiles = reinterpret_cast<int4*>(p);
  return v;
}

// Launches the builder on `st` (grouped_plan.cu); argument checks are the caller's.
int build_grouped_plan(const int64_t* m_offsets_dev, int64_t groups, int64_t rows, void* plan, cudaStream_t st);

constexpr int64_t PLAN_MAX_GROUPS = 65536;
constexpr int64_t PLAN_MAX_ROWS = (int64_t)1 << 30;

}  // namespace mt
