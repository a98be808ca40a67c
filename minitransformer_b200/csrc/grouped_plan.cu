// Builds the plan of a grouped call on the device: from the G + 1 row offsets of the groups
// (device memory) one CTA derives the padded token offsets, the (row block, group) tile
// entries of the grouped GEMMs for 256- and 128-row blocks and the 128-token tiles of the
// grouped transposed quantize. Every grouped entry point then reads its tables and counts from
// the plan, so none of them copies from host memory or needs the offsets on the host.
#include "grouped_plan.cuh"
#include "mt_common.cuh"

namespace mt {

constexpr int PLAN_THREADS = 256;

// Number of `blk`-row blocks that rows [lo, hi) touch (hi > lo).
__device__ __forceinline__ int64_t blocks_touched(int64_t lo, int64_t hi, int64_t blk) {
  return (hi - 1) / blk - lo / blk + 1;
}

__global__ void __launch_bounds__(PLAN_THREADS) grouped_plan_kernel(const int64_t* __restrict__ m_offsets, int64_t G,
                                                                    int64_t rows, void* plan, int* status) {
  __shared__ int64_t s_cnt[4][PLAN_THREADS];   // per thread: entries256, entries128, qtiles, padded rows
  __shared__ int s_bad;
  const PlanView v = plan_view(plan, rows, G);
  const int tid = threadIdx.x;
  const int64_t chunk = (G + PLAN_THREADS - 1) / PLAN_THREADS;
  const int64_t g0 = min(G, (int64_t)tid * chunk), g1 = min(G, g0 + chunk);
  if (tid == 0) s_bad = (m_offsets[0] != 0 || m_offsets[G] != rows) ? 1 : 0;
  __syncthreads();

  int64_t c256 = 0, c128 = 0, cq = 0, pad = 0;
  bool bad = false;
  for (int64_t g = g0; g < g1; ++g) {
    const int64_t lo = m_offsets[g], hi = m_offsets[g + 1];
    if (hi < lo || lo < 0 || hi > rows) { bad = true; continue; }
    if (hi == lo) continue;
    c256 += blocks_touched(lo, hi, 256);
    c128 += blocks_touched(lo, hi, 128);
    cq += (hi - lo + 127) / 128;
    pad += (hi - lo + 127) / 128 * 128;
  }
  if (bad) s_bad = 1;
  s_cnt[0][tid] = c256; s_cnt[1][tid] = c128; s_cnt[2][tid] = cq; s_cnt[3][tid] = pad;
  __syncthreads();
  // exclusive prefix sums over the threads' counts (4 x 256 values: one thread per quantity)
  if (tid < 4) {
    int64_t run = 0;
    for (int i = 0; i < PLAN_THREADS; ++i) {
      const int64_t c = s_cnt[tid][i];
      s_cnt[tid][i] = run;
      run += c;
    }
    if (tid == 0) v.header->n_entries256 = s_bad ? 0 : (int32_t)run;
    if (tid == 1) v.header->n_entries128 = s_bad ? 0 : (int32_t)run;
    if (tid == 2) v.header->n_qtiles = s_bad ? 0 : (int32_t)run;
    if (tid == 3) { v.header->padded_rows = run; v.pad_offsets[G] = run; }
  }
  __syncthreads();
  if (tid == 0) {
    v.header->magic = PLAN_MAGIC;
    v.header->groups = (int32_t)G;
    v.header->rows = rows;
    v.header->error = s_bad;
    v.offsets[G] = rows;
    if (s_bad) atomicOr(status, DS_BAD_PLAN);
  }
  if (s_bad) return;

  int64_t i256 = s_cnt[0][tid], i128 = s_cnt[1][tid], iq = s_cnt[2][tid], p = s_cnt[3][tid];
  const int64_t q_total = (int64_t)v.header->n_qtiles;   // written before the barrier above
  for (int64_t g = g0; g < g1; ++g) {
    const int64_t lo = m_offsets[g], hi = m_offsets[g + 1];
    v.offsets[g] = lo;
    v.pad_offsets[g] = p;
    if (hi == lo) continue;
    for (int64_t rb = lo / 256; rb <= (hi - 1) / 256; ++rb, ++i256) {
      v.e256_rb[i256] = (int32_t)rb;
      v.e256_group[i256] = (int32_t)g;
    }
    for (int64_t rb = lo / 128; rb <= (hi - 1) / 128; ++rb, ++i128) {
      v.e128_rb[i128] = (int32_t)rb;
      v.e128_group[i128] = (int32_t)g;
    }
    for (int64_t r = lo; r < hi; r += 128, ++iq, p += 128)
      v.qtiles[iq] = make_int4((int)r, (int)min((int64_t)128, hi - r), (int)p, (iq == q_total - 1) ? 1 : 0);
  }
}

int build_grouped_plan(const int64_t* m_offsets_dev, int64_t groups, int64_t rows, void* plan, cudaStream_t st) {
  int* status = device_status_ptr();
  if (!status) return fail(MT_ERR_CUDA, "device status word not reachable");
  grouped_plan_kernel<<<1, PLAN_THREADS, 0, st>>>(m_offsets_dev, groups, rows, plan, status);
  MT_CUDA(cudaGetLastError());
  return MT_OK;
}

}  // namespace mt

extern "C" {

int64_t mt_grouped_plan_bytes(int64_t rows, int64_t groups) {
  if (rows < 0 || groups <= 0 || rows > mt::PLAN_MAX_ROWS || groups > mt::PLAN_MAX_GROUPS) return 0;
  return mt::plan_bytes(rows, groups);
}

int mt_grouped_plan_build(const int64_t* m_offsets, int64_t groups, int64_t rows, void* plan, int64_t plan_bytes,
                          mt_stream_t stream) {
  const char* name = "mt_grouped_plan_build";
  MT_REQUIRE(groups > 0 && groups <= mt::PLAN_MAX_GROUPS, "%s: group count %lld out of range", name, (long long)groups);
  MT_REQUIRE(rows >= 0 && rows <= mt::PLAN_MAX_ROWS, "%s: row count %lld out of range", name, (long long)rows);
  MT_REQUIRE(m_offsets && plan, "%s: null pointer", name);
  MT_REQUIRE(mt::aligned16(plan) && (reinterpret_cast<uintptr_t>(m_offsets) & 7) == 0, "%s: misaligned pointer", name);
  MT_REQUIRE(plan_bytes >= mt::plan_bytes(rows, groups), "%s: plan buffer too small (%lld < %lld bytes)", name,
             (long long)plan_bytes, (long long)mt::plan_bytes(rows, groups));
  return mt::build_grouped_plan(m_offsets, groups, rows, plan, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
