// Tensor-parallel exchange steps over NVLink peer memory, for the ranks of one node (one GPU per
// process, at most MT_MAX_PEERS of them). Every rank owns a small control block and whatever data
// buffers the caller shares; the callers pass tables of the peers' mapped addresses. All
// cross-GPU traffic here is plain peer loads and stores (no multicast of any kind).
//
//   peer barrier        flag exchange through the control blocks; orders a producer kernel on
//                       every rank before a consumer kernel on every rank
//   abs-max exchange    the barrier carrying a few fp32 values, reduced with max: every rank
//                       quantizes its token shard with the abs-max of the whole tensor
//   pull all-gather     copies the peers' shards of several byte tensors into local buffers
//   partial-sum reduce  sums the slices the peers' GEMM epilogues pushed into this rank's staging
//                       buffer (the reduce half of a reduce-scatter), optionally emitting the
//                       abs-max of the result for the next quantize
// Every wait on a peer is bounded: on expiry the kernel raises DS_PEER_WAIT in the device status
// word and returns.
#include <string.h>

#include <algorithm>

#include "mt_common.cuh"

namespace mt {

constexpr int PEER_CHANNELS = 8;
// Control block layout (bytes): flags[channel][src] u32, values[channel][parity][src][4] f32, then
// epoch[channel] u32: the number of exchanges this rank has done on the channel. The epoch lives
// on the device (each exchange kernel increments it), so that a captured sequence of exchanges
// can be replayed: every replay signals and waits for fresh values.
constexpr int CTRL_FLAGS_BYTES = PEER_CHANNELS * MT_MAX_PEERS * 4;
constexpr int CTRL_VALUES_BYTES = PEER_CHANNELS * 2 * MT_MAX_PEERS * 4 * 4;
constexpr int CTRL_EPOCH_OFFSET = CTRL_FLAGS_BYTES + CTRL_VALUES_BYTES;
static_assert(CTRL_EPOCH_OFFSET + PEER_CHANNELS * 4 <= MT_PEER_CTRL_BYTES, "control block too small");

struct PeerTable {
  void* p[MT_MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until *flag has reached `epoch` (wrap-around safe) or the limit has passed.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, int* status, uint64_t timeout_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
    if ((++spins & 63u) == 0 && global_timer_ns() - t0 > timeout_ns) {
      atomicOr(status, DS_PEER_WAIT);
      return false;
    }
  }
  return true;
}

// One warp: lane t signals peer t and waits for peer t's signal. With nvals > 0 the lane first
// writes this rank's values into the peer's control block and afterwards reads the peer's values
// from its own block; vals[] is replaced by the maximum over all ranks.
__global__ void __launch_bounds__(32) peer_exchange_kernel(PeerTable ctrl, int me, int n, int channel, float* vals,
                                                           int nvals, int* status, uint64_t timeout_ns) {
  const int t = threadIdx.x;
  pdl_trigger();
  pdl_wait();   // what this rank announces to its peers is the work of the kernels before this one
  // this exchange's number: one more than the last one on this channel (only this kernel, one
  // launch at a time per channel, touches the counter)
  uint32_t* counter = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ctrl.p[me]) + CTRL_EPOCH_OFFSET) + channel;
  uint32_t epoch = 0;
  if (t == 0) {
    epoch = *counter + 1;
    *counter = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  const int parity = epoch & 1;
  float mine[4] = {0.f, 0.f, 0.f, 0.f}, got[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < nvals; ++i) mine[i] = vals[i];
  bool ok = true;
  if (t < n) {
    uint8_t* remote = static_cast<uint8_t*>(ctrl.p[t]);
    if (nvals > 0) {
      float* rv = reinterpret_cast<float*>(remote + CTRL_FLAGS_BYTES) + ((channel * 2 + parity) * MT_MAX_PEERS + me) * 4;
      for (int i = 0; i < nvals; ++i) rv[i] = mine[i];
    }
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(remote) + channel * MT_MAX_PEERS + me, epoch);
    uint8_t* local = static_cast<uint8_t*>(ctrl.p[me]);
    ok = wait_flag(reinterpret_cast<uint32_t*>(local) + channel * MT_MAX_PEERS + t, epoch, status, timeout_ns);
    if (ok && nvals > 0) {
      const volatile float* lv =
          reinterpret_cast<const volatile float*>(local + CTRL_FLAGS_BYTES) + ((channel * 2 + parity) * MT_MAX_PEERS + t) * 4;
      for (int i = 0; i < nvals; ++i) got[i] = lv[i];
    }
  }
  if (nvals > 0) {
    const bool all_ok = __all_sync(0xffffffffu, ok);
    for (int i = 0; i < nvals; ++i) {
      float m = got[i];
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (t == 0 && all_ok) vals[i] = m;
    }
  }
}

// ---- pull all-gather ----
struct GatherSeg {
  int64_t src_off;      // byte offset of this tensor's shard inside every rank's shared buffer
  uint8_t* dst;         // local destination; rank r's shard lands at dst + r * bytes
  int64_t bytes;        // shard size, a multiple of 16
};
struct GatherArgs {
  PeerTable src;        // the ranks' shared buffers (this rank's own entry included)
  GatherSeg seg[MT_MAX_GATHER_SEGS];
  int nseg, n, me;
};

__device__ __forceinline__ uint4 ld_peer_v4(const uint4* p) {
  uint4 v;   // relaxed system-scope load: never served from a stale L1 line of an earlier step
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Work is cut into units of THREADS * 128 bytes of one (segment, rank); consecutive units belong to
// different ranks, so the CTAs running at one time pull from all peers at once (a single peer at a
// time leaves the copy bound by the round-trip latency of one link), and every rank starts with
// the peer after it. Two shapes: 128-thread CTAs for a copy that has the GPU to itself, and
// 1024-thread CTAs that each claim a whole SM (through a large dynamic shared-memory request) for
// a copy that runs beside a persistent GEMM whose grid leaves that many SMs free: a GEMM CTA
// fills the register file of its SM, so the two kernels cannot share SMs, and a copy spread thinly
// over all SMs would hold up the GEMM's CTAs instead.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) peer_gather_kernel(const GatherArgs a) {
  constexpr int UNIT = THREADS * 16 * 8;   // 8 loads of 16 bytes in flight per thread
  pdl_trigger();
  pdl_wait();
  int64_t first = 0;   // first unit of the current segment
  int64_t u = blockIdx.x;
  for (int s = 0; s < a.nseg; ++s) {
    const GatherSeg g = a.seg[s];
    const int64_t chunks = (g.bytes + UNIT - 1) / UNIT;
    const int64_t units = chunks * a.n;
    for (; u < first + units; u += gridDim.x) {
      const int64_t local = u - first;
      const int r = (a.me + 1 + (int)(local % a.n)) % a.n;
      const int64_t off = (local / a.n) * UNIT;
      const int64_t vecs = min((int64_t)UNIT, g.bytes - off) >> 4;
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.src.p[r]) + g.src_off + off);
      uint4* dst = reinterpret_cast<uint4*>(g.dst + (int64_t)r * g.bytes + off);
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t i = threadIdx.x + k * THREADS;
        if (i < vecs) v[k] = ld_peer_v4(src + i);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int64_t i = threadIdx.x + k * THREADS;
        if (i < vecs) dst[i] = v[k];
      }
    }
    first += units;
  }
}
constexpr int GATHER_EXCLUSIVE_SMEM = 160 * 1024;   // more than half an SM: one such CTA per SM

// ---- reduce of pushed partial sums ----
// stage is [n][rows][cols] bf16 in this rank's memory (slice s written by rank s's GEMM epilogue);
// out[r][c] = bf16(sum_s stage[s][r][c]), summed in fp32 in rank order.
__global__ void __launch_bounds__(256) peer_reduce_kernel(const __nv_bfloat16* __restrict__ stage, int n, int64_t elems,
                                                          __nv_bfloat16* __restrict__ out, float* amax_out) {
  const int64_t vecs = elems >> 3;   // 8 bf16 per 16 bytes
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  pdl_trigger();
  pdl_wait();
  const uint4* src = reinterpret_cast<const uint4*>(stage);
  uint4* dst = reinterpret_cast<uint4*>(out);
  uint32_t am = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += nthreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int s = 0; s < n; ++s) {
      const uint4 v = __ldcg(src + (int64_t)s * vecs + i);   // L2 is where the peers' stores landed
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      o[j] = *reinterpret_cast<uint32_t*>(&h);
      asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(am) : "r"(am), "r"(o[j]));
    }
    dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (amax_out != nullptr) {
    am &= 0x7FFF7FFFu;
    const float m = fmaxf(__uint_as_float(am << 16), __uint_as_float(am & 0xFFFF0000u));
    const uint32_t bits = __reduce_max_sync(0xffffffffu, __float_as_uint(m));
    if ((threadIdx.x & 31) == 0 && bits != 0) atomicMax(reinterpret_cast<unsigned int*>(amax_out), bits);
  }
}

static int check_peers(const char* name, const void* const* table, int n, int me) {
  MT_REQUIRE(table != nullptr, "%s: null peer table", name);
  MT_REQUIRE(n >= 1 && n <= MT_MAX_PEERS && me >= 0 && me < n, "%s: rank %d of %d is out of range (at most %d ranks)", name,
             me, n, MT_MAX_PEERS);
  for (int r = 0; r < n; ++r) MT_REQUIRE(table[r] != nullptr && aligned16(table[r]), "%s: peer %d: null or misaligned address", name, r);
  return MT_OK;
}

static PeerTable make_table(const void* const* table, int n) {
  PeerTable t{};
  for (int r = 0; r < n; ++r) t.p[r] = const_cast<void*>(table[r]);
  return t;
}

}  // namespace mt

extern "C" {

int mt_ipc_export(const void* ptr, uint8_t* handle_out, int64_t* offset_out) {
  MT_REQUIRE(ptr && handle_out && offset_out, "mt_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == MT_IPC_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  MT_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  // the handle names the whole allocation `ptr` lies in: report where inside it `ptr` is
  CUdeviceptr base = 0;
  size_t size = 0;
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = nullptr;
  if (!range_fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return mt::fail(MT_ERR_CUDA, "mt_ipc_export: cuMemGetAddressRange entry point not available");
    range_fn = reinterpret_cast<RangeFn>(p);
  }
  if (range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
    return mt::fail(MT_ERR_CUDA, "mt_ipc_export: address range lookup failed");
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = (int64_t)(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return MT_OK;
}

int mt_ipc_import(const uint8_t* handle, int64_t offset, void** ptr_out) {
  MT_REQUIRE(handle && ptr_out && offset >= 0, "mt_ipc_import: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* base = nullptr;
  MT_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr_out = static_cast<uint8_t*>(base) + offset;
  return MT_OK;
}

int mt_ipc_close(void* ptr, int64_t offset) {
  MT_REQUIRE(ptr && offset >= 0, "mt_ipc_close: bad argument");
  MT_CUDA(cudaIpcCloseMemHandle(static_cast<uint8_t*>(ptr) - offset));
  return MT_OK;
}

int mt_peer_barrier(const void* const* ctrl, int n, int me, int channel, mt_stream_t stream) {
  int rc = mt::check_peers("mt_peer_barrier", ctrl, n, me);
  if (rc != MT_OK) return rc;
  MT_REQUIRE(channel >= 0 && channel < mt::PEER_CHANNELS, "mt_peer_barrier: channel %d out of range", channel);
  int* status = mt::device_status_ptr();
  if (!status) return mt::fail(MT_ERR_CUDA, "device status word not reachable");
  MT_CUDA(mt::launch_pdl(mt::peer_exchange_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                         mt::make_table(ctrl, n), me, n, channel, (float*)nullptr, 0, status, (uint64_t)2000000000ull));
  return MT_OK;
}

int mt_peer_allreduce_max(const void* const* ctrl, int n, int me, int channel, float* vals, int nvals,
                          mt_stream_t stream) {
  int rc = mt::check_peers("mt_peer_allreduce_max", ctrl, n, me);
  if (rc != MT_OK) return rc;
  MT_REQUIRE(channel >= 0 && channel < mt::PEER_CHANNELS, "mt_peer_allreduce_max: channel %d out of range", channel);
  MT_REQUIRE(vals != nullptr && nvals >= 1 && nvals <= 4, "mt_peer_allreduce_max: 1 to 4 values");
  int* status = mt::device_status_ptr();
  if (!status) return mt::fail(MT_ERR_CUDA, "device status word not reachable");
  MT_CUDA(mt::launch_pdl(mt::peer_exchange_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                         mt::make_table(ctrl, n), me, n, channel, vals, nvals, status, (uint64_t)2000000000ull));
  return MT_OK;
}

int mt_peer_gather(const void* const* shared, int n, int me, const int64_t* src_offsets, void* const* dsts,
                   const int64_t* shard_bytes, int nseg, int ctas, int whole_sms, mt_stream_t stream) {
  const char* name = "mt_peer_gather";
  int rc = mt::check_peers(name, shared, n, me);
  if (rc != MT_OK) return rc;
  MT_REQUIRE(src_offsets && dsts && shard_bytes && nseg >= 1 && nseg <= MT_MAX_GATHER_SEGS, "%s: 1 to %d segments", name,
             MT_MAX_GATHER_SEGS);
  MT_REQUIRE(ctas >= 1 && ctas <= 4096, "%s: CTA count %d out of range", name, ctas);
  mt::GatherArgs a{};
  a.src = mt::make_table(shared, n);
  a.nseg = nseg; a.n = n; a.me = me;
  for (int s = 0; s < nseg; ++s) {
    MT_REQUIRE(dsts[s] && mt::aligned16(dsts[s]) && src_offsets[s] >= 0 && src_offsets[s] % 16 == 0 && shard_bytes[s] >= 0 &&
               shard_bytes[s] % 16 == 0, "%s: segment %d: addresses and sizes must be multiples of 16 bytes", name, s);
    a.seg[s].src_off = src_offsets[s];
    a.seg[s].dst = static_cast<uint8_t*>(dsts[s]);
    a.seg[s].bytes = shard_bytes[s];
  }
  if (whole_sms) {
    auto kern = mt::peer_gather_kernel<1024>;
    static bool attr_set[mt::MT_MAX_DEVICES] = {};
    const int slot = mt::current_device_slot();
    if (!attr_set[slot]) {
      MT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, mt::GATHER_EXCLUSIVE_SMEM));
      attr_set[slot] = true;
    }
    // launched as clusters of two, which the hardware places on the two SMs of one TPC: the
    // CTA pairs of the GEMM beside it need whole TPCs, so the copy should not break up more
    // of them than it has to
    MT_REQUIRE(ctas % 2 == 0, "%s: a whole-SM copy takes an even number of CTAs", name);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(1024);
    cfg.dynamicSmemBytes = mt::GATHER_EXCLUSIVE_SMEM;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    MT_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  } else {
    MT_CUDA(mt::launch_pdl(mt::peer_gather_kernel<128>, dim3((unsigned)ctas), dim3(128), 0, static_cast<cudaStream_t>(stream), a));
  }
  MT_CUDA(cudaGetLastError());
  return MT_OK;
}

int mt_peer_reduce_bf16(const void* stage, int n, int64_t rows, int64_t cols, void* out, float* amax_out,
                        mt_stream_t stream) {
  const char* name = "mt_peer_reduce_bf16";
  MT_REQUIRE(stage && out && mt::aligned16(stage) && mt::aligned16(out), "%s: null or misaligned pointer", name);
  MT_REQUIRE(n >= 1 && n <= MT_MAX_PEERS && rows >= 0 && cols >= 0 && (rows * cols) % 8 == 0,
             "%s: up to %d slices of rows * cols (a multiple of 8) elements", name, MT_MAX_PEERS);
  if (rows * cols == 0) return MT_OK;
  const int64_t vecs = rows * cols / 8;
  const int blocks = (int)std::min<int64_t>((vecs + 255) / 256, 148 * 8);
  MT_CUDA(mt::launch_pdl(mt::peer_reduce_kernel, dim3((unsigned)blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                         static_cast<const __nv_bfloat16*>(stage), n, rows * cols, static_cast<__nv_bfloat16*>(out), amax_out));
  return MT_OK;
}

}  // extern "C"
