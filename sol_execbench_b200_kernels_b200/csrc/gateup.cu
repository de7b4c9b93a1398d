// Host side of libgateup.so: argument checks, TMA descriptor encoding, the
// shape heuristic and the extern "C" entry points declared in include/gateup.h.
// Takes over what the reference does in its pybind `run` and
// `launch_fp8_mlp_gate_up` (variants/cuda_cpp_v4/binding.cpp:18-81,
// variants/cuda_cpp_v4/kernel.cu:185-233, 271-341), for any (M, K, N) with
// K and N multiples of 128.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "../../include/gateup.h"
#include "gateup_stream.cuh"
#include "gateup_pair.cuh"
#include "gateup_tile.cuh"
#include "quantize_act.cuh"
#include "reduce_gather.cuh"

namespace gu {
namespace {

// ---------------------------------------------------------------------------
// driver entry point for tensor-map encoding (no link-time libcuda dependency,
// so the library also loads on a machine without a driver)
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t cols, rows, pitch_bytes;
  uint32_t box_cols, box_rows, dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && cols == o.cols && rows == o.rows && pitch_bytes == o.pitch_bytes &&
           box_cols == o.box_cols && box_rows == o.box_rows && dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9e3779b97f4a7c15ull;
    h ^= (k.cols + 0x632be59bd9b4e019ull) * 0xff51afd7ed558ccdull;
    h ^= (k.rows << 17) ^ (k.pitch_bytes << 3) ^ (uint64_t(k.box_rows) << 40) ^ (uint64_t(k.box_cols) << 52) ^ k.dtype;
    return static_cast<size_t>(h ^ (h >> 29));
  }
};

std::mutex g_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;  // encoded descriptors, keyed by what they describe

// Row-major 2-D tensor [rows, cols] with a row pitch, box [box_rows, box_cols],
// 128-byte swizzle (box_cols * element size must be 128 bytes).
int get_map(CUtensorMap* out, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* ptr, uint64_t cols,
            uint64_t rows, uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows) {
  MapKey key{ptr, cols, rows, pitch_bytes, box_cols, box_rows, static_cast<uint32_t>(dtype)};
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *out = it->second;
      return GU_OK;
    }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return GU_ECUDA;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  (void)elem_bytes;
  CUresult r = fn(out, dtype, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return GU_ECUDA;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, *out);
  return GU_OK;
}

struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  int max_smem_optin = 0;
  int pair_clusters = 0;  // CTA pairs of the pair kernel that are resident at once (0: pairs cannot be launched)
  bool attrs_set = false;
};
DeviceInfo g_dev[64];

int device_info(DeviceInfo** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GU_ECUDA;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return GU_ECUDA;
    if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return GU_ECUDA;
    if (cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
      return GU_ECUDA;
    d.ready = true;
  }
  if (d.cc_major != 10) return GU_EDEVICE;
  if (!d.attrs_set) {
    const int smem = d.max_smem_optin;
    if (cudaFuncSetAttribute(gateup_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_tile_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(blockwise_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_tile_fp8out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(blockwise_gemm_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_stream_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_stream_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_stream_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaFuncSetAttribute(blockwise_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_pair_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_pair_sk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gateup_pair_fp8out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(blockwise_gemm_pair_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess) {
      cudaGetLastError();
      return GU_ECUDA;
    }
    {
      // how many two-CTA clusters of the pair kernel the device holds at once (one CTA per SM)
      cudaLaunchConfig_t cfg;
      std::memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3(2 * static_cast<unsigned>(d.sm_count), 1, 1);
      cfg.blockDim = dim3(kPairThreads, 1, 1);
      cfg.dynamicSmemBytes = kPairSmemBytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, gateup_pair_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        clusters = 0;
      }
      d.pair_clusters = clusters;
    }
    d.attrs_set = true;
  }
  *out = &d;
  return GU_OK;
}

// One CTA whose only wait is on a barrier that nothing ever arrives on: the bounded-wait protocol of the real
// kernels (mbar_wait, WaitCtx::fail, the CTA abort flag) run to its time limit, with no copy or MMA in flight.
constexpr unsigned kWaitProbe = 31;
__global__ void wait_probe_kernel() {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtx ctx{smem_u32(&abort_flag), false, false};
  if (threadIdx.x == 0) mbar_wait(ctx, smem_u32(&bar), 0u, kWaitProbe);  // gives up after the wait limit
  __syncthreads();
  // every other thread finds the CTA aborting and returns at once, as the roles of the real kernels do
  if (threadIdx.x != 0) mbar_wait(ctx, smem_u32(&bar), 0u, kWaitProbe);
}

std::atomic<unsigned int> g_epoch{0};

// A stamp no earlier call of this process has used for its hand-off flags; never 0.
unsigned int next_epoch() {
  unsigned int e = g_epoch.fetch_add(1, std::memory_order_relaxed) + 1;
  if (e == 0) e = g_epoch.fetch_add(1, std::memory_order_relaxed) + 1;
  return e;
}
std::atomic<long long> g_launches{0};

constexpr int kSmemBudget = 227 * 1024;

inline int stream_mpad(int64_t m) { return m <= 16 ? 16 : (m <= 32 ? 32 : 64); }

// Ring depth of the streaming kernel: as deep as shared memory allows, 0 if fewer than 3 stages fit.
int stream_stages(int mpad, int64_t kb) {
  const int64_t stage = 2 * kOperandTileBytes + int64_t(mpad) * 128;
  const int64_t fixed = 512 + kb * mpad * 4 + 1024;
  int64_t s = (kSmemBudget - fixed) / stage;
  if (s > kStreamMaxStages) s = kStreamMaxStages;
  return s >= 3 ? static_cast<int>(s) : 0;
}

// SM count of the current device, or the B200's 148 when no device can be asked (sizing queries on a CPU box).
int sm_count_or_default() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
    return sms;
  cudaGetLastError();
  return 148;
}

// Tile kernel schedule.  The stream-K schedule (whole rounds data-parallel, the last one to two rounds' worth of
// tiles cut into equal unit ranges) balances awkward tile counts, but measured on B200 its hand-off cost
// (publish, gather, a second launch) cancels the gain at every size tried: 128 x 4096 x 14336 takes 38.9 us
// against 30.7 us data-parallel, 512 rows 89.1 against 86.0, 1024 rows 148.5 against 145.4.  So the heuristic
// keeps the data-parallel schedule; GU_PLAN_TILE_SK still selects stream-K explicitly.
bool tile_prefers_stream_k(int64_t, int64_t, int64_t, int) { return false; }

size_t tile_stream_k_bytes() { return kTileFlagBytes + size_t(kTileMaxGrid) * kTilePartialFloats * sizeof(float); }

bool shape_ok(int64_t m, int64_t k, int64_t n) {
  return m >= 1 && k >= 128 && n >= 128 && (k % 128) == 0 && (n % 128) == 0 && m < (1ll << 31) &&
         k < (1ll << 31) && n < (1ll << 31);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// CTAs of `threads` threads of `kernel` that one SM holds at once (at least 1), by the runtime's occupancy query
template <typename Kernel>
int resident_ctas(Kernel kernel, int threads) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
  return n;
}

int check_problem(const gu_problem* pr) {
  if (!pr) return GU_EINVAL_NULL;
  if (!pr->x || !pr->scale_x || !pr->gate_w || !pr->scale_gate || !pr->up_w || !pr->scale_up || !pr->output)
    return GU_EINVAL_NULL;
  if (!shape_ok(pr->m, pr->k, pr->n)) return GU_EINVAL_SHAPE;
  if (pr->ld_output < pr->n) return GU_EINVAL_SHAPE;
  if (!aligned16(pr->x) || !aligned16(pr->gate_w) || !aligned16(pr->up_w) || !aligned16(pr->output) ||
      (reinterpret_cast<uintptr_t>(pr->scale_x) & 3u) || (reinterpret_cast<uintptr_t>(pr->scale_gate) & 3u) ||
      (reinterpret_cast<uintptr_t>(pr->scale_up) & 3u) || (pr->ld_output % 8) != 0)
    return GU_EINVAL_ALIGN;
  return GU_OK;
}

int launch_tile(const gu_problem* pr, const DeviceInfo& dev, cudaStream_t stream, bool stream_k) {
  const int64_t m = pr->m, k = pr->k, n = pr->n;
  CUtensorMap tm_x, tm_g, tm_u, tm_o;
  int rc;
  if ((rc = get_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->x, k, m, k, 128, 128)) != GU_OK) return rc;
  if ((rc = get_map(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->gate_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = get_map(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->up_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = get_map(&tm_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pr->output, n, m, pr->ld_output * 2, 64, 128)) !=
      GU_OK)
    return rc;

  TileParams p;
  p.scale_x = pr->scale_x;
  p.scale_gate = pr->scale_gate;
  p.scale_up = pr->scale_up;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.num_m_blocks = static_cast<int>((m + kTileM - 1) / kTileM);
  p.num_n_blocks = static_cast<int>(n / kTileN);
  const int64_t tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
  if (tiles * (k / 128) >= (1ll << 31)) return GU_EINVAL_SHAPE;  // the schedules count (tile, K block) units in 32 bits
  p.num_tiles = static_cast<int>(tiles);
  // raster group: as many M blocks as keep the group's X tiles (128 x K bytes each) within ~24 MiB of L2
  int64_t gm = (24ll << 20) / (128 * k);
  if (gm < 1) gm = 1;
  if (gm > p.num_m_blocks) gm = p.num_m_blocks;
  p.group_m = static_cast<int>(gm);

  p.flags = nullptr;
  p.partials = nullptr;
  p.epoch = 0;
  p.tile_begin = 0;
  p.out_count = 1;
  p.out_rank = 0;
  p.out_col0 = 0;
  p.n_blocks128 = 0;
  p.scale_out = nullptr;
  p.blocks_per_owner = 1;
  p.slot_rows = 0;
  p.out_rows = static_cast<int>(m);
  p.out_cols = static_cast<int>(n);
  const int total_tiles = p.num_tiles;
  const int sms = dev.sm_count;
  // Hybrid schedule: whole rounds of tiles run data-parallel; the last round plus the remainder (between one and
  // two rounds' worth of tiles, or everything when there is less than one round) is split into equal unit ranges.
  // (Splitting only the remainder was measured too: a tile cut 32 ways makes its owner gather 31 partials one
  // after the other, 134 us against 85 us data-parallel at M=512, K=4096, N=14336.)
  int dp_tiles = total_tiles;
  if (stream_k) {
    const int rounds = total_tiles / sms;
    dp_tiles = (total_tiles % sms == 0) ? total_tiles : (rounds >= 1 ? (rounds - 1) * sms : 0);
  }
  if (dp_tiles > 0) {
    p.num_tiles = dp_tiles;
    const int grid = dp_tiles < sms ? dp_tiles : sms;
    gateup_tile_kernel<false><<<grid, kTileThreads, kTileSmemBytes, stream>>>(tm_x, tm_g, tm_u, tm_o, p);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (cudaGetLastError() != cudaSuccess) return GU_ECUDA;
  }
  if (dp_tiles < total_tiles) {
    p.tile_begin = dp_tiles;
    p.num_tiles = total_tiles - dp_tiles;
    int64_t grid = sms < kTileMaxGrid ? sms : kTileMaxGrid;
    const int64_t units = int64_t(p.num_tiles) * p.kb;
    if (units < grid) grid = units;
    // words [256, 512) of the flag block: the streaming kernel stamps words [0, 256) of the same workspace with
    // epochs of its own counter, and a stale stamp of one kernel must never look like the other's epoch
    p.flags = static_cast<unsigned int*>(pr->workspace) + 256;
    p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(pr->workspace) + kTileFlagBytes);
    p.epoch = next_epoch();
    gateup_tile_kernel<true><<<static_cast<int>(grid), kTileThreads, kTileSmemBytes, stream>>>(tm_x, tm_g, tm_u, tm_o, p);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (cudaGetLastError() != cudaSuccess) return GU_ECUDA;
  }
  return GU_OK;
}

// CTA-pair kernel: 256-token x 128-column tiles, one per two-CTA cluster.
// Stream-K schedule of the pair kernel (whole rounds as whole tiles, the last whole round plus the remainder cut into
// equal unit ranges).  Possible when no tile spans more than two ranges (at least as many tiles as clusters).  Its
// hand-off (one 128 KiB publish and one 128 KiB fix-up per CTA, a K block more on the critical path, and the last
// tile's SwiGLU on two warps only) costs about 8 us per launch, measured on B200 at K=4096, N=14336 against whole
// tiles: 512 tokens (3.03 rounds) 73.8 against 77.8 us, 1024 (6.05) 123.7 against 127.3, 2048 (12.1) 229.4 against
// 231.5, 4096 (24.2) within the noise; 256 tokens (1.51 rounds, no whole round before the cut) 55.2 against 47.1, and
// 2 - 4 us lost where the tiles divide evenly.  So the heuristic wants two rounds or more, at least 10 % of the
// device idle in the last round of whole tiles, and a last round less than 0.3 full.
bool pair_can_stream_k(int tiles, int clusters) {
  // one flag word and one 128 KiB slot of the scratch per CTA
  return clusters >= 2 && tiles >= clusters && 2 * clusters <= kPairMaxCtas && 2 * clusters <= kTileMaxGrid;
}
bool pair_prefers_stream_k(int tiles, int clusters) {
  if (!pair_can_stream_k(tiles, clusters) || tiles < 2 * clusters || tiles % clusters == 0) return false;
  const int rounds = (tiles + clusters - 1) / clusters;
  // (the hand-off is worth about 0.7 of a round: 3.57 rounds at K=2048 ran 55.8 us cut against 53.2 us whole)
  return double(tiles) / (double(rounds) * clusters) < 0.90 && double(tiles) / clusters + 0.7 < double(rounds);
}

int launch_pair(const gu_problem* pr, const DeviceInfo& dev, cudaStream_t stream, int stream_k /* 0 no, 1 yes, -1 by the heuristic */) {
  const int64_t m = pr->m, k = pr->k, n = pr->n;
  if (dev.pair_clusters < 1) return GU_EINVAL_PLAN;
  CUtensorMap tm_x, tm_g, tm_u, tm_o;
  int rc;
  if ((rc = get_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->x, k, m, k, 128, 128)) != GU_OK) return rc;
  if ((rc = get_map(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->gate_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = get_map(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->up_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = get_map(&tm_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pr->output, n, m, pr->ld_output * 2, 64, 128)) !=
      GU_OK)
    return rc;

  TileParams p;
  std::memset(&p, 0, sizeof(p));
  p.scale_x = pr->scale_x;
  p.scale_gate = pr->scale_gate;
  p.scale_up = pr->scale_up;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.num_m_blocks = static_cast<int>((m + 2 * kTileM - 1) / (2 * kTileM));  // 256-token pair blocks
  p.num_n_blocks = static_cast<int>(n / kTileN);
  const int64_t tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
  if (tiles * (k / 128) >= (1ll << 31)) return GU_EINVAL_SHAPE;
  p.num_tiles = static_cast<int>(tiles);
  // raster group: as many pair blocks as keep the group's X rows (256 x K bytes each) within ~24 MiB of L2
  int64_t gm = (24ll << 20) / (256 * k);
  if (gm < 1) gm = 1;
  if (gm > p.num_m_blocks) gm = p.num_m_blocks;
  p.group_m = static_cast<int>(gm);
  p.out_count = 1;
  p.blocks_per_owner = 1;
  p.out_rows = static_cast<int>(m);
  p.out_cols = static_cast<int>(n);

  const int clusters = p.num_tiles < dev.pair_clusters ? p.num_tiles : dev.pair_clusters;
  const bool have_ws = pr->workspace && pr->workspace_bytes >= tile_stream_k_bytes() && aligned16(pr->workspace);
  bool sk = false;
  if (stream_k == 1) {
    if (!have_ws) return GU_EWORKSPACE;
    if (!pair_can_stream_k(p.num_tiles, clusters)) return GU_EINVAL_PLAN;
    sk = true;
  } else if (stream_k == -1) {
    // without scratch the data-parallel schedule is used: slower on awkward tile counts, never wrong
    sk = have_ws && pair_prefers_stream_k(p.num_tiles, clusters);
  }
  if (sk) {
    // whole rounds but the last run as whole tiles; the last whole round and the remainder are cut into unit ranges
    const int rounds = p.num_tiles / clusters;
    p.tile_begin = (rounds - 1) * clusters;
    p.flags = static_cast<unsigned int*>(pr->workspace);
    p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(pr->workspace) + kTileFlagBytes);
    gateup_pair_sk_kernel<<<2 * clusters, kPairThreads, kPairSmemBytes, stream>>>(tm_x, tm_g, tm_u, tm_o, p);
  } else {
    gateup_pair_kernel<<<2 * clusters, kPairThreads, kPairSmemBytes, stream>>>(tm_x, tm_g, tm_u, tm_o, p);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

// The tile plan's kernel for a shape: CTA pairs once there is more than one 128-token block (a lone block would
// leave the second CTA of every pair without rows), the lone-CTA kernel otherwise.
bool tile_prefers_pairs(int64_t m, const DeviceInfo& dev) { return m > kTileM && dev.pair_clusters >= 1; }

// The choice between the two tile kernels for more than one 128-token block.  The lone-CTA kernel needs about 1.21
// times as long for the same work (its MMAs read every weight row from the CTA's own shared memory) but it schedules
// 128-token blocks on single SMs, starts and ends a few microseconds sooner (worth about 16 K blocks) and has four
// epilogue warps per 128 x 128 outputs where the pair kernel has two, so it wins where the pair kernel's rounds come
// out badly — an odd number of 128-token blocks (a third block costs the pair kernel a whole 256-token block) — or
// where a tile has so few K blocks that the pair kernel's epilogue takes longer than its K loop.  Costs are counted
// in K blocks of the pair kernel: rounds x max(K blocks per tile, the epilogue's length in K blocks); the pair
// kernel's stream-K schedule costs the fraction of rounds it runs plus 0.7 of a round.  Measured on B200 over 129 ...
// 4096 tokens.  Gate/up, bf16 output, (K, N) = (4096, 14336), (8192, 28672), (7168, 2304), (2048, 5632), (3584,
// 18944), (5120, 13824), (1024, 4096), (4096, 4736): the kernel picked this way is within 7 % of the fastest
// everywhere; with pairs for every M > 128 it was up to 66 % behind (384 tokens at (2048, 5632): 30.7 us against
// 18.4 us) and 9 - 14 % behind at 320 - 384 tokens on the large shapes.  Gate/up with e4m3 output: the pair kernel's
// two epilogue warps need about 29 K blocks' time per tile, so at K = 2048 the lone kernel is 21 - 105 % faster at
// every M (4096 tokens: 118.8 against 144.3 us), at K = 4096 only on odd block counts (384 tokens: 68.1 against
// 79.9 us).  Single GEMM, (K, N) = (14336, 4096), (5632, 2048), (4096, 4096): pairs except where the lone kernel
// saves a round (1152 tokens: 71.8 against 105.5 us).  Both kernels give the same bits when no tile is cut along K.
enum TileOp { kOpGateUp = GU_OP_GATEUP, kOpGateUpFp8 = GU_OP_GATEUP_FP8, kOpGemm = GU_OP_GEMM };
bool tile_prefers_lone(int op, int64_t m, int64_t kb, int64_t col_tiles, int sm_count, int pair_clusters, bool scratch) {
  if (m <= kTileM || pair_clusters < 1) return true;
  const int64_t lone_tiles = ((m + kTileM - 1) / kTileM) * col_tiles;
  const int64_t pair_tiles = ((m + 2 * kTileM - 1) / (2 * kTileM)) * col_tiles;
  if (pair_tiles >= (1ll << 31) || sm_count < 1) return false;
  const double lone_rounds = double((lone_tiles + sm_count - 1) / sm_count);
  const int clusters = pair_tiles < pair_clusters ? static_cast<int>(pair_tiles) : pair_clusters;
  double pair_rounds = double((pair_tiles + clusters - 1) / clusters);
  if (op == kOpGateUp && scratch && pair_prefers_stream_k(static_cast<int>(pair_tiles), clusters)) {
    const double cut = double(pair_tiles) / clusters + 0.7;
    if (cut < pair_rounds) pair_rounds = cut;
  }
  // epilogue lengths in K blocks (pair, lone) and the lone kernel's head start
  const double pair_epi = op == kOpGateUp ? 18.0 : op == kOpGateUpFp8 ? 29.0 : 0.0;
  const double lone_epi = op == kOpGateUpFp8 ? 20.0 : 0.0;
  const double head_start = op == kOpGemm ? 0.0 : 16.0;
  const double kbd = double(kb);
  const double pair_cost = pair_rounds * (kbd > pair_epi ? kbd : pair_epi);
  const double lone_cost = 1.21 * lone_rounds * (kbd > lone_epi ? kbd : lone_epi);
  return lone_cost <= pair_cost + head_start - 0.1 * kbd;
}

// Tile geometry of a pair launch: 256-token pair blocks x `col_tiles` column tiles, raster groups that keep a
// group's activation rows (256 x K bytes per pair block) within ~24 MiB of L2.  Returns the number of clusters to
// launch, or 0 when the schedule's 32-bit (tile, K block) count would overflow.
int pair_geometry(TileParams& p, const DeviceInfo& dev, int64_t m, int64_t k, int col_tiles) {
  p.num_m_blocks = static_cast<int>((m + 2 * kTileM - 1) / (2 * kTileM));
  p.num_n_blocks = col_tiles;
  const int64_t tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
  if (tiles * (k / 128) >= (1ll << 31)) return 0;
  p.num_tiles = static_cast<int>(tiles);
  int64_t gm = (24ll << 20) / (256 * k);
  if (gm < 1) gm = 1;
  if (gm > p.num_m_blocks) gm = p.num_m_blocks;
  p.group_m = static_cast<int>(gm);
  return p.num_tiles < dev.pair_clusters ? p.num_tiles : dev.pair_clusters;
}

template <int MPAD>
int launch_stream_t(const gu_problem* pr, const DeviceInfo& dev, cudaStream_t stream, int stages) {
  const int64_t m = pr->m, k = pr->k, n = pr->n;
  CUtensorMap tm_x, tm_g, tm_u;
  int rc;
  if ((rc = get_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->x, k, m, k, 128, MPAD)) != GU_OK) return rc;
  if ((rc = get_map(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->gate_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = get_map(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->up_w, k, n, k, 128, 128)) != GU_OK) return rc;

  StreamParams p;
  p.scale_x = pr->scale_x;
  p.scale_gate = pr->scale_gate;
  p.scale_up = pr->scale_up;
  p.out = static_cast<__nv_bfloat16*>(pr->output);
  p.ld_out = pr->ld_output;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>(n / 128);
  p.stages = stages;
  p.flags = static_cast<unsigned int*>(pr->workspace);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(pr->workspace) + kStreamFlagBytes);

  const int64_t units = int64_t(p.nb) * p.kb;
  int64_t grid = dev.sm_count < kStreamMaxGrid ? dev.sm_count : kStreamMaxGrid;
  if (units < grid) grid = units;
  const uint32_t smem = StreamCfg<MPAD>::smem_bytes(stages, p.kb);
  gateup_stream_kernel<MPAD><<<static_cast<int>(grid), kStreamThreads, smem, stream>>>(tm_x, tm_g, tm_u, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}


// ---------------------------------------------------------------------------
// Built-in scratch for gu_run_decode_static.
//
// Some hosts of this library may not allocate device memory at all: a serving
// runtime that claims all of HBM for its own arena at start-up and forbids
// cudaMalloc afterwards, or a decode loop that cannot afford the device-wide
// synchronisation an allocation implies.  For them the stream-K hand-off scratch
// of the decode kernel lives in this file-scope array instead of in a
// caller-supplied workspace.  It is sized for at most kStaticMaxTokens tokens
// (4 KiB of flags + 256 ranges x 2 x 16 x 128 fp32 = 4 MiB + 4 KiB), and every
// GPU that loads the library carries it until the process exits.
//
// In host code the array's name is only a stand-in for the symbol; the device
// address is obtained with cudaGetSymbolAddress, once per device, with that
// device current (static_scratch_ptr below), and passed to the kernel.
// ---------------------------------------------------------------------------
constexpr int kStaticMaxTokens = 16;
constexpr size_t kStaticScratchBytes =
    kStreamFlagBytes + size_t(kStreamMaxGrid) * 2 * kStaticMaxTokens * 128 * sizeof(float);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

void* g_static_ptr[64] = {nullptr};

int static_scratch_ptr(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GU_ECUDA;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) {
      cudaGetLastError();
      return GU_ECUDA;
    }
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return GU_OK;
}

// Descriptor encoding straight into caller storage: no cache entry, so no host allocation either.
int encode_map_uncached(CUtensorMap* out, const void* ptr, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return GU_ECUDA;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GU_OK : GU_ECUDA;
}

}  // namespace
}  // namespace gu

extern "C" {

int gu_version(void) { return GU_VERSION; }

const char* gu_error_string(int code) {
  switch (code) {
    case GU_OK: return "ok";
    case GU_EINVAL_NULL: return "a required pointer is null";
    case GU_EINVAL_SHAPE: return "unsupported shape: need M >= 1, K and N positive multiples of 128, ld_output >= N";
    case GU_EINVAL_ALIGN: return "pointers must be 16-byte aligned and ld_output a multiple of 8";
    case GU_EINVAL_PLAN: return "unknown plan, or the plan cannot run this shape on this device";
    case GU_EWORKSPACE: return "workspace missing or too small (see gu_workspace_bytes)";
    case GU_ECUDA: return "a CUDA call failed";
    case GU_EDEVICE: return "the current device is not compute capability 10.x";
    case GU_ETIMEOUT: return "a bounded device-side wait gave up";
    case GU_ESTATIC_LIMIT: return "gu_run_decode_static: at most 16 tokens fit the built-in scratch";
    case GU_EBOUNDS: return "the range-checked debug build found an index or coordinate outside its extent";
    default: return "unknown error";
  }
}

int gu_select_plan(int64_t m, int64_t k, int64_t n) {
  if (!gu::shape_ok(m, k, n)) return GU_EINVAL_SHAPE;
  // Measured crossover on B200 (both kernels on the same shapes): with up to 16 tokens the weight-streaming
  // kernel wins or ties once the weights exceed ~64 MB (its equal unit ranges keep all SMs streaming whatever
  // N/128 is); with 17-32 tokens it still wins on large weights (M=32, K=8192, N=28672: 84 us against 94 us)
  // but loses on mid-sized ones (K=4096, N=14336: 34.6 us against 28.8 us); from 33 tokens on the tile kernel
  // is faster everywhere (its consumers do one FMA per element, the streaming kernel's do two).
  const int64_t weight_bytes = 2 * n * k;
  const bool can_stream = m <= 64 && gu::stream_stages(gu::stream_mpad(m), k / 128) > 0;
  if (can_stream && ((m <= 16 && weight_bytes >= (64ll << 20)) || (m <= 32 && weight_bytes >= (256ll << 20))))
    return GU_PLAN_STREAM;
  return GU_PLAN_TILE;
}

int gu_select_tile_kernel(int op, int64_t m, int64_t k, int64_t n, int with_workspace) {
  if (!gu::shape_ok(m, k, n)) return GU_EINVAL_SHAPE;
  if (op != GU_OP_GATEUP && op != GU_OP_GATEUP_FP8 && op != GU_OP_GEMM) return GU_EINVAL_PLAN;
  const int sms = gu::sm_count_or_default(), clusters = sms / 2;
  const int64_t col_tiles = op == GU_OP_GEMM ? (n / 128 + 1) / 2 : n / gu::kTileN;
  if (gu::tile_prefers_lone(op, m, k / 128, col_tiles, sms, clusters, with_workspace != 0)) {
    const bool cut = op == GU_OP_GATEUP && with_workspace && m <= gu::kTileM && gu::tile_prefers_stream_k(m, k, n, sms);
    return cut ? GU_PLAN_TILE_SK : GU_PLAN_TILE_DP;
  }
  const int64_t tiles = ((m + 2 * gu::kTileM - 1) / (2 * gu::kTileM)) * col_tiles;
  const int used = tiles < clusters ? static_cast<int>(tiles) : clusters;
  return op == GU_OP_GATEUP && with_workspace && gu::pair_prefers_stream_k(static_cast<int>(tiles), used)
             ? GU_PLAN_TILE_PAIR_SK
             : GU_PLAN_TILE_PAIR;
}

size_t gu_workspace_bytes(int64_t m, int64_t k, int64_t n, int plan) {
  if (!gu::shape_ok(m, k, n)) return 0;
  if (plan == GU_PLAN_AUTO) plan = gu_select_plan(m, k, n);
  if (plan == GU_PLAN_STREAM && m <= 64)
    return gu::kStreamFlagBytes + size_t(gu::kStreamMaxGrid) * 2 * gu::stream_mpad(m) * 128 * sizeof(float);
  if (plan == GU_PLAN_TILE_SK || plan == GU_PLAN_TILE_PAIR_SK) return gu::tile_stream_k_bytes();
  if (plan == GU_PLAN_TILE) {
    // what the tile plan would launch on a B200 (one cluster per two SMs): scratch only where stream-K is chosen
    const int clusters = gu::sm_count_or_default() / 2;
    const int64_t tiles = ((m + 255) / 256) * (n / 128);
    if (m > gu::kTileM && tiles < (1ll << 31) && gu::pair_prefers_stream_k(static_cast<int>(tiles), clusters) &&
        !gu::tile_prefers_lone(gu::kOpGateUp, m, k / 128, n / gu::kTileN, gu::sm_count_or_default(), clusters, true))
      return gu::tile_stream_k_bytes();
    if (m <= gu::kTileM && gu::tile_prefers_stream_k(m, k, n, gu::sm_count_or_default())) return gu::tile_stream_k_bytes();
  }
  return 0;
}

int gu_workspace_init(void* workspace, size_t bytes, void* stream) {
  if (!workspace || bytes == 0) return GU_OK;
  const size_t n = bytes < gu::kStreamFlagBytes ? bytes : gu::kStreamFlagBytes;
  return cudaMemsetAsync(workspace, 0, n, static_cast<cudaStream_t>(stream)) == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_run(const gu_problem* pr, void* stream_v) {
  int rc = gu::check_problem(pr);
  if (rc != GU_OK) return rc;
  int plan = pr->plan;
  if (plan == GU_PLAN_AUTO) plan = gu_select_plan(pr->m, pr->k, pr->n);
  if (plan != GU_PLAN_TILE && plan != GU_PLAN_STREAM && plan != GU_PLAN_TILE_DP && plan != GU_PLAN_TILE_SK &&
      plan != GU_PLAN_TILE_PAIR && plan != GU_PLAN_TILE_PAIR_SK)
    return GU_EINVAL_PLAN;
  gu::DeviceInfo* dev = nullptr;
  if ((rc = gu::device_info(&dev)) != GU_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (plan == GU_PLAN_TILE_PAIR) return gu::launch_pair(pr, *dev, stream, 0);
  if (plan == GU_PLAN_TILE_PAIR_SK) return gu::launch_pair(pr, *dev, stream, 1);
  const bool have_ws = pr->workspace && pr->workspace_bytes >= gu::tile_stream_k_bytes() && gu::aligned16(pr->workspace);
  if (plan == GU_PLAN_TILE && pr->m > gu::kTileM) {
    if (!gu::tile_prefers_lone(gu::kOpGateUp, pr->m, pr->k / 128, pr->n / gu::kTileN, dev->sm_count, dev->pair_clusters,
                               have_ws))
      return gu::launch_pair(pr, *dev, stream, -1);
    plan = GU_PLAN_TILE_DP;  // whole 128-token tiles on single SMs
  }
  if (plan != GU_PLAN_STREAM) {
    bool sk = false;
    if (plan == GU_PLAN_TILE_SK) {
      if (!have_ws) return GU_EWORKSPACE;
      sk = true;
    } else if (plan == GU_PLAN_TILE) {
      // without scratch the data-parallel schedule is used: slower on awkward tile counts, never wrong
      sk = have_ws && gu::tile_prefers_stream_k(pr->m, pr->k, pr->n, dev->sm_count);
    }
    return gu::launch_tile(pr, *dev, stream, sk);
  }

  if (pr->m > 64) return GU_EINVAL_PLAN;
  const int mpad = gu::stream_mpad(pr->m);
  const int stages = gu::stream_stages(mpad, pr->k / 128);
  if (stages == 0) return GU_EINVAL_PLAN;
  const size_t need = gu_workspace_bytes(pr->m, pr->k, pr->n, GU_PLAN_STREAM);
  if (!pr->workspace || pr->workspace_bytes < need || !gu::aligned16(pr->workspace)) return GU_EWORKSPACE;
  switch (mpad) {
    case 16: return gu::launch_stream_t<16>(pr, *dev, stream, stages);
    case 32: return gu::launch_stream_t<32>(pr, *dev, stream, stages);
    default: return gu::launch_stream_t<64>(pr, *dev, stream, stages);
  }
}

int gu_run_concat(const void* x, const float* scale_x, const void* w2n, const float* scale_w2n, void* output,
                  int64_t m, int64_t k, int64_t n, int64_t ld_output, void* workspace, size_t workspace_bytes,
                  int plan, void* stream) {
  if (!w2n || !scale_w2n) return GU_EINVAL_NULL;
  if (!gu::shape_ok(m, k, n)) return GU_EINVAL_SHAPE;
  gu_problem pr;
  std::memset(&pr, 0, sizeof(pr));
  pr.x = x;
  pr.scale_x = scale_x;
  pr.gate_w = w2n;
  pr.scale_gate = scale_w2n;
  pr.up_w = static_cast<const uint8_t*>(w2n) + size_t(n) * size_t(k);
  pr.scale_up = scale_w2n + size_t(n / 128) * size_t(k / 128);
  pr.output = output;
  pr.m = m;
  pr.k = k;
  pr.n = n;
  pr.ld_output = ld_output;
  pr.workspace = workspace;
  pr.workspace_bytes = workspace_bytes;
  pr.plan = plan;
  return gu_run(&pr, stream);
}

int gu_run_decode_static(const gu_problem* pr, void* stream_v) {
  int rc = gu::check_problem(pr);
  if (rc != GU_OK) return rc;
  if (pr->m > gu::kStaticMaxTokens) return GU_ESTATIC_LIMIT;
  const int stages = gu::stream_stages(16, pr->k / 128);
  if (stages == 0) return GU_EINVAL_PLAN;
  gu::DeviceInfo* dev = nullptr;
  if ((rc = gu::device_info(&dev)) != GU_OK) return rc;   // first call per device: function attributes
  void* scratch = nullptr;
  if ((rc = gu::static_scratch_ptr(&scratch)) != GU_OK) return rc;  // first call per device: symbol address

  const int64_t m = pr->m, k = pr->k, n = pr->n;
  CUtensorMap tm_x, tm_g, tm_u;
  if ((rc = gu::encode_map_uncached(&tm_x, pr->x, k, m, k, 128, 16)) != GU_OK) return rc;
  if ((rc = gu::encode_map_uncached(&tm_g, pr->gate_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::encode_map_uncached(&tm_u, pr->up_w, k, n, k, 128, 128)) != GU_OK) return rc;

  gu::StreamParams p;
  p.scale_x = pr->scale_x;
  p.scale_gate = pr->scale_gate;
  p.scale_up = pr->scale_up;
  p.out = static_cast<__nv_bfloat16*>(pr->output);
  p.ld_out = pr->ld_output;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>(n / 128);
  p.stages = stages;
  // The array keeps whatever the previous call left in it.  Nothing has to be cleared: a flag only
  // counts when it equals this launch's epoch, a value no earlier launch has written (the array, with
  // the launch counter that epochs come from, starts zeroed at module load and 0 is never an epoch), and
  // partial slots are fully rewritten before their flag is stamped.
  p.flags = static_cast<unsigned int*>(scratch);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + gu::kStreamFlagBytes);

  const int64_t units = int64_t(p.nb) * p.kb;
  int64_t grid = dev->sm_count < gu::kStreamMaxGrid ? dev->sm_count : gu::kStreamMaxGrid;
  if (units < grid) grid = units;
  const uint32_t smem = gu::StreamCfg<16>::smem_bytes(stages, p.kb);
  gu::gateup_stream_kernel<16><<<static_cast<int>(grid), gu::kStreamThreads, smem,
                                 static_cast<cudaStream_t>(stream_v)>>>(tm_x, tm_g, tm_u, p);
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_run_gather(const gu_problem* pr, void* const* rank_outputs, int world, int rank, int64_t ld_full,
                  void* stream_v) {
  int rc = gu::check_problem(pr);
  if (rc != GU_OK) return rc;
  if (!rank_outputs) return GU_EINVAL_NULL;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return GU_EINVAL_SHAPE;
  const int64_t m = pr->m, k = pr->k, n = pr->n, n_full = n * world;
  if (ld_full < n_full) return GU_EINVAL_SHAPE;
  if (ld_full % 8 != 0) return GU_EINVAL_ALIGN;
  for (int r = 0; r < world; ++r) {
    if (!rank_outputs[r]) return GU_EINVAL_NULL;
    if (!gu::aligned16(rank_outputs[r])) return GU_EINVAL_ALIGN;
  }
  gu::DeviceInfo* dev = nullptr;
  if ((rc = gu::device_info(&dev)) != GU_OK) return rc;

  CUtensorMap tm_x, tm_g, tm_u;
  gu::PeerMaps peers;
  std::memset(&peers, 0, sizeof(peers));
  if ((rc = gu::get_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->x, k, m, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->gate_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->up_w, k, n, k, 128, 128)) != GU_OK) return rc;
  for (int r = 0; r < world; ++r) {
    // each rank's full [M, N * world] buffer; stores land at this rank's column offset
    if ((rc = gu::get_map(&peers.m[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rank_outputs[r], n_full, m, ld_full * 2,
                          64, 128)) != GU_OK)
      return rc;
  }

  gu::TileParams p;
  p.scale_x = pr->scale_x;
  p.scale_gate = pr->scale_gate;
  p.scale_up = pr->scale_up;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.num_m_blocks = static_cast<int>((m + gu::kTileM - 1) / gu::kTileM);
  p.num_n_blocks = static_cast<int>(n / gu::kTileN);
  const int64_t tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
  if (tiles * (k / 128) >= (1ll << 31)) return GU_EINVAL_SHAPE;
  p.num_tiles = static_cast<int>(tiles);
  int64_t gm = (24ll << 20) / (128 * k);
  if (gm < 1) gm = 1;
  if (gm > p.num_m_blocks) gm = p.num_m_blocks;
  p.group_m = static_cast<int>(gm);
  p.tile_begin = 0;
  p.flags = nullptr;
  p.partials = nullptr;
  p.epoch = 0;
  p.n_blocks128 = 0;
  p.scale_out = nullptr;
  p.blocks_per_owner = 1;
  p.slot_rows = 0;
  p.out_count = world;
  p.out_rank = rank;
  p.out_col0 = static_cast<int>(int64_t(rank) * n);

  if (gu::tile_prefers_pairs(m, *dev)) {
    const int clusters = gu::pair_geometry(p, *dev, m, k, static_cast<int>(n / gu::kTileN));
    if (clusters < 1) return GU_EINVAL_SHAPE;
    gu::gateup_pair_gather_kernel<<<2 * clusters, gu::kPairThreads, gu::kPairSmemBytes,
                                    static_cast<cudaStream_t>(stream_v)>>>(tm_x, tm_g, tm_u, peers, p);
    gu::g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
  }
  const int grid = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
  gu::gateup_tile_gather_kernel<<<grid, gu::kTileThreads, gu::kTileSmemBytes, static_cast<cudaStream_t>(stream_v)>>>(
      tm_x, tm_g, tm_u, peers, p);
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_blockwise_gemm_scatter(const void* a, const float* scale_a, const void* b, const float* scale_b,
                              void* const* rank_slots, int world, int rank, int64_t m, int64_t k, int64_t n,
                              void* stream_v) {
  if (!a || !scale_a || !b || !scale_b || !rank_slots) return GU_EINVAL_NULL;
  if (!gu::shape_ok(m, k, n) || world < 1 || world > 8 || rank < 0 || rank >= world) return GU_EINVAL_SHAPE;
  if (m % (128 * int64_t(world)) != 0) return GU_EINVAL_SHAPE;  // every rank owns the same whole number of token blocks
  if (!gu::aligned16(a) || !gu::aligned16(b) || (reinterpret_cast<uintptr_t>(scale_a) & 3u) ||
      (reinterpret_cast<uintptr_t>(scale_b) & 3u))
    return GU_EINVAL_ALIGN;
  for (int r = 0; r < world; ++r) {
    if (!rank_slots[r]) return GU_EINVAL_NULL;
    if (!gu::aligned16(rank_slots[r])) return GU_EINVAL_ALIGN;
  }
  gu::DeviceInfo* dev = nullptr;
  int rc = gu::device_info(&dev);
  if (rc != GU_OK) return rc;
  const int64_t slot_rows = m / world;

  CUtensorMap tm_a, tm_b;
  gu::PeerMaps peers;
  std::memset(&peers, 0, sizeof(peers));
  if ((rc = gu::get_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, k, m, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, k, n, k, 128, 128)) != GU_OK) return rc;
  for (int r = 0; r < world; ++r) {
    // rank r's buffer: `world` slots of [slot_rows, n] bf16, one per sending rank
    if ((rc = gu::get_map(&peers.m[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rank_slots[r], n, slot_rows * world, n * 2,
                          64, 128)) != GU_OK)
      return rc;
  }
  gu::TileParams p;
  p.scale_x = scale_a;
  p.scale_gate = scale_b;
  p.scale_up = scale_b;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.n_blocks128 = static_cast<int>(n / 128);
  p.scale_out = nullptr;
  p.num_m_blocks = static_cast<int>(m / gu::kTileM);
  p.num_n_blocks = (p.n_blocks128 + 1) / 2;
  const int64_t tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
  if (tiles * (k / 128) >= (1ll << 31)) return GU_EINVAL_SHAPE;
  p.num_tiles = static_cast<int>(tiles);
  int64_t gm = (24ll << 20) / (128 * k);
  if (gm < 1) gm = 1;
  if (gm > p.num_m_blocks) gm = p.num_m_blocks;
  p.group_m = static_cast<int>(gm);
  p.tile_begin = 0;
  p.flags = nullptr;
  p.partials = nullptr;
  p.epoch = 0;
  p.out_count = world;
  p.out_rank = rank;
  p.out_col0 = 0;
  p.blocks_per_owner = p.num_m_blocks / world;  // in 128-token blocks, whichever kernel runs
  p.slot_rows = static_cast<int>(slot_rows);

  if (gu::tile_prefers_pairs(m, *dev)) {
    const int clusters = gu::pair_geometry(p, *dev, m, k, (p.n_blocks128 + 1) / 2);
    if (clusters < 1) return GU_EINVAL_SHAPE;
    gu::blockwise_gemm_pair_scatter_kernel<<<2 * clusters, gu::kPairThreads, gu::kPairSmemBytes,
                                             static_cast<cudaStream_t>(stream_v)>>>(tm_a, tm_b, peers, p);
    gu::g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
  }
  const int grid = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
  gu::blockwise_gemm_scatter_kernel<<<grid, gu::kTileThreads, gu::kTileSmemBytes, static_cast<cudaStream_t>(stream_v)>>>(
      tm_a, tm_b, peers, p);
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_reduce_gather(const void* slots, void* const* rank_outputs, int world, int rank, int64_t m, int64_t h,
                     void* stream_v) {
  if (!slots || !rank_outputs) return GU_EINVAL_NULL;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || m < 1 || h < 8 || m % world != 0 || h % 8 != 0)
    return GU_EINVAL_SHAPE;
  if (!gu::aligned16(slots)) return GU_EINVAL_ALIGN;
  gu::DeviceInfo* dev = nullptr;
  int rc = gu::device_info(&dev);
  if (rc != GU_OK) return rc;
  gu::ReduceGatherParams p;
  std::memset(&p, 0, sizeof(p));
  p.slots = static_cast<const uint4*>(slots);
  if (!rank_outputs[rank]) return GU_EINVAL_NULL;
  for (int r = 0; r < world; ++r) {
    // a null entry other than this rank's own is a destination that does not want the rows (reduce-scatter form)
    if (rank_outputs[r] && !gu::aligned16(rank_outputs[r])) return GU_EINVAL_ALIGN;
    p.outputs[r] = static_cast<uint4*>(rank_outputs[r]);
  }
  const int64_t slot_rows = m / world;
  p.words_per_slot = slot_rows * h / 8;
  p.out_word0 = int64_t(rank) * p.words_per_slot;
  p.world = world;
  long long grid = (p.words_per_slot + 255) / 256;
  const long long cap = static_cast<long long>(dev->sm_count) * 8;
  if (grid > cap) grid = cap;
  gu::reduce_gather_kernel<<<static_cast<int>(grid), 256, 0, static_cast<cudaStream_t>(stream_v)>>>(p);
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_peer_barrier(void* const* rank_flags, int world, int rank, uint64_t limit_ns, void* stream_v) {
  if (!rank_flags) return GU_EINVAL_NULL;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return GU_EINVAL_SHAPE;
  gu::PeerBarrierParams p;
  std::memset(&p, 0, sizeof(p));
  for (int r = 0; r < world; ++r) {
    if (!rank_flags[r]) return GU_EINVAL_NULL;
    if (reinterpret_cast<uintptr_t>(rank_flags[r]) & 3u) return GU_EINVAL_ALIGN;
    p.flags[r] = static_cast<unsigned int*>(rank_flags[r]);
  }
  p.world = world;
  p.rank = rank;
  p.limit_ns = limit_ns ? limit_ns : 2000000000ull;
  gu::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_v)>>>(p);
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_quantize_activation(const void* x, int x_is_f32, int64_t ld_x, void* q, float* scale, int64_t m, int64_t k,
                           void* stream_v) {
  if (!x || !q || !scale) return GU_EINVAL_NULL;
  if (m < 1 || k < 128 || (k % 128) != 0 || ld_x < k) return GU_EINVAL_SHAPE;
  const int64_t elem = x_is_f32 ? 4 : 2;
  if (!gu::aligned16(x) || !gu::aligned16(q) || (reinterpret_cast<uintptr_t>(scale) & 3u) || (ld_x * elem) % 16 != 0)
    return GU_EINVAL_ALIGN;
  gu::DeviceInfo* dev = nullptr;
  int rc = gu::device_info(&dev);
  if (rc != GU_OK) return rc;
  const long long blocks = static_cast<long long>(m) * (k / 128);
  if (blocks >= (1ll << 31)) return GU_EINVAL_SHAPE;  // the kernel counts 1x128 blocks in 32 bits
  const long long per_cta = (gu::kQuantThreads / 16) * (x_is_f32 ? gu::quant_unroll<float>() : gu::quant_unroll<__nv_bfloat16>());
  long long grid = (blocks + per_cta - 1) / per_cta;
  // one wave: as many CTAs as are resident at once (the kernel's registers allow 4 of 256 threads per SM; a grid
  // of 8 per SM ran as two waves and paid two ramps)
  static const int resident[2][2] = {
      {gu::resident_ctas(gu::quantize_act_kernel<__nv_bfloat16, false>, gu::kQuantThreads),
       gu::resident_ctas(gu::quantize_act_kernel<__nv_bfloat16, true>, gu::kQuantThreads)},
      {gu::resident_ctas(gu::quantize_act_kernel<float, false>, gu::kQuantThreads),
       gu::resident_ctas(gu::quantize_act_kernel<float, true>, gu::kQuantThreads)}};
  const long long cap = static_cast<long long>(dev->sm_count) * resident[x_is_f32 ? 1 : 0][ld_x != k ? 1 : 0];
  if (grid > cap) grid = cap;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int g = static_cast<int>(grid);
  const uint32_t nblk = static_cast<uint32_t>(blocks), kb = static_cast<uint32_t>(k / 128);
  uint8_t* qb = static_cast<uint8_t*>(q);
  const bool pitched = ld_x != k;
  if (x_is_f32) {
    const float* xf = static_cast<const float*>(x);
    if (pitched) gu::quantize_act_kernel<float, true><<<g, gu::kQuantThreads, 0, stream>>>(xf, qb, scale, nblk, ld_x, kb);
    else gu::quantize_act_kernel<float, false><<<g, gu::kQuantThreads, 0, stream>>>(xf, qb, scale, nblk, ld_x, kb);
  } else {
    const __nv_bfloat16* xh = static_cast<const __nv_bfloat16*>(x);
    if (pitched) gu::quantize_act_kernel<__nv_bfloat16, true><<<g, gu::kQuantThreads, 0, stream>>>(xh, qb, scale, nblk, ld_x, kb);
    else gu::quantize_act_kernel<__nv_bfloat16, false><<<g, gu::kQuantThreads, 0, stream>>>(xh, qb, scale, nblk, ld_x, kb);
  }
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_run_fp8out(const gu_problem* pr, void* out_q, float* out_scale, void* stream_v) {
  if (!pr || !out_q || !out_scale) return GU_EINVAL_NULL;
  if (!pr->x || !pr->scale_x || !pr->gate_w || !pr->scale_gate || !pr->up_w || !pr->scale_up) return GU_EINVAL_NULL;
  if (!gu::shape_ok(pr->m, pr->k, pr->n)) return GU_EINVAL_SHAPE;
  if (!gu::aligned16(pr->x) || !gu::aligned16(pr->gate_w) || !gu::aligned16(pr->up_w) || !gu::aligned16(out_q) ||
      (reinterpret_cast<uintptr_t>(pr->scale_x) & 3u) || (reinterpret_cast<uintptr_t>(pr->scale_gate) & 3u) ||
      (reinterpret_cast<uintptr_t>(pr->scale_up) & 3u) || (reinterpret_cast<uintptr_t>(out_scale) & 3u))
    return GU_EINVAL_ALIGN;
  gu::DeviceInfo* dev = nullptr;
  int rc = gu::device_info(&dev);
  if (rc != GU_OK) return rc;
  const int64_t m = pr->m, k = pr->k, n = pr->n;
  CUtensorMap tm_x, tm_g, tm_u, tm_q;
  if ((rc = gu::get_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->x, k, m, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_g, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->gate_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, pr->up_w, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, out_q, n, m, n, 128, 128)) != GU_OK) return rc;

  gu::TileParams p;
  p.scale_x = pr->scale_x;
  p.scale_gate = pr->scale_gate;
  p.scale_up = pr->scale_up;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.num_m_blocks = static_cast<int>((m + gu::kTileM - 1) / gu::kTileM);
  p.num_n_blocks = static_cast<int>(n / gu::kTileN);
  const int64_t tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
  if (tiles * (k / 128) >= (1ll << 31)) return GU_EINVAL_SHAPE;
  p.num_tiles = static_cast<int>(tiles);
  int64_t gm = (24ll << 20) / (128 * k);
  if (gm < 1) gm = 1;
  if (gm > p.num_m_blocks) gm = p.num_m_blocks;
  p.group_m = static_cast<int>(gm);
  p.tile_begin = 0;
  p.flags = nullptr;
  p.partials = nullptr;
  p.epoch = 0;
  p.out_count = 1;
  p.out_rank = 0;
  p.out_col0 = 0;
  p.n_blocks128 = static_cast<int>(n / 128);
  p.scale_out = out_scale;
  p.blocks_per_owner = 1;
  p.slot_rows = 0;

  if (!gu::tile_prefers_lone(gu::kOpGateUpFp8, m, k / 128, n / gu::kTileN, dev->sm_count, dev->pair_clusters, false)) {
    const int clusters = gu::pair_geometry(p, *dev, m, k, static_cast<int>(n / gu::kTileN));
    if (clusters < 1) return GU_EINVAL_SHAPE;
    gu::gateup_pair_fp8out_kernel<<<2 * clusters, gu::kPairThreads, gu::kPairSmemBytes,
                                    static_cast<cudaStream_t>(stream_v)>>>(tm_x, tm_g, tm_u, tm_q, p);
    gu::g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
  }
  const int grid = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
  gu::gateup_tile_fp8out_kernel<<<grid, gu::kTileThreads, gu::kTileSmemBytes, static_cast<cudaStream_t>(stream_v)>>>(
      tm_x, tm_g, tm_u, tm_q, p);
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_blockwise_gemm(const void* a, const float* scale_a, const void* b, const float* scale_b, void* c, int64_t m,
                      int64_t k, int64_t n, int64_t ld_c, void* stream_v) {
  if (!a || !scale_a || !b || !scale_b || !c) return GU_EINVAL_NULL;
  if (!gu::shape_ok(m, k, n) || ld_c < n) return GU_EINVAL_SHAPE;
  if (!gu::aligned16(a) || !gu::aligned16(b) || !gu::aligned16(c) || (reinterpret_cast<uintptr_t>(scale_a) & 3u) ||
      (reinterpret_cast<uintptr_t>(scale_b) & 3u) || (ld_c % 8) != 0)
    return GU_EINVAL_ALIGN;
  gu::DeviceInfo* dev = nullptr;
  int rc = gu::device_info(&dev);
  if (rc != GU_OK) return rc;

  CUtensorMap tm_a, tm_b, tm_c;
  if ((rc = gu::get_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, k, m, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, k, n, k, 128, 128)) != GU_OK) return rc;
  if ((rc = gu::get_map(&tm_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, n, m, ld_c * 2, 64, 128)) != GU_OK) return rc;

  gu::TileParams p;
  p.scale_x = scale_a;
  p.scale_gate = scale_b;
  p.scale_up = scale_b;
  p.m = static_cast<int>(m);
  p.kb = static_cast<int>(k / 128);
  p.n_blocks128 = static_cast<int>(n / 128);
  p.scale_out = nullptr;
  p.blocks_per_owner = 1;
  p.slot_rows = 0;
  p.out_rows = static_cast<int>(m);
  p.out_cols = static_cast<int>(n);
  if (!gu::tile_prefers_lone(gu::kOpGemm, m, k / 128, (n / 128 + 1) / 2, dev->sm_count, dev->pair_clusters, false)) {
    // CTA pairs: 256-token x 256-column tiles, one per two-CTA cluster
    p.num_m_blocks = static_cast<int>((m + 2 * gu::kTileM - 1) / (2 * gu::kTileM));
    p.num_n_blocks = (p.n_blocks128 + 1) / 2;
    const int64_t pair_tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
    if (pair_tiles * (k / 128) >= (1ll << 31)) return GU_EINVAL_SHAPE;
    p.num_tiles = static_cast<int>(pair_tiles);
    int64_t pgm = (24ll << 20) / (256 * k);
    if (pgm < 1) pgm = 1;
    if (pgm > p.num_m_blocks) pgm = p.num_m_blocks;
    p.group_m = static_cast<int>(pgm);
    p.tile_begin = 0;
    p.flags = nullptr;
    p.partials = nullptr;
    p.epoch = 0;
    p.out_count = 1;
    p.out_rank = 0;
    p.out_col0 = 0;
    const int clusters = p.num_tiles < dev->pair_clusters ? p.num_tiles : dev->pair_clusters;
    gu::blockwise_gemm_pair_kernel<<<2 * clusters, gu::kPairThreads, gu::kPairSmemBytes,
                                     static_cast<cudaStream_t>(stream_v)>>>(tm_a, tm_b, tm_c, p);
    gu::g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
  }
  p.num_m_blocks = static_cast<int>((m + gu::kTileM - 1) / gu::kTileM);
  p.num_n_blocks = (p.n_blocks128 + 1) / 2;  // a CTA tile spans two 128-column blocks of B
  const int64_t tiles = int64_t(p.num_m_blocks) * p.num_n_blocks;
  if (tiles * (k / 128) >= (1ll << 31)) return GU_EINVAL_SHAPE;
  p.num_tiles = static_cast<int>(tiles);
  int64_t gm = (24ll << 20) / (128 * k);
  if (gm < 1) gm = 1;
  if (gm > p.num_m_blocks) gm = p.num_m_blocks;
  p.group_m = static_cast<int>(gm);
  p.tile_begin = 0;
  p.flags = nullptr;
  p.partials = nullptr;
  p.epoch = 0;
  p.out_count = 1;
  p.out_rank = 0;
  p.out_col0 = 0;

  const int grid = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
  gu::blockwise_gemm_kernel<<<grid, gu::kTileThreads, gu::kTileSmemBytes, static_cast<cudaStream_t>(stream_v)>>>(
      tm_a, tm_b, tm_c, p);
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_last_status(int* detail, int clear) {
  unsigned int host[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return GU_ECUDA;
  if (cudaMemcpyFromSymbol(host, gu::g_status, sizeof(host)) != cudaSuccess) return GU_ECUDA;
  if (detail) *detail = static_cast<int>(host[1]);
  if (clear && host[0] != 0) {
    unsigned int zero[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbol(gu::g_status, zero, sizeof(zero)) != cudaSuccess) return GU_ECUDA;
  }
  if (host[0] == 0) return GU_OK;
  return host[0] == gu::kStatusBounds ? GU_EBOUNDS : GU_ETIMEOUT;
}

int gu_is_range_checked_build(void) {
#ifdef GU_BOUNDS
  return 1;
#else
  return 0;
#endif
}

int64_t gu_launch_count(void) { return gu::g_launches.load(std::memory_order_relaxed); }

int gu_set_wait_limit_ns(uint64_t ns) {
  const unsigned long long v = ns ? ns : 2000000000ull;
  if (cudaDeviceSynchronize() != cudaSuccess) return GU_ECUDA;
  return cudaMemcpyToSymbol(gu::g_wait_limit_ns, &v, sizeof(v)) == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_wait_probe(void* stream_v) {
  gu::wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream_v)>>>();
  gu::g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? GU_OK : GU_ECUDA;
}

int gu_trace_read(uint64_t* out, int capacity, int clear) {
#ifdef GU_TRACE
  if (!out || capacity < 0) return GU_EINVAL_NULL;
  unsigned long long host[32 + 256];
  if (cudaDeviceSynchronize() != cudaSuccess) return GU_ECUDA;
  if (cudaMemcpyFromSymbol(host, gu::g_trace, 32 * sizeof(host[0])) != cudaSuccess) return GU_ECUDA;
  if (cudaMemcpyFromSymbol(host + 32, gu::g_events, 256 * sizeof(host[0])) != cudaSuccess) return GU_ECUDA;
  const int n = capacity < 288 ? capacity : 288;
  for (int i = 0; i < n; ++i) out[i] = host[i];
  if (clear) {
    std::memset(host, 0, sizeof(host));
    if (cudaMemcpyToSymbol(gu::g_trace, host, 32 * sizeof(host[0])) != cudaSuccess) return GU_ECUDA;
  }
  return n;
#else
  (void)out;
  (void)capacity;
  (void)clear;
  return 0;
#endif
}

}  // extern "C"
