// C ABI of libfused_swiglu_sm100.so (declared in include/fused_swiglu.h):
// argument checking, TMA tensor-map construction, UMMA descriptor constants and
// kernel launches.  No device memory is allocated here: scratch (dg/du, the
// workspace of a split last wave, multi-GPU receive buffers) is the caller's.  State
// kept by the library: process-wide options, a cache of device attributes and of
// encoded tensor maps, and per device a status word, a clock probe, a ring of pacing
// counters and the fixed scratch of fsw_backward_static_scratch (all `__device__`
// variables of the library image).
#include "../../include/fused_swiglu.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>

#include "fsw_gemm.cuh"

namespace fsw {

// ------------------------------------------------------------------ errors --
static thread_local char t_err[512] = "";

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return code;
}

#define FSW_CUDA(call)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (call);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return fail(FSW_ECUDA, "%s failed: %s", #call, cudaGetErrorString(e_));            \
  } while (0)

// ----------------------------------------------------------------- options --
struct Options {
  int64_t cta_group = 0;  // CTAs per MMA: 1, 2, or 0 = choose per launch
  int64_t nsub = 0;       // accumulator regions per tile: 1, 2 (needs a CTA pair), or 0 = choose
  int64_t group_m = 0;           // rasterisation group height in tiles; 0 = choose per launch
  int64_t wait_limit_ms = 2000;  // bound on every device-side wait
  int64_t stall_producer = 0;    // test hook: make the consumers' waits run out
  int64_t gemm_max_sms = 0;      // cap on SMs a GEMM launch occupies (0 = all of them)
  int64_t l2_a = 2, l2_b = 2;    // L2 eviction priority of A / B operand loads (0 normal,
                                 // 1 first, 2 last).  Evict-last keeps operand panels, which
                                 // other CTAs of the wave are about to read, ahead of output
                                 // lines: +1.5-3.6 % forward, +1-3 % dX and dW in round-robin
                                 // A/B runs at the power cap.
  int64_t l2_out = 1;            // ... of the forward's g/u/out stores: evict first, they are
                                 // not read again by this launch (measured: 5 % fewer DRAM
                                 // reads, +1.2 % sustained forward throughput)
  int64_t l2_promo = 2;          // TMA L2 promotion of operand and output maps: 0 none,
                                 // 1 = 128 bytes, 2 = 256 bytes
  int64_t pace_kb = 32;          // producers of all CTAs meet every pace_kb K blocks so that
                                 // the two dies keep sharing operand panels in L2 (0 = off)
  int64_t pace_limit_us = 50;    // longest wait at one meeting point
  int64_t ew_blocks_per_sm = 32;  // grid cap of the elementwise kernel, per SM
  int64_t split_k = 1;            // 0: never split the last wave of tiles along K
  int64_t ew_ahead = 0;           // row tiles the gate-gradient side job may run ahead (0 = one wave + 2)
  int64_t gate_in_dx = 1;         // 0: fsw_backward_dx_gate runs the elementwise step as a launch of its own
  int64_t scatter_gap_ns = -1;    // pause between peer-store instructions of the dX scatter; -1 = from the tile's length
};
static Options g_opt;
// Kernels this library has launched in this process (read through fsw_get_option("kernel_launches")).
static std::atomic<long long> g_kernel_launches{0};

// Status word the kernels write when a bounded wait gives up.
__device__ uint32_t g_status_word;
// Arrival counter and off switch of the producers' pacing (see Pacer).  Every paced
// launch takes the next of kPaceSlots pairs, so launches that overlap on one device
// (other streams, other host threads) do not disturb each other's counts.
constexpr int kPaceSlots = 16;
__device__ unsigned int g_pace[2 * kPaceSlots];
// Ticket and per-row-tile counters of the gate-gradient side job of MODE_DXE launches;
// a ring of slots, one per launch in turn (see g_pace).
constexpr int kEwSlots = 4;
constexpr int kEwMaxRowTiles = 8192;
__device__ unsigned int g_ew_ctrl[kEwSlots * (2 + kEwMaxRowTiles)];
// SM cycles and nanoseconds that CTA 0 of the last GEMM launch was resident.
__device__ unsigned long long g_clk_probe[8];

// ------------------------------------------------------------ device cache --
constexpr int kMaxDevices = 64;
struct DeviceInfo {
  bool ready = false;
  int sm_count = 0, cc_major = 0, cc_minor = 0;
  int64_t smem_optin = 0;
  int max_pairs = 0;  // co-resident 2-CTA clusters of the GEMM kernels
  uint32_t* status = nullptr;
  unsigned long long* clk_probe = nullptr;
  unsigned int* pace = nullptr;
  unsigned int* ew_ctrl = nullptr;
  unsigned int ew_next = 0;     // next slot of g_ew_ctrl to hand out
  unsigned int pace_next = 0;   // next slot of g_pace to hand out
  unsigned int pace_last = 0;   // slot the last paced launch used
};
static DeviceInfo g_dev[kMaxDevices];
static std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

template <int MODE, int CG, int NSUB, typename T, bool ACC16>
static cudaError_t prepare_kernel() {
  return cudaFuncSetAttribute(gemm_kernel<MODE, CG, NSUB, T, ACC16>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              TileCfg<MODE, CG, NSUB>::SMEM_BYTES);
}

template <int MODE, int CG, int NSUB>
static cudaError_t prepare_mode() {
  cudaError_t e;
  if ((e = prepare_kernel<MODE, CG, NSUB, __nv_bfloat16, false>()) != cudaSuccess) return e;
  if ((e = prepare_kernel<MODE, CG, NSUB, __half, false>()) != cudaSuccess) return e;
  return prepare_kernel<MODE, CG, NSUB, __half, true>();
}

static int ensure_device(DeviceInfo** out) {
  int dev = 0;
  FSW_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FSW_EINVAL, "device index %d out of range", dev);
  // The tensor-map encoder is a driver call and needs the device's context current on
  // THIS thread; a thread that has made no runtime call with side effects yet (an
  // autograd worker whose first call lands here) has none.  cudaSetDevice binds it.
  static thread_local int t_bound_device = -1;
  if (t_bound_device != dev) {
    FSW_CUDA(cudaSetDevice(dev));
    t_bound_device = dev;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    FSW_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    FSW_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    if (d.cc_major != 10)
      return fail(FSW_EDEVICE,
                  "device %d is compute capability %d.%d; this library runs on 10.x (B200) only",
                  dev, d.cc_major, d.cc_minor);
    int v = 0;
    FSW_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    FSW_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    d.smem_optin = v;
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      FSW_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
        return fail(FSW_EUNAVAILABLE, "driver does not provide cuTensorMapEncodeTiled");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    FSW_CUDA((prepare_mode<MODE_FWD, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_DX, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_DW, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_FWD, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_DX, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_DW, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_FWD, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_FWDST, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_FWDST, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_FWDST, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_DX, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_DW, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_DXE, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_DXE, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_DXE, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_DXG, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_DXG, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_DXG, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_NN, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_NT, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_TN, 1, 1>()));
    FSW_CUDA((prepare_mode<MODE_NN, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_NT, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_TN, 2, 1>()));
    FSW_CUDA((prepare_mode<MODE_NN, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_NT, 2, 2>()));
    FSW_CUDA((prepare_mode<MODE_TN, 2, 2>()));
    void* sp = nullptr;
    FSW_CUDA(cudaGetSymbolAddress(&sp, g_status_word));
    d.status = static_cast<uint32_t*>(sp);
    FSW_CUDA(cudaGetSymbolAddress(&sp, g_clk_probe));
    d.clk_probe = static_cast<unsigned long long*>(sp);
    FSW_CUDA(cudaGetSymbolAddress(&sp, g_pace));
    d.pace = static_cast<unsigned int*>(sp);
    FSW_CUDA(cudaGetSymbolAddress(&sp, g_ew_ctrl));
    d.ew_ctrl = static_cast<unsigned int*>(sp);
    // How many CTA pairs can be resident at once (a GPC with an odd SM count
    // leaves one SM without a partner).
    {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * d.sm_count, 1, 1);
      cfg.blockDim = dim3(TileCfg<MODE_FWD, 2, 2>::THREADS, 1, 1);
      cfg.dynamicSmemBytes = TileCfg<MODE_FWD, 2, 2>::SMEM_BYTES;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      cudaError_t e = cudaOccupancyMaxActiveClusters(
          &n, gemm_kernel<MODE_FWD, 2, 2, __nv_bfloat16, false>, &cfg);
      if (e != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = d.sm_count / 2;
      }
      d.max_pairs = n;
    }
    d.ready = true;
  }
  *out = &d;
  return FSW_OK;
}

// ------------------------------------------------------------- tensor maps --
// Encoded maps are kept in a small direct-mapped cache keyed by everything the
// encoding depends on, so a training loop that calls with the same buffers every
// step encodes each map once.  (An encoding holds only the address and geometry,
// so an entry stays valid even if the buffer is freed and the address reused for
// a tensor of the same geometry.)
struct MapKey {
  const void* ptr;
  uint64_t inner, outer, row_elems;
  uint32_t box_inner, box_outer;
  int32_t dtype, l2_promo;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && row_elems == o.row_elems &&
           box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype &&
           l2_promo == o.l2_promo;
  }
};
constexpr int kMapCacheSlots = 256;
struct MapCacheEntry {
  bool valid = false;
  MapKey key;
  CUtensorMap map;
};
static MapCacheEntry g_map_cache[kMapCacheSlots];
static std::mutex g_map_mu;
static uint64_t g_map_hits = 0, g_map_misses = 0;

static uint32_t map_slot(const MapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= (k.inner * 0xC2B2AE3D27D4EB4Full) ^ (k.outer * 0x165667B19E3779F9ull) ^
       (k.row_elems * 0x27D4EB2F165667C5ull) ^
       ((uint64_t)k.box_outer << 40) ^ ((uint64_t)k.box_inner << 32) ^ ((uint64_t)k.dtype << 8) ^
       (uint64_t)k.l2_promo;
  h ^= h >> 29;
  h *= 0xBF58476D1CE4E5B9ull;
  h ^= h >> 32;
  return (uint32_t)(h % kMapCacheSlots);
}

// Row-major (outer, inner) array of 16-bit elements; box = box_outer rows of 64
// elements (128 bytes, 128-byte swizzle) or of 32 elements (64 bytes, 64-byte swizzle).
// `row_elems` is the distance between rows in elements when the map covers a column
// range of a wider array (0 = dense, rows are `inner` elements apart).
static int make_map(CUtensorMap* m, const void* ptr, int dtype, uint64_t inner, uint64_t outer,
                    uint32_t box_outer, const char* what, uint32_t box_inner = 64,
                    uint64_t row_elems = 0) {
  const MapKey key = {ptr, inner, outer, row_elems, box_inner, box_outer, dtype, (int32_t)g_opt.l2_promo};
  const uint32_t slot = map_slot(key);
  {
    std::lock_guard<std::mutex> lock(g_map_mu);
    const MapCacheEntry& e = g_map_cache[slot];
    if (e.valid && e.key == key) {
      *m = e.map;
      ++g_map_hits;
      return FSW_OK;
    }
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {(row_elems ? row_elems : inner) * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(
      m, dtype == FSW_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
      const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      box_inner == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
      key.l2_promo == 0   ? CU_TENSOR_MAP_L2_PROMOTION_NONE
      : key.l2_promo == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                          : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FSW_ECUDA, "cuTensorMapEncodeTiled(%s: inner=%llu outer=%llu box_outer=%u) -> %d",
                what, (unsigned long long)inner, (unsigned long long)outer, box_outer, (int)r);
  {
    std::lock_guard<std::mutex> lock(g_map_mu);
    MapCacheEntry& e = g_map_cache[slot];
    e.key = key;
    e.map = *m;
    e.valid = true;
    ++g_map_misses;
  }
  return FSW_OK;
}

// UMMA instruction descriptor, kind::f16: D format [4,6), A format [7,10),
// B format [10,13), A major bit 15, B major bit 16, N>>3 at [17,23), M>>4 at [24,29).
static uint32_t make_idesc(int dtype, bool acc16, int a_major, int b_major, int m, int n) {
  uint32_t d = 0;
  d |= (acc16 ? 0u : 1u) << 4;
  d |= (dtype == FSW_BF16 ? 1u : 0u) << 7;
  d |= (dtype == FSW_BF16 ? 1u : 0u) << 10;
  d |= static_cast<uint32_t>(a_major) << 15;
  d |= static_cast<uint32_t>(b_major) << 16;
  d |= static_cast<uint32_t>(n >> 3) << 17;
  d |= static_cast<uint32_t>(m >> 4) << 24;
  return d;
}

// UMMA shared-memory descriptor without the start address: leading byte offset
// at [16,30), stride byte offset at [32,46) (both >>4), version 1 at bit 46,
// layout type SWIZZLE_128B (2) at [61,64).
static uint64_t make_sdesc(uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

static void fill_operand_desc(int major, uint64_t* desc, uint32_t* kadv) {
  if (major == MAJOR_K) {
    // rows of 64 elements = one 128-byte swizzle row; 8-row groups 1024 B apart;
    // a K=16 step moves 32 bytes inside the swizzle row.
    *desc = make_sdesc(16u, 1024u);
    *kadv = 32u;
  } else {
    // 64(MN) x 64(K) boxes: K rows of 128 bytes; 8-row K groups 1024 B apart
    // (stride offset); the next 64 MN elements are one whole box (8192 B) away
    // (leading offset); a K=16 step is 16 rows = 2048 bytes.
    *desc = make_sdesc(8192u, 1024u);
    *kadv = 2048u;
  }
}

// ---------------------------------------------------------------- launches --
template <int MODE, int CG, int NSUB, typename T, bool ACC16>
static cudaError_t launch_one(const GemmParams& p, int grid, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(TileCfg<MODE, CG, NSUB>::THREADS, 1, 1);
  cfg.dynamicSmemBytes = TileCfg<MODE, CG, NSUB>::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ++g_kernel_launches;
  return cudaLaunchKernelEx(&cfg, gemm_kernel<MODE, CG, NSUB, T, ACC16>, p);
}

template <int MODE, int CG, int NSUB>
static cudaError_t launch_cg(const GemmParams& p, int grid, int dtype, bool acc16,
                             cudaStream_t st) {
  if (dtype == FSW_BF16) return launch_one<MODE, CG, NSUB, __nv_bfloat16, false>(p, grid, st);
  if (acc16) return launch_one<MODE, CG, NSUB, __half, true>(p, grid, st);
  return launch_one<MODE, CG, NSUB, __half, false>(p, grid, st);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_common(int64_t T, int64_t dm, int64_t di, int dtype, int accum) {
  if (dtype != FSW_BF16 && dtype != FSW_FP16) return fail(FSW_EINVAL, "unknown dtype %d", dtype);
  if (accum != FSW_ACC_F32 && accum != FSW_ACC_F16)
    return fail(FSW_EINVAL, "unknown accumulate mode %d", accum);
  if (accum == FSW_ACC_F16 && dtype != FSW_FP16)
    return fail(FSW_EINVAL, "fp16 accumulation needs fp16 tensors");
  if (T < 0 || dm <= 0 || di <= 0)
    return fail(FSW_EINVAL, "bad shape T=%lld dm=%lld di=%lld", (long long)T, (long long)dm,
                (long long)di);
  if ((dm & 7) || (di & 7))
    return fail(FSW_EINVAL, "d_model (%lld) and d_intermediate (%lld) must be multiples of 8",
                (long long)dm, (long long)di);
  if (T >= (1ll << 31) || dm >= (1ll << 31) || di >= (1ll << 31))
    return fail(FSW_EINVAL, "extent exceeds 2^31-1");
  return FSW_OK;
}

// Tile configuration for one launch.  Unless pinned by the options, take the
// configuration with the best (wave efficiency x relative speed): 256x512 tiles per
// CTA pair are fastest on large problems (the others sustain about 0.84x / 0.75x
// of their rate) but leave SMs idle when the problem has fewer tiles than workers
// or just over a whole number of waves.
struct TileChoice {
  int cg, nsub;
};
// SMs a launch may occupy: the call's own cap if it has one, else the process-wide
// "gemm_max_sms" option, else all of them.
static int sm_budget(const DeviceInfo* d, int max_sms) {
  int64_t cap = max_sms > 0 ? max_sms : g_opt.gemm_max_sms;
  return (cap > 0 && cap < d->sm_count) ? (int)cap : d->sm_count;
}

static TileChoice choose_tiles(int mode, int64_t rows, int64_t cols, const DeviceInfo* d,
                               int max_sms = 0, bool can_split = false) {
  const int want_cg = (int)g_opt.cta_group, want_ns = (int)g_opt.nsub;
  const int region_n = (mode == MODE_FWD || mode == MODE_DW) ? 128 : 256;
  const struct {
    int cg, nsub;
    double speed;
  } cand[3] = {{2, 2, 1.0}, {2, 1, 0.84}, {1, 1, 0.75}};
  TileChoice best = {2, 2};
  double best_score = -1.0;
  for (const auto& c : cand) {
    if (want_cg != 0 && c.cg != want_cg) continue;
    if (want_ns != 0 && c.nsub != want_ns && !(c.cg == 1 && want_cg == 1)) continue;
    int workers = (c.cg == 2) ? d->max_pairs : d->sm_count;
    {
      const int cap = sm_budget(d, max_sms) / c.cg;
      if (cap < workers) workers = cap < 1 ? 1 : cap;
    }
    const double tiles = (double)((rows + 128 * c.cg - 1) / (128 * c.cg)) *
                         (double)((cols + region_n * c.nsub - 1) / (region_n * c.nsub));
    double waves = (double)(int64_t)((tiles + workers - 1) / workers);
    // With a workspace the 256x512 configuration splits its last partial wave along K
    // over all workers, so it loses (almost) nothing to a ragged tile count.
    if (can_split && c.cg == 2 && c.nsub == 2 && tiles > workers / 4) waves = tiles / workers + 0.05;
    const double score = c.speed * tiles / (waves * workers);
    if (score > best_score) {
      best_score = score;
      best = {c.cg, c.nsub};
    }
  }
  return best;
}

// Plan of the split of the last partial wave along K for `tiles` tiles of `ipt` K
// iterations each on `pairs` CTA pairs: true if it pays.  Costs beyond the pieces'
// own iterations: one more (short) kernel and a round trip of the pieces through
// the workspace, put at 15 K iterations plus 0.3 per piece.
static bool plan_split(long long tiles, int pairs, long long ipt, int* first_tile, int* share,
                       long long* total) {
  const long long whole = (tiles / pairs) * pairs;
  const long long rem = tiles - whole;
  if (rem <= 0) return false;
  const long long tot = rem * ipt;
  const long long sh = (tot + pairs - 1) / pairs;
  const double cost = (double)sh + 15.0 + 0.3 * (double)(pairs + rem);
  if (!(cost < 0.9 * (double)ipt) || sh < 1 || tot >= (1ll << 40)) return false;
  *first_tile = (int)whole;
  *share = (int)sh;
  *total = tot;
  return true;
}

static int64_t splitk_workspace_bytes(const DeviceInfo* d) {
  return (int64_t)d->max_pairs * 2 * kSplitSlotFloats * (int64_t)sizeof(float);
}

template <int MODE>
static int run_gemm(GemmParams& p, int rows, int dtype, bool acc16, cudaStream_t st,
                    DeviceInfo* d, TileChoice tc, int max_sms = 0, void* ws = nullptr,
                    int64_t ws_bytes = 0) {
  const int cg = tc.cg;
  const int nsub = tc.nsub;
  const int tile_m = 128 * cg;
  const int tile_n = ((is_fwd(MODE) || MODE == MODE_DW) ? 128 : 256) * nsub;
  p.num_m_tiles = (rows + tile_m - 1) / tile_m;
  p.num_n_tiles = (p.N + tile_n - 1) / tile_n;
  if (p.ldc == 0) p.ldc = p.N;
  p.status = d->status;
  p.clk_probe = d->clk_probe;
  p.l2_a = (int)g_opt.l2_a;
  p.l2_b = (int)g_opt.l2_b;
  p.l2_out = (int)g_opt.l2_out;
  p.wait_limit_ns = (unsigned long long)g_opt.wait_limit_ms * 1000000ull;
  p.stall_producer = (int)g_opt.stall_producer;
  const int a_major = (MODE == MODE_DW || MODE == MODE_TN) ? MAJOR_MN : MAJOR_K;
  const int b_major = (is_dx(MODE) || MODE == MODE_NT || MODE == MODE_DXG) ? MAJOR_K : MAJOR_MN;
  fill_operand_desc(a_major, &p.a_desc, &p.a_kadv);
  fill_operand_desc(b_major, &p.b_desc, &p.b_kadv);
  p.idesc = make_idesc(dtype, acc16, a_major, b_major, 128 * cg, 256);
  const long long tiles = (long long)p.num_m_tiles * p.num_n_tiles;
  if (tiles <= 0) return FSW_OK;
  if (tiles >= (1ll << 31)) return fail(FSW_EINVAL, "too many tiles");
  cudaError_t e;
  const int avail_sms = sm_budget(d, max_sms);
  // Rasterisation: tiles are issued group_m rows at a time, sweeping the columns.
  // The tiles in flight then form roughly a group_m x (workers / group_m) block and
  // read group_m A panels (256 rows each) + that many B panels (512 rows each) from
  // HBM per wave; with the producers paced (see Pacer) measured DRAM reads match
  // this count.  The GPU runs at its power cap, so HBM traffic saved comes back as
  // SM clock: a poor group height costs up to 25 % of throughput.
  //   - at most 9 column tiles (dX of d_model 4096; an 8-way shard): every wave
  //     streams nearly all of B anyway, 1-2 rows are best;
  //   - otherwise the height that makes the block square in elements,
  //     sqrt(2 * workers) = 12 for 74 CTA pairs of 256x512 tiles, adjusted so that the groups are of
  //     equal height; one group if that is at most 1.5 heights (dW, whose rows are
  //     d_model).
  // Checked by sweeps of group_m on the Llama-3-8B and -70B MLP shapes and their
  // 1/2, 1/4, 1/8 column shards.
  {
    const int workers = (cg == 2) ? avail_sms / 2 : avail_sms;
    int gm = (int)g_opt.group_m;
    if (gm < 1) {
      if (p.num_n_tiles * 8 <= workers) {
        gm = workers / (p.num_n_tiles * 4);
      } else {
        const int aspect = (cg == 2 && nsub == 1) ? 1 : 2;  // tile columns / tile rows
        int g0 = 1;
        while ((g0 + 1) * (g0 + 1) <= aspect * workers) ++g0;  // floor(sqrt(aspect * workers))
        if (2 * p.num_m_tiles <= 3 * g0) {
          gm = p.num_m_tiles;
        } else {
          const int groups = (p.num_m_tiles + g0 / 2) / g0;
          gm = (p.num_m_tiles + groups - 1) / groups;
        }
      }
    }
    if (gm < 1) gm = 1;
    if (gm > p.num_m_tiles) gm = p.num_m_tiles;
    p.group_m = gm;
  }
  // Pacing only pays when the launch runs several waves of tiles on most of the GPU.
  p.pace = nullptr;
  p.pace_kb = 0;
  p.pace_limit_ns = (unsigned int)(g_opt.pace_limit_us * 1000);
  {
    const long long workers = (cg == 2) ? avail_sms / 2 : avail_sms;
    if (g_opt.pace_kb > 0 && tiles > workers) {
      unsigned int slot;
      {
        std::lock_guard<std::mutex> lock(g_mu);
        slot = d->pace_next++ % kPaceSlots;
        d->pace_last = slot;
      }
      p.pace = d->pace + 2 * slot;
      p.pace_kb = (int)g_opt.pace_kb;
      e = cudaMemsetAsync(p.pace, 0, 2 * sizeof(unsigned int), st);
      if (e != cudaSuccess) return fail(FSW_ECUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
    }
  }
  if (cg == 2) {
    int max_pairs = d->max_pairs < avail_sms / 2 ? d->max_pairs : avail_sms / 2;
    if (max_pairs < 1) max_pairs = 1;
    int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
    // Split the last partial wave along K over all pairs when the caller gave a
    // workspace and the tail would otherwise idle most of the GPU.
    constexpr int nseg = (is_dx(MODE) || MODE == MODE_DXG) ? 2 : 1;
    const long long ipt = (long long)nseg * p.num_k_blocks;
    p.sk_total_iters = 0;
    if (nsub == 2 && ws != nullptr && g_opt.split_k != 0 &&
        ws_bytes >= (int64_t)max_pairs * 2 * kSplitSlotFloats * (int64_t)sizeof(float) &&
        (reinterpret_cast<uintptr_t>(ws) & 15u) == 0) {
      if (plan_split(tiles, max_pairs, ipt, &p.sk_first_tile, &p.sk_iters_per_cluster,
                     &p.sk_total_iters)) {
        p.sk_ws = static_cast<float*>(ws);
        pairs = max_pairs;
      }
    }
    e = (nsub == 2) ? launch_cg<MODE, 2, 2>(p, 2 * pairs, dtype, acc16, st)
                    : launch_cg<MODE, 2, 1>(p, 2 * pairs, dtype, acc16, st);
    if (e == cudaSuccess && p.sk_total_iters > 0) {
      const int rem = (int)(tiles - p.sk_first_tile);
      constexpr bool dual = (MODE == MODE_DW);
      const float4* w4 = reinterpret_cast<const float4*>(p.sk_ws);
      ++g_kernel_launches;
      if (is_fwd(MODE) && dtype == FSW_BF16)
        splitk_reduce_swiglu_kernel<__nv_bfloat16><<<rem * 16, 256, 0, st>>>(
            w4, p.store_gu ? p.c0_ptr : nullptr, p.c1_ptr, p.c2_ptr, p.M, p.N, p.num_m_tiles,
            p.num_n_tiles, p.group_m, p.sk_first_tile, (int)ipt, p.sk_iters_per_cluster);
      else if (is_fwd(MODE))
        splitk_reduce_swiglu_kernel<__half><<<rem * 16, 256, 0, st>>>(
            w4, p.store_gu ? p.c0_ptr : nullptr, p.c1_ptr, p.c2_ptr, p.M, p.N, p.num_m_tiles,
            p.num_n_tiles, p.group_m, p.sk_first_tile, (int)ipt, p.sk_iters_per_cluster);
      else if (dtype == FSW_BF16)
        splitk_reduce_kernel<__nv_bfloat16, dual><<<rem * 16, 256, 0, st>>>(
            w4, p.c0_ptr, p.c1_ptr, p.M, p.N, p.ldc, p.num_m_tiles, p.num_n_tiles, p.group_m,
            p.sk_first_tile, (int)ipt, p.sk_iters_per_cluster);
      else
        splitk_reduce_kernel<__half, dual><<<rem * 16, 256, 0, st>>>(
            w4, p.c0_ptr, p.c1_ptr, p.M, p.N, p.ldc, p.num_m_tiles, p.num_n_tiles, p.group_m,
            p.sk_first_tile, (int)ipt, p.sk_iters_per_cluster);
      e = cudaGetLastError();
    }
  } else {
    const int ctas = (int)(tiles < avail_sms ? tiles : avail_sms);
    e = launch_cg<MODE, 1, 1>(p, ctas, dtype, acc16, st);
  }
  if (e != cudaSuccess) return fail(FSW_ECUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return FSW_OK;
}

// ------------------------------------------------ gate-gradient elementwise --
// du = dout * silu(g); dg = (dout * u) * silu'(g).  g is upcast to fp32 for the
// sigmoid; silu, silu' and every product are rounded to the 16-bit type, as in
// the reference kernel.
template <typename T>
__device__ __forceinline__ void gate_grad_one(float dout, float g, float u, float& dg, float& du) {
  const float sg = sigmoid_f32(g);
  const float silu_f = g * sg;
  const float silu = round16<T>(silu_f);
  const float dsilu = round16<T>(fmaf(silu_f, 1.0f - sg, sg));  // sg + g*sg*(1-sg)
  du = round16<T>(dout * silu);
  dg = round16<T>(round16<T>(dout * u) * dsilu);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) {
  return __half2float(v);
}

constexpr int kGateGradUnroll = 4;  // 16-byte vectors per thread and tensor in flight

template <typename T>
__global__ void __launch_bounds__(256) gate_grad_kernel(const T* __restrict__ dout,
                                                       const T* __restrict__ g,
                                                       const T* __restrict__ u, T* __restrict__ dg,
                                                       T* __restrict__ du, int64_t numel) {
  const int64_t nvec = numel >> 3;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint4* d4 = reinterpret_cast<const uint4*>(dout);
  const uint4* g4 = reinterpret_cast<const uint4*>(g);
  const uint4* u4 = reinterpret_cast<const uint4*>(u);
  int64_t v = tid;
  // main loop: kGateGradUnroll independent vectors per thread, all loads issued
  // before the first use
  for (; v + (kGateGradUnroll - 1) * stride < nvec; v += kGateGradUnroll * stride) {
    uint4 vd[kGateGradUnroll], vg[kGateGradUnroll], vu[kGateGradUnroll];
#pragma unroll
    for (int j = 0; j < kGateGradUnroll; ++j) {
      vd[j] = ld_stream(d4 + v + j * stride);
      vg[j] = ld_stream(g4 + v + j * stride);
      vu[j] = ld_stream(u4 + v + j * stride);
    }
#pragma unroll
    for (int j = 0; j < kGateGradUnroll; ++j) {
      uint4 odg, odu;
      gate_grad_vec<T>(vd[j], vg[j], vu[j], odg, odu);
      reinterpret_cast<uint4*>(dg)[v + j * stride] = odg;
      reinterpret_cast<uint4*>(du)[v + j * stride] = odu;
    }
  }
  for (; v < nvec; v += stride) {
    uint4 odg, odu;
    gate_grad_vec<T>(ld_stream(d4 + v), ld_stream(g4 + v), ld_stream(u4 + v), odg, odu);
    reinterpret_cast<uint4*>(dg)[v] = odg;
    reinterpret_cast<uint4*>(du)[v] = odu;
  }
  // tail of fewer than 8 elements
  if (blockIdx.x == 0 && threadIdx.x < (numel & 7)) {
    const int64_t i = (nvec << 3) + threadIdx.x;
    float dgv, duv;
    gate_grad_one<T>(to_f32(dout[i]), to_f32(g[i]), to_f32(u[i]), dgv, duv);
    const uint32_t a = pack2<T>(dgv, 0.f), b = pack2<T>(duv, 0.f);
    reinterpret_cast<unsigned short*>(dg)[i] = static_cast<unsigned short>(a & 0xFFFFu);
    reinterpret_cast<unsigned short*>(du)[i] = static_cast<unsigned short>(b & 0xFFFFu);
  }
}

// dg = dout * t, du = dout * s from the activations saved by a forward with save_st:
// two packed multiplies per pair, each rounding once.
template <typename T>
__global__ void __launch_bounds__(256) gate_grad_st_kernel(const uint4* __restrict__ dout,
                                                          const uint4* __restrict__ s,
                                                          const uint4* __restrict__ t, uint4* __restrict__ dg,
                                                          uint4* __restrict__ du, int64_t nvec) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    const uint4 d = ld_stream(dout + v), a = ld_stream(s + v), b = ld_stream(t + v);
    uint4 og, ou;
    og.x = mul2<T>(d.x, b.x); og.y = mul2<T>(d.y, b.y); og.z = mul2<T>(d.z, b.z); og.w = mul2<T>(d.w, b.w);
    ou.x = mul2<T>(d.x, a.x); ou.y = mul2<T>(d.y, a.y); ou.z = mul2<T>(d.z, a.z); ou.w = mul2<T>(d.w, a.w);
    dg[v] = og;
    du[v] = ou;
  }
}

}  // namespace fsw

using namespace fsw;

// ===================================================================== C ABI ==
extern "C" {

const char* fsw_last_error(void) { return t_err; }

int fsw_query_device(int device, int* sm_count, int* cc_major, int* cc_minor,
                     int64_t* smem_optin_bytes) {
  int n = 0, maj = 0, min = 0, smem = 0;
  FSW_CUDA(cudaDeviceGetAttribute(&maj, cudaDevAttrComputeCapabilityMajor, device));
  FSW_CUDA(cudaDeviceGetAttribute(&min, cudaDevAttrComputeCapabilityMinor, device));
  FSW_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
  FSW_CUDA(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  if (sm_count) *sm_count = n;
  if (cc_major) *cc_major = maj;
  if (cc_minor) *cc_minor = min;
  if (smem_optin_bytes) *smem_optin_bytes = smem;
  if (maj != 10)
    return fail(FSW_EDEVICE,
                "device %d is compute capability %d.%d; this library runs on 10.x (B200) only",
                device, maj, min);
  return FSW_OK;
}

int64_t fsw_status(void) {
  DeviceInfo* d = nullptr;
  int rc = ensure_device(&d);
  if (rc != FSW_OK) return rc;
  FSW_CUDA(cudaDeviceSynchronize());
  uint32_t v = 0, zero = 0;
  FSW_CUDA(cudaMemcpy(&v, d->status, sizeof(v), cudaMemcpyDeviceToHost));
  if (v != 0) {
    FSW_CUDA(cudaMemcpy(d->status, &zero, sizeof(zero), cudaMemcpyHostToDevice));
    fail(FSW_ETIMEOUT, "a kernel gave up on a bounded wait: code %u in CTA %u", v & 0xFFu, v >> 8);
  }
  return (int64_t)v;
}

int fsw_set_option(const char* name, int64_t value) {
  if (name == nullptr) return fail(FSW_EINVAL, "option name is NULL");
  std::lock_guard<std::mutex> lock(g_mu);
  if (!strcmp(name, "cta_group")) {
    if (value < 0 || value > 2) return fail(FSW_EINVAL, "cta_group must be 0 (automatic), 1 or 2");
    g_opt.cta_group = value;
  } else if (!strcmp(name, "nsub")) {
    if (value < 0 || value > 2) return fail(FSW_EINVAL, "nsub must be 0 (automatic), 1 or 2");
    g_opt.nsub = value;
  } else if (!strcmp(name, "group_m")) {
    if (value < 0 || value > (1 << 20)) return fail(FSW_EINVAL, "group_m must be >= 0 (0 = automatic)");
    g_opt.group_m = value;
  } else if (!strcmp(name, "wait_limit_ms")) {
    if (value < 1 || value > 60000) return fail(FSW_EINVAL, "wait_limit_ms must be in [1, 60000]");
    g_opt.wait_limit_ms = value;
  } else if (!strcmp(name, "stall_producer")) {
    if (value != 0 && value != 1) return fail(FSW_EINVAL, "stall_producer must be 0 or 1");
    g_opt.stall_producer = value;
  } else if (!strcmp(name, "gemm_max_sms")) {
    if (value < 0) return fail(FSW_EINVAL, "gemm_max_sms must be >= 0");
    g_opt.gemm_max_sms = value;
  } else if (!strcmp(name, "l2_a") || !strcmp(name, "l2_b") || !strcmp(name, "l2_out")) {
    if (value < 0 || value > 2) return fail(FSW_EINVAL, "%s must be 0, 1 or 2", name);
    (name[3] == 'a' ? g_opt.l2_a : name[3] == 'b' ? g_opt.l2_b : g_opt.l2_out) = value;
  } else if (!strcmp(name, "pace_kb")) {
    if (value < 0 || value > (1 << 20)) return fail(FSW_EINVAL, "pace_kb must be >= 0 (0 = no pacing)");
    g_opt.pace_kb = value;
  } else if (!strcmp(name, "pace_limit_us")) {
    if (value < 1 || value > 100000) return fail(FSW_EINVAL, "pace_limit_us must be in [1, 100000]");
    g_opt.pace_limit_us = value;
  } else if (!strcmp(name, "l2_promo")) {
    if (value < 0 || value > 2) return fail(FSW_EINVAL, "l2_promo must be 0, 1 or 2");
    g_opt.l2_promo = value;
  } else if (!strcmp(name, "split_k")) {
    if (value != 0 && value != 1) return fail(FSW_EINVAL, "split_k must be 0 or 1");
    g_opt.split_k = value;
  } else if (!strcmp(name, "ew_ahead")) {
    if (value < 0 || value > 100000) return fail(FSW_EINVAL, "ew_ahead must be in [0, 100000]");
    g_opt.ew_ahead = value;
  } else if (!strcmp(name, "gate_in_dx")) {
    if (value != 0 && value != 1) return fail(FSW_EINVAL, "gate_in_dx must be 0 or 1");
    g_opt.gate_in_dx = value;
  } else if (!strcmp(name, "scatter_gap_ns")) {
    if (value < -1 || value > 100000) return fail(FSW_EINVAL, "scatter_gap_ns must be in [-1, 100000]");
    g_opt.scatter_gap_ns = value;
  } else if (!strcmp(name, "ew_blocks_per_sm")) {
    if (value < 1 || value > 64) return fail(FSW_EINVAL, "ew_blocks_per_sm must be in [1, 64]");
    g_opt.ew_blocks_per_sm = value;
  } else {
    return fail(FSW_EINVAL, "unknown option '%s'", name);
  }
  return FSW_OK;
}

int64_t fsw_get_option(const char* name) {
  if (name == nullptr) return -1;
  if (!strcmp(name, "cta_group")) return g_opt.cta_group;
  if (!strcmp(name, "group_m")) return g_opt.group_m;
  if (!strcmp(name, "nsub")) return g_opt.nsub;
  if (!strcmp(name, "ew_blocks_per_sm")) return g_opt.ew_blocks_per_sm;
  if (!strcmp(name, "split_k")) return g_opt.split_k;
  if (!strcmp(name, "scatter_gap_ns")) return g_opt.scatter_gap_ns;
  if (!strcmp(name, "gate_in_dx")) return g_opt.gate_in_dx;
  if (!strcmp(name, "ew_ahead")) return g_opt.ew_ahead;
  if (!strcmp(name, "gemm_max_sms")) return g_opt.gemm_max_sms;
  if (!strcmp(name, "wait_limit_ms")) return g_opt.wait_limit_ms;
  if (!strcmp(name, "stall_producer")) return g_opt.stall_producer;
  if (!strcmp(name, "l2_a")) return g_opt.l2_a;
  if (!strcmp(name, "l2_b")) return g_opt.l2_b;
  if (!strcmp(name, "l2_out")) return g_opt.l2_out;
  if (!strcmp(name, "l2_promo")) return g_opt.l2_promo;
  if (!strcmp(name, "pace_kb")) return g_opt.pace_kb;
  if (!strcmp(name, "pace_limit_us")) return g_opt.pace_limit_us;
  if (!strcmp(name, "pace_off")) {
    // 1 if the last paced launch on the current device switched its pacing off; synchronises
    DeviceInfo* d = nullptr;
    if (ensure_device(&d) != FSW_OK) return -1;
    unsigned int v[2] = {0, 0};
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpy(v, d->pace + 2 * d->pace_last, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess)
      return -1;
    return v[1];
  }
  if (!strcmp(name, "kernel_launches")) return (int64_t)g_kernel_launches.load();
  if (!strcmp(name, "map_cache_hits")) return (int64_t)g_map_hits;
  if (!strcmp(name, "map_cache_misses")) return (int64_t)g_map_misses;
  if (!strcmp(name, "last_sm_khz")) {
    // Synchronises; average SM clock (kHz) seen by CTA 0 of the last GEMM launch.
    DeviceInfo* d = nullptr;
    if (ensure_device(&d) != FSW_OK) return -1;
    unsigned long long v[2] = {0, 0};
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpy(v, d->clk_probe, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return v[1] ? (int64_t)(v[0] * 1000000ull / v[1]) : -1;
  }
  if (!strncmp(name, "probe", 5) && name[5] >= '0' && name[5] <= '7' && name[6] == 0) {
    // Raw diagnostic counters of the last GEMM launch (see FSW_PROFILE); synchronises.
    DeviceInfo* d = nullptr;
    if (ensure_device(&d) != FSW_OK) return -1;
    unsigned long long v[8] = {};
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpy(v, d->clk_probe, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return (int64_t)v[name[5] - '0'];
  }
  if (!strcmp(name, "max_pairs") || !strcmp(name, "sm_count") || !strcmp(name, "stages")) {
    // facts about the current device (initialises it on first use)
    DeviceInfo* d = nullptr;
    if (ensure_device(&d) != FSW_OK) return -1;
    if (!strcmp(name, "max_pairs")) return d->max_pairs;
    if (!strcmp(name, "sm_count")) return d->sm_count;
    if (g_opt.cta_group == 1) return TileCfg<MODE_FWD, 1, 1>::STAGES;
    return g_opt.nsub == 1 ? TileCfg<MODE_FWD, 2, 1>::STAGES : TileCfg<MODE_FWD, 2, 2>::STAGES;
  }
  return -1;
}

int fsw_forward(const void* x, const void* w_gate, const void* w_up, void* out, void* g, void* u,
                int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream) {
  return fsw_forward_ws(x, w_gate, w_up, out, g, u, T, dm, di, nullptr, 0, dtype, accum, stream);
}

static int forward_impl(const void* x, const void* w_gate, const void* w_up, void* out, void* g, void* u,
                        int64_t T, int64_t dm, int64_t di, void* workspace, int64_t workspace_bytes,
                        int dtype, int accum, void* stream, int save_st);

int fsw_forward_ws(const void* x, const void* w_gate, const void* w_up, void* out, void* g, void* u,
                   int64_t T, int64_t dm, int64_t di, void* workspace, int64_t workspace_bytes,
                   int dtype, int accum, void* stream) {
  return forward_impl(x, w_gate, w_up, out, g, u, T, dm, di, workspace, workspace_bytes, dtype, accum,
                      stream, 0);
}

int fsw_forward_st(const void* x, const void* w_gate, const void* w_up, void* out, void* s, void* t,
                   int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream) {
  if (!s || !t) return fail(FSW_EINVAL, "s and t are required");
  // (the second pass of a split last wave only knows the g / u form, so no workspace here)
  return forward_impl(x, w_gate, w_up, out, s, t, T, dm, di, nullptr, 0, dtype, accum, stream, 1);
}

static int forward_impl(const void* x, const void* w_gate, const void* w_up, void* out, void* g, void* u,
                        int64_t T, int64_t dm, int64_t di, void* workspace, int64_t workspace_bytes,
                        int dtype, int accum, void* stream, int save_st) {
  int rc = check_common(T, dm, di, dtype, accum);
  if (rc != FSW_OK) return rc;
  if (T == 0) return FSW_OK;  // nothing to compute; empty tensors may have NULL storage
  if (!x || !w_gate || !w_up || !out) return fail(FSW_EINVAL, "x, w_gate, w_up and out are required");
  if ((g == nullptr) != (u == nullptr))
    return fail(FSW_EINVAL, "g and u must both be given or both be NULL");
  if (!aligned16(x) || !aligned16(w_gate) || !aligned16(w_up) || !aligned16(out) || !aligned16(g) ||
      !aligned16(u))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  DeviceInfo* d = nullptr;
  if ((rc = ensure_device(&d)) != FSW_OK) return rc;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = make_map(&p.a0, x, dtype, dm, T, 128, "x")) != FSW_OK) return rc;
  p.a1 = p.a0;
  if ((rc = make_map(&p.b0, w_gate, dtype, di, dm, 64, "w_gate")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b1, w_up, dtype, di, dm, 64, "w_up")) != FSW_OK) return rc;
  if ((rc = make_map(&p.sg, g ? g : out, dtype, di, T, 32, "g (store)", 32)) != FSW_OK) return rc;
  if ((rc = make_map(&p.su, u ? u : out, dtype, di, T, 32, "u (store)", 32)) != FSW_OK) return rc;
  if ((rc = make_map(&p.so, out, dtype, di, T, 32, "out (store)", 32)) != FSW_OK) return rc;
  p.M = (int)T;
  p.N = (int)di;
  p.num_k_blocks = (int)((dm + 63) / 64);
  p.store_gu = g != nullptr;
  p.c0_ptr = g;
  p.c1_ptr = u;
  p.c2_ptr = out;
  if (save_st)
    return run_gemm<MODE_FWDST>(p, (int)T, dtype, accum == FSW_ACC_F16, static_cast<cudaStream_t>(stream),
                                d, choose_tiles(MODE_FWD, T, di, d));
  return run_gemm<MODE_FWD>(p, (int)T, dtype, accum == FSW_ACC_F16,
                            static_cast<cudaStream_t>(stream), d,
                            choose_tiles(MODE_FWD, T, di, d, 0, workspace != nullptr), 0, workspace,
                            workspace_bytes);
}

int fsw_backward_elementwise(const void* dout, const void* g, const void* u, void* dg, void* du,
                             int64_t numel, int dtype, void* stream) {
  if (dtype != FSW_BF16 && dtype != FSW_FP16) return fail(FSW_EINVAL, "unknown dtype %d", dtype);
  if (numel < 0) return fail(FSW_EINVAL, "numel < 0");
  if (numel == 0) return FSW_OK;
  if (!dout || !g || !u || !dg || !du) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(dout) || !aligned16(g) || !aligned16(u) || !aligned16(dg) || !aligned16(du))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  DeviceInfo* d = nullptr;
  int rc = ensure_device(&d);
  if (rc != FSW_OK) return rc;
  const int64_t nvec = numel >> 3;
  int64_t blocks = (nvec + 255) / 256;
  const int64_t cap = (int64_t)d->sm_count * (g_opt.ew_blocks_per_sm > 0 ? g_opt.ew_blocks_per_sm : 32);
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ++g_kernel_launches;
  if (dtype == FSW_BF16)
    gate_grad_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(g),
        static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(dg),
        static_cast<__nv_bfloat16*>(du), numel);
  else
    gate_grad_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __half*>(dout), static_cast<const __half*>(g),
        static_cast<const __half*>(u), static_cast<__half*>(dg), static_cast<__half*>(du), numel);
  FSW_CUDA(cudaGetLastError());
  return FSW_OK;
}

int fsw_backward_elementwise_st(const void* dout, const void* s, const void* t, void* dg, void* du,
                                int64_t numel, int dtype, void* stream) {
  if (dtype != FSW_BF16 && dtype != FSW_FP16) return fail(FSW_EINVAL, "unknown dtype %d", dtype);
  if (numel < 0 || (numel & 7)) return fail(FSW_EINVAL, "numel must be a non-negative multiple of 8");
  if (numel == 0) return FSW_OK;
  if (!dout || !s || !t || !dg || !du) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(dout) || !aligned16(s) || !aligned16(t) || !aligned16(dg) || !aligned16(du))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  DeviceInfo* d = nullptr;
  int rc = ensure_device(&d);
  if (rc != FSW_OK) return rc;
  const int64_t nvec = numel >> 3;
  int64_t blocks = (nvec + 255) / 256;
  const int64_t cap = (int64_t)d->sm_count * 32;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ++g_kernel_launches;
  if (dtype == FSW_BF16)
    gate_grad_st_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const uint4*>(dout), static_cast<const uint4*>(s), static_cast<const uint4*>(t),
        static_cast<uint4*>(dg), static_cast<uint4*>(du), nvec);
  else
    gate_grad_st_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const uint4*>(dout), static_cast<const uint4*>(s), static_cast<const uint4*>(t),
        static_cast<uint4*>(dg), static_cast<uint4*>(du), nvec);
  FSW_CUDA(cudaGetLastError());
  return FSW_OK;
}

// dX GEMM with the gate-gradient step inside: the A tiles dout * t and dout * s are
// produced by the kernel's own warps; dg and du are also written out for the dW GEMM.
int fsw_backward_dx_fused(const void* dout, const void* s, const void* t, const void* w_gate,
                          const void* w_up, void* dx, void* dg, void* du, int64_t T, int64_t dm,
                          int64_t di, int dtype, void* stream) {
  int rc = check_common(T, dm, di, dtype, FSW_ACC_F32);
  if (rc != FSW_OK) return rc;
  if (T == 0) return FSW_OK;
  if (!dout || !s || !t || !w_gate || !w_up || !dx || !dg || !du) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(dout) || !aligned16(s) || !aligned16(t) || !aligned16(w_gate) || !aligned16(w_up) ||
      !aligned16(dx) || !aligned16(dg) || !aligned16(du))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  DeviceInfo* d = nullptr;
  if ((rc = ensure_device(&d)) != FSW_OK) return rc;
  const TileChoice tc = choose_tiles(MODE_DX, T, dm, d);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  // A has no tensor map (the warps read dout, s, t with plain loads); the maps of B are MODE_DX's
  if ((rc = make_map(&p.b0, w_gate, dtype, di, dm, 256 / tc.cg, "w_gate")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b1, w_up, dtype, di, dm, 256 / tc.cg, "w_up")) != FSW_OK) return rc;
  p.a0 = p.a1 = p.b0;
  p.c0_ptr = dx;
  p.M = (int)T;
  p.N = (int)dm;
  p.num_k_blocks = (int)((di + 63) / 64);
  p.gg_dout = dout;
  p.gg_s = s;
  p.gg_t = t;
  p.gg_dg = dg;
  p.gg_du = du;
  p.gg_k = (int)di;
  return run_gemm<MODE_DXG>(p, (int)T, dtype, false, static_cast<cudaStream_t>(stream), d, tc);
}

// Gate-gradient step and dX in one launch: the elementwise work is done once, by the
// GEMM kernel's own epilogue warps while they wait for accumulators, ahead of the tiles
// that read dg and du.  Results are those of fsw_backward_elementwise + fsw_backward_dx_ws.
int fsw_backward_dx_gate(const void* dout, const void* g, const void* u, const void* w_gate,
                         const void* w_up, void* dx, void* dg, void* du, int64_t T, int64_t dm,
                         int64_t di, void* workspace, int64_t workspace_bytes, int dtype, void* stream) {
  int rc = check_common(T, dm, di, dtype, FSW_ACC_F32);
  if (rc != FSW_OK) return rc;
  if (T == 0) return FSW_OK;
  if (!dout || !g || !u || !w_gate || !w_up || !dx || !dg || !du) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(dout) || !aligned16(g) || !aligned16(u) || !aligned16(w_gate) || !aligned16(w_up) ||
      !aligned16(dx) || !aligned16(dg) || !aligned16(du))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  DeviceInfo* d = nullptr;
  if ((rc = ensure_device(&d)) != FSW_OK) return rc;
  const TileChoice tc = choose_tiles(MODE_DX, T, dm, d, 0, workspace != nullptr);
  const int64_t row_tiles = (T + 255) / 256;
  if (tc.cg != 2 || row_tiles > kEwMaxRowTiles || g_opt.gate_in_dx == 0) {
    // the side job is written for 256-row tiles of CTA pairs: otherwise two launches
    if ((rc = fsw_backward_elementwise(dout, g, u, dg, du, T * di, dtype, stream)) != FSW_OK) return rc;
    return fsw_backward_dx_ws(dg, du, w_gate, w_up, dx, T, dm, di, workspace, workspace_bytes, dtype,
                              FSW_ACC_F32, stream);
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = make_map(&p.a0, dg, dtype, di, T, 128, "dg")) != FSW_OK) return rc;
  if ((rc = make_map(&p.a1, du, dtype, di, T, 128, "du")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b0, w_gate, dtype, di, dm, 256 / tc.cg, "w_gate")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b1, w_up, dtype, di, dm, 256 / tc.cg, "w_up")) != FSW_OK) return rc;
  p.c0_ptr = dx;
  p.M = (int)T;
  p.N = (int)dm;
  p.num_k_blocks = (int)((di + 63) / 64);
  p.ew_dout = dout;
  p.ew_g = g;
  p.ew_u = u;
  p.ew_dg = dg;
  p.ew_du = du;
  p.ew_cols = (int)di;
  p.ew_qpm = (int)(256 * di / 2048);
  {
    // one wave of tiles ahead: the row tiles that a wave of SM pairs works on at once, plus two
    const int64_t n_tiles = (dm + 511) / 512;
    const int64_t ahead = g_opt.ew_ahead > 0 ? g_opt.ew_ahead : (d->max_pairs + n_tiles - 1) / n_tiles + 2;
    p.ew_ahead = (int)(ahead < 1 ? 1 : ahead);
  }
  unsigned int slot;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    slot = d->ew_next++ % kEwSlots;
  }
  p.ew_ctrl = d->ew_ctrl + (size_t)slot * (2 + kEwMaxRowTiles);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FSW_CUDA(cudaMemsetAsync(p.ew_ctrl, 0, (size_t)(2 + row_tiles) * sizeof(unsigned int), st));
  return run_gemm<MODE_DXE>(p, (int)T, dtype, false, st, d, tc, 0, workspace, workspace_bytes);
}

int fsw_backward_dx(const void* dg, const void* du, const void* w_gate, const void* w_up, void* dx,
                    int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream) {
  return fsw_backward_dx_ws(dg, du, w_gate, w_up, dx, T, dm, di, nullptr, 0, dtype, accum, stream);
}

int fsw_backward_dx_ws(const void* dg, const void* du, const void* w_gate, const void* w_up,
                       void* dx, int64_t T, int64_t dm, int64_t di, void* workspace,
                       int64_t workspace_bytes, int dtype, int accum, void* stream) {
  int rc = check_common(T, dm, di, dtype, accum);
  if (rc != FSW_OK) return rc;
  if (T == 0) return FSW_OK;
  if (!dg || !du || !w_gate || !w_up || !dx) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(dg) || !aligned16(du) || !aligned16(w_gate) || !aligned16(w_up) || !aligned16(dx))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  DeviceInfo* d = nullptr;
  if ((rc = ensure_device(&d)) != FSW_OK) return rc;
  const TileChoice tc = choose_tiles(MODE_DX, T, dm, d, 0, workspace != nullptr);
  const int cg = tc.cg;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = make_map(&p.a0, dg, dtype, di, T, 128, "dg")) != FSW_OK) return rc;
  if ((rc = make_map(&p.a1, du, dtype, di, T, 128, "du")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b0, w_gate, dtype, di, dm, 256 / cg, "w_gate")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b1, w_up, dtype, di, dm, 256 / cg, "w_up")) != FSW_OK) return rc;
  p.c0_ptr = dx;
  p.M = (int)T;
  p.N = (int)dm;
  p.num_k_blocks = (int)((di + 63) / 64);
  return run_gemm<MODE_DX>(p, (int)T, dtype, accum == FSW_ACC_F16,
                           static_cast<cudaStream_t>(stream), d, tc, 0, workspace, workspace_bytes);
}

// dX GEMM whose epilogue stores the partial sums into the owning ranks' buffers.
int fsw_backward_dx_scatter(const void* dg, const void* du, const void* w_gate, const void* w_up,
                            void* const* recv_ptrs, int world, int rank, int64_t T, int64_t dm,
                            int64_t di, int dtype, int accum, void* stream) {
  int rc = check_common(T, dm, di, dtype, accum);
  if (rc != FSW_OK) return rc;
  if (world < 2 || world > kMaxScatterRanks || rank < 0 || rank >= world)
    return fail(FSW_EINVAL, "world size %d (2..%d) / rank %d", world, kMaxScatterRanks, rank);
  if (T <= 0 || T % world != 0 || (T / world) % 32 != 0)
    return fail(FSW_EINVAL, "T = %lld must split into %d equal parts of a multiple of 32 rows",
                (long long)T, world);
  if (!dg || !du || !w_gate || !w_up || !recv_ptrs) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(dg) || !aligned16(du) || !aligned16(w_gate) || !aligned16(w_up))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  for (int r = 0; r < world; ++r)
    if (recv_ptrs[r] == nullptr || !aligned16(recv_ptrs[r]))
      return fail(FSW_EINVAL, "receive buffer of rank %d is NULL or not 16-byte aligned", r);
  DeviceInfo* d = nullptr;
  if ((rc = ensure_device(&d)) != FSW_OK) return rc;
  const TileChoice tc = choose_tiles(MODE_DX, T, dm, d);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = make_map(&p.a0, dg, dtype, di, T, 128, "dg")) != FSW_OK) return rc;
  if ((rc = make_map(&p.a1, du, dtype, di, T, 128, "du")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b0, w_gate, dtype, di, dm, 256 / tc.cg, "w_gate")) != FSW_OK) return rc;
  if ((rc = make_map(&p.b1, w_up, dtype, di, dm, 256 / tc.cg, "w_up")) != FSW_OK) return rc;
  p.M = (int)T;
  p.N = (int)dm;
  p.num_k_blocks = (int)((di + 63) / 64);
  for (int r = 0; r < world; ++r) p.scatter[r] = recv_ptrs[r];
  p.scatter_world = world;
  p.scatter_rank = rank;
  p.scatter_rows = (int)(T / world);
  // Spread a tile's 32 store instructions per warp over about 60 % of the tile's K loop
  // (0.8 us per K block of a 256x512 tile at the sustained rate).
  if (g_opt.scatter_gap_ns >= 0) {
    p.scatter_gap_ns = (unsigned int)g_opt.scatter_gap_ns;
  } else {
    const double tile_ns = 2.0 * p.num_k_blocks * 800.0;
    double gap = 0.6 * tile_ns / 32.0;
    p.scatter_gap_ns = (unsigned int)(gap > 4000.0 ? 4000.0 : gap);
  }
  // start at the rows of the next rank; this rank's own rows (local stores) come last
  {
    const int tile_m = 128 * tc.cg;
    const int m_tiles = (int)((T + tile_m - 1) / tile_m);
    p.m_rotate = (int)((((int64_t)(rank + 1) % world) * (T / world)) / tile_m) % m_tiles;
  }
  return run_gemm<MODE_DX>(p, (int)T, dtype, accum == FSW_ACC_F16,
                           static_cast<cudaStream_t>(stream), d, tc);
}

int fsw_dx_reduce(const void* recv, const void* own_slice, void* const* peer_flag_ptrs, void* my_flags,
                  int world, int rank, uint32_t seq, int64_t rows, int64_t dm, void* dx_rows, int dtype,
                  void* stream) {
  if (dtype != FSW_BF16 && dtype != FSW_FP16) return fail(FSW_EINVAL, "unknown dtype %d", dtype);
  if (world < 2 || world > kMaxScatterRanks || rank < 0 || rank >= world)
    return fail(FSW_EINVAL, "world size %d (2..%d) / rank %d", world, kMaxScatterRanks, rank);
  if (rows <= 0 || dm <= 0 || (dm & 7)) return fail(FSW_EINVAL, "bad shape rows=%lld dm=%lld", (long long)rows, (long long)dm);
  if (!recv || !peer_flag_ptrs || !my_flags || !dx_rows) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(recv) || !aligned16(own_slice) || !aligned16(dx_rows) ||
      (reinterpret_cast<uintptr_t>(my_flags) & 3u))
    return fail(FSW_EINVAL, "pointers must be aligned (16 bytes; flags 4 bytes)");
  PeerFlags pf;
  memset(&pf, 0, sizeof(pf));
  for (int r = 0; r < world; ++r) {
    if (peer_flag_ptrs[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_flag_ptrs[r]) & 3u))
      return fail(FSW_EINVAL, "flag pointer of rank %d is NULL or misaligned", r);
    pf.p[r] = static_cast<unsigned int*>(peer_flag_ptrs[r]);
  }
  DeviceInfo* d = nullptr;
  int rc = ensure_device(&d);
  if (rc != FSW_OK) return rc;
  const long long vecs = rows * dm / 8;
  long long blocks = (vecs + 255) / 256;
  const long long cap = (long long)d->sm_count * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned long long limit = (unsigned long long)g_opt.wait_limit_ms * 1000000ull;
  ++g_kernel_launches;
  if (dtype == FSW_BF16)
    dx_slices_reduce_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const uint4*>(recv), static_cast<const uint4*>(own_slice),
        static_cast<__nv_bfloat16*>(dx_rows), vecs, world, rank, seq, pf, static_cast<unsigned int*>(my_flags), d->status, limit);
  else
    dx_slices_reduce_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const uint4*>(recv), static_cast<const uint4*>(own_slice),
        static_cast<__half*>(dx_rows), vecs, world, rank, seq, pf,
        static_cast<unsigned int*>(my_flags), d->status, limit);
  FSW_CUDA(cudaGetLastError());
  return FSW_OK;
}

int fsw_wait_flags(void* flags, int n, uint32_t seq, void* stream) {
  if (!flags || (reinterpret_cast<uintptr_t>(flags) & 3u) || n < 1 || n > 32)
    return fail(FSW_EINVAL, "bad flag array");
  DeviceInfo* d = nullptr;
  int rc = ensure_device(&d);
  if (rc != FSW_OK) return rc;
  ++g_kernel_launches;
  wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned int*>(flags), n, seq, d->status,
      (unsigned long long)g_opt.wait_limit_ms * 1000000ull);
  FSW_CUDA(cudaGetLastError());
  return FSW_OK;
}

// Columns [col0, col0 + ncols) of both weight gradients; all pointers are to the
// full arrays, whose rows are di elements long.
static int backward_dw_columns(const void* x, const void* dg, const void* du, void* dw_gate,
                               void* dw_up, int64_t T, int64_t dm, int64_t di, int64_t col0,
                               int64_t ncols, int max_sms, void* ws, int64_t ws_bytes, int dtype,
                               int accum, void* stream) {
  int rc = check_common(T, dm, di, dtype, accum);
  if (rc != FSW_OK) return rc;
  if (max_sms < 0) return fail(FSW_EINVAL, "max_sms must be >= 0 (0 = no cap of its own)");
  if (col0 < 0 || ncols < 0 || col0 + ncols > di || (col0 % 8) != 0 || (ncols % 8) != 0)
    return fail(FSW_EINVAL, "column range [%lld, +%lld) must lie in [0, %lld) and be multiples of 8",
                (long long)col0, (long long)ncols, (long long)di);
  if (!dw_gate || !dw_up) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(x) || !aligned16(dg) || !aligned16(du) || !aligned16(dw_gate) || !aligned16(dw_up))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  DeviceInfo* d = nullptr;
  if ((rc = ensure_device(&d)) != FSW_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ncols == 0) return FSW_OK;
  char* wg_out = static_cast<char*>(dw_gate) + col0 * 2;
  char* wu_out = static_cast<char*>(dw_up) + col0 * 2;
  if (T == 0) {
    // An empty reduction: the gradients are exactly zero.
    FSW_CUDA(cudaMemset2DAsync(wg_out, (size_t)di * 2, 0, (size_t)ncols * 2, (size_t)dm, st));
    FSW_CUDA(cudaMemset2DAsync(wu_out, (size_t)di * 2, 0, (size_t)ncols * 2, (size_t)dm, st));
    return FSW_OK;
  }
  if (!x || !dg || !du) return fail(FSW_EINVAL, "NULL pointer");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  if ((rc = make_map(&p.a0, x, dtype, dm, T, 64, "x^T")) != FSW_OK) return rc;
  p.a1 = p.a0;
  if ((rc = make_map(&p.b0, static_cast<const char*>(dg) + col0 * 2, dtype, ncols, T, 64, "dg", 64,
                     di)) != FSW_OK)
    return rc;
  if ((rc = make_map(&p.b1, static_cast<const char*>(du) + col0 * 2, dtype, ncols, T, 64, "du", 64,
                     di)) != FSW_OK)
    return rc;
  p.c0_ptr = wg_out;
  p.c1_ptr = wu_out;
  p.M = (int)dm;
  p.N = (int)ncols;
  p.ldc = (int)di;
  p.num_k_blocks = (int)((T + 63) / 64);
  return run_gemm<MODE_DW>(p, (int)dm, dtype, accum == FSW_ACC_F16, st, d,
                           choose_tiles(MODE_DW, dm, ncols, d, max_sms, ws != nullptr), max_sms, ws,
                           ws_bytes);
}

int fsw_backward_dw(const void* x, const void* dg, const void* du, void* dw_gate, void* dw_up,
                    int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream) {
  return backward_dw_columns(x, dg, du, dw_gate, dw_up, T, dm, di, 0, di, 0, nullptr, 0, dtype,
                             accum, stream);
}

int fsw_backward_dw_columns(const void* x, const void* dg, const void* du, void* dw_gate,
                            void* dw_up, int64_t T, int64_t dm, int64_t di, int64_t col0,
                            int64_t ncols, int max_sms, void* workspace, int64_t workspace_bytes,
                            int dtype, int accum, void* stream) {
  if (workspace_bytes < 0) return fail(FSW_EINVAL, "workspace_bytes < 0");
  return backward_dw_columns(x, dg, du, dw_gate, dw_up, T, dm, di, col0, ncols, max_sms, workspace,
                             workspace_bytes, dtype, accum, stream);
}

int64_t fsw_workspace_bytes(void) {
  DeviceInfo* d = nullptr;
  int rc = ensure_device(&d);
  if (rc != FSW_OK) return rc;
  return splitk_workspace_bytes(d);
}

int fsw_backward(const void* dout, const void* x, const void* w_gate, const void* w_up,
                 const void* g, const void* u, void* dg_scratch, void* du_scratch, void* dx,
                 void* dw_gate, void* dw_up, int64_t T, int64_t dm, int64_t di, int dtype,
                 int accum, void* stream) {
  int rc = check_common(T, dm, di, dtype, accum);
  if (rc != FSW_OK) return rc;
  if ((rc = fsw_backward_elementwise(dout, g, u, dg_scratch, du_scratch, T * di, dtype, stream)) !=
      FSW_OK)
    return rc;
  if ((rc = fsw_backward_dx(dg_scratch, du_scratch, w_gate, w_up, dx, T, dm, di, dtype,
                            FSW_ACC_F32, stream)) != FSW_OK)
    return rc;
  return fsw_backward_dw(x, dg_scratch, du_scratch, dw_gate, dw_up, T, dm, di, dtype, accum,
                         stream);
}

// Host copy of the kernels' tile rasterisation, for tests of the scheduling math.
int fsw_debug_decode_tile(int t, int num_m_tiles, int num_n_tiles, int group_m, int* m_tile,
                          int* n_tile) {
  if (!m_tile || !n_tile || num_m_tiles < 1 || num_n_tiles < 1 || group_m < 1 || t < 0 ||
      (int64_t)t >= (int64_t)num_m_tiles * num_n_tiles)
    return fail(FSW_EINVAL, "bad tile query");
  decode_tile_order(t, num_m_tiles, num_n_tiles, group_m, *m_tile, *n_tile);
  return FSW_OK;
}

// Host copy of the kernels' work distribution with a split last wave, for tests:
// the plan for `num_m_tiles x num_n_tiles` tiles of `iters_per_tile` K iterations on
// `pairs` CTA pairs (returns 1 and fills plan[3] = {first split tile, iterations per
// pair, total split iterations} if the split pays, else 0), and, with item != NULL,
// work item `idx` of pair `cluster` under that plan as item[6] = {valid, m_tile,
// n_tile, it0, it1, slot}.
int fsw_debug_split_work(int num_m_tiles, int num_n_tiles, int group_m, int iters_per_tile,
                         int pairs, int cluster, int idx, int64_t* plan, int* item) {
  if (num_m_tiles < 1 || num_n_tiles < 1 || group_m < 1 || iters_per_tile < 1 || pairs < 1 || !plan)
    return fail(FSW_EINVAL, "bad split query");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.num_m_tiles = num_m_tiles;
  p.num_n_tiles = num_n_tiles;
  p.group_m = group_m;
  const long long tiles = (long long)num_m_tiles * num_n_tiles;
  const bool split = plan_split(tiles, pairs, iters_per_tile, &p.sk_first_tile,
                                &p.sk_iters_per_cluster, &p.sk_total_iters);
  if (!split) p.sk_total_iters = 0;
  plan[0] = p.sk_first_tile;
  plan[1] = p.sk_iters_per_cluster;
  plan[2] = p.sk_total_iters;
  if (item != nullptr) {
    // without a split the kernel launches min(tiles, pairs) pairs
    const int clusters = split ? pairs : (int)(tiles < pairs ? tiles : pairs);
    WorkItem w = {0, 0, 0, 0, -1};
    const bool ok = cluster >= 0 && cluster < clusters && idx >= 0 &&
                    next_work(p, iters_per_tile, cluster, clusters, idx, w);
    item[0] = ok ? 1 : 0;
    item[1] = w.m_tile;
    item[2] = w.n_tile;
    item[3] = w.it0;
    item[4] = w.it1;
    item[5] = w.slot;
  }
  return split ? 1 : 0;
}

// The descriptor constants a launch would use, for known-answer tests of the encoders.
int fsw_debug_descriptors(int dtype, int accum, int a_major, int b_major, int m, int n,
                          uint32_t* idesc, uint64_t* sdesc_k_major, uint64_t* sdesc_mn_major) {
  if ((dtype != FSW_BF16 && dtype != FSW_FP16) || (a_major | b_major) >> 1 || !idesc ||
      !sdesc_k_major || !sdesc_mn_major)
    return fail(FSW_EINVAL, "bad descriptor query");
  *idesc = make_idesc(dtype, accum == FSW_ACC_F16, a_major, b_major, m, n);
  uint32_t kadv = 0;
  fill_operand_desc(MAJOR_K, sdesc_k_major, &kadv);
  fill_operand_desc(MAJOR_MN, sdesc_mn_major, &kadv);
  return FSW_OK;
}

// Plain GEMM C (M,N) = op(A) @ op(B) on row-major 16-bit arrays, for the projection
// that follows SwiGLU in an MLP block and its two gradients.
int fsw_gemm(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int trans_a,
             int trans_b, int dtype, int accum, void* stream) {
  return fsw_gemm_ws(a, b, c, M, N, K, trans_a, trans_b, nullptr, 0, dtype, accum, stream);
}

int fsw_gemm_ws(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int trans_a,
                int trans_b, void* workspace, int64_t workspace_bytes, int dtype, int accum,
                void* stream) {
  if (dtype != FSW_BF16 && dtype != FSW_FP16) return fail(FSW_EINVAL, "unknown dtype %d", dtype);
  if (accum != FSW_ACC_F32 && !(accum == FSW_ACC_F16 && dtype == FSW_FP16))
    return fail(FSW_EINVAL, "bad accumulate mode %d for dtype %d", accum, dtype);
  if (trans_a && trans_b) return fail(FSW_EINVAL, "A^T @ B^T is not provided");
  if (M < 0 || N <= 0 || K < 0 || M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31))
    return fail(FSW_EINVAL, "bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  // every row of A, B and C must be a multiple of 16 bytes
  const int64_t a_inner = trans_a ? M : K, b_inner = trans_b ? K : N;
  if ((a_inner & 7) || (b_inner & 7) || (N & 7))
    return fail(FSW_EINVAL, "row lengths (%lld, %lld, %lld) must be multiples of 8",
                (long long)a_inner, (long long)b_inner, (long long)N);
  if (M == 0) return FSW_OK;
  if (!c) return fail(FSW_EINVAL, "NULL pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceInfo* d = nullptr;
  int rc = ensure_device(&d);
  if (rc != FSW_OK) return rc;
  if (K == 0) {
    FSW_CUDA(cudaMemsetAsync(c, 0, (size_t)M * N * 2, st));
    return FSW_OK;
  }
  if (!a || !b) return fail(FSW_EINVAL, "NULL pointer");
  if (!aligned16(a) || !aligned16(b) || !aligned16(c))
    return fail(FSW_EINVAL, "pointers must be 16-byte aligned");
  const int mode = trans_a ? MODE_TN : (trans_b ? MODE_NT : MODE_NN);
  const TileChoice tc = choose_tiles(mode, M, N, d, 0, workspace != nullptr);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  // A: K-major -> rows of 64 k, 128 rows per box; MN-major -> 64 m x 64 k boxes
  if ((rc = make_map(&p.a0, a, dtype, a_inner, trans_a ? K : M, trans_a ? 64 : 128, "A")) != FSW_OK)
    return rc;
  p.a1 = p.a0;
  // B: K-major (given as (N,K)) -> 256/cg rows per box; MN-major -> 64 n x 64 k boxes
  if ((rc = make_map(&p.b0, b, dtype, b_inner, trans_b ? N : K, trans_b ? 256 / tc.cg : 64, "B")) !=
      FSW_OK)
    return rc;
  p.b1 = p.b0;
  p.sg = p.su = p.so = p.a0;
  p.c0_ptr = c;
  p.M = (int)M;
  p.N = (int)N;
  p.num_k_blocks = (int)((K + 63) / 64);
  const bool acc16 = accum == FSW_ACC_F16;
  if (mode == MODE_NN) return run_gemm<MODE_NN>(p, (int)M, dtype, acc16, st, d, tc, 0, workspace, workspace_bytes);
  if (mode == MODE_NT) return run_gemm<MODE_NT>(p, (int)M, dtype, acc16, st, d, tc, 0, workspace, workspace_bytes);
  return run_gemm<MODE_TN>(p, (int)M, dtype, acc16, st, d, tc, 0, workspace, workspace_bytes);
}

// ------------------------------------------------- backward without allocation --
// Scratch for fsw_backward_static_scratch: dg and du, each up to
// FSW_STATIC_SCRATCH_ELEMS 16-bit elements, 256-byte aligned.  The array lives in
// the library image, so every GPU that loads the library holds these 16 MiB until
// the process exits.  In host code `g_static_scratch` is only a handle for
// cudaGetSymbolAddress; the device address is resolved once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[2ull * FSW_STATIC_SCRATCH_ELEMS * 2ull];
static unsigned char* g_static_scratch_ptr[fsw::kMaxDevices] = {};

int fsw_backward_static_scratch(const void* dout, const void* x, const void* w_gate,
                                const void* w_up, const void* g, const void* u, void* dx,
                                void* dw_gate, void* dw_up, int64_t T, int64_t dm, int64_t di,
                                int dtype, int accum, void* stream) {
  int rc = check_common(T, dm, di, dtype, accum);
  if (rc != FSW_OK) return rc;
  if (T * di > (int64_t)FSW_STATIC_SCRATCH_ELEMS)
    return fail(FSW_EINVAL,
                "T*d_intermediate = %lld exceeds the built-in scratch of %lld elements per tensor; "
                "use fsw_backward with caller-provided scratch for this size",
                (long long)(T * di), (long long)FSW_STATIC_SCRATCH_ELEMS);
  int dev = 0;
  FSW_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FSW_EINVAL, "device index %d out of range", dev);
  unsigned char* base = nullptr;
  {
    // First call on this device: turn the symbol into this device's address.
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_static_scratch_ptr[dev] == nullptr) {
      void* sp = nullptr;
      FSW_CUDA(cudaGetSymbolAddress(&sp, g_static_scratch));
      g_static_scratch_ptr[dev] = static_cast<unsigned char*>(sp);
    }
    base = g_static_scratch_ptr[dev];
  }
  // dg first, du after it on the next 256-byte boundary.  Both are fully
  // overwritten by the elementwise step before the GEMMs read them, so nothing
  // needs clearing between calls.
  const size_t dg_bytes = ((size_t)(T * di) * 2 + 255) & ~(size_t)255;
  void* dg = base;
  void* du = base + dg_bytes;
  return fsw_backward(dout, x, w_gate, w_up, g, u, dg, du, dx, dw_gate, dw_up, T, dm, di, dtype,
                      accum, stream);
}

}  // extern "C"
