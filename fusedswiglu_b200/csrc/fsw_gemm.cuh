// Persistent, warp-specialised tcgen05 GEMM used by all three tensor-core
// phases of fused SwiGLU on sm_100a.
//
//   MODE_FWD : [g | u] = x @ [W_gate | W_up]         (A K-major, B MN-major)
//              epilogue writes g, u and out = silu(g) * u
//   MODE_DX  : dX = dg @ W_gate^T + du @ W_up^T      (A K-major, B K-major)
//              one accumulator, the K loop runs over both products
//   MODE_DW  : [dW_gate | dW_up] = x^T @ [dg | du]   (A MN-major, B MN-major)
//   MODE_DXG : MODE_DX with the gate-gradient step inside: its A tiles dg = dout * t and
//              du = dout * s are not loaded but produced by the epilogue warps from
//              dout and the activations s = silu(g), t = u * silu'(g) that the forward
//              saved (GemmParams::save_st), straight into the swizzled operand stage;
//              the tiles of the first column of tiles also write dg and du out, for the
//              dW GEMM
// and, for the projection that follows SwiGLU in an MLP block, three plain
// single-product GEMMs C = op(A) @ op(B) on row-major arrays:
//   MODE_NN  : A (M,K) @ B (K,N)      (A K-major,  B MN-major)
//   MODE_NT  : A (M,K) @ B (N,K)^T    (A K-major,  B K-major)
//   MODE_TN  : A (K,M)^T @ B (K,N)    (A MN-major, B MN-major)
//
// One CTA owns 128 rows x 512 fp32 columns of tensor memory, used as two
// 256-column accumulator regions.
//   NSUB == 1: a tile is 128 x 256 per CTA; the two regions alternate between
//              consecutive tiles, so the epilogue of tile i overlaps the MMAs of
//              tile i+1.
//   NSUB == 2: a tile is 128 x 512 per CTA and fills both regions; per K block
//              the A tile is staged once and used by two N=256 MMAs, which cuts
//              L2->shared-memory traffic per flop by a quarter.  There is no
//              spare tensor memory, so the SwiGLU epilogue first copies its
//              accumulators (rounded to 16 bits) into registers and releases the
//              region, then does its math and stores beside the next tile's MMAs;
//              the plain epilogues are short next to their K loops and are left
//              un-overlapped.
// With CG == 2 two CTAs of a cluster form a pair: each stages its own 128 rows
// of A and half of every B sub-tile; the pair leader issues M=256 x N=256 MMAs
// that read both CTAs' shared memory and write both CTAs' tensor memory.  No TMA
// multicast is used anywhere.
//
// Warp roles: warp 0 = TMA producer (one thread), warp 1 = TMEM owner and MMA
// issuer (one thread), warps 2.. = epilogue (TMEM -> registers -> 16-bit results
// -> per-warp swizzled shared-memory buffer -> global memory; the plain GEMMs read
// the buffer back for row-coalesced 16-byte stores, the SwiGLU epilogue hands it to
// TMA stores).
//
// Every mbarrier wait is bounded: after the wait limit the waiting thread records a
// code in `status`, raises the CTA's abort flag and every role leaves its loop;
// the CTA then lets in-flight copies drain, frees its tensor memory and returns.
#pragma once

#include "fsw_ptx.cuh"

namespace fsw {

enum : int { MODE_FWD = 0, MODE_DX = 1, MODE_DW = 2, MODE_NN = 3, MODE_NT = 4, MODE_TN = 5, MODE_DXG = 6, MODE_FWDST = 7, MODE_DXE = 8 };
// MODE_FWDST is MODE_FWD that saves s = silu(g) and t = u * silu'(g) where g and u would go.
__host__ __device__ constexpr bool is_fwd(int mode) { return mode == MODE_FWD || mode == MODE_FWDST; }
// MODE_DXE is MODE_DX whose otherwise idle epilogue warps also do the gate-gradient
// elementwise step (dg, du from dout, g, u), once per element, ahead of the tiles that
// read dg and du through TMA; see GemmParams::ew_*.
__host__ __device__ constexpr bool is_dx(int mode) { return mode == MODE_DX || mode == MODE_DXE; }
enum : int { MAJOR_K = 0, MAJOR_MN = 1 };

// Codes written to the status word when a bounded wait gives up.
enum : uint32_t {
  WAIT_OK = 0,
  WAIT_PRODUCER_EMPTY = 1,
  WAIT_MMA_FULL = 2,
  WAIT_MMA_TMEM_EMPTY = 3,
  WAIT_EPI_TMEM_FULL = 4,
  WAIT_XFORM_EMPTY = 6,   // (5 is WAIT_PEER_PARTIALS, below)
  WAIT_MMA_XFORM = 7,
  WAIT_GATE_GRAD_ROWS = 8,
};

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // default limit per wait: 2 s
constexpr uint64_t kDrainNs = 20000000ull;        // 20 ms drain on the abort path

struct GemmParams {
  CUtensorMap a0, a1;      // A operand(s); a1 only in MODE_DX (second product)
  CUtensorMap b0, b1;      // B operands (gate, up)
  // MODE_FWD store maps for g, u and out: boxes of 32 rows x 32 columns, 64-byte swizzle
  CUtensorMap sg, su, so;
  uint64_t a_desc, b_desc; // UMMA shared-memory descriptors with a zero start address
  uint32_t a_kadv, b_kadv; // bytes to advance the start address per K=16 step
  uint32_t idesc;          // UMMA instruction descriptor
  int M, N;                // output extents: rows, columns (per output tensor)
  int ldc;                 // elements between output rows (N unless a column range is written)
  int num_m_tiles, num_n_tiles, group_m;
  int num_k_blocks;        // 64-wide K blocks per product
  int store_gu;            // MODE_FWD: also write g and u
  // MODE_DXG: dout, s, t (T x di, row-major, read with plain loads) and the dg / du
  // arrays that the tiles of column 0 write
  const void *gg_dout, *gg_s, *gg_t;
  void *gg_dg, *gg_du;
  int gg_k;                // di: row length of the five arrays above
  // MODE_DXE: the elementwise step as a side job of the epilogue warps.  The (T, di)
  // arrays are cut, in the order the row tiles are visited, into quanta of 2048
  // elements (256 * di is a multiple of 2048, so no quantum straddles two row tiles):
  // row tile number v in visiting order owns quanta [v * ew_qpm, (v + 1) * ew_qpm).  Idle
  // epilogue warps of all CTAs take quanta from ew_ctrl[0] (an atomic ticket), compute
  // dg and du, and add 1 to ew_ctrl[2 + v]; a tile's TMA producer waits - time-limited -
  // until its row tile's count has reached ew_qpm before it loads dg / du tiles.  The
  // side job stays at most ew_ahead row tiles ahead of the furthest row tile any producer
  // has asked for (ew_ctrl[1] - 1): done all at once it would stream through L2 at HBM
  // speed and evict the operand panels the tiles share.
  const void *ew_dout, *ew_g, *ew_u;
  void *ew_dg, *ew_du;
  unsigned int* ew_ctrl;
  int ew_qpm;              // quanta per row tile = 256 * di / 2048
  int ew_ahead;            // row tiles the side job may run ahead
  int ew_cols;             // di
  int l2_a, l2_b;          // L2 eviction priority of A / B loads: 0 normal, 1 first, 2 last
  int l2_out;              // same for the forward's output stores
  uint32_t* status;        // device status word (0 = ok)
  void *c0_ptr, *c1_ptr, *c2_ptr;  // outputs (see the mode table above); row stride N
  unsigned long long* clk_probe;   // [2]: SM cycles and nanoseconds CTA 0 was resident
  unsigned long long wait_limit_ns;  // every mbarrier wait gives up after this long
  int stall_producer;              // test hook: the TMA producer issues nothing, so the
                                   // consumers' bounded waits run out and the error path runs
  // Advisory pacing of the TMA producers (nullptr or pace_kb 0 = free-running):
  // pace[0] counts arrivals, pace[1] != 0 switches pacing off for the launch.
  unsigned int* pace;
  int pace_kb;                     // K blocks between two meeting points
  unsigned int pace_limit_ns;      // longest a producer waits at a meeting point
  // Split of the last, partial wave of tiles along K (sk_total_iters == 0: none).
  // Tiles [0, sk_first_tile) - a whole number of waves - are computed one per CTA
  // pair as usual.  The K iterations of the remaining tiles, taken as one range of
  // sk_total_iters = tiles_left * iterations_per_tile, are cut into equal shares of
  // sk_iters_per_cluster; pair c takes [c * share, (c + 1) * share), which touches at
  // most two tiles, and writes each piece's fp32 accumulators to slot 2 * c + piece
  // of sk_ws.  splitk_reduce_kernel then adds the pieces of each tile in a fixed order.
  int sk_first_tile;
  int sk_iters_per_cluster;
  long long sk_total_iters;
  float* sk_ws;
  // MODE_DX across several GPUs (scatter_world > 1): rows [r * scatter_rows,
  // (r + 1) * scatter_rows) of dX belong to rank r, and the epilogue stores this
  // rank's partial sums for them straight into rank r's receive buffer scatter[r]
  // (peer memory mapped into this process; plain 16-byte stores over NVLink), which
  // is laid out [source rank][scatter_rows][N].  c0_ptr is not written.
  void* scatter[8];
  int scatter_world, scatter_rank, scatter_rows;
  // Pause between two store instructions of a warp that go to peer memory.  Without it
  // all CTAs emit a tile's rows in one burst at the end of each wave of tiles; NVLink
  // (~690 GB/s for SM-issued stores, measured) drains that for tens of microseconds,
  // the stores back up into the SMs' request path and the TMA loads of the next tile
  // queue behind them.  Spread over most of a tile's K loop the same bytes never
  // exceed the link's rate.
  unsigned int scatter_gap_ns;
  // Tile rows are visited starting at row tile m_rotate (mod num_m_tiles): with the
  // scatter every rank starts at another owner's rows, so that at any moment the
  // ranks store to different GPUs instead of all to the same one.
  int m_rotate;
};
constexpr int kMaxScatterRanks = 8;

// One piece of work of a CTA pair: K iterations [it0, it1) of tile (m_tile, n_tile).
// slot < 0: the whole tile, results go to the output arrays; otherwise a partial
// sum that goes to workspace slot `slot`.
struct WorkItem {
  int m_tile, n_tile, it0, it1, slot;
};
constexpr int kSplitSlotFloats = 2 * 128 * 512;  // one slot: both CTAs' 128 x 512 accumulators

// Epilogue warps: 4 (one per TMEM lane quadrant) or 8 (two per quadrant).
#ifndef FSW_EPI_WARPS
#define FSW_EPI_WARPS 8
#endif
constexpr int kSmemBudget = 232448;  // 227 KB opt-in limit per CTA

// Timing experiments only (results are garbage when set): run the MMA loop on
// whatever is in shared memory without any TMA load, or skip the epilogue's
// math and stores.  All default to off and are never set in the shipped build.
#ifndef FSW_DBG_SKIP_LOADS
#define FSW_DBG_SKIP_LOADS 0
#endif
#ifndef FSW_DBG_SKIP_EPILOGUE
#define FSW_DBG_SKIP_EPILOGUE 0
#endif
#ifndef FSW_DBG_SKIP_B_LOADS
#define FSW_DBG_SKIP_B_LOADS 0
#endif
// Cycle accounting (diagnostic builds only): the MMA thread and one epilogue warp
// of CTA 0 add up the SM cycles they spend in each wait and write them to
// clk_probe[2..7].
#ifndef FSW_PROFILE
#define FSW_PROFILE 0
#endif
// Measurement builds only: the plain epilogue releases tensor memory after its last
// read instead of reading everything into registers first (see drain_plain).
#ifndef FSW_PLAIN_ONE_PHASE
#define FSW_PLAIN_ONE_PHASE 0
#endif

template <int MODE, int CG, int NSUB>
struct TileCfg {
  static_assert(NSUB == 1 || (NSUB == 2 && CG == 2), "512-column tiles need a CTA pair");
  static constexpr int A_MAJOR = (MODE == MODE_DW || MODE == MODE_TN) ? MAJOR_MN : MAJOR_K;
  static constexpr int B_MAJOR = (is_dx(MODE) || MODE == MODE_NT || MODE == MODE_DXG) ? MAJOR_K : MAJOR_MN;
  // the A operand is written by the epilogue warps instead of TMA
  static constexpr bool A_BY_WARPS = (MODE == MODE_DXG);
  // dual: the accumulator columns of a region are [128 from b0 | 128 from b1]
  static constexpr bool DUAL_B = (is_fwd(MODE) || MODE == MODE_DW);
  static constexpr int BM = 128;          // accumulator rows per CTA
  static constexpr int BN = 256;          // columns of one accumulator region (MMA N)
  static constexpr int BK = 64;           // one 128-byte swizzle row of 16-bit elements
  static constexpr int SUB_ROWS = BN / CG;            // B n-extent per region staged by a CTA
  static constexpr int SUB_B_BYTES = SUB_ROWS * BK * 2;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = NSUB * SUB_B_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int CHUNK_BYTES = 64 * BK * 2;  // one MN-major 64x64 box
  static constexpr int EPI_WARPS = FSW_EPI_WARPS;
  static_assert(EPI_WARPS == 4 || EPI_WARPS == 8, "4 or 8 epilogue warps");
  static constexpr int EPI_BUF_BYTES = 32 * 128;  // 32 rows x 64 16-bit columns per warp
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUF_BYTES;
  static constexpr int BAR_BYTES = 512;
  // as many operand stages as fit beside the epilogue staging
  static constexpr int STAGES = (kSmemBudget - 1024 - BAR_BYTES - EPI_BYTES) / STAGE_BYTES;
  static_assert(STAGES >= 2 && STAGES <= 12, "unexpected stage count");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int TMEM_COLS = 512;
  static constexpr int NSEG = (is_dx(MODE) || MODE == MODE_DXG) ? 2 : 1;
  // Output columns covered by one accumulator region / one tile, per output tensor.
  static constexpr int REGION_N = DUAL_B ? 128 : 256;
  static constexpr int TILE_N = REGION_N * NSUB;
  static constexpr int TILE_M = BM * CG;
  // Arrivals that free one accumulator region.
  static constexpr int TEMPTY_COUNT = (NSUB == 2 ? 4 : EPI_WARPS) * CG;
};

// ------------------------------------------------------------- conversions --
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T>
__device__ __forceinline__ float round16(float v);
template <>
__device__ __forceinline__ float round16<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round16<__half>(float v) {
  return __half2float(__float2half_rn(v));
}

// 1 / (1 + 2^(-x*log2(e))) with the two special-function-unit approximations
// (relative error ~1e-7, far below a 16-bit ulp).  x -> -inf gives exactly 0,
// x -> +inf exactly 1.
__device__ __forceinline__ float sigmoid_f32(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}

// ------------------------------------------------------------ bounded wait --
struct AbortCtl {
  volatile uint32_t* flag;  // shared-memory abort flag of this CTA
  uint32_t* status;         // global status word
  uint64_t limit_ns;        // how long one wait may last
};

// Wait by ONE thread.
__device__ __forceinline__ bool bounded_wait_thread(uint32_t bar, uint32_t parity,
                                                    const AbortCtl& ctl, uint32_t code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0u) {
      if (*ctl.flag != 0u) return false;
      if (ptx::globaltimer_ns() - t0 > ctl.limit_ns) {
        *ctl.flag = code;
        atomicCAS(ctl.status, 0u, code | (static_cast<uint32_t>(blockIdx.x) << 8));
        return false;
      }
    }
  }
}

// Wait by a whole (converged) warp; the verdict is made warp-uniform.
__device__ __forceinline__ bool bounded_wait_warp(uint32_t bar, uint32_t parity,
                                                  const AbortCtl& ctl, uint32_t code) {
  return __all_sync(0xffffffffu, bounded_wait_thread(bar, parity, ctl, code));
}

// Advisory pacing.  The SMs of the two dies of a B200 do not run this kernel at
// exactly the same speed (measured: 1.5-3 % apart), so the CTAs of one die pull
// ahead by a few microseconds per tile.  Once the lead exceeds the time a line
// survives in L2 (about 50 us at the rates this kernel streams) the two dies stop
// sharing operand panels and every panel is fetched from HBM twice.  The producers
// therefore meet every pace_kb K blocks: each adds 1 to a counter and waits until
// all CTAs that work on the same wave of tiles have done so.  The meeting carries
// no data and is not needed for correctness.  A wait ends after pace_limit_ns at
// the latest and the CTA goes on (it has been counted, so later meetings still
// work); a CTA whose waits ran out three times switches pacing off for the whole
// launch (pace[1]).  CTAs that are late or not resident (SMs taken by another
// kernel) therefore cost a few short waits, never a hang and never an error.
struct Pacer {
  unsigned int* ctr;
  int kb;
  unsigned int limit_ns;
  bool on;
  int misses;
  __device__ __forceinline__ void meet(unsigned int target, const AbortCtl& ctl) {
    atomicAdd(ctr, 1u);
    volatile unsigned int* v = ctr;
    if (v[0] >= target) return;
    const uint64_t t0 = ptx::globaltimer_ns();
    for (;;) {
      if (v[0] >= target) return;
      if (v[1] != 0u || *ctl.flag != 0u) {
        on = false;
        return;
      }
      if (ptx::globaltimer_ns() - t0 > limit_ns) {
        if (++misses >= 3) {
          v[1] = 1u;
          on = false;
        }
        return;
      }
    }
  }
};

// Linear tile index -> (m_tile, n_tile); m is grouped so that concurrently
// running tiles share A row panels and B column panels in L2.
__host__ __device__ __forceinline__ void decode_tile_order(int t, int num_m_tiles, int num_n_tiles,
                                                           int group_m, int& m_tile, int& n_tile) {
  const int per_group = group_m * num_n_tiles;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int rest = num_m_tiles - first_m;
  const int gsz = rest < group_m ? rest : group_m;
  const int r = t - g * per_group;
  m_tile = first_m + r % gsz;
  n_tile = r / gsz;
}
__device__ __forceinline__ void decode_tile(int t, const GemmParams& p, int& m_tile, int& n_tile) {
  decode_tile_order(t, p.num_m_tiles, p.num_n_tiles, p.group_m, m_tile, n_tile);
}

// The idx-th work item of pair `cluster_id` (false when it has no more).  Every role
// of both CTAs of the pair walks the same sequence.
__host__ __device__ __forceinline__ bool next_work(const GemmParams& p, int iters_per_tile,
                                                   int cluster_id, int num_clusters, int idx,
                                                   WorkItem& w) {
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int whole = p.sk_total_iters > 0 ? p.sk_first_tile : num_tiles;
  const int t = cluster_id + idx * num_clusters;
  if (t < whole) {
    decode_tile_order(t, p.num_m_tiles, p.num_n_tiles, p.group_m, w.m_tile, w.n_tile);
    w.m_tile += p.m_rotate;
    if (w.m_tile >= p.num_m_tiles) w.m_tile -= p.num_m_tiles;
    w.it0 = 0;
    w.it1 = iters_per_tile;
    w.slot = -1;
    return true;
  }
  if (p.sk_total_iters == 0) return false;
  const int piece = idx - whole / num_clusters;  // `whole` is a multiple of num_clusters
  if (piece < 0 || piece > 1) return false;
  const long long u0 = static_cast<long long>(cluster_id) * p.sk_iters_per_cluster;
  long long u1 = u0 + p.sk_iters_per_cluster;
  if (u1 > p.sk_total_iters) u1 = p.sk_total_iters;
  if (u0 >= u1) return false;
  const int a = static_cast<int>(u0 / iters_per_tile);  // first tile of the split range this pair touches
  const long long a_end = static_cast<long long>(a + 1) * iters_per_tile;
  int tile;
  if (piece == 0) {
    tile = a;
    w.it0 = static_cast<int>(u0 - static_cast<long long>(a) * iters_per_tile);
    w.it1 = static_cast<int>((u1 < a_end ? u1 : a_end) - static_cast<long long>(a) * iters_per_tile);
  } else {
    if (u1 <= a_end) return false;
    tile = a + 1;
    w.it0 = 0;
    w.it1 = static_cast<int>(u1 - a_end);
  }
  decode_tile_order(p.sk_first_tile + tile, p.num_m_tiles, p.num_n_tiles, p.group_m, w.m_tile, w.n_tile);
  w.slot = 2 * cluster_id + piece;
  return true;
}


// ---------------------------------------------------------------- epilogue --
// tcgen05.ld hands every thread 32 consecutive columns of ONE accumulator row, so
// a direct store would scatter each warp-wide store over 32 rows.  The epilogue
// instead transposes through a 4 KB per-warp shared-memory buffer: threads write
// their row (XOR-swizzled 16-byte chunks, conflict-free), then read it back so that
// 4 (or 8) consecutive lanes cover one row and every global store instruction
// writes whole 64- or 128-byte row segments.
struct EpiCtx {
  int lane;
  int row0;       // first global output row of this warp
  uint32_t buf;   // this warp's 4 KB staging buffer
};

// 32 rows x 32 columns (64-byte rows) held as 16 packed words per thread.
__device__ __forceinline__ void stage_rows64(uint32_t buf, int lane, const uint32_t (&w)[16]) {
  const uint32_t base = buf + lane * 64u;
  const uint32_t x = (lane >> 1) & 3u;
#pragma unroll
  for (int c = 0; c < 4; ++c)
    ptx::st_shared_v4(base + ((c ^ x) << 4), w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}
// Write the staged 32x32 block to out[row0.., col0..] (row stride N elements).
__device__ __forceinline__ void flush_rows64(uint32_t buf, int lane, void* out, int row0, int col0,
                                             int M, int N) {
  const int c = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 8 * i + (lane >> 2);
    uint32_t a, b, cc, d;
    ptx::ld_shared_v4(buf + r * 64u + ((c ^ ((r >> 1) & 3)) << 4), a, b, cc, d);
    const int row = row0 + r, col = col0 + c * 8;
    if (row < M && col < N)
      ptx::st_global_v4(static_cast<char*>(out) + (static_cast<size_t>(row) * N + col) * 2, a, b, cc,
                        d);
  }
}
// 32 rows x 64 columns (128-byte rows) held as 32 packed words per thread.
__device__ __forceinline__ void stage_rows128(uint32_t buf, int lane, const uint32_t (&w)[32]) {
  const uint32_t base = buf + lane * 128u;
  const uint32_t x = lane & 7u;
#pragma unroll
  for (int c = 0; c < 8; ++c)
    ptx::st_shared_v4(base + ((c ^ x) << 4), w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}
__device__ __forceinline__ void flush_rows128(uint32_t buf, int lane, void* out, int row0, int col0,
                                              int M, int N, int ld, unsigned int gap_ns = 0) {
  const int c = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (gap_ns != 0) __nanosleep(gap_ns);
    const int r = 4 * i + (lane >> 3);
    uint32_t a, b, cc, d;
    ptx::ld_shared_v4(buf + r * 128u + ((c ^ (r & 7)) << 4), a, b, cc, d);
    const int row = row0 + r, col = col0 + c * 8;
    if (row < M && col < N)
      ptx::st_global_v4(static_cast<char*>(out) + (static_cast<size_t>(row) * ld + col) * 2, a, b, cc,
                        d);
  }
}

// Unpack a packed pair of 16-bit values to fp32.
template <typename T>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi);
template <>
__device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
  lo = __uint_as_float(w << 16);
  hi = __uint_as_float(w & 0xFFFF0000u);
}
template <>
__device__ __forceinline__ void unpack2<__half>(uint32_t w, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  lo = f.x;
  hi = f.y;
}

// Product of two packed 16-bit pairs, each lane rounded once to the 16-bit type -
// bit-identical to multiplying in fp32 (the product of two 16-bit values is exact
// there) and rounding.
template <typename T>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b);
template <>
__device__ __forceinline__ uint32_t mul2<__nv_bfloat16>(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                   *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t mul2<__half>(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// Read 16 accumulator columns and round them to 8 packed 16-bit pairs.
template <typename T, bool ACC16>
__device__ __forceinline__ void load_pack16(uint32_t taddr, uint32_t* dst8) {
  uint32_t r[16];
  ptx::tmem_ld_32x16(taddr, r);
  ptx::tmem_ld_wait();
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    if (ACC16)  // fp16 accumulators sit in the low half of each 32-bit column
      dst8[q] = __byte_perm(r[2 * q], r[2 * q + 1], 0x5410);
    else
      dst8[q] = pack2<T>(__uint_as_float(r[2 * q]), __uint_as_float(r[2 * q + 1]));
  }
}

// Read 16 gate and 16 up columns with both loads in flight, rounded to 8 + 8 pairs.
template <typename T, bool ACC16>
__device__ __forceinline__ void load_pack16x2(uint32_t taddr_g, uint32_t taddr_u, uint32_t* g8,
                                              uint32_t* u8) {
  uint32_t rg[16], ru[16];
  ptx::tmem_ld_32x16(taddr_g, rg);
  ptx::tmem_ld_32x16(taddr_u, ru);
  ptx::tmem_ld_wait();
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    if (ACC16) {
      g8[q] = __byte_perm(rg[2 * q], rg[2 * q + 1], 0x5410);
      u8[q] = __byte_perm(ru[2 * q], ru[2 * q + 1], 0x5410);
    } else {
      g8[q] = pack2<T>(__uint_as_float(rg[2 * q]), __uint_as_float(rg[2 * q + 1]));
      u8[q] = pack2<T>(__uint_as_float(ru[2 * q]), __uint_as_float(ru[2 * q + 1]));
    }
  }
}

// SwiGLU epilogue over 64-column boxes jb in [jb_begin, jb_begin + NJB) of one
// 256-column region laid out [128 gate | 128 up].
//
// Phase A reads the warp's accumulators, rounds them to the 16-bit g and u that are
// stored anyway, keeps them packed in registers and calls `release`, so the MMA
// issuer can refill the region while phase B runs.  Phase B computes
// out = round(round(silu_f32(g16)) * u16) - the rounding order of the reference's
// PyTorch oracle (test_swiglu.py:47-55), every op rounding to the tensor dtype -
// and hands g, u and out to TMA stores as 32x32 boxes from the warp's two swizzled
// 2 KB staging buffers.  A buffer is rewritten only after the bulk group that read it
// has finished reading; phase B overlaps the next tile's MMAs, so these waits are
// off the critical path.
template <class C, typename T, bool ACC16, int NJB, bool SAVE_ST, class Release>
__device__ __forceinline__ void drain_swiglu(const GemmParams& p, const EpiCtx& e, uint32_t taddr,
                                             int n0, int jb_begin, Release release) {
  const uint32_t buf0 = e.buf, buf1 = e.buf + 2048u;
  const bool rows_ok = e.row0 < p.M;
  const uint64_t pol_out = ptx::make_l2_policy(p.l2_out);
  uint32_t G[NJB * 32], U[NJB * 32];
#pragma unroll
  for (int c = 0; c < NJB * 4; ++c)
    load_pack16x2<T, ACC16>(taddr + jb_begin * 64 + c * 16, taddr + 128 + jb_begin * 64 + c * 16,
                            &G[c * 8], &U[c * 8]);
  release();
#pragma unroll
  for (int c = 0; c < NJB * 2; ++c) {
    const uint32_t* pg = &G[c * 16];
    const uint32_t* pu = &U[c * 16];
    const int col = n0 + jb_begin * 64 + c * 32;
    const bool in_range = rows_ok && col < p.N;
    uint32_t po[16];
    if (SAVE_ST) {
      // s = silu(g), rounded: a factor of out, and what is saved in place of g
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        float g0, g1;
        unpack2<T>(pg[q], g0, g1);
        po[q] = pack2<T>(g0 * sigmoid_f32(g0), g1 * sigmoid_f32(g1));
      }
    }
    if (p.store_gu) {
      if (e.lane == 0) ptx::tma_store_wait_read<0>();
      __syncwarp();
      if (SAVE_ST) {
        stage_rows64(buf0, e.lane, po);
        uint32_t pt[16];  // t = u * silu'(g); silu'(g) = sg + silu * (1 - sg), rounded, times u, rounded
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          float g0, g1;
          unpack2<T>(pg[q], g0, g1);
          const float s0 = sigmoid_f32(g0), s1 = sigmoid_f32(g1);
          pt[q] = mul2<T>(pu[q], pack2<T>(fmaf(g0 * s0, 1.0f - s0, s0), fmaf(g1 * s1, 1.0f - s1, s1)));
        }
        stage_rows64(buf1, e.lane, pt);
      } else {
        stage_rows64(buf0, e.lane, *reinterpret_cast<const uint32_t(*)[16]>(pg));
        stage_rows64(buf1, e.lane, *reinterpret_cast<const uint32_t(*)[16]>(pu));
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (e.lane == 0 && in_range) {
        ptx::tma_store_2d_hint(&p.sg, buf0, col, e.row0, pol_out);
        ptx::tma_store_2d_hint(&p.su, buf1, col, e.row0, pol_out);
        ptx::tma_store_commit();
      }
    }
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      if (SAVE_ST) {
        po[q] = mul2<T>(po[q], pu[q]);
      } else {
        float g0, g1;
        unpack2<T>(pg[q], g0, g1);
        po[q] = mul2<T>(pack2<T>(g0 * sigmoid_f32(g0), g1 * sigmoid_f32(g1)), pu[q]);
      }
    }
    if (e.lane == 0) ptx::tma_store_wait_read<0>();
    __syncwarp();
    stage_rows64(buf0, e.lane, po);
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (e.lane == 0 && in_range) {
      ptx::tma_store_2d_hint(&p.so, buf0, col, e.row0, pol_out);
      ptx::tma_store_commit();
    }
  }
}

// Plain epilogue over 64-column boxes jb in [jb_begin, jb_begin + NJB) of one
// 256-column region.  MODE_DW: boxes 0,1 -> c0, boxes 2,3 -> c1, at n0 + 64*(jb&1);
// every other mode: all four boxes belong to c0 at columns n0 + 64*jb.  Two phases,
// like the SwiGLU epilogue: first every box is read from tensor memory, rounded and
// kept packed in registers (32 words per box) and `release` is called, so the MMA
// issuer can start the next tile; then the boxes are transposed through the staging
// buffer and written with row-coalesced stores beside the next tile's MMAs.  That
// matters when a tile's K loop is short (column shards) and when the stores are slow
// (the multi-GPU scatter writes them to peer memory over NVLink).
template <class C, int MODE, typename T, bool ACC16, int NJB, class Release>
__device__ __forceinline__ void drain_plain(const GemmParams& p, const EpiCtx& e, uint32_t taddr,
                                            int n0, int jb_begin, Release release) {
  uint32_t pk[NJB * 32];
  auto read_box = [&](int j) {
#pragma unroll
    for (int c = 0; c < 4; c += 2)
      load_pack16x2<T, ACC16>(taddr + (jb_begin + j) * 64 + c * 16, taddr + (jb_begin + j) * 64 + (c + 1) * 16,
                              &pk[j * 32 + c * 8], &pk[j * 32 + (c + 1) * 8]);
  };
  if (!FSW_PLAIN_ONE_PHASE) {
#pragma unroll
    for (int j = 0; j < NJB; ++j) read_box(j);
    release();
  }
  void* scatter_out = nullptr;
  unsigned int gap_ns = 0;
  if (is_dx(MODE) && p.scatter_world > 1) {
    // The warp's 32 rows have one owner (scatter_rows is a multiple of 32).  Row t of
    // dX is row (rank * scatter_rows + t - owner * scatter_rows) of the owner's buffer.
    int owner = e.row0 / p.scatter_rows;
    if (owner >= p.scatter_world) owner = p.scatter_world - 1;  // rows >= M: nothing is stored
    const long long shift = static_cast<long long>(p.scatter_rank - owner) * p.scatter_rows;
    scatter_out = static_cast<char*>(p.scatter[owner]) + shift * p.ldc * 2;
    if (owner != p.scatter_rank) gap_ns = p.scatter_gap_ns;
  }
#pragma unroll
  for (int j = 0; j < NJB; ++j) {
    const int jb = jb_begin + j;
    const int col = (MODE == MODE_DW) ? (n0 + (jb & 1) * 64) : (n0 + jb * 64);
    void* out = (MODE == MODE_DW && jb >= 2) ? p.c1_ptr : p.c0_ptr;
    if (is_dx(MODE) && p.scatter_world > 1) out = scatter_out;
    if (FSW_PLAIN_ONE_PHASE) {  // measurement build: read, release after the last read, store box by box
      read_box(j);
      if (j == NJB - 1) release();
    }
    stage_rows128(e.buf, e.lane, *reinterpret_cast<const uint32_t(*)[32]>(&pk[j * 32]));
    __syncwarp();
    flush_rows128(e.buf, e.lane, out, e.row0, col, p.M, p.N, p.ldc, gap_ns);
    __syncwarp();
  }
}

// Split-K piece: copy one 256-column accumulator region, as fp32, to the piece's
// workspace slot.  The slot is laid out in the order tensor memory is read - for
// every (CTA, lane quadrant, region, 16-column chunk) four float4 vectors per lane,
// lanes adjacent - so each store instruction of a warp writes 512 contiguous bytes.
// splitk_reduce_kernel reads the same layout.
__device__ __forceinline__ size_t splitk_vec_index(int slot, int cta, int q, int r, int c, int j,
                                                   int lane) {
  return ((((((static_cast<size_t>(slot) * 2 + cta) * 4 + q) * 2 + r) * 16 + c) * 4 + j) * 32) + lane;
}
template <bool ACC16, class Release>
__device__ __forceinline__ void drain_partial(const GemmParams& p, int lane, uint32_t taddr, int slot,
                                              int cta, int q, int r, int c_begin, int c_count,
                                              Release release) {
  float4* ws = reinterpret_cast<float4*>(p.sk_ws);
#pragma unroll 1
  for (int c = c_begin; c < c_begin + c_count; ++c) {
    uint32_t v[16];
    ptx::tmem_ld_32x16(taddr + c * 16, v);
    ptx::tmem_ld_wait();
    if (c == c_begin + c_count - 1) release();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (ACC16)  // fp16 accumulators sit in the low half of each 32-bit column
          w[e] = __float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(v[4 * j + e] & 0xFFFFu))));
        else
          w[e] = v[4 * j + e];
      }
      ptx::st_global_v4(ws + splitk_vec_index(slot, cta, q, r, c, j, lane), w[0], w[1], w[2], w[3]);
    }
  }
}

// ---------------------------------------------- gate-gradient arithmetic --
// 16-byte streaming load / store: every operand is touched once per launch.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// One 16-byte vector (8 elements).  Only g is widened to fp32 (sigmoid); the
// products are packed 16-bit multiplies, each rounding once like the fp32 form.
template <typename T>
__device__ __forceinline__ void gate_grad_vec(const uint4& vd, const uint4& vg, const uint4& vu,
                                              uint4& odg, uint4& odu) {
  const uint32_t* wd = reinterpret_cast<const uint32_t*>(&vd);
  const uint32_t* wg = reinterpret_cast<const uint32_t*>(&vg);
  const uint32_t* wu = reinterpret_cast<const uint32_t*>(&vu);
  uint32_t* wdg = reinterpret_cast<uint32_t*>(&odg);
  uint32_t* wdu = reinterpret_cast<uint32_t*>(&odu);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float g0, g1;
    unpack2<T>(wg[e], g0, g1);
    const float s0 = sigmoid_f32(g0), s1 = sigmoid_f32(g1);
    const float silu0 = g0 * s0, silu1 = g1 * s1;
    const uint32_t silu = pack2<T>(silu0, silu1);
    const uint32_t dsilu = pack2<T>(fmaf(silu0, 1.0f - s0, s0), fmaf(silu1, 1.0f - s1, s1));
    wdu[e] = mul2<T>(wd[e], silu);
    wdg[e] = mul2<T>(mul2<T>(wd[e], wu[e]), dsilu);
  }
}

// ------------------------------------------ A tiles produced by the warps --
// MODE_DXG.  One K block of the A operand is 128 rows x 64 elements = 1024 chunks of
// 16 bytes; the EPI_WARPS * 32 threads take chunks tid, tid + 256, ... (8 lanes cover
// one row's 128 bytes, so global accesses are whole 128-byte segments).  The chunk of
// row r, 16-byte column c goes to byte r * 128 + ((c ^ (r & 7)) << 4) of the stage:
// the 128-byte swizzle that TMA would have written and the MMA descriptor expects.
struct GateGradTile {
  uint4 d[4], a[4];  // dout and the saved activation (t or s) for this thread's four chunks
};
__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
template <int THREADS>
__device__ __forceinline__ void gate_grad_issue(const GemmParams& p, int tid, int m0, int k0, bool second_is_s,
                                                GateGradTile& g) {
  const char* second = static_cast<const char*>(second_is_s ? p.gg_s : p.gg_t);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int chunk = tid + THREADS * i;
    const int row = m0 + (chunk >> 3), col = k0 + (chunk & 7) * 8;
    if (row < p.M && col < p.gg_k) {  // gg_k is a multiple of 8: a chunk is all in or all out
      const size_t off = (static_cast<size_t>(row) * p.gg_k + col) * 2;
      g.d[i] = ldg_nc16(static_cast<const char*>(p.gg_dout) + off);
      g.a[i] = ldg_nc16(second + off);
    } else {
      g.d[i] = make_uint4(0u, 0u, 0u, 0u);
      g.a[i] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}
template <typename T, int THREADS>
__device__ __forceinline__ void gate_grad_write(const GemmParams& p, int tid, int m0, int k0, uint32_t a_dst,
                                                const GateGradTile& g, void* grad_out) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int chunk = tid + THREADS * i;
    const int r = chunk >> 3, c = chunk & 7;
    const uint32_t w0 = mul2<T>(g.d[i].x, g.a[i].x), w1 = mul2<T>(g.d[i].y, g.a[i].y);
    const uint32_t w2 = mul2<T>(g.d[i].z, g.a[i].z), w3 = mul2<T>(g.d[i].w, g.a[i].w);
    ptx::st_shared_v4(a_dst + r * 128u + ((c ^ (r & 7)) << 4), w0, w1, w2, w3);
    if (grad_out != nullptr) {
      const int row = m0 + r, col = k0 + c * 8;
      if (row < p.M && col < p.gg_k)
        ptx::st_global_v4(static_cast<char*>(grad_out) + (static_cast<size_t>(row) * p.gg_k + col) * 2, w0, w1,
                          w2, w3);
    }
  }
}

// One quantum of the MODE_DXE side job, by a whole warp: 2048 elements = 256 vectors of
// 8; lane l takes vectors l, l + 32, ... (8 of them, in two rounds of 4 so that 12 loads
// are in flight per lane).  Quantum `q` belongs to row tile (q / ew_qpm + m_rotate) mod
// num_m_tiles, the order in which the tiles visit the rows; a quantum beyond the end of the
// arrays (ragged last row tile) is empty.  Finishing a quantum - after a fence, so that
// the results are visible GPU-wide first - adds 1 to the row tile's count.
template <typename T, int TILE_M>
__device__ __forceinline__ void gate_grad_quantum(const GemmParams& p, unsigned int q, int lane) {
  const unsigned int v = q / static_cast<unsigned int>(p.ew_qpm);
  const unsigned int j = q - v * static_cast<unsigned int>(p.ew_qpm);
  int m = static_cast<int>(v) + p.m_rotate;
  if (m >= p.num_m_tiles) m -= p.num_m_tiles;
  const long long total_vec = static_cast<long long>(p.M) * p.ew_cols / 8;
  const long long first = (static_cast<long long>(m) * TILE_M * p.ew_cols) / 8 + static_cast<long long>(j) * 256;
  const uint4* d4 = static_cast<const uint4*>(p.ew_dout);
  const uint4* g4 = static_cast<const uint4*>(p.ew_g);
  const uint4* u4 = static_cast<const uint4*>(p.ew_u);
  uint4* dg4 = static_cast<uint4*>(p.ew_dg);
  uint4* du4 = static_cast<uint4*>(p.ew_du);
#pragma unroll 1
  for (int round = 0; round < 2; ++round) {
    uint4 vd[4], vg[4], vu[4];
    bool in[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long idx = first + (round * 4 + i) * 32 + lane;
      in[i] = idx < total_vec;
      if (in[i]) {
        vd[i] = ld_stream(d4 + idx);
        vg[i] = ld_stream(g4 + idx);
        vu[i] = ld_stream(u4 + idx);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (in[i]) {
        const long long idx = first + (round * 4 + i) * 32 + lane;
        uint4 odg, odu;
        gate_grad_vec<T>(vd[i], vg[i], vu[i], odg, odu);
        dg4[idx] = odg;
        du4[idx] = odu;
      }
    }
  }
  __threadfence();
  __syncwarp();
  if (lane == 0) atomicAdd(p.ew_ctrl + 2 + v, 1u);
}

// ------------------------------------------------------------------ kernel --
template <int MODE, int CG, int NSUB, typename T, bool ACC16>
__global__ void __launch_bounds__(64 + 32 * FSW_EPI_WARPS, 1)
    gemm_kernel(const __grid_constant__ GemmParams p) {
  using C = TileCfg<MODE, CG, NSUB>;
  constexpr int STAGES = C::STAGES;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
  const uint32_t smem_base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - raw_u32);

  const uint32_t epi_base = smem_base + STAGES * C::STAGE_BYTES;
  const uint32_t bar_base = epi_base + C::EPI_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  // A_BY_WARPS: "the warps have written stage s's A tile" (all epilogue warps of both CTAs arrive)
  auto xf_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 5 + s); };
  const uint32_t misc_off = (bar_base - smem_base) + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + misc_off);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + misc_off + 4);
  const AbortCtl ctl{abort_flag, p.status, p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CG == 2) ? ptx::cluster_ctarank() : 0u;
  // CTA 0 measures the SM clock it actually ran at (cycles / wall time).
  long long probe_c0 = 0;
  uint64_t probe_t0 = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    probe_c0 = clock64();
    probe_t0 = ptx::globaltimer_ns();
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), C::TEMPTY_COUNT);
    }
    if (C::A_BY_WARPS)
      for (int s = 0; s < STAGES; ++s) ptx::mbar_init(xf_bar(s), C::EPI_WARPS * CG);
    *abort_flag = 0u;
    ptx::fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&p.a0);
    ptx::prefetch_tensormap(&p.b0);
    ptx::prefetch_tensormap(&p.b1);
    if (is_dx(MODE)) ptx::prefetch_tensormap(&p.a1);
    if (is_fwd(MODE)) {
      ptx::prefetch_tensormap(&p.sg);
      ptx::prefetch_tensormap(&p.su);
      ptx::prefetch_tensormap(&p.so);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc<CG>(bar_base + 8u * (2 * STAGES + 4), C::TMEM_COLS);
    ptx::tmem_relinquish<CG>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (CG == 2) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_clusters = gridDim.x / CG;
  const int cluster_id = blockIdx.x / CG;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_kb = p.num_k_blocks;

  if (warp == 0) {
    // ======================= TMA producer (one thread) =======================
    if (lane == 0 && !FSW_DBG_SKIP_LOADS && !p.stall_producer) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint64_t pol_a = ptx::make_l2_policy(p.l2_a);
      const uint64_t pol_b = ptx::make_l2_policy(p.l2_b);
      Pacer pacer{p.pace, p.pace_kb, p.pace_limit_ns, p.pace != nullptr && p.pace_kb > 0, 0};
      const int kb_per_tile = C::NSEG * num_kb;
      int ew_ready_tile = -1;  // MODE_DXE: row tile whose gate gradient is known to be complete
      const unsigned int meets_per_tile =
          pacer.on ? static_cast<unsigned int>((kb_per_tile + pacer.kb - 1) / pacer.kb) : 0u;
      WorkItem w;
      for (int idx = 0; ok && next_work(p, kb_per_tile, cluster_id, num_clusters, idx, w); ++idx) {
        const int m0 = w.m_tile * C::TILE_M + cta_rank * C::BM;
        const int n0 = w.n_tile * C::TILE_N;
        if (MODE == MODE_DXE && w.m_tile != ew_ready_tile) {
          // dg / du rows of this row tile are produced by the epilogue warps of all CTAs
          int v = w.m_tile - p.m_rotate;
          if (v < 0) v += p.num_m_tiles;
          const unsigned int* cnt = p.ew_ctrl + 2 + v;
          atomicMax(p.ew_ctrl + 1, static_cast<unsigned int>(v) + 1u);  // how far the tiles have got
          const uint64_t t0 = ptx::globaltimer_ns();
          for (;;) {
            unsigned int c;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(c) : "l"(cnt) : "memory");
            if (c >= static_cast<unsigned int>(p.ew_qpm)) break;
            if (*ctl.flag != 0u) {
              ok = false;
              break;
            }
            if (ptx::globaltimer_ns() - t0 > ctl.limit_ns) {
              *ctl.flag = WAIT_GATE_GRAD_ROWS;
              atomicCAS(ctl.status, 0u, WAIT_GATE_GRAD_ROWS | (static_cast<uint32_t>(blockIdx.x) << 8));
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          // the rows were written through the generic proxy; TMA reads them through the async proxy
          asm volatile("fence.proxy.async;" ::: "memory");
          ew_ready_tile = w.m_tile;
        }
        // Whole tiles run in waves of num_clusters; every wave before the last is full,
        // and with a split tail every whole-tile wave is.
        const bool pace_item = pacer.on && w.slot < 0;
        const int left = (p.sk_total_iters > 0 ? p.sk_first_tile : num_tiles) - idx * num_clusters;
        const unsigned int in_wave = static_cast<unsigned int>((left < num_clusters ? left : num_clusters) * CG);
        const unsigned int before = static_cast<unsigned int>(idx) * meets_per_tile * gridDim.x;
        int until_meet = 0;
        unsigned int meet_no = 0;
        for (int it = w.it0; it < w.it1; ++it) {
          {
            const int seg = (C::NSEG == 2 && it >= num_kb) ? 1 : 0;
            const int kb = it - seg * num_kb;
            if (pace_item && pacer.on && --until_meet < 0) {
              until_meet = pacer.kb - 1;
              pacer.meet(before + (++meet_no) * in_wave, ctl);
            }
            ok = bounded_wait_thread(empty_bar(s), ph ^ 1u, ctl, WAIT_PRODUCER_EMPTY);
            if (!ok) break;
            const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
            const uint32_t b_dst = a_dst + C::A_BYTES;
            const int k0 = kb * C::BK;
            uint32_t fb = full_bar(s);
            if (CG == 2) fb = ptx::mapa(fb, 0);
            if (cta_rank == 0)
              ptx::mbar_arrive_expect_tx(full_bar(s),
                                         CG * (FSW_DBG_SKIP_B_LOADS ? C::A_BYTES
                                               : C::A_BY_WARPS      ? C::B_BYTES
                                                                    : C::STAGE_BYTES));
            auto load_pol = [&](uint32_t dst, const CUtensorMap* tm, int x, int y, uint64_t pol) {
              if (CG == 2)
                ptx::tma_load_2d_pair(dst, tm, fb, x, y, pol);
              else
                ptx::tma_load_2d(dst, tm, fb, x, y, pol);
            };
            auto load_a = [&](uint32_t dst, const CUtensorMap* tm, int x, int y) {
              load_pol(dst, tm, x, y, pol_a);
            };
            auto load = [&](uint32_t dst, const CUtensorMap* tm, int x, int y) {
              load_pol(dst, tm, x, y, pol_b);
            };
            // ---- A tile: 128 rows x 64 k
            if (C::A_BY_WARPS) {
              // written by the epilogue warps (see the transform loop below)
            } else if (C::A_MAJOR == MAJOR_K) {
              load_a(a_dst, (is_dx(MODE) && seg == 1) ? &p.a1 : &p.a0, k0, m0);
            } else {
#pragma unroll
              for (int c = 0; c < C::BM / 64; ++c)
                load_a(a_dst + c * C::CHUNK_BYTES, &p.a0, m0 + c * 64, k0);
            }
            // ---- B: one SUB_ROWS x 64 sub-tile per accumulator region
            if (!FSW_DBG_SKIP_B_LOADS) {
#pragma unroll
              for (int r = 0; r < NSUB; ++r) {
                const uint32_t dst = b_dst + r * C::SUB_B_BYTES;
                if (C::B_MAJOR == MAJOR_K) {
                  load(dst, seg == 1 ? &p.b1 : &p.b0, k0,
                       n0 + r * C::REGION_N + cta_rank * C::SUB_ROWS);
                } else if (!C::DUAL_B) {
                  // one MN-major B: this CTA's SUB_ROWS columns of region r
#pragma unroll
                  for (int c = 0; c < C::SUB_ROWS / 64; ++c)
                    load(dst + c * C::CHUNK_BYTES, &p.b0,
                         n0 + r * C::REGION_N + cta_rank * C::SUB_ROWS + c * 64, k0);
                } else if (CG == 1) {
#pragma unroll
                  for (int c = 0; c < 4; ++c)
                    load(dst + c * C::CHUNK_BYTES, c < 2 ? &p.b0 : &p.b1, n0 + (c & 1) * 64, k0);
                } else {
#pragma unroll
                  for (int c = 0; c < 2; ++c)
                    load(dst + c * C::CHUNK_BYTES, cta_rank ? &p.b1 : &p.b0,
                         n0 + r * C::REGION_N + c * 64, k0);
                }
              }
            }
            if (++s == STAGES) {
              s = 0;
              ph ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ================ MMA issuer (one thread of the pair leader) ================
    if (cta_rank == 0 && lane == 0) {
      int s = 0, a = 0;
      uint32_t ph = 0, aph = 0;
      bool ok = true;
      long long prof_full = 0, prof_tempty = 0, prof_t0 = 0;
      auto commit = [&](uint32_t bar) {
        if (CG == 2)
          ptx::mma_commit_pair(bar, 3);
        else
          ptx::mma_commit(bar);
      };
      WorkItem w;
      for (int idx = 0; ok && next_work(p, C::NSEG * num_kb, cluster_id, num_clusters, idx, w); ++idx) {
        if (NSUB == 1) {
          ok = bounded_wait_thread(tempty_bar(a), aph ^ 1u, ctl, WAIT_MMA_TMEM_EMPTY);
          if (!ok) break;
          ptx::tc_fence_after_sync();
        }
        const int iters = w.it1 - w.it0;  // a split piece starts its own accumulation at zero
        for (int it = 0; it < iters; ++it) {
          if (FSW_PROFILE) prof_t0 = clock64();
          if (!FSW_DBG_SKIP_LOADS) ok = bounded_wait_thread(full_bar(s), ph, ctl, WAIT_MMA_FULL);
          if (ok && C::A_BY_WARPS) ok = bounded_wait_thread(xf_bar(s), ph, ctl, WAIT_MMA_XFORM);
          if (FSW_PROFILE) prof_full += clock64() - prof_t0;
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = smem_base + s * C::STAGE_BYTES;
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int r = 0; r < NSUB; ++r) {
            if (NSUB == 2 && it == 0) {
              // both regions belong to this tile; region r must have been drained
              if (FSW_PROFILE) prof_t0 = clock64();
              ok = bounded_wait_thread(tempty_bar(r), aph ^ 1u, ctl, WAIT_MMA_TMEM_EMPTY);
              if (FSW_PROFILE) prof_tempty += clock64() - prof_t0;
              if (!ok) break;
              ptx::tc_fence_after_sync();
            }
            const uint32_t d_tmem = tmem_base + (NSUB == 2 ? r : a) * C::BN;
#pragma unroll
            for (int k = 0; k < C::BK / 16; ++k) {
              const uint64_t ad = p.a_desc | (((a_addr + k * p.a_kadv) & 0x3FFFFu) >> 4);
              const uint64_t bd =
                  p.b_desc | (((b_addr + r * C::SUB_B_BYTES + k * p.b_kadv) & 0x3FFFFu) >> 4);
              ptx::mma_f16_ss<CG>(d_tmem, ad, bd, p.idesc, (it | k) != 0 ? 1u : 0u);
            }
          }
          if (!ok) break;
          commit(empty_bar(s));
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        if (NSUB == 2) {
          commit(tfull_bar(0));
          aph ^= 1u;
        } else {
          commit(tfull_bar(a));
          a ^= 1;
          if (a == 0) aph ^= 1u;
        }
      }
      if (FSW_PROFILE && blockIdx.x == 0 && p.clk_probe != nullptr) {
        p.clk_probe[2] = prof_full;
        p.clk_probe[3] = prof_tempty;
      }
    }
  } else {
    // ======================= epilogue =======================
    const int q = warp & 3;     // TMEM lane quadrant this warp may read
    const int ew = warp - 2;    // epilogue warp index
    const int chalf = ew >> 2;  // with 8 warps: 0 or 1
    constexpr int kSplit = C::EPI_WARPS / 4;
    EpiCtx e;
    e.lane = lane;
    e.buf = epi_base + ew * C::EPI_BUF_BYTES;
    int a = 0;
    uint32_t aph = 0;
    bool ok = true;
    int xs = 0;        // A_BY_WARPS: stage and phase of the next A tile the warps write
    uint32_t xph = 0;
    bool ew_more = (MODE == MODE_DXE);  // MODE_DXE: quanta of the side job may be left
    const unsigned int ew_total = (MODE == MODE_DXE)
                                      ? static_cast<unsigned int>(p.num_m_tiles) * static_cast<unsigned int>(p.ew_qpm)
                                      : 0u;
    long long prof_wait = 0, prof_drain = 0, prof_t0 = 0, prof_tiles = 0;
    WorkItem w;
    for (int idx = 0; ok && next_work(p, C::NSEG * num_kb, cluster_id, num_clusters, idx, w); ++idx) {
      e.row0 = w.m_tile * C::TILE_M + cta_rank * C::BM + q * 32;
      const int n0 = w.n_tile * C::TILE_N;
      if (C::A_BY_WARPS) {
        // Produce this item's A tiles: dg = dout * t for the first num_kb iterations,
        // du = dout * s for the rest.  Loads run kPrefetch iterations ahead of their use.
        constexpr int kThreads = C::EPI_WARPS * 32;
        constexpr int kPrefetch = 2;
        const int tid = ew * 32 + lane;
        const int m0 = w.m_tile * C::TILE_M + cta_rank * C::BM;
        const bool write_out = (w.n_tile == 0);  // one tile per row of tiles emits dg / du for the dW GEMM
        GateGradTile gt[kPrefetch];
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) {
          const int it = w.it0 + j;
          if (it < w.it1)
            gate_grad_issue<kThreads>(p, tid, m0, (it >= num_kb ? it - num_kb : it) * C::BK, it >= num_kb, gt[j]);
        }
        for (int base = w.it0; base < w.it1 && ok; base += kPrefetch) {
#pragma unroll
          for (int j = 0; j < kPrefetch; ++j) {
            const int it = base + j;
            if (it < w.it1 && ok) {
              const bool second = it >= num_kb;
              const int k0 = (second ? it - num_kb : it) * C::BK;
              ok = bounded_wait_warp(empty_bar(xs), xph ^ 1u, ctl, WAIT_XFORM_EMPTY);
              if (ok) {
                gate_grad_write<T, kThreads>(p, tid, m0, k0, smem_base + xs * C::STAGE_BYTES, gt[j],
                                             write_out ? (second ? p.gg_du : p.gg_dg) : nullptr);
                const int nx = it + kPrefetch;
                if (nx < w.it1)
                  gate_grad_issue<kThreads>(p, tid, m0, (nx >= num_kb ? nx - num_kb : nx) * C::BK, nx >= num_kb,
                                            gt[j]);
                ptx::fence_proxy_async_smem();  // the MMA reads the tile through the async proxy
                __syncwarp();
                if (lane == 0) {
                  if (CG == 2)
                    ptx::mbar_arrive_cluster(ptx::mapa(xf_bar(xs), 0));
                  else
                    ptx::mbar_arrive(xf_bar(xs));
                }
                if (++xs == STAGES) {
                  xs = 0;
                  xph ^= 1u;
                }
              }
            }
          }
        }
        if (!ok) break;
      }
      if (MODE == MODE_DXE) {
        // Until this item's accumulators are complete, take quanta of the gate-gradient step.
        while (ew_more) {
          const uint32_t ready = ptx::mbar_try_wait(tfull_bar(NSUB == 2 ? 0 : a), aph) ? 1u : 0u;
          if (__shfl_sync(0xffffffffu, ready, 0) != 0u) break;
          unsigned int qn = 0xFFFFFFFFu;
          if (lane == 0) {
            const volatile unsigned int* c = p.ew_ctrl;
            const unsigned int limit = (c[1] + static_cast<unsigned int>(p.ew_ahead)) * static_cast<unsigned int>(p.ew_qpm);
            if (c[0] >= ew_total)
              qn = ew_total;                       // nothing left
            else if (c[0] < limit)
              qn = atomicAdd(p.ew_ctrl, 1u);       // may overshoot the limit by a few quanta: harmless
          }
          qn = __shfl_sync(0xffffffffu, qn, 0);
          if (qn == 0xFFFFFFFFu) {                 // far enough ahead for now
            __nanosleep(500);
            continue;
          }
          if (qn >= ew_total) {
            ew_more = false;
            break;
          }
          gate_grad_quantum<T, C::TILE_M>(p, qn, lane);
        }
      }
      if (FSW_PROFILE) prof_t0 = clock64();
      ok = bounded_wait_warp(tfull_bar(NSUB == 2 ? 0 : a), aph, ctl, WAIT_EPI_TMEM_FULL);
      if (FSW_PROFILE) {
        const long long now = clock64();
        prof_wait += now - prof_t0;
        prof_t0 = now;
        ++prof_tiles;
      }
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);

      // Which accumulator regions this warp drains and which 64-column boxes of
      // each.  NSUB==1: region `a`, boxes split between the two warps of a
      // quadrant.  NSUB==2: with 8 warps one region per warp, with 4 both.
      const int r_begin = (NSUB == 2) ? (kSplit == 2 ? chalf : 0) : a;
      const int r_end = (NSUB == 2) ? (kSplit == 2 ? chalf + 1 : 2) : a + 1;
      for (int r = r_begin; r < r_end; ++r) {
        const uint32_t taddr = lane_base + r * C::BN;
        const int rn0 = n0 + (NSUB == 2 ? r * C::REGION_N : 0);
        auto release = [&]() {
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (CG == 2)
              ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(r), 0));
            else
              ptx::mbar_arrive(tempty_bar(r));
          }
        };
        const bool split = (NSUB == 1 && kSplit == 2);
        if (FSW_DBG_SKIP_EPILOGUE) {
          release();
        } else if (NSUB == 2 && w.slot >= 0) {
          drain_partial<ACC16>(p, lane, taddr, w.slot, static_cast<int>(cta_rank), q, r, 0, 16, release);
        } else if (is_fwd(MODE)) {
          if (split)
            drain_swiglu<C, T, ACC16, 1, MODE == MODE_FWDST>(p, e, taddr, rn0, chalf, release);
          else
            drain_swiglu<C, T, ACC16, 2, MODE == MODE_FWDST>(p, e, taddr, rn0, 0, release);
        } else {
          if (split)
            drain_plain<C, MODE, T, ACC16, 2>(p, e, taddr, rn0, 2 * chalf, release);
          else
            drain_plain<C, MODE, T, ACC16, 4>(p, e, taddr, rn0, 0, release);
        }
      }
      if (FSW_PROFILE) prof_drain += clock64() - prof_t0;
      if (NSUB == 2) {
        aph ^= 1u;
      } else {
        a ^= 1;
        if (a == 0) aph ^= 1u;
      }
    }
    if (MODE == MODE_DXE) {
      // a CTA pair with few or no tiles still helps until the queue is empty
      while (ew_more && ok) {
        unsigned int qn = 0;
        if (lane == 0) qn = atomicAdd(p.ew_ctrl, 1u);
        qn = __shfl_sync(0xffffffffu, qn, 0);
        if (qn >= ew_total)
          ew_more = false;
        else
          gate_grad_quantum<T, C::TILE_M>(p, qn, lane);
      }
    }
    if (is_fwd(MODE)) {
      // all bulk stores of this warp must have completed before the CTA exits
      if (lane == 0) ptx::tma_store_wait_all<0>();
      __syncwarp();
    }
    if (FSW_PROFILE && blockIdx.x == 0 && warp == 2 && lane == 0 && p.clk_probe != nullptr) {
      p.clk_probe[4] = prof_wait;
      p.clk_probe[5] = prof_drain;
      p.clk_probe[6] = prof_tiles;
    }
  }

  // ======================= teardown =======================
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    // A wait gave up: give copies and MMAs still in flight time to land before
    // shared and tensor memory are handed back.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < kDrainNs) __nanosleep(1000);
  }
  if (CG == 2) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<CG>(tmem_base, C::TMEM_COLS);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && p.clk_probe != nullptr) {
    p.clk_probe[0] = static_cast<unsigned long long>(clock64() - probe_c0);
    p.clk_probe[1] = ptx::globaltimer_ns() - probe_t0;
  }
}

// ------------------------------------------------------ split-K second pass --
// Adds the fp32 pieces that gemm_kernel left in the workspace for each tile of the
// split tail (see GemmParams::sk_*) in ascending K order and writes the 16-bit
// results.  One block per (tile, CTA half, lane quadrant, accumulator region); a warp
// takes 16-column chunks, lanes are rows, so workspace reads are contiguous.
template <typename T, bool DUAL>
__global__ void __launch_bounds__(256)
    splitk_reduce_kernel(const float4* __restrict__ ws, void* c0, void* c1, int M, int N, int ldc,
                         int num_m_tiles, int num_n_tiles, int group_m, int first_tile,
                         int iters_per_tile, int share) {
  const int b = blockIdx.x;
  const int r = b & 1, q = (b >> 1) & 3, cta = (b >> 3) & 1, j = b >> 4;
  const int lane = threadIdx.x & 31, wv = threadIdx.x >> 5;
  const long long t0 = static_cast<long long>(j) * iters_per_tile;
  const int c_lo = static_cast<int>(t0 / share);
  const int c_hi = static_cast<int>((t0 + iters_per_tile - 1) / share);
  int m_tile, n_tile;
  decode_tile_order(first_tile + j, num_m_tiles, num_n_tiles, group_m, m_tile, n_tile);
  const int row = m_tile * 256 + cta * 128 + q * 32 + lane;
#pragma unroll 1
  for (int cc = 2 * wv; cc < 2 * wv + 2; ++cc) {
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int cl = c_lo; cl <= c_hi; ++cl) {
      const int first = static_cast<int>((static_cast<long long>(cl) * share) / iters_per_tile);
      const int slot = 2 * cl + (first == j ? 0 : 1);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const float4 f = ws[splitk_vec_index(slot, cta, q, r, cc, v, lane)];
        acc[4 * v] += f.x;
        acc[4 * v + 1] += f.y;
        acc[4 * v + 2] += f.z;
        acc[4 * v + 3] += f.w;
      }
    }
    // Column of the chunk in the output: a dual region is [128 of c0 | 128 of c1].
    int col;
    void* out;
    if (DUAL) {
      const int in_region = cc * 16;
      out = in_region >= 128 ? c1 : c0;
      col = n_tile * 256 + r * 128 + (in_region & 127);
    } else {
      out = c0;
      col = n_tile * 512 + r * 256 + cc * 16;
    }
    if (row < M) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (col + 8 * h < N) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) w[e] = pack2<T>(acc[8 * h + 2 * e], acc[8 * h + 2 * e + 1]);
          ptx::st_global_v4(static_cast<char*>(out) + (static_cast<size_t>(row) * ldc + col + 8 * h) * 2,
                            w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
}

// Second pass for the forward: the pieces hold partial sums of [128 gate | 128 up]
// accumulator regions.  Warp w of a block adds gate chunk w and up chunk w + 8 (the
// same 16 output columns), rounds g and u to the 16-bit type and applies the same
// epilogue arithmetic as drain_swiglu: out = round(round(silu_f32(g16)) * u16).
template <typename T>
__global__ void __launch_bounds__(256)
    splitk_reduce_swiglu_kernel(const float4* __restrict__ ws, void* g_out, void* u_out, void* out,
                                int M, int N, int num_m_tiles, int num_n_tiles, int group_m,
                                int first_tile, int iters_per_tile, int share) {
  const int b = blockIdx.x;
  const int r = b & 1, q = (b >> 1) & 3, cta = (b >> 3) & 1, j = b >> 4;
  const int lane = threadIdx.x & 31, wv = threadIdx.x >> 5;
  const long long t0 = static_cast<long long>(j) * iters_per_tile;
  const int c_lo = static_cast<int>(t0 / share);
  const int c_hi = static_cast<int>((t0 + iters_per_tile - 1) / share);
  int m_tile, n_tile;
  decode_tile_order(first_tile + j, num_m_tiles, num_n_tiles, group_m, m_tile, n_tile);
  const int row = m_tile * 256 + cta * 128 + q * 32 + lane;
  const int col = n_tile * 256 + r * 128 + wv * 16;
  float ag[16], au[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) ag[i] = au[i] = 0.f;
  for (int cl = c_lo; cl <= c_hi; ++cl) {
    const int first = static_cast<int>((static_cast<long long>(cl) * share) / iters_per_tile);
    const int slot = 2 * cl + (first == j ? 0 : 1);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const float4 fg = ws[splitk_vec_index(slot, cta, q, r, wv, v, lane)];
      const float4 fu = ws[splitk_vec_index(slot, cta, q, r, wv + 8, v, lane)];
      ag[4 * v] += fg.x;
      ag[4 * v + 1] += fg.y;
      ag[4 * v + 2] += fg.z;
      ag[4 * v + 3] += fg.w;
      au[4 * v] += fu.x;
      au[4 * v + 1] += fu.y;
      au[4 * v + 2] += fu.z;
      au[4 * v + 3] += fu.w;
    }
  }
  if (row >= M) return;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (col + 8 * h >= N) continue;
    uint32_t pg[4], pu[4], po[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      pg[e] = pack2<T>(ag[8 * h + 2 * e], ag[8 * h + 2 * e + 1]);
      pu[e] = pack2<T>(au[8 * h + 2 * e], au[8 * h + 2 * e + 1]);
      float g0, g1;
      unpack2<T>(pg[e], g0, g1);
      po[e] = mul2<T>(pack2<T>(g0 * sigmoid_f32(g0), g1 * sigmoid_f32(g1)), pu[e]);
    }
    const size_t off = (static_cast<size_t>(row) * N + col + 8 * h) * 2;
    if (g_out != nullptr) {
      ptx::st_global_v4(static_cast<char*>(g_out) + off, pg[0], pg[1], pg[2], pg[3]);
      ptx::st_global_v4(static_cast<char*>(u_out) + off, pu[0], pu[1], pu[2], pu[3]);
    }
    ptx::st_global_v4(static_cast<char*>(out) + off, po[0], po[1], po[2], po[3]);
  }
}

// ------------------------------------------- reduction of scattered dX partials --
// Second half of the dX reduce-scatter over NVLink.  Every rank's dX GEMM has stored
// its partial sums for this rank's rows into slice [source rank] of `recv` (see
// GemmParams::scatter).  This kernel, launched on the same stream right after that
// GEMM, (1) tells every peer that this rank's partials are complete - they are: the
// GEMM kernel has finished - by storing the step number `seq` into the peer's flag
// word [this rank], (2) waits, with a time limit, until all peers have said the same
// here, and (3) adds the `world` slices in fp32 in rank order and writes the 16-bit
// result.  A wait that runs out records WAIT_PEER_PARTIALS in the status word and the
// block returns without writing (the host reads the status).
constexpr uint32_t WAIT_PEER_PARTIALS = 5;
struct PeerFlags {
  unsigned int* p[kMaxScatterRanks];  // p[r]: rank r's flag words (peer memory)
};

template <typename T>
__global__ void __launch_bounds__(256)
    dx_slices_reduce_kernel(const uint4* __restrict__ recv, const uint4* __restrict__ own_slice,
                            T* __restrict__ out, long long vecs_per_slice, int world, int rank, unsigned int seq, const PeerFlags peer_flags,
                            volatile unsigned int* my_flags, uint32_t* status,
                            unsigned long long wait_limit_ns) {
  __shared__ int give_up;
  if (threadIdx.x == 0) give_up = 0;
  if (blockIdx.x == 0 && threadIdx.x < world) {
    // the partials were written by an earlier kernel on this stream; order them before
    // the flag for observers on other GPUs
    __threadfence_system();
    unsigned int* f = peer_flags.p[threadIdx.x] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
  }
  __syncthreads();
  if (threadIdx.x < world) {
    const uint64_t t0 = ptx::globaltimer_ns();
    for (;;) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];"
                   : "=r"(v)
                   : "l"(const_cast<unsigned int*>(my_flags) + threadIdx.x)
                   : "memory");
      // flags only grow; compare in wrap-around arithmetic
      if (static_cast<int>(v - seq) >= 0) break;
      if (ptx::globaltimer_ns() - t0 > wait_limit_ns) {
        give_up = 1;
        atomicCAS(status, 0u, WAIT_PEER_PARTIALS | (static_cast<uint32_t>(threadIdx.x) << 8));
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (give_up) return;
  // every slice vector of a thread is loaded before the first is used
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs_per_slice;
       v += stride) {
    uint4 w[kMaxScatterRanks];
#pragma unroll
    for (int s = 0; s < kMaxScatterRanks; ++s) {
      if (s < world) {
        // this rank's own partial may sit outside the receive buffer (it never left the GPU)
        const uint4* src = (s == rank && own_slice != nullptr)
                               ? own_slice + v
                               : recv + static_cast<long long>(s) * vecs_per_slice + v;
        // a coherent load (not the read-only path): peers wrote these lines until just
        // before the flags were seen
        asm volatile("ld.global.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w[s].x), "=r"(w[s].y), "=r"(w[s].z), "=r"(w[s].w)
                     : "l"(src)
                     : "memory");
      }
    }
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxScatterRanks; ++s) {
      if (s < world) {
        const uint32_t ww[4] = {w[s].x, w[s].y, w[s].z, w[s].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo, hi;
          unpack2<T>(ww[e], lo, hi);
          acc[2 * e] += lo;
          acc[2 * e + 1] += hi;
        }
      }
    }
    uint4 o;
    o.x = pack2<T>(acc[0], acc[1]);
    o.y = pack2<T>(acc[2], acc[3]);
    o.z = pack2<T>(acc[4], acc[5]);
    o.w = pack2<T>(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[v] = o;
  }
}

// Time-limited wait until every word of flags[0..n) has reached `seq`; used to learn
// that the peers' copies of their reduced rows into this rank's buffer have landed.
__global__ void wait_flags_kernel(volatile unsigned int* flags, int n, unsigned int seq, uint32_t* status,
                                  unsigned long long wait_limit_ns) {
  if (threadIdx.x >= n) return;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];"
                 : "=r"(v)
                 : "l"(const_cast<unsigned int*>(flags) + threadIdx.x)
                 : "memory");
    if (static_cast<int>(v - seq) >= 0) return;
    if (ptx::globaltimer_ns() - t0 > wait_limit_ns) {
      atomicCAS(status, 0u, WAIT_PEER_PARTIALS | (static_cast<uint32_t>(threadIdx.x) << 8) | 0x80u);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace fsw
