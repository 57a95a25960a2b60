/*
 * C ABI of libfused_swiglu_sm100.so: fused SwiGLU forward and backward for
 * NVIDIA B200 (sm_100a), hand-written TMA + tcgen05 kernels.
 *
 * This header is the drop-in boundary for the GPU work that the Python package
 * `fused_swiglu` (fattorib/fusedswiglu) performs through Triton and cuBLAS.  Each
 * entry point names the reference interface it replaces, by file:line within
 * that project.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current CUDA device, 16-byte
 *     aligned, to a dense row-major array; the library allocates nothing;
 *   - T = batch * sequence tokens, dm = d_model, di = d_intermediate;
 *     x is (T, dm); w_gate and w_up are (dm, di); g, u, out, dout are (T, di);
 *     dm and di must be multiples of 8 (16-byte rows); T may be any value >= 0;
 *   - dtype: FSW_BF16 or FSW_FP16 is the storage type of every tensor;
 *     accum: FSW_ACC_F32, or FSW_ACC_F16 (fp16 tensors only) for an fp16
 *     tensor-memory accumulator;
 *   - `stream` is a cudaStream_t passed as void*; all work is asynchronous on it;
 *   - return value: FSW_OK or a negative FSW_E* code; fsw_last_error() gives the
 *     message for the calling thread.  Nothing aborts or throws.
 */
#ifndef FUSED_SWIGLU_H_
#define FUSED_SWIGLU_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { FSW_BF16 = 0, FSW_FP16 = 1 };
enum { FSW_ACC_F32 = 0, FSW_ACC_F16 = 1 };
enum {
  FSW_OK = 0,
  FSW_EINVAL = -1,      /* bad pointer, shape, dtype or accumulate mode          */
  FSW_EDEVICE = -2,     /* current device is not compute capability 10.x         */
  FSW_ECUDA = -3,       /* a CUDA runtime or driver call failed                  */
  FSW_ETIMEOUT = -4,    /* a kernel gave up on a bounded wait (see fsw_status)   */
  FSW_EUNAVAILABLE = -5 /* the driver lacks cuTensorMapEncodeTiled               */
};

/*
 * Forward:  g = x @ w_gate, u = x @ w_up, out = silu(g) * u, one dual GEMM.
 * Replaces fused_swiglu_fwd + swiglu_kernel (fused_swiglu/kernels/kernels_bf16.py:41-206,
 * fused_swiglu/kernels/kernels_fp16.py:41-216).  `g` and `u` may both be NULL to
 * skip saving the activations (inference); `out` is required.
 * accum = FSW_ACC_F16 corresponds to fast_accum=True (kernels_fp16.py:69-75).
 */
int fsw_forward(const void* x, const void* w_gate, const void* w_up, void* out, void* g, void* u,
                int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream);

/*
 * Gate-gradient elementwise step: du = dout * silu(g), dg = dout * u * silu'(g),
 * with the reference's rounding points.  Replaces elementwise_backward +
 * elementwise_backward_kernel (kernels_bf16.py:210-255, kernels_fp16.py:220-265).
 * Unlike the reference launcher it also processes a tail of numel % 128 elements.
 */
int fsw_backward_elementwise(const void* dout, const void* g, const void* u, void* dg, void* du,
                             int64_t numel, int dtype, void* stream);

/*
 * Input gradient: dx = dg @ w_gate^T + du @ w_up^T as ONE accumulated GEMM.
 * Replaces the two cuBLAS matmuls and the add at fused_swiglu/swiglu.py:45.
 */
int fsw_backward_dx(const void* dg, const void* du, const void* w_gate, const void* w_up, void* dx,
                    int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream);

/*
 * Caller-provided workspace for the GEMMs that can use one (the `_ws` entry points
 * and fsw_backward_dw_columns).  A GEMM's output tiles rarely fill a whole number
 * of waves of the GPU's SM pairs; without a workspace the last, partial wave leaves
 * SMs idle (a quarter of the launch when d_intermediate is split over 8 GPUs).
 * With one, the K loops of the last wave's tiles are divided evenly over all SM
 * pairs, the fp32 partial sums go through the workspace, and a short second kernel
 * adds them in a fixed order (results are deterministic; they can differ from the
 * no-workspace result in the last bit of those tiles, because the fp32 additions
 * associate differently).  fsw_workspace_bytes() is the size that suffices for any
 * launch on the current device (1 MiB per SM pair, 74 MiB on a B200); a smaller,
 * NULL or misaligned (16 bytes) workspace just means the launch does not split.
 * The buffer is scratch: its contents mean nothing after the call, and calls that
 * may overlap on the GPU need different buffers.  Option "split_k" = 0 turns the
 * splitting off process-wide.  No counterpart in the reference.
 */
int64_t fsw_workspace_bytes(void);
int fsw_forward_ws(const void* x, const void* w_gate, const void* w_up, void* out, void* g, void* u,
                   int64_t T, int64_t dm, int64_t di, void* workspace, int64_t workspace_bytes,
                   int dtype, int accum, void* stream);
int fsw_backward_dx_ws(const void* dg, const void* du, const void* w_gate, const void* w_up,
                       void* dx, int64_t T, int64_t dm, int64_t di, void* workspace,
                       int64_t workspace_bytes, int dtype, int accum, void* stream);

/*
 * Weight gradients: dw_gate = x^T @ dg, dw_up = x^T @ du, reduced over all T
 * tokens in one dual GEMM.  Replaces fused_bmm + bmm_kernel
 * (kernels_bf16.py:280-412, kernels_fp16.py:290-422) and the batch sum
 * `unbroadcast` (fused_swiglu/swiglu.py:11-13,56-57).
 */
int fsw_backward_dw(const void* x, const void* dg, const void* du, void* dw_gate, void* dw_up,
                    int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream);

/*
 * fsw_backward_dw restricted to columns [col0, col0 + ncols) of dw_gate and dw_up
 * (col0 and ncols multiples of 8).  All pointers are to the FULL arrays: dg and du
 * (T, di), dw_gate and dw_up (dm, di); only the named columns are read and written,
 * and, without a workspace, get exactly the values fsw_backward_dw would give them
 * (`workspace` may be NULL; see fsw_workspace_bytes above).  `max_sms` > 0
 * caps the SMs this one launch occupies (0 = no cap of its own; the process-wide
 * "gemm_max_sms" option, if set, then applies).  Lets a caller cut the
 * weight-gradient GEMM into pieces, e.g. to run one piece beside a collective on
 * fewer SMs and the rest on the whole GPU, without touching process-wide state.
 * No counterpart in the reference, whose fused_bmm always covers all of
 * d_intermediate.
 */
int fsw_backward_dw_columns(const void* x, const void* dg, const void* du, void* dw_gate,
                            void* dw_up, int64_t T, int64_t dm, int64_t di, int64_t col0,
                            int64_t ncols, int max_sms, void* workspace, int64_t workspace_bytes,
                            int dtype, int accum, void* stream);

/*
 * Whole backward on one stream: elementwise step into the caller's scratch
 * (`dg_scratch`, `du_scratch`, each T*di elements), then dx, then dw.
 * Replaces FusedSwiGLU.backward (fused_swiglu/swiglu.py:34-58).
 * accum applies to the dw GEMM; dx always accumulates in fp32, as cuBLAS does on
 * the reference path.
 */
int fsw_backward(const void* dout, const void* x, const void* w_gate, const void* w_up,
                 const void* g, const void* u, void* dg_scratch, void* du_scratch, void* dx,
                 void* dw_gate, void* dw_up, int64_t T, int64_t dm, int64_t di, int dtype,
                 int accum, void* stream);

/*
 * The gate-gradient step inside the dX GEMM ("dg = dout*u*silu'(g) and du = dout*silu(g)
 * computed on-chip").  Replaces elementwise_backward (kernels_bf16.py:210-255) and the
 * two matmuls of swiglu.py:45 by ONE launch.
 *
 * fsw_forward_st is fsw_forward that saves, in place of g and u, the two factors the
 * backward needs: s = round(silu(g)) and t = round(u * round(silu'(g))), both from
 * the 16-bit g and u.  Then dg = round(dout * t) and du = round(dout * s): one
 * multiply each (the reference rounds dout*u first and multiplies by silu'(g) second,
 * kernels_bf16.py:230-231; the two orders differ by one rounding of a 16-bit product).
 *
 * fsw_backward_dx_fused computes dx = dg @ w_gate^T + du @ w_up^T without reading dg
 * or du: the kernel's epilogue warps load dout, t and s tiles, multiply, and write the
 * products straight into the swizzled shared-memory operand stage of the tensor-core
 * pipeline.  The tiles of the first column of output tiles also store dg and du (T, di)
 * for fsw_backward_dw, which follows.  fp32 accumulation.
 *
 * fsw_backward_elementwise_st is the same dg/du step as a kernel of its own (numel a
 * multiple of 8).
 */
int fsw_forward_st(const void* x, const void* w_gate, const void* w_up, void* out, void* s, void* t,
                   int64_t T, int64_t dm, int64_t di, int dtype, int accum, void* stream);
int fsw_backward_dx_fused(const void* dout, const void* s, const void* t, const void* w_gate,
                          const void* w_up, void* dx, void* dg, void* du, int64_t T, int64_t dm,
                          int64_t di, int dtype, void* stream);
int fsw_backward_elementwise_st(const void* dout, const void* s, const void* t, void* dg, void* du,
                                int64_t numel, int dtype, void* stream);

/*
 * fsw_backward_elementwise and fsw_backward_dx_ws as ONE launch (replaces
 * kernels_bf16.py:210-255 + swiglu.py:45): the dX GEMM's epilogue warps, idle while a
 * tile's K loop runs, compute dg and du (same arithmetic and rounding points as
 * fsw_backward_elementwise, once per element) ahead of the tiles that read them; a tile's
 * loads wait - time-limited - until the rows they need are complete.  dg and du (T, di)
 * are outputs here, for fsw_backward_dw.  Results are bit-identical to the two separate
 * calls.  Falls back to them when the launch would not use 256-row tiles of SM pairs or
 * T exceeds 2 Mi rows, or with option "gate_in_dx" = 0.
 */
int fsw_backward_dx_gate(const void* dout, const void* g, const void* u, const void* w_gate,
                         const void* w_up, void* dx, void* dg, void* du, int64_t T, int64_t dm,
                         int64_t di, void* workspace, int64_t workspace_bytes, int dtype, void* stream);

/*
 * dX reduced across GPUs inside the kernels (no counterpart in the reference, which
 * is single-GPU).  With d_intermediate split over `world` ranks (2..8) every rank's
 * dX GEMM yields a partial sum of the whole (T, dm) gradient.  Rank r owns rows
 * [r*T/world, (r+1)*T/world); T/world must be a multiple of 32.
 *
 * fsw_backward_dx_scatter is fsw_backward_dx whose epilogue stores each tile's rows
 * directly into the owner's receive buffer over NVLink (plain stores to peer memory;
 * no TMA or multicast touches peer memory): recv_ptrs[r] is rank r's buffer, laid
 * out [source rank][T/world][dm], mapped into this process (CUDA IPC / symmetric
 * memory; the caller maps it).  recv_ptrs is a HOST array of `world` device pointers.
 *
 * fsw_dx_reduce, called on the same stream right after it, stores `seq` into flag
 * word [rank] of every rank (peer_flag_ptrs: HOST array of `world` device pointers to
 * each rank's `world` 32-bit flag words), waits until all `world` words of my_flags
 * have reached `seq` - i.e. every peer's partials for these rows have arrived - and
 * writes the fp32 sum of the `world` slices of `recv` (this rank's buffer), rounded
 * once, to dx_rows (T/world, dm); if own_slice is not NULL, slice [rank] is read from
 * there instead (a caller that moves the partials with copies need not copy its own).  `seq` must grow by one per step, and the receive
 * buffers and flag arrays must alternate between two sets from step to step (a rank
 * may be one step ahead of a peer, never two).  The wait gives up after
 * "wait_limit_ms": the kernel then records a code in the status word (fsw_status)
 * and leaves dx_rows unwritten; nothing hangs.
 *
 * fsw_wait_flags waits the same way until flags[0..n) have all reached seq.
 */
int fsw_backward_dx_scatter(const void* dg, const void* du, const void* w_gate, const void* w_up,
                            void* const* recv_ptrs, int world, int rank, int64_t T, int64_t dm,
                            int64_t di, int dtype, int accum, void* stream);
int fsw_dx_reduce(const void* recv, const void* own_slice, void* const* peer_flag_ptrs, void* my_flags,
                  int world, int rank, uint32_t seq, int64_t rows, int64_t dm, void* dx_rows, int dtype,
                  void* stream);
int fsw_wait_flags(void* flags, int n, uint32_t seq, void* stream);

/*
 * Plain GEMM on row-major 16-bit arrays with the same tcgen05 kernel:
 *   trans_a = 0, trans_b = 0:  c (M,N) = a (M,K) @ b (K,N)
 *   trans_a = 0, trans_b = 1:  c (M,N) = a (M,K) @ b (N,K)^T
 *   trans_a = 1, trans_b = 0:  c (M,N) = a (K,M)^T @ b (K,N)
 * Every row length (of a, b and c) must be a multiple of 8 elements.  This is the
 * down projection y = out @ w_down that follows SwiGLU in an MLP block, and its two
 * gradients.  It has no counterpart in the reference, which stops at `out`
 * (a user of the reference calls a library GEMM for it).
 */
int fsw_gemm(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int trans_a,
             int trans_b, int dtype, int accum, void* stream);
/* The same with a workspace for the split of the last wave (see fsw_workspace_bytes). */
int fsw_gemm_ws(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int trans_a,
                int trans_b, void* workspace, int64_t workspace_bytes, int dtype, int accum,
                void* stream);

/*
 * fsw_backward for callers that have no scratch memory to give and may not
 * allocate any.  (No counterpart in the reference, whose launchers allocate
 * fresh dg/du tensors on every call.)
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they need
 * the backward: an inference/training runtime whose device memory is planned up
 * front and handed out from a fixed arena, a plugin's enqueue hook that is
 * forbidden to allocate, or a latency-critical loop that cannot afford the
 * device-wide synchronisation cudaMalloc and cudaFree imply.  For them the dg/du
 * scratch lives in a fixed array inside the library instead of in an argument:
 *
 *   - limit: T * di <= FSW_STATIC_SCRATCH_ELEMS (4 Mi elements; 16 MiB for dg and
 *     du together, held by every GPU that loads the library until the process
 *     exits).  Larger problems get FSW_EINVAL with a message naming the limit;
 *     use fsw_backward with your own scratch for those;
 *   - the call allocates nothing: no cudaMalloc/cudaFree, no allocating library
 *     routine.  Inputs and outputs are still the caller's buffers;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current).  Make that first call
 *     before starting any stream capture;
 *   - every call on a device shares the one array.  Its contents after a call are
 *     that call's dg/du; the next call overwrites all it reads, so nothing has to
 *     be cleared.  Two calls that overlap on the GPU (different streams, or
 *     different host threads) race on it: serialise them.
 * Arguments and results are otherwise those of fsw_backward.
 */
#define FSW_STATIC_SCRATCH_ELEMS (4 * 1024 * 1024)
int fsw_backward_static_scratch(const void* dout, const void* x, const void* w_gate,
                                const void* w_up, const void* g, const void* u, void* dx,
                                void* dw_gate, void* dw_up, int64_t T, int64_t dm, int64_t di,
                                int dtype, int accum, void* stream);

/* Message for the last non-zero return on the calling thread ("" if none). */
const char* fsw_last_error(void);

/*
 * Device facts for `device`: SM count, compute capability, opt-in shared memory
 * per block.  Any output pointer may be NULL.  Returns FSW_EDEVICE if the device
 * is not compute capability 10.x (there is no fallback path).
 */
int fsw_query_device(int device, int* sm_count, int* cc_major, int* cc_minor,
                     int64_t* smem_optin_bytes);

/*
 * Synchronises the current device and returns the kernels' status word, clearing
 * it: 0 when every bounded wait completed, otherwise (cta << 8 | code) of the
 * first wait that gave up.  Returns a negative FSW_E* code on CUDA failure.
 */
int64_t fsw_status(void);

/*
 * Tuning and debugging knobs.  They are PROCESS-WIDE: a value set here applies to
 * every later call from any thread on any device, so a host with several threads
 * should set them once at start-up (per-call needs, like an SM cap for one launch,
 * are arguments of the entry points instead).  Apart from these options the
 * library keeps only caches (device attributes, encoded tensor maps) and, per
 * device, one status word (fsw_status), one clock probe ("last_sm_khz") and a ring
 * of pacing counters; entry points may be called concurrently from several threads
 * and on several streams and devices.  Main names: "cta_group" (1 or 2 CTAs
 * per MMA, 0 = automatic), "nsub" (1 or 2 accumulator regions per tile, 0 =
 * automatic), "group_m" (tile rasterisation group height in tiles, 0 = automatic),
 * "gemm_max_sms" (cap on the SMs a GEMM launch occupies, 0 = all; used to leave room
 * for a concurrent collective), "pace_kb" (the TMA producers of all CTAs of a GEMM
 * meet every pace_kb K blocks so that both dies of the GPU stream the same operand
 * panels at the same time and share them in L2; 0 = free-running; advisory, never
 * changes results), "pace_limit_us" (longest wait at one meeting), "l2_a", "l2_b",
 * "l2_out" (L2 eviction priority of operand loads and forward stores: 0 normal,
 * 1 evict first, 2 evict last), "ew_blocks_per_sm".  Read-only facts through
 * fsw_get_option: "sm_count", "max_pairs", "stages", "last_sm_khz", "pace_off" (1 if
 * the last paced launch gave its pacing up), "map_cache_hits", "map_cache_misses",
 * "kernel_launches" (kernels launched by the library in this process so far).  Returns FSW_EINVAL for an unknown name
 * or value.  fsw_get_option returns the current value or -1.
 */
int fsw_set_option(const char* name, int64_t value);
int64_t fsw_get_option(const char* name);

/*
 * Testing aid (runs on the host, needs no GPU): the (m_tile, n_tile) that the
 * kernels' rasterisation assigns to linear tile index t for a grid of
 * num_m_tiles x num_n_tiles tiles issued group_m rows at a time.
 */
int fsw_debug_decode_tile(int t, int num_m_tiles, int num_n_tiles, int group_m, int* m_tile,
                          int* n_tile);

/*
 * Testing aid (host only): the kernels' distribution of work when the last partial
 * wave of tiles is split along K (see fsw_workspace_bytes).  For a grid of
 * num_m_tiles x num_n_tiles tiles of iters_per_tile K iterations on `pairs` SM
 * pairs: returns 1 if the launch would split (0 if not, negative on bad arguments)
 * and fills plan[3] = {first split tile, K iterations per pair, total split
 * iterations}; with item != NULL also work item `idx` of pair `cluster` as
 * item[6] = {valid, m_tile, n_tile, first iteration, end iteration, workspace slot
 * or -1 for a whole tile}.
 */
int fsw_debug_split_work(int num_m_tiles, int num_n_tiles, int group_m, int iters_per_tile,
                         int pairs, int cluster, int idx, int64_t* plan, int* item);

/*
 * Testing aid (host only): the tcgen05 instruction descriptor for the given types,
 * operand majorness (0 = K-major, 1 = MN-major) and MMA shape, and the two
 * shared-memory matrix descriptors (without start address) the kernels use.
 */
int fsw_debug_descriptors(int dtype, int accum, int a_major, int b_major, int m, int n,
                          uint32_t* idesc, uint64_t* sdesc_k_major, uint64_t* sdesc_mn_major);

#ifdef __cplusplus
}
#endif
#endif /* FUSED_SWIGLU_H_ */
