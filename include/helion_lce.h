/* C ABI of the B200 (sm_100a) fused linear-cross-entropy library (libhelion_lce.so).
 *
 * The library replaces the GPU work behind two public functions of the reference,
 *   tritium.linear_cross_entropy           (tritium/ops/cross_entropy.py:716-725)
 *   tritium.linear_cross_entropy_backward  (tritium/ops/cross_entropy.py:863-959)
 * i.e. loss = cross_entropy(hidden @ weight^T, target) and its gradients, without ever writing the
 * N x V logits to memory. The reference has no FFI of its own (it launches Triton kernels from
 * Python); each entry point below names the reference host function whose launches it replaces.
 *
 * Conventions
 *   - every pointer is a device pointer owned by the caller unless stated otherwise; the library
 *     allocates nothing at call time and keeps no reference after the call returns. The one piece of
 *     device memory it owns is compiled into its image: the 16 MiB scratch array of
 *     lce_forward_stats_static (plus a 4-byte status word and 16 KB of completion counters used by
 *     one-launch forwards of very small problems), held by every GPU that loads the library;
 *   - a call only enqueues work on `stream` (a cudaStream_t passed as void*) of the current
 *     device and returns; it never synchronises. Kernels of one call may be launched with programmatic
 *     stream serialization (they wait on the device for their predecessor before they read its results);
 *     towards the work before and after the call the stream order is the ordinary one;
 *   - return value 0 = enqueued; anything else is a synchronous argument / launch error, see
 *     lce_strerror(). There is no CPU fallback: a device that is not sm_100 yields LCE_ERR_ARCH;
 *   - x is [N, H] row-major, w is [V_local, H] row-major (rows vocab_start .. vocab_start+V_local
 *     of the full weight when the vocabulary is sharded), targets are GLOBAL vocabulary indices;
 *   - `ws` is scratch memory of at least the matching *_workspace_bytes(); its contents are
 *     undefined before and after a call, and calls that overlap in time need distinct scratch.
 */
#ifndef HELION_LCE_H_
#define HELION_LCE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LCE_VERSION 2

/* element type of x, w, dx, dw */
#define LCE_DTYPE_BF16 0
#define LCE_DTYPE_F16 1
#define LCE_DTYPE_F32 2

/* loss reduction (torch.nn.functional.cross_entropy semantics) */
#define LCE_REDUCTION_NONE 0
#define LCE_REDUCTION_MEAN 1
#define LCE_REDUCTION_SUM 2

/* flags */
#define LCE_FLAG_FORCE_SIMT 1u /* CUDA-core kernels even where the tcgen05 path applies        */
#define LCE_FLAG_FORCE_TC 2u   /* tcgen05 kernels or LCE_ERR_ARG; never a silent switch         */
#define LCE_FLAG_DX_F32 4u     /* dx is float32 [N, H]: a partial sum another rank will reduce   */
#define LCE_FLAG_NO_DX 8u      /* skip dX (dx may be NULL)                                       */
#define LCE_FLAG_NO_DW 16u     /* skip dW (dw may be NULL)                                       */
#define LCE_FLAG_ONE_CTA 32u   /* tcgen05 cta_group::1 (one CTA per 128x256 tile) instead of the
                                  default CTA pairs (cta_group::2, 256x256 tiles)                  */

/* status codes */
#define LCE_OK 0
#define LCE_ERR_ARG 1          /* NULL pointer, negative size, unknown enum                      */
#define LCE_ERR_ALIGN 2        /* tcgen05 path forced but a pointer / pitch is not 16-byte aligned */
#define LCE_ERR_WS_TOO_SMALL 3
#define LCE_ERR_ARCH 4         /* current device is not compute capability 10.x                  */
#define LCE_ERR_CUDA 5         /* a CUDA runtime / driver call failed                            */
#define LCE_ERR_TOO_LARGE 6    /* a dimension exceeds what 32-bit tile indexing supports         */
#define LCE_ERR_STATIC_SCRATCH 7 /* lce_forward_stats_static: problem exceeds the built-in scratch  */

int lce_version(void);
const char* lce_strerror(int code);
/* Name of the CUDA error behind the calling thread's most recent LCE_ERR_CUDA from a kernel launch
 * ("cudaSuccess" if there was none). */
const char* lce_last_cuda_error(void);

/* Number of kernels this library has launched since it was loaded (host-side counter, all devices
 * and streams). Lets a harness state how many of the library's own kernels ran inside a timed
 * region. No counterpart in the reference. */
unsigned long long lce_launch_count(void);

/* Reads (and optionally clears) the per-device status word that kernels set when one of their
 * bounded waits ran out (0 = no such event). Synchronises the device; meant for tests. */
int lce_device_status(int* status_out, int clear);

/* ---- forward ---------------------------------------------------------------------------------
 * Replaces the launches of _linear_cross_entropy_forward (tritium/ops/cross_entropy.py:563-640):
 * the partial-forward kernel (:192-248) or the direct kernel (:134-189).
 * Writes per-row softmax statistics of the LOCAL vocabulary shard, component-major:
 *   stats[0*N + i] = max_j z[i,j]   stats[1*N + i] = sum_j exp(z[i,j] - max)
 *   stats[2*N + i] = z[i, target_i] if vocab_start <= target_i < vocab_start + V_local else -inf
 */
size_t lce_forward_workspace_bytes(int64_t N, int64_t H, int64_t V_local, int dtype, unsigned flags);
int lce_forward_stats(const void* x, const void* w, const void* target, int target_is_i64,
                      int64_t N, int64_t H, int64_t V_local, int64_t vocab_start, int dtype,
                      float* stats, void* ws, size_t ws_bytes, unsigned flags, void* stream);

/* Same computation and same `stats` output as lce_forward_stats, but with no workspace argument:
 * the partial statistics go through a fixed 16 MiB array that is compiled into the library
 * (lce_forward_stats_static_capacity() returns its size). No counterpart in the reference.
 *
 * It exists for hosts that cannot hand the library scratch memory at call time - a serving or
 * training process whose device memory was carved up once at start-up, so that a later allocation
 * would fail or fragment someone else's pool, or a thread that must not block on the device-wide
 * synchronisation an allocation can imply. The call itself allocates nothing and frees nothing, on
 * the device or through any library.
 *
 *   - Limit: ceil(V_local / T) * 3 * roundup(N, 64) * 4 bytes must fit in the 16 MiB, with T = 256 on
 *     the tcgen05 path and T = 128 on the CUDA-core path (e.g. N = 4096 with V_local = 50304 in bf16).
 *     Larger problems return LCE_ERR_STATIC_SCRATCH and launch nothing.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture. Later calls reuse the cached address.
 *   - Every GPU that loads the library holds the 16 MiB until the process exits.
 *   - All calls on a device share the one array, which still holds the previous call's values. No
 *     entry needs clearing: each value read was written earlier in the same call. But two calls
 *     that can overlap on the GPU (different streams, no dependency) would race on it; serialise
 *     them, or use lce_forward_stats with separate workspaces. */
size_t lce_forward_stats_static_capacity(void);
int lce_forward_stats_static(const void* x, const void* w, const void* target, int target_is_i64,
                             int64_t N, int64_t H, int64_t V_local, int64_t vocab_start, int dtype,
                             float* stats, unsigned flags, void* stream);

/* Replaces _linear_cross_entropy_reduce_forward_kernel (tritium/ops/cross_entropy.py:251-293):
 * merges the statistics of R shards (stats is [R][3][N], shard r at stats + r*3*N; R = 1 on one
 * GPU) in shard order and produces
 *   lse[i]  = logsumexp over the full vocabulary (fp32 [N], also for ignored rows)
 *   loss    = one float for MEAN / SUM, N floats for NONE (0 for ignored rows)
 *   valid_count (optional, may be NULL) = number of rows with target != ignore_index, as float
 * The sum over rows uses a fixed tree, so the loss is bit-identical from run to run (the
 * reference accumulates with atomics). ws: lce_finalize_workspace_bytes(N). */
size_t lce_finalize_workspace_bytes(int64_t N);
int lce_finalize(const float* stats, int R, const void* target, int target_is_i64, int64_t N,
                 int64_t ignore_index, int reduction, float* lse, float* loss, float* valid_count,
                 void* ws, size_t ws_bytes, void* stream);

/* Forward in one call for an unsharded vocabulary: lce_forward_stats followed by lce_finalize, with the
 * merge and the finalize fused (the statistics never reach memory). Replaces the whole of
 * _linear_cross_entropy_forward (tritium/ops/cross_entropy.py:563-640). Outputs as lce_finalize.
 * N must be > 0. */
size_t lce_forward_loss_workspace_bytes(int64_t N, int64_t H, int64_t V, int dtype, unsigned flags);
int lce_forward_loss(const void* x, const void* w, const void* target, int target_is_i64, int64_t N,
                     int64_t H, int64_t V, int dtype, int64_t ignore_index, int reduction, float* lse,
                     float* loss, float* valid_count, void* ws, size_t ws_bytes, unsigned flags,
                     void* stream);

/* ---- backward --------------------------------------------------------------------------------
 * Replaces linear_cross_entropy_backward (tritium/ops/cross_entropy.py:863-959): the fused
 * small-shape kernel (:296-382) and the chunk loop of F.linear / in-place softmax-gradient /
 * mm / addmm (:927-957).
 *   G  = (softmax(z) - onehot(target)) * scale_i, rounded to the input dtype
 *        scale_i = grad_out / valid_count (MEAN), grad_out (SUM), grad_out[i] (NONE); 0 if ignored
 *   dx = G  @ w   [N, H]        (input dtype, or float32 partial with LCE_FLAG_DX_F32)
 *   dw = G^T @ x  [V_local, H]  (input dtype)
 * grad_out is read on the device: one float for MEAN / SUM, N floats for NONE.
 * G is staged block by block through `ws` (block_bytes caps one block; 0 = default 256 MiB), and
 * partial sums over blocks are added in a fixed order in fp32, so results are deterministic.
 * dx_events: NULL, or one cudaEvent_t per row chunk of lce_backward_plan(); event i is recorded on
 * `stream` as soon as the dx rows of chunk i are final (before the remaining dW work), so that a
 * caller can start reducing partial dx across ranks on another stream while this call's GEMMs run.
 * dw_sumsq: NULL, or one float that receives the sum of squares of dw as stored (the head's share of the
 * gradient norm that helion.clip_grad_norm computes, helion/training.py:36-49, by reading every gradient
 * again): the dW GEMM's epilogue adds up the squares of the values it stores, one partial per (tile, warp),
 * and a last small launch adds the partials in index order - no second pass over the V x H gradient, and the
 * same bits on every run. dw must then be 16-byte aligned. */
/* Optional fusion of the cross-rank dX reduction into the dX GEMM (vocabulary-parallel runs; new, the
 * reference is single-GPU). With a non-NULL `scatter` (and LCE_FLAG_DX_F32) lce_backward does not write
 * `dx`: the epilogue of the dX GEMM stores every finished fp32 row directly into the staging buffer of
 * the rank that owns the row in a reduce-scatter over row slices (rows_per_rank = ceil(N / world),
 * owner = row / rows_per_rank), through peer pointers over NVLink. staging[k] is rank k's buffer of
 * world * rows_per_rank * H floats, 16-byte aligned (peer-mapped device memory, e.g. symmetric memory);
 * this rank writes slot `rank` of each. Plain stores only: no TMA and no multicast touch peer memory, and
 * no kernel waits on another GPU - the caller orders the ranks (a barrier) before lce_dx_reduce_gather
 * sums the world slots of this rank's rows in rank order, rounds once and stores the result into every
 * rank's final dX buffer (out_ptrs[k], [N, H] in `dtype`). */
typedef struct {
    void* staging[8];
    int rank;
    int world;
} lce_peer_scatter;

int lce_dx_reduce_gather(const void* staging, int world, int rank, int64_t N, int64_t H, int dtype,
                         void* const* out_ptrs, void* stream);

/* The reduce half alone: sums the world slots of this rank's row slice (rows rank * rows_per_rank ..) of
 * ITS OWN staging buffer in rank order, rounds once and writes the slice to local memory, out =
 * [rows_per_rank, H] in `dtype`, 16-byte aligned. The caller then all-gathers the slices (any collective
 * library), which also tells every rank that all slices are final. New; the reference is single-GPU. */
int lce_dx_reduce_slice(const void* staging, int world, int rank, int64_t N, int64_t H, int dtype,
                        void* out, void* stream);

/* Workspace sizes and the split of a short contraction over CTAs are computed for a GPU of 148 SMs
 * (74 CTA pairs), B200's count, whatever device is current: the plan, and with it the summation order
 * and the result bits, are then the same on every device the library accepts. */
size_t lce_backward_workspace_bytes(int64_t N, int64_t H, int64_t V_local, int dtype, unsigned flags,
                                    size_t block_bytes);
int lce_backward(const void* x, const void* w, const void* target, int target_is_i64,
                 const float* lse, const float* grad_out, int64_t N, int64_t H, int64_t V_local,
                 int64_t vocab_start, int dtype, int64_t ignore_index, int reduction, void* dx,
                 void* dw, void* ws, size_t ws_bytes, unsigned flags, size_t block_bytes,
                 void* const* dx_events, const lce_peer_scatter* scatter, float* dw_sumsq, void* stream);

/* The block grid lce_backward will use for these arguments (x and w only decide, by their
 * alignment, which kernel family runs): out[0] = rows per row chunk, out[1] = vocabulary columns per
 * band, out[2] = number of row chunks, out[3] = number of bands. Host-only. No counterpart in the
 * reference (its chunk size is _linear_ce_backward_chunk_size, tritium/ops/cross_entropy.py:515-519). */
int lce_backward_plan(int64_t N, int64_t H, int64_t V_local, int dtype, unsigned flags,
                      size_t block_bytes, const void* x, const void* w, int64_t* out);

/* ---- cross-entropy on materialised logits -------------------------------------------------------
 * The plain op of the same reference file: tritium.cross_entropy (tritium/ops/cross_entropy.py:708-713,
 * kernel :36-68) and tritium.cross_entropy_backward (:792-799, kernel :71-100). logits is [N, V]
 * row-major in `dtype`. Outputs as lce_finalize: lse[N], loss (1 float, or N for NONE), optional
 * valid_count. dlogits has the dtype of logits. One pass over the logits each way (bandwidth-bound);
 * no limit on V (the reference refuses next_pow2(V) > 131072). N must be > 0 in the forward. */
size_t lce_ce_workspace_bytes(int64_t N, int64_t V, int dtype);
int lce_ce_forward(const void* logits, const void* target, int target_is_i64, int64_t N, int64_t V,
                   int dtype, int64_t ignore_index, int reduction, float* lse, float* loss,
                   float* valid_count, void* ws, size_t ws_bytes, void* stream);
int lce_ce_backward(const void* logits, const void* target, int target_is_i64, const float* lse,
                    const float* grad_out, int64_t N, int64_t V, int dtype, int64_t ignore_index,
                    int reduction, void* dlogits, void* ws, size_t ws_bytes, void* stream);

/* ---- plain matrix product --------------------------------------------------------------------------
 * c[M, N] = A[M, K] * B[K, N] in `dtype` with fp32 accumulation, on the GEMM cores of the fused op
 * (tcgen05 for 16-bit inputs with 16-byte aligned bases and pitches, CUDA cores otherwise; a short M with
 * a long K is split along K and summed in a fixed order). Replaces the launches of tritium.matmul /
 * matmul_vec (tritium/ops/matmul.py:47-129, 252-309): forward, and both backward products through the
 * layout flags. Either operand may be given transposed:
 *   a_mn_major = 0: a[m * lda + k]      1: a[k * lda + m]
 *   b_mn_major = 1: b[k * ldb + n]      0: b[n * ldb + k]        c[m * ldc + n]
 * ws: lce_matmul_workspace_bytes() bytes (0 unless K is split). */
size_t lce_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype, unsigned flags);
int lce_matmul(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int a_mn_major,
               int64_t lda, int b_mn_major, int64_t ldb, int64_t ldc, int dtype, void* ws, size_t ws_bytes,
               unsigned flags, void* stream);

/* ---- consumers of dW --------------------------------------------------------------------------------
 * lce_adamw_step replaces the launch of tritium.adamw_step (tritium/ops/adamw.py:21-54, :113-151): in-place
 * AdamW on `param` (n elements of `dtype`, grad the same dtype) with fp32 moments, same arithmetic in fp32.
 * grad_scale: NULL, or a device scalar multiplied into the gradient first (the clipping coefficient of
 * helion.clip_grad_norm, helion/training.py:36-49, applied without a separate pass over the gradients).
 * lce_sumsq: out (+)= sum of x[i]^2 (fp32, fixed summation order: identical bits from run to run), the
 * quantity behind clip_grad_norm; ws: lce_sumsq_workspace_bytes(). All pointers 16-byte aligned. */
int lce_adamw_step(void* param, const void* grad, float* exp_avg, float* exp_avg_sq, int64_t n, int dtype,
                   float lr, float beta1, float beta2, float eps, float weight_decay, int64_t step,
                   const float* grad_scale, void* stream);
size_t lce_sumsq_workspace_bytes(void);
int lce_sumsq(const void* x, int64_t n, int dtype, float* out, int accumulate, void* ws, size_t ws_bytes,
              void* stream);

/* ---- greedy decoding head ----------------------------------------------------------------------------
 * token[row] = vocab_start + argmax_v (x[row] . w[v]) (the lowest index on ties), logprob[row] = log softmax of
 * the row at that token, lse[row] (NULL: not written) = the row's logsumexp - the logits are never materialised.
 * Replaces, for greedy sampling, the logits product of the reference's decode step
 * (examples/common.py:127-131, :380-384: tritium.matmul / matmul_vec on lm_head.T.contiguous(), a V x H
 * transpose copy and an N x V write per step). ws: lce_forward_workspace_bytes(N, H, V, dtype, flags). */
int lce_greedy_head(const void* x, const void* w, int64_t N, int64_t H, int64_t V, int64_t vocab_start, int dtype,
                    int64_t* token, float* logprob, float* lse, void* ws, size_t ws_bytes, unsigned flags,
                    void* stream);

/* Sampling head: for every row the k (1..64) largest SCALED logits y = inv_temperature * x . w[v] with their
 * GLOBAL vocabulary indices (vocab_start + local row of w), largest first and the lower index first among
 * equal values, and lse[i] = logsumexp_v y[i, v] over this shard - what temperature / top-k / nucleus
 * sampling needs, without the N x V logits reaching memory. top_val is float32 [N, k], top_idx int64 [N, k]
 * (-inf / -1 where the shard has fewer than k rows), lse float32 [N]. The result is exact: a vocabulary tile
 * that holds more of the k best than the GEMM epilogue keeps per tile (8) is detected in the per-row merge and
 * recomputed there. Takes the place of the reference's decode step, which forms all logits with
 * tritium.matmul_vec on lm_head.T.contiguous() and runs torch.topk / torch.sort over them
 * (examples/common.py:288-301, 380-396). ws: lce_topk_workspace_bytes(). */
size_t lce_topk_workspace_bytes(int64_t N, int64_t H, int64_t V_local, int dtype, unsigned flags);
int lce_topk_head(const void* x, const void* w, int64_t N, int64_t H, int64_t V_local, int64_t vocab_start,
                  int dtype, int k, float inv_temperature, float* top_val, int64_t* top_idx, float* lse,
                  void* ws, size_t ws_bytes, unsigned flags, void* stream);

/* ---- producer of the hidden states -----------------------------------------------------------------
 * lce_rmsnorm_forward replaces the launches of tritium.rmsnorm and tritium.residual_rmsnorm
 * (tritium/ops/rmsnorm.py:29-84, :325-349, :749-778) on [n_rows, hidden] row-major tensors of `dtype`:
 *   z = x (+ residual);  rstd = 1 / sqrt(mean(z^2) + eps);  out = z * rstd * weight     (fp32 arithmetic)
 * residual, residual_out: both NULL (plain rmsnorm) or both set (residual_out = z rounded to dtype).
 * rstd: NULL or [n_rows] float32 (what the reference saves for backward).
 * lce_rmsnorm_backward replaces tritium.rmsnorm_backward and the backward of both autograd functions
 * (tritium/ops/rmsnorm.py:105-280, :383-616, :697-734):
 *   dx = rstd * dy * weight - (rstd^3 / hidden) * x * sum(dy * weight * x)   (+ dresidual, when not NULL)
 *   dweight = sum over rows of dy * x * rstd      (NULL: not computed)
 * x is the normalised tensor (residual_out for the residual form). rstd NULL: recomputed from x and eps.
 * One pass over dy and x; dweight is summed in a fixed order (identical bits from run to run, where the
 * reference uses atomics below hidden = 512). ws: lce_rmsnorm_backward_workspace_bytes(), needed only
 * when dweight is wanted. hidden is limited by memory only (the reference stops at 65536). */
int lce_rmsnorm_forward(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                        float* rstd, int64_t n_rows, int64_t hidden, float eps, int dtype, void* stream);
size_t lce_rmsnorm_backward_workspace_bytes(int64_t n_rows, int64_t hidden, int dtype);
/* How a call would run (host arithmetic only; no device needed): op 0 rmsnorm forward, 1 residual forward,
 * 2 backward, 3 backward with dresidual; aligned = all pointers 16-byte aligned. out[0] form (0 shared-memory
 * ring, 1 register-resident rows, 2 two-pass wide rows), out[1] 16-byte vectors per thread, out[2] threads per
 * CTA, out[3] rows per step, out[4] CTAs per SM / out[5] stages / out[6] dynamic shared memory bytes of the
 * ring (0 otherwise), out[7] CTAs launched on a device of sm_count SMs. The counterpart of the reference's
 * block-size and staged-dweight heuristics (tritium/ops/rmsnorm.py:338, :371-380). */
int lce_rmsnorm_plan(int64_t n_rows, int64_t hidden, int dtype, int op, int aligned, int sm_count, int64_t* out);
int lce_rmsnorm_backward(const void* dy, const void* x, const void* weight, const float* rstd,
                         const void* dresidual, void* dx, void* dweight, int64_t n_rows, int64_t hidden, float eps,
                         int dtype, void* ws, size_t ws_bytes, void* stream);

/* ---- test hook (not part of the product interface) -------------------------------------------
 * Test infrastructure only: nothing above depends on it, a binding for the reference needs no stub
 * for it, and it may change without notice.
 * out[M, N] (float32, row-major) = A * B^T on the tcgen05 GEMM core used by every kernel above,
 * for 16-bit inputs. a_mn_major = 0: a is [M, K] row-major; 1: a is [K, M] row-major. Same for b
 * with N. No counterpart in the reference; exists so the operand-layout handling can be tested
 * in isolation. */
/* Tuning knobs of the tcgen05 launches, process-wide, for measurements: band_mb = MiB of operand panels the
 * tile order keeps resident in L2 (default 32), l2_hint_mode = 0 no eviction hints, 1 resident operand
 * evict_last + streaming operand evict_first, 2 evict_last only (default), dyn_waves = launches of at least
 * this many waves of tiles draw their tiles from a counter instead of round-robin (default 32, 0 = never).
 * A value that is out of range (band_mb <= 0, the others < 0) leaves that knob as it is. Results do not depend
 * on any of them. Test infrastructure like lce_debug_gemm. */
void lce_set_tuning(int band_mb, int l2_hint_mode, int dyn_waves);

/* Wait-expiry test hook (test infrastructure): every wait inside the kernels is bounded (2 s by default) and
 * unwinds with a code in the device status word when the bound is hit. This sets, on the current device, the
 * bound to limit_ns (0 = back to the default) and makes the producers announce announce_extra_bytes more on
 * a barrier than their copies deliver (0 = normal operation), so that a test can watch the bound being hit
 * with nothing left in flight: all copies land, no barrier completes, nothing traps or faults, and the
 * kernel returns. Synchronises the device. Always call it again with (0, 0) afterwards. */
int lce_debug_wait_test(unsigned long long limit_ns, unsigned announce_extra_bytes);

int lce_debug_gemm(const void* a, const void* b, float* out, int64_t M, int64_t N, int64_t K,
                   int a_mn_major, int b_mn_major, int dtype, unsigned flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HELION_LCE_H_ */
