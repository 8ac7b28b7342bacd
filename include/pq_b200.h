/* pq_b200.h -- C ABI of libpq_b200.so: the INT8 deployment hot path of PyraQuant
 * (deploy/int8_exec.py and the token gather/scatter of flux/routing.py) as hand-written
 * sm_100a CUDA.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless stated;
 *   - the return value is a pq_status (0 = PQ_OK); nothing throws, nothing prints;
 *   - no allocation, no implicit synchronisation: kernels are enqueued on `stream`
 *     (a cudaStream_t passed as void*; NULL = the legacy default stream) and the call
 *     returns at once; outputs are caller-allocated;
 *   - argument checks (null / shape / alignment / dtype) run on the host before any launch:
 *     a non-zero status means nothing was enqueued;
 *   - safe to call from any host thread; the only process-wide state is the tuning knobs of
 *     pq_set_option and a small cache of weight tensor maps guarded by a mutex.
 *
 * dtype codes: 0 = bfloat16, 1 = float16 (activations, low-rank factors, outputs).
 */
#ifndef PQ_B200_H_
#define PQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pq_status {
  PQ_OK = 0,
  PQ_ERR_NULL = 1,        /* a required pointer is NULL */
  PQ_ERR_SHAPE = 2,       /* a size is negative, zero where it may not be, or too large */
  PQ_ERR_ALIGN = 3,       /* a pointer or leading dimension breaks the stated alignment */
  PQ_ERR_DTYPE = 4,       /* unknown dtype code */
  PQ_ERR_CUDA = 5,        /* a CUDA runtime/driver call failed (see pq_last_cuda_error) */
  PQ_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up (read from a status word) */
  PQ_ERR_UNSUPPORTED = 7, /* valid arguments, but a combination this build does not implement */
  PQ_ERR_WORKSPACE = 8    /* workspace missing or too small */
} pq_status;

#define PQ_DTYPE_BF16 0
#define PQ_DTYPE_FP16 1

/* Library version (major*10000 + minor*100 + patch). */
int pq_version(void);
/* Static, human-readable text for a status code. */
const char* pq_status_str(int status);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread. */
int pq_last_cuda_error(void);

/* Internal tuning / test knobs, 0 = automatic unless stated:
 *   "quant_tpr"         threads per row of the quantisation kernel (32, 64, 128, 256);
 *   "gemm_stages"       depth of the operand ring of the single-CTA kernels;
 *   "gemm_block_n"      column tile of the single-CTA kernels (128 or 256);
 *   "gemm_pm","gemm_pn" shape of the CTA grid of the tile schedule;
 *   "gemm_max_ctas"     upper bound of CTAs (or CTA pairs x 2) launched;
 *   "gemm_epi_warps"    epilogue warps per CTA of the CTA-pair kernel: 0 = automatic (16 up to K = 1536 without a low-rank
 *                       term, where the epilogue outlasts the K loop; else 8), 8 or 16;
 *   "gemm_tma_store"    1 (default) = sixteen-warp tiles of plain calls store through shared memory + TMA, 0 = never;
 *   "gemm_pair"         0 = never use the CTA-pair kernel, 1 = automatic (default), 2 = whenever it is legal;
 *   "gemm_debug_timing" 1 = the CTA-pair kernel runs in its debug instantiation (the production kernel contains no
 *                       counters) and writes per-role cycle counters to workspace + 256 (needs ws_bytes >= 256 + 4096*64).
 *   "gemm_tail_pairs"   1 (default) = SM pairs that the rectangular pair grid leaves over take a tail region of the tile
 *                       matrix (the last row tiles of the last column round), 0 = they stay idle;
 *   "gemm_panel_mb"     CTA-pair kernel with several column rounds: megabytes of activation rows per row panel of the tile
 *                       schedule (the rows of a panel stay in L2 across the rounds); 0 = one panel over all rows;
 *   "gemm_l2_hints"     CTA-pair kernel, L2 eviction priorities: bit 0 weights evict-last, bit 1 activations evict-first,
 *                       bit 2 activations evict-last, bit 3 streaming output stores;
 *   "g32_variant"       group-32 GEMM: bit 0 = eight epilogue warps instead of sixteen; bit 1 = scalar instead of packed
 *                       fp32 operations; bit 3 = data path only (measurements; the output is meaningless).
 * Unknown keys return PQ_ERR_UNSUPPORTED.  Not part of the reference API. */
int pq_set_option(const char* key, int value);
int pq_get_option(const char* key, int* value);

/* Per-token symmetric INT8 quantisation:  s[m] = max(max_k |x[m,k]|, 1e-8) / 127,
 * q[m,k] = clamp(round_half_even(x[m,k] / s[m]), -127, 127), IEEE fp32 division.
 * Replaces quant_rows + _quant_rows_kernel (deploy/int8_exec.py:216-230, :78-101).
 * x [M,K] with row stride ldx (elements), last dim contiguous; q [M,K] contiguous; s [M].
 * Needs K % 8 == 0, ldx % 8 == 0, x and q 16-byte aligned.  M == 0 is a no-op. */
int pq_quant_rows(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                  int8_t* q, float* s, void* stream);

/* Same quantisation applied to gathered rows: row m of the output is row row_idx[m] of the
 * canvas (the active-leaf + halo token rows of build_patch_buckets, flux/routing.py:253-315,
 * fused with the quantisation of deploy/int8_exec.py:216-230).  row_idx[m] < 0 marks a padding
 * row: it is written as zeros with the scale of an all-zero row.  0 <= row_idx[m] < rows. */
int pq_gather_quant_rows(const void* canvas, int dtype, int64_t rows, int64_t K, int64_t ld,
                         const int32_t* row_idx, int64_t M, int8_t* q, float* s, void* stream);

/* Plain gather without quantisation (the copy of flux/routing.py:288-311): out[m,:] =
 * canvas[row_idx[m],:], zeros for row_idx[m] < 0.  K % 8 == 0, 16-byte aligned rows. */
int pq_gather_rows(const void* canvas, int dtype, int64_t rows, int64_t K, int64_t ld,
                   const int32_t* row_idx, int64_t M, void* out, int64_t ldo, void* stream);

/* Group-32 variant: one scale per 32 consecutive input channels,
 * s[m,g] = max(max_{k in g} |x|, 1e-8) / 127  (ExtActQuant "dyn_group",
 * pyraquant/external_quant.py:104-109 with group 32, 8 bits, signed).  s is [M, K/32]. K % 32 == 0. */
int pq_quant_rows_g32(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                      int8_t* q, float* s, void* stream);

/* adaLN prologue fused into the per-token quantisation (no counterpart kernel in the reference, which runs
 * LayerNorm, multiply, add and the Linear's quantisation as four kernels):
 *   z[m,:] = LayerNorm(x[m,:]) * (1 + scale[b,:]) + shift[b,:],  b = m / rows_per_sample (0 when rows_per_sample == 0),
 *   (q, s) = pq_quant_rows(z),
 * the input of the feed-forward's first Linear in the FLUX blocks (flux/transformer_flux.py:195 `norm2 =
 * nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)`, :236-239).  LayerNorm without affine parameters, row
 * statistics in fp32; every step rounds to the activation type where the reference's 16-bit tensors round.
 *   x [M,K] row stride ldx; scale, shift [samples, K] row stride ld_mod, same dtype as x;
 *   x_mod: NULL, or [M,K] (row stride ldxm) that receives z (the low-rank down-projection reads it);
 *   K % 8 == 0, K <= 16384, strides % 8 == 0, 16-byte aligned x, scale, shift, x_mod. */
int pq_adaln_quant_rows(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                        const void* scale, const void* shift, int64_t ld_mod, int64_t rows_per_sample, float eps,
                        void* x_mod, int64_t ldxm, int8_t* q, float* s, void* stream);

/* Dequantisation of materialised accumulators: out[m,n] = float(acc[m,n]) * (s_row[m] * s_col[n])
 * (+ bias[n]) rounded to out_dtype.  Replaces dequant_epilogue / _dequant_epilogue_kernel
 * (deploy/int8_exec.py:233-243, :104-127); kept for API parity, the fused GEMM never needs it.
 * acc int32 [M,N] contiguous, out [M,N] contiguous. */
int pq_dequant_epilogue(const int32_t* acc, const float* s_row, const float* s_col, const float* bias,
                        void* out, int out_dtype, int64_t M, int64_t N, void* stream);

/* Fused INT8 GEMM:  out[m,n] = float(sum_k xq[m,k] * w[n,k]) * (s_row[m] * s_col[n])
 *                              (+ sum_r t[m,r] * lb[r,n])  (+ bias[n]),  rounded to out_dtype.
 * Replaces int8_gemm_fused / _int8_gemm_fused_kernel_impl (deploy/int8_exec.py:202-212, :144-183)
 * and, with t/lb given, int8_gemm_lr / _int8_gemm_lr_impl (:327-336, :272-314); same operation
 * order as :303-309.  tcgen05 kind::i8 with int32 accumulators in tensor memory.
 *   xq [M,K] int8 row stride ldx;  w [N,K] int8 row stride ldw;  both K-contiguous, 16-byte aligned
 *   bases, ldx % 16 == 0, ldw % 16 == 0, K % 16 == 0;
 *   s_row [M], s_col [N], bias [N] or NULL: fp32;
 *   t [M,R] (row stride ldt) and lb [R,N] (row stride ldb) in lr_dtype, both NULL or both set,
 *   R == 32 (the reference's rank) when set;
 *   lb_t: NULL, or the transpose of lb as a contiguous [N,R] matrix (16-byte aligned).  With it the rank-32
 *   term is computed by tcgen05.mma kind::f16 on the tensor cores; without it by warp-level mma.sync in the
 *   epilogue, which is markedly slower for small K.  Same result up to fp32 summation order;
 *   out [M,N] row stride ldo in out_dtype;
 *   dbg_acc: NULL, or int32 [M,N] contiguous that receives the raw accumulators (tests);
 *   workspace: NULL or >= PQ_GEMM_WORKSPACE_BYTES device bytes; word 0 is a status word that the
 *   kernel sets non-zero if a bounded wait gave up (read it with pq_read_status_word).
 * M == 0 is a no-op. */
#define PQ_GEMM_WORKSPACE_BYTES 256
int pq_int8_gemm(const int8_t* xq, int64_t ldx, const float* s_row,
                 const int8_t* w, int64_t ldw, const float* s_col, const float* bias,
                 const void* t, int64_t ldt, const void* lb, int64_t ldb, const void* lb_t, int R, int lr_dtype,
                 void* out, int out_dtype, int64_t ldo,
                 int64_t M, int64_t N, int64_t K,
                 void* workspace, size_t ws_bytes, int32_t* dbg_acc, void* stream);

/* pq_int8_gemm with a variant epilogue (no counterpart in the reference, whose callers run these as separate
 * elementwise kernels after the Linear).  `epilogue` is a combination of
 *   PQ_EPI_ACCUMULATE  out = round(out + round(y)): the second half of a Linear split along its inputs
 *                      (SplitInLinear.forward, pyraquant/external_quant.py:191-192) adds onto the first half's output;
 *   PQ_EPI_GELU_TANH   out = round(gelu_tanh(round(y))): the tanh-form GELU that follows proj_mlp
 *                      (flux/transformer_flux.py:135), tanh by the hardware approximation;
 * (activation first when both are set).  y is the pq_int8_gemm result before rounding, round() rounds to out_dtype.
 * Needs the CTA-pair kernel: lb_t given when t is, N % 32 == 0, ldo % 8 == 0, out 16-byte aligned; otherwise
 * PQ_ERR_UNSUPPORTED and nothing is launched.  epilogue == 0 is pq_int8_gemm. */
#define PQ_EPI_ACCUMULATE 1
#define PQ_EPI_GELU_TANH 2
#define PQ_EPI_GATE 4          /* set by pq_int8_gemm_gated; not accepted by pq_int8_gemm_ex */
int pq_int8_gemm_ex(const int8_t* xq, int64_t ldx, const float* s_row,
                    const int8_t* w, int64_t ldw, const float* s_col, const float* bias,
                    const void* t, int64_t ldt, const void* lb, int64_t ldb, const void* lb_t, int R, int lr_dtype,
                    void* out, int out_dtype, int64_t ldo,
                    int64_t M, int64_t N, int64_t K, int epilogue,
                    void* workspace, size_t ws_bytes, void* stream);

/* Tail of a FLUX block in the Linear's epilogue (no counterpart kernel in the reference, which runs a multiply and an
 * add after the Linear): with PQ_EPI_ACCUMULATE,
 *   out[m,n] = round(out[m,n] + round(gate[b,n] * round(y[m,n]))),   b = m / rows_per_sample (0 when that is 0),
 * i.e. `residual + gate.unsqueeze(1) * proj_out(x)` with the residual stream in `out`, updated in place
 * (flux/transformer_flux.py:145-149 for the single-stream blocks; :224-225, :240-242 for attention and feed-forward
 * outputs of the double-stream blocks).  Every step rounds to out_dtype where the reference's 16-bit tensors round; fp16
 * sums are clipped to +-65504 as the block does.  Without PQ_EPI_ACCUMULATE the product alone is stored.
 * gate [samples, N] in out_dtype, row stride ld_gate (% 8 == 0, >= N), 16-byte aligned.  Other rules as pq_int8_gemm_ex. */
int pq_int8_gemm_gated(const int8_t* xq, int64_t ldx, const float* s_row,
                       const int8_t* w, int64_t ldw, const float* s_col, const float* bias,
                       const void* t, int64_t ldt, const void* lb, int64_t ldb, const void* lb_t, int R, int lr_dtype,
                       const void* gate, int64_t ld_gate, int64_t rows_per_sample,
                       void* out, int out_dtype, int64_t ldo,
                       int64_t M, int64_t N, int64_t K, int epilogue,
                       void* workspace, size_t ws_bytes, void* stream);

/* pq_int8_gemm_ex whose epilogue stores every output tile to n_out_more further buffers as well (no counterpart in
 * the reference, which runs on one GPU).  `out_more` is a HOST array of n_out_more (<= PQ_MAX_OUT_MORE) device
 * pointers; buffer d receives exactly what `out` receives, at the same offsets (same [M,N] extent, row stride ldo,
 * 16-byte aligned).  Meant for the row-sharded Linear on several GPUs of one node: `out` and out_more[d] are this
 * rank's row block inside the full output buffers of this GPU and of its peers (peer memory mapped into the process,
 * written with plain stores), so the all-gather of the outputs happens tile by tile inside the GEMM instead of after
 * it.  The call only enqueues the kernel: peers may read their buffer once this GPU's stream has passed the kernel and
 * the ranks have synchronised (the caller's job).  Same shape rules as pq_int8_gemm_ex (CTA-pair kernel, N % 32 == 0,
 * ldo % 8 == 0, 16-byte-aligned outputs, lb_t given with t); n_out_more == 0 is pq_int8_gemm_ex. */
#define PQ_MAX_OUT_MORE 7
int pq_int8_gemm_bcast(const int8_t* xq, int64_t ldx, const float* s_row,
                       const int8_t* w, int64_t ldw, const float* s_col, const float* bias,
                       const void* t, int64_t ldt, const void* lb, int64_t ldb, const void* lb_t, int R, int lr_dtype,
                       void* out, void* const* out_more, int n_out_more, int out_dtype, int64_t ldo,
                       int64_t M, int64_t N, int64_t K, int epilogue,
                       void* workspace, size_t ws_bytes, void* stream);

/* Routed two-tier GEMM (the per-leaf precision routing of flux/run_flux.py:117-123 collapsed to a
 * hard choice at the Linear): rows [0, M_hi) use weight set 0 (the INT8 codes), rows [M_hi, M)
 * use weight set 1 (the codes re-rounded to the nested 4-bit grid,
 * pyraquant/quantizers_weight.py:182-199, still stored as int8).  Everything else as pq_int8_gemm;
 * low-rank factors and bias are shared by both tiers. */
int pq_int8_gemm_grouped(const int8_t* xq, int64_t ldx, const float* s_row,
                         const int8_t* w_hi, const float* s_col_hi,
                         const int8_t* w_lo, const float* s_col_lo, int64_t ldw,
                         const float* bias,
                         const void* t, int64_t ldt, const void* lb, int64_t ldb, const void* lb_t, int R,
                         int lr_dtype, void* out, int out_dtype, int64_t ldo,
                         int64_t M_hi, int64_t M, int64_t N, int64_t K,
                         void* workspace, size_t ws_bytes, void* stream);

/* Group-32 W8A8 GEMM (SDXL round-to-nearest arm):
 *   out[m,n] = sum_g s_a[m,g] * s_w[g,n] * (sum_{k in group g} xq[m,k] * w[n,k])  (+ bias[n])
 * with the weight grid of qdq_weight(w, 8, 32) (pyraquant/quantizers_weight.py:96-109) and the
 * activation grid of pq_quant_rows_g32 (pyraquant/external_quant.py:104-109).  Per-group int32 partial
 * sums are exact; the fp32 combination runs in ascending group order as
 * sum = fma(float(partial), s_a * s_w, sum).  No counterpart kernel exists in the reference (its
 * SDXL deployment arm is per-channel; the group-32 grid is only simulated there).
 *   s_a [M, K/32] fp32 contiguous (as written by pq_quant_rows_g32);
 *   s_w [K/32, N] fp32 contiguous (group-major: the transpose of the [N, K/32] scale table);
 *   K % 128 == 0, N % 4 == 0, ldx % 16 == 0, ldw % 16 == 0, 16-byte aligned xq, w, s_a, s_w. */
int pq_int8_gemm_g32(const int8_t* xq, int64_t ldx, const float* s_a,
                     const int8_t* w, int64_t ldw, const float* s_w, const float* bias,
                     void* out, int out_dtype, int64_t ldo,
                     int64_t M, int64_t N, int64_t K,
                     void* workspace, size_t ws_bytes, void* stream);

/* Down-projection of the rank-32 branch: t[m, 0:R] = round(sum_k x[m,k] * A[k, 0:R]), fp32 accumulation on the
 * tensor cores, result rounded to `dtype`.  Replaces `x2.to(lr_A.dtype) @ lr_A` (deploy/int8_exec.py:390), a torch
 * matmul in the reference; same value up to fp32 summation order.  R = 32 for one layer; 64, 96 or 128 when the
 * factors of layers that read the same input stand side by side (x is then read once for all of them).  A is passed
 * transposed: a_t [R, K] with row stride lda (K-contiguous).  x [M, K] row stride ldx, t [M, R] row stride ldt, all
 * in `dtype`; K % 8 == 0, ldx % 8 == 0, lda % 8 == 0, ldt % 8 == 0, 16-byte aligned bases.  workspace as for
 * pq_int8_gemm (status word).  PQ_ERR_UNSUPPORTED for any other R. */
int pq_lowrank_down(const void* x, int dtype, int64_t ldx, const void* a_t, int64_t lda, int R, void* t, int64_t ldt,
                    int64_t M, int64_t K, void* workspace, size_t ws_bytes, void* stream);

/* pq_quant_rows and pq_lowrank_down on an input that is the concatenation of two tensors along K,
 *   x[m, :] = [x0[m, 0:K0] | x1[m, 0:K1]],
 * without materialising it: `proj_out(torch.cat([attn_output, mlp_hidden_states], dim=2))` of the single-stream FLUX
 * blocks (flux/transformer_flux.py:143-145) reads its two sources in place.  Results are those of the plain entry points on
 * the concatenated tensor, bit for bit.  K0 % 8 == 0, K1 % 8 == 0, K0 + K1 <= 16384 for the quantisation; K0 % 64 == 0
 * for the down-projection; row strides % 8 == 0; 16-byte aligned bases.  No counterpart in the reference. */
int pq_quant_rows_cat(const void* x0, int64_t K0, int64_t ldx0, const void* x1, int64_t K1, int64_t ldx1,
                      int dtype, int64_t M, int8_t* q, float* s, void* stream);
int pq_lowrank_down_cat(const void* x0, int64_t K0, int64_t ldx0, const void* x1, int64_t K1, int64_t ldx1,
                        int dtype, const void* a_t, int64_t lda, int R, void* t, int64_t ldt, int64_t M,
                        void* workspace, size_t ws_bytes, void* stream);

/* Low-tier weights at rest in 4 bits: expands packed nested-4-bit codes (pyraquant/quantizers_weight.py:182-199;
 * the reference keeps this tier for storage/BOPs accounting only, deploy/run_flux_latency.py:16-18) to the int8
 * operand the GEMMs read.  Byte b of row n holds element 2b in its low nibble and element 2b+1 in its high nibble,
 * two's complement.  packed [N, K/2] row stride ldp bytes, out [N, K] row stride ldo; K % 32 == 0, ldp % 16 == 0,
 * ldo % 16 == 0, 16-byte aligned bases.  No counterpart in the reference. */
int pq_unpack_int4(const uint8_t* packed, int64_t ldp, int8_t* out, int64_t ldo, int64_t N, int64_t K, void* stream);

/* Feathered scatter of routed rows back over the cached canvas, in place: the pull form of
 * fuse_patch_predictions (flux/routing.py:328-379).  For canvas token j with contributor list
 * e in [ptr[j], ptr[j+1]):  local = sum_e beta[e] * y[src[e], :], bsum = sum_e beta[e] (both
 * accumulated in the canvas dtype, in list order, like the reference's bf16 accumulators), then
 *   canvas[j] = (1 - clamp(bsum,0,1)) * canvas[j] + clamp(bsum,0,1) * (local / max(bsum, 1e-8)).
 * Every intermediate is rounded to the canvas dtype where the reference's 16-bit tensors round (bit-identical
 * results for finite data).  A token whose factor 1 - clamp(bsum,0,1) rounds to zero takes nothing from the canvas and
 * its old row is not read (0 * b + u == u for every finite b; an Inf/NaN already on the canvas under such a token does
 * not propagate, unlike in the reference's formula).
 * Tokens without contributors are left untouched.  `tokens` is the list of canvas rows that have
 * at least one contributor (n_tokens of them); ptr has n_tokens + 1 entries and indexes src/beta.
 * y [M_act, C] row stride ldy; canvas [rows, C] row stride ldc.  C % 8 == 0, 16-byte aligned. */
int pq_scatter_rows(const void* y, int64_t ldy, int64_t M_act,
                    const int32_t* tokens, const int32_t* ptr, const int32_t* src, const float* beta,
                    int64_t n_tokens, void* canvas, int64_t ldc, int64_t rows, int64_t C,
                    int dtype, void* stream);

/* Linear forward for callers that cannot allocate device memory (no counterpart in the reference, which
 * allocates its intermediates with torch.empty on every call):
 *   out = fused_gemm(quant_rows(x), w, s_col, bias)      -- Int8Linear without a low-rank branch.
 * Some callers may not call cudaMalloc at all: a server that gave all device memory to its own pool, code inside
 * a stream capture, a plugin with a fixed memory budget.  They still need somewhere to put the int8 codes and
 * row scales that exist only between the two kernels; here that place is a fixed __device__ array inside the
 * library (pq_noalloc_scratch_bytes() bytes, about 16 MiB, held on every GPU that loads the library until the
 * process exits).  The call performs no cudaMalloc/cudaFree and uses no allocating library routine.
 * Limits: M <= PQ_NOALLOC_MAX_ROWS and M * K <= PQ_NOALLOC_MAX_CODE_BYTES, else PQ_ERR_WORKSPACE; otherwise
 * the rules of pq_quant_rows and pq_int8_gemm apply (x and out in `dtype`).
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current): make that first call before starting any stream capture.
 * All calls share the one array: two calls whose kernels can overlap on the GPU (different streams, or
 * different host threads on different streams) race on it -- serialise them.  *status_word (optional)
 * receives the device address whose first word the GEMM sets if a bounded wait gives up; it is cleared at the
 * start of every call and can be read with pq_read_status_word. */
#define PQ_NOALLOC_MAX_ROWS 16384
#define PQ_NOALLOC_MAX_CODE_BYTES (16u * 1024u * 1024u)
size_t pq_noalloc_scratch_bytes(void);
int pq_int8_linear_noalloc(const void* x, int dtype, int64_t ldx,
                           const int8_t* w, int64_t ldw, const float* s_col, const float* bias,
                           void* out, int64_t ldo, int64_t M, int64_t N, int64_t K,
                           void** status_word, void* stream);

/* Copies the workspace status word to the host after synchronising `stream` and maps it to a
 * pq_status (PQ_OK or PQ_ERR_TIMEOUT); *raw receives the word itself (role and barrier that gave
 * up) when raw != NULL.  The word is cleared when `clear` is non-zero. */
int pq_read_status_word(void* workspace, int32_t* raw, int clear, void* stream);

/* Diagnostic for the bounded waits (no counterpart in the reference): launches one warp in which a thread waits,
 * through the same bounded wait the GEMM roles use, on a barrier that nothing ever completes.  After `budget_us`
 * microseconds (1 .. 100000) the wait gives up, the kernel writes the status word (role 5) and returns normally; the
 * context stays usable.  pq_read_status_word then reports PQ_ERR_TIMEOUT.  Shows the path from a wait that runs out
 * to the host-visible error without a GPU fault, trap or endless loop. */
int pq_wait_probe(void* workspace, size_t ws_bytes, int budget_us, void* stream);

/* Tensor-pipe ceiling probe: every CTA issues `iters` tcgen05.mma kind::i8 128x256x32 instructions
 * on shared-memory operands with no global traffic and writes elapsed clock cycles per CTA to
 * cycles[ctas] (int64).  The operands are all ones; a negative `iters` runs |iters| iterations on pseudo-random
 * operand bytes instead (tensor-core power, and with it the clock the GPU holds, depends on the data).  Used by the
 * benchmark for the measured INT8 ceiling. */
int pq_i8_mma_issue_loop(int ctas, int iters, long long* cycles, void* workspace, size_t ws_bytes,
                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PQ_B200_H_ */
