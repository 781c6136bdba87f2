/*
 * lookupffn.h -- C ABI of liblookupffn.so, the sm_100a implementation of the
 * LookupFFN layer's hot path (hash projection -> codes/weights -> weighted
 * gather-add, and the gather's backward).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller unless the name ends
 *     in _host; nothing is allocated behind the caller's back unless a function
 *     says so; buffers are dense row-major.
 *   - every function returns LFFN_OK (0) or a negative LFFN_ERR_* code and never
 *     aborts; lffn_last_error_string() gives the message for the calling thread.
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) and is asynchronous unless stated otherwise.
 *   - paths below are relative to src/roberta/models/prenorm_lookup/ of
 *     mlpen/LookupFFN; each entry point names the reference interface it replaces.
 */
#ifndef LOOKUPFFN_H_
#define LOOKUPFFN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LFFN_VERSION 100

#define LFFN_OK 0
#define LFFN_ERR_INVALID_ARG (-1) /* null pointer, non-positive size, bad enum            */
#define LFFN_ERR_UNSUPPORTED (-2) /* a shape the kernels do not cover (message says which) */
#define LFFN_ERR_CUDA (-3)        /* a CUDA runtime call or launch failed                  */
#define LFFN_ERR_INDEX_RANGE (-4) /* device status word reports an index outside [0, S)   */
#define LFFN_ERR_SCRATCH (-5)     /* scratch buffer missing or too small                   */

/* storage types */
#define LFFN_F32 0
#define LFFN_BF16 1

/* bit order of a code: MSB first is the reference (compute_code_score/kernel.py:32-34,
 * torch_extension.cc:35); LSB first is code = sum_j [v_j > 0] << j. */
#define LFFN_BIT_MSB_FIRST 0
#define LFFN_BIT_LSB_FIRST 1

/* how gather weights are derived from the projection z[t, 0..k) */
#define LFFN_WEIGHT_SCORE 0     /* sum|z| / prod(1 + exp(-2|z|))  (compute_code_score/kernel.py:51-53) */
#define LFFN_WEIGHT_ONES 1      /* 1                                                                   */
#define LFFN_WEIGHT_SOFT_FLIP 2 /* k+1 candidates per table: hard code and its k single-bit flips,
                                   weights prod_j sigma(|z_j|/tau) with factor j replaced by
                                   1 - sigma(|z_j|/tau) for flip j                                    */

/* bits of the device status word (lffn_device_status) */
#define LFFN_STATUS_INDEX_RANGE 1u /* a gather/scatter index was outside [0, S); the row was skipped */
#define LFFN_STATUS_STRUCTURE 2u   /* an index left its table's row range in the sorted backward     */
#define LFFN_STATUS_TIMEOUT 4u     /* a bounded wait inside a kernel ran out; that launch's outputs are incomplete */

typedef void *lffn_stream_t;

/*
 * Description of the hashing stage = modules BH4 + Hashing (lookup.py:10-77) with the
 * CUDA/training semantics of bh4_cuda (bh4/kernel.py:23-36):
 *   u      = x zero-padded from d_in to D columns (D a power of two, 64 <= D <= 2048)
 *   y_r    = u; repeat S times { y_r <- blockdiag(w[r, j]) y_r ; y_r <- H_D y_r * had_scale }
 *   z      = fl(fl(mix_a * concat_r y_r) + fl(mix_b * tile(u, R)))[:, :T*k] + proj_bias
 *   codes and weights from z viewed as [T, k]
 * proj_w is [R, S, D/BS, BS, BS] fp32.  BS = 1 is a diagonal (random +-1 entries give
 * H diag(s2) H diag(s1) x for S = 2); BS = 64, S = 4, mix 0.7/0.3, had_scale 1 is the reference.
 * transpose_w = 0 multiplies by w[nb][o][i] ("bni,noi->bno", bh4/kernel.py:32), 1 by w[nb][i][o]
 * (the convention of the reference's CPU extension, bh4/cpu/kernel.py:91).
 * H is the unnormalised Sylvester matrix; butterflies run from stride D/2 down to 1, the order
 * of bh4/fast_hadamard_transform/extension/cuda_kernel.cu:234-252, so sign bits reproduce.
 */
typedef struct lffn_hash_desc {
    int32_t d_in;
    int32_t D;
    int32_t BS;
    int32_t S;
    int32_t R;
    int32_t transpose_w;
    float had_scale;
    float mix_a;
    float mix_b;
    int32_t T; /* number of tables of the whole layer */
    int32_t k; /* code length, table has 2^k rows, 1 <= k <= 16 */
    int32_t bit_order;
    int32_t weight_mode;
    float tau;
    const float *proj_w;
    const float *proj_bias; /* [T*k] or NULL */
} lffn_hash_desc;

int lffn_version(void);
const char *lffn_last_error_string(void);

/*
 * Tracing, off by default (the reference carries per-stage wall-clock timers around projection, code/score and
 * gather, commented out: lookup.py:67-75,103-106).
 *   LFFN_TRACE_NVTX         every entry point brackets its host-side work with an NVTX range named after it, so
 *                           a timeline tool shows which call enqueued which kernels
 *   LFFN_TRACE_STAGE_TIMES  lffn_layer_fwd / lffn_layer_fwd_ln_residual record CUDA events before the hash kernel,
 *                           between the two kernels and after the gather; lffn_trace_last_layer_times waits for
 *                           the last such call on the current device and returns the two durations in ms
 * The flags are process-wide.  With stage times on, whole-layer calls on one device should come from one stream at
 * a time (the events are per device); lffn_layer_fwd_host issues many such calls and leaves the last chunk's times.
 */
#define LFFN_TRACE_NVTX 1u
#define LFFN_TRACE_STAGE_TIMES 2u
int lffn_trace_configure(uint32_t flags);
int lffn_trace_last_layer_times(float *hash_ms, float *gather_ms);

/* Reads and clears the status word of the current device with one atomic exchange on `stream`, then
 * synchronises `stream`.  A flag raised concurrently by a kernel on another stream is never lost: it is either in
 * this value or in the next one. */
int lffn_device_status(uint32_t *status_out, lffn_stream_t stream);

/*
 * Self-test of the kernels' bounded waits (no reference counterpart).  Launches one tiny kernel whose only wait is
 * on a barrier nobody will ever signal, with `poll_limit` polls (1 .. 2^20); the wait gives up, the kernel sets
 * LFFN_STATUS_TIMEOUT in the device status word and ends normally.  Shows that a wait that runs out surfaces as a
 * status bit and leaves the device usable.  No memory is touched and nothing else is in flight.
 */
int lffn_selftest_bounded_wait(int32_t poll_limit, lffn_stream_t stream);

/*
 * Measurement probe (no reference counterpart; not on the layer's path): reads the bytes at `buf` `repeats`
 * times with the gather kernel's kind of access -- coalesced 16-byte read-only loads that bypass L1 -- and nothing
 * else in the loop.  With a buffer that fits L2 and several repeats, bytes read / elapsed time is an L2 read
 * bandwidth.  How much an SM keeps in flight decides the rate, so there are four configurations: mode 0 = 12 loads
 * per thread at the gather kernel's own residency (4 CTAs of 128 threads per SM); modes 1, 2, 3 = 8, 16, 4 loads
 * per thread with as many CTAs per SM as fit.  The benchmark quotes the gather against the best of them.  A launch
 * reads the largest whole number of grid-wide slabs that fits in `bytes`; *bytes_read_per_repeat (host pointer, may
 * be NULL) receives that amount.  `sink` is one device word that keeps the loads observable (practically never
 * written).
 */
int lffn_probe_read(const void *buf, size_t bytes, int32_t repeats, int32_t mode, uint32_t *sink,
                    size_t *bytes_read_per_repeat, lffn_stream_t stream);

/*
 * Walsh-Hadamard transform of each row, out = x H_D * scale.  Replaces
 * fast_hadamard_transform_kernel.fast_hadamard_transform(inp)
 * (bh4/fast_hadamard_transform/extension/torch_extension.cpp:5-32, kernel.py:39-44,78-89).
 * x, out: [N, D] of `dtype` (LFFN_F32 or LFFN_BF16, arithmetic in fp32); in place allowed.
 */
int lffn_fwht(const void *x, void *out, int64_t N, int32_t D, int32_t dtype, float scale, lffn_stream_t stream);

/*
 * Hashing stage for tables [t_begin, t_begin + t_count): replaces
 * Hashing.forward = BH4.forward + compute_code_score (lookup.py:64-77, bh4/kernel.py:10-36,
 * compute_code_score/kernel.py:22-55) plus the table offsets of LookupFFN.gather (lookup.py:126).
 *   x        [N, d_in] of x_dtype
 *   idx_out  int32 [N, t_count*m]  row index = code + (t - t_begin) * 2^k  (m = 1, or k+1 for SOFT_FLIP)
 *   w_out    fp32  [N, t_count*m]
 *   z_out    fp32  [N, t_count*k] or NULL: the projected coordinates, for diagnostics and backward
 * idx_out and w_out may both be NULL when only z_out is wanted (the projection alone = bh4(x, w),
 * bh4/kernel.py:10-21, with mix_a = 1, mix_b = 0, no bias, k = 1, T = R*D).
 */
int lffn_hash_fwd(const lffn_hash_desc *desc, const void *x, int32_t x_dtype, int64_t N, int32_t t_begin,
                  int32_t t_count, int32_t *idx_out, float *w_out, float *z_out, lffn_stream_t stream);

/*
 * The same with the module's LayerNorm (lookup.py:84,99: nn.LayerNorm(hidden_size, eps) applied before the hash)
 * done inside the kernel's load of x: u = (x - mean) * rstd * ln_gamma + ln_beta over the d_in columns, biased
 * variance, eps inside the square root, fp32 arithmetic.  ln_gamma [d_in] fp32 (NULL: no LayerNorm, i.e.
 * lffn_hash_fwd), ln_beta [d_in] fp32 or NULL.  Saves the [N, d_in] round trip of a separate LayerNorm kernel.
 */
int lffn_hash_fwd_ln(const lffn_hash_desc *desc, const float *ln_gamma, const float *ln_beta, float ln_eps,
                     const void *x, int32_t x_dtype, int64_t N, int32_t t_begin, int32_t t_count, int32_t *idx_out,
                     float *w_out, float *z_out, lffn_stream_t stream);

/*
 * Codes and weights from already projected coordinates z [N, T, k] fp32: replaces
 * compute_code_score(hash_scores, training) (compute_code_score/kernel.py:22-30) and
 * ccs_cpu.compute_code_score (torch_extension.cc:14-42).  add_offsets adds t * 2^k (lookup.py:126).
 */
int lffn_code_weights(const float *z, int64_t N, int32_t T, int32_t k, int32_t bit_order, int32_t weight_mode,
                      float tau, int32_t add_offsets, int32_t *idx_out, float *w_out, lffn_stream_t stream);

/*
 * Gradient of those weights with respect to z: dz [N, T, k] from dw [N, T*m].  Replaces what autograd derives
 * from compute_code_score_torch (compute_code_score/kernel.py:43-55); the codes carry no gradient.
 */
int lffn_code_weights_bwd(const float *z, const float *dw, int64_t N, int32_t T, int32_t k, int32_t weight_mode,
                          float tau, float *dz, lffn_stream_t stream);

/*
 * Backward pass of the block-diagonal projection z = BH4(x) for training: what autograd derives from bh4_cuda's
 * chain of torch.einsum("bni,noi->bno") and Hadamard transforms (bh4/kernel.py:23-36; the transform's backward is
 * the transform, bh4/fast_hadamard_transform/kernel.py:47-54) and from the mix / slice / bias of lookup.py:29-39.
 *   desc       the projection as for lffn_hash_fwd with T*k = the number of output columns of z, BS = 64,
 *              D in {256, 512, 1024}, transpose_w = 1 and desc->proj_w the weights in [R, S, D/64, i, o] order
 *              (the copy the forward fast path uses); desc->proj_bias is not read
 *   proj_w_oi  the same weights in the parameter's own order [R, S, D/64, o, i]
 *   x          [N, d_in] of x_dtype, the input of the forward call;   dz  fp32 [N, T*k], the upstream gradient
 *   du         fp32 [N, D]: gradient with respect to the zero-padded input (its first d_in columns are dx), or NULL
 *   dw         fp32 [R, S, D/64, 64, 64] in the parameter's order, or NULL;   dbias  fp32 [T*k], or NULL
 *   saved_acts the stage inputs kept by lffn_proj_fwd_train for the same x, or NULL: they are then recomputed
 *   ws         workspace of lffn_proj_bwd_ws_bytes(desc, N) bytes, 256-byte aligned
 * fp32 fused multiply-adds throughout, no atomics: results are the same from run to run.
 *
 * lffn_proj_fwd_train is the forward pass for training: z [N, T*k] (= lffn_hash_fwd with z_out only, desc->proj_bias
 * added) and, in `acts` (lffn_proj_acts_bytes(desc, N) bytes: R * S * ceil(N/32) tiles of [D][32] fp32), the input of
 * every stage, which is what autograd keeps for the reference's einsum chain.  Handing them to lffn_proj_bwd saves
 * the recomputation (about a tenth of a training step of the layer) at the price of that memory.
 */
size_t lffn_proj_bwd_ws_bytes(const lffn_hash_desc *desc, int64_t N);
size_t lffn_proj_acts_bytes(const lffn_hash_desc *desc, int64_t N);
int lffn_proj_fwd_train(const lffn_hash_desc *desc, const void *x, int32_t x_dtype, int64_t N, float *z, float *acts,
                        size_t acts_bytes, lffn_stream_t stream);
int lffn_proj_bwd(const lffn_hash_desc *desc, const float *proj_w_oi, const void *x, int32_t x_dtype, int64_t N,
                  const float *dz, float *du, float *dw, float *dbias, const float *saved_acts, void *ws,
                  size_t ws_bytes, lffn_stream_t stream);

/*
 * Backward of the layer's LayerNorm (lookup.py:84,99: torch.nn.LayerNorm over the hidden dimension; in the reference
 * autograd's native_layer_norm_backward): x, du, dx fp32 [N, d]; gamma, dgamma, dbeta fp32 [d]; d in {256, 512, 768,
 * 1024}.  The statistics are recomputed from x.  Deterministic (partial column sums added in a fixed order).
 * ws: lffn_layernorm_bwd_ws_bytes(d) bytes of device scratch.
 */
size_t lffn_layernorm_bwd_ws_bytes(int32_t d);
/* dbias[c] = sum_n dy[n, c]: gradient of the `outputs + self.bias` of lookup.py:108 (autograd's sum in the reference);
 * dy fp32 [N, cols]; deterministic.  ws: lffn_bias_grad_ws_bytes(cols) bytes of device scratch. */
size_t lffn_bias_grad_ws_bytes(int32_t cols);
int lffn_bias_grad(const float *dy, int64_t N, int32_t cols, float *dbias, void *ws, size_t ws_bytes, lffn_stream_t stream);
int lffn_layernorm_bwd(const float *x, const float *du, const float *gamma, int64_t N, int32_t d, float eps, float *dx,
                       float *dgamma, float *dbeta, void *ws, size_t ws_bytes, lffn_stream_t stream);

/*
 * out[n, :] = sum_i w[n, i] * tables[idx[n, i], :] (+ bias): replaces
 * gather_add.weighted_vector_gather_add_fp32/_fp16 (gather/cuda/extension/torch_extension.cpp:6-33,
 * gather/cuda/kernel.py:22-70) and gather_add_cpu.weighted_vector_gather_add_* (gather/cpu/
 * torch_extension.cpp:17-96), with `+ bias` of lookup.py:108 folded in.
 *   idx int32 [N, I], w fp32 [N, I], tables [S, d] of table_dtype, out [N, d] of out_dtype.
 * d must be a multiple of 4 (fp32 tables) or 8 (bf16 tables).  out need not be zeroed.
 * Accumulation is fp32, one fused multiply-add per row in index order.  Indices outside [0, S)
 * are skipped and flagged in the device status word.
 */
int lffn_gather_fwd(const int32_t *idx, const float *w, const void *tables, int32_t table_dtype, void *out,
                    int32_t out_dtype, int64_t N, int32_t I, int64_t S, int32_t d, const float *bias,
                    lffn_stream_t stream);

/*
 * The same with the caller's residual connection folded into the epilogue: out = fl(fl(sum + bias) + residual),
 * the `self.dropout(self.FFN(attn_output)) + attn_output` of EncoderLayer.forward (layer.py:75-78) in inference
 * (dropout is the identity there).  residual [N, d] of out_dtype, or NULL; it may be `out` itself (in place).
 */
int lffn_gather_fwd_residual(const int32_t *idx, const float *w, const void *tables, int32_t table_dtype, void *out,
                             int32_t out_dtype, int64_t N, int32_t I, int64_t S, int32_t d, const float *bias,
                             const void *residual, lffn_stream_t stream);

/*
 * Gather fused with the reduce-scatter of the table-sharded mode (no reference counterpart: the reference is
 * data-parallel only).  Every rank calls it with its own tables and index lists for ALL N tokens; the row of
 * token n goes to the rank that owns it, n / rows_per_owner, through out_ptrs, a DEVICE array of n_owners fp32
 * buffer addresses, one per rank, all mapped into this process (peer / symmetric memory over NVLink; the local
 * one included).
 *   slab = -1: buffers are [rows_per_owner, d]; the row is ADDED in place: the warp parks its fp32 row in shared
 *              memory and one bulk reduction (cp.reduce.async.bulk, f32 add) carries it to the owner.  The buffers
 *              must hold their initial value (zeros or the bias) on every rank before any rank starts; the order
 *              of summation across ranks is not fixed.
 *   slab = -2: the same in-place add, carried out with 16-byte vector reductions (red.global.add.v4.f32): many
 *              small packets instead of one large one (slower over NVLink; kept for comparison).
 *   slab >= 0: buffers are [n_owners, rows_per_owner, d]; the row is STORED into slab `slab` (the caller's rank):
 *              with plain 16-byte stores, or, when LFFN_SCATTER_SLAB_BULK is or-ed into `slab`, as one bulk copy
 *              (cp.async.bulk) from the row parked in shared memory.  The owner then sums its slabs in rank order:
 *              deterministic, and no read-modify-write on the remote side.
 * first_owner in [0, n_owners): the call walks the tokens starting with those of this owner and wraps around.
 * Ranks that run at the same time should pass different values ((rank + 1) % n_owners): then at any moment every
 * rank sends to a different owner and all NVLink ports are busy, instead of all ranks converging on one owner.
 * The result does not depend on it.
 * Either way a buffer is complete once every rank's call has finished: the caller synchronises the ranks on the
 * host; the kernel itself never waits on a peer.
 */
#define LFFN_SCATTER_SLAB_BULK 0x40000000
int lffn_gather_fwd_scatter(const int32_t *idx, const float *w, const void *tables, int32_t table_dtype,
                            float *const *out_ptrs, int32_t n_owners, int64_t rows_per_owner, int32_t slab,
                            int32_t first_owner, int64_t N, int32_t I, int64_t S, int32_t d, lffn_stream_t stream);

/*
 * dw[n, i] = <dy[n, :], tables[idx[n, i], :]>: replaces gather_add.indexed_inner_product_fp32/_fp16
 * (gather/cuda/extension/torch_extension.cpp:35-62, gather/cuda/kernel.py:72-122).
 * dy fp32 [N, d]; dw fp32 [N, I].
 */
int lffn_gather_bwd_weights(const int32_t *idx, const float *dy, const void *tables, int32_t table_dtype, float *dw,
                            int64_t N, int32_t I, int64_t S, int32_t d, lffn_stream_t stream);

/*
 * dtables[idx[n, i], :] += w[n, i] * dy[n, :] with dtables [S, d] fp32 zeroed first by this call:
 * replaces gather_add.weighted_vector_scatter_add_fp32/_fp16 (gather/cuda/extension/
 * torch_extension.cpp:64-91, gather/cuda/kernel.py:124-173).  Any index list; uses vector
 * reductions in L2, so the summation order (not the set of terms) varies between runs.
 */
int lffn_gather_bwd_tables(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N, int32_t I,
                           int64_t S, int32_t d, lffn_stream_t stream);

/*
 * Same result, deterministic and without atomics on the output, for index lists with the layer's
 * structure: I = T * m entries per token and idx[n, t*m + c] in [t * rows, (t+1) * rows).
 * Entries are counting-sorted per table into `scratch`, then every output row is summed in
 * ascending (n, c) order and written once.  lffn_gather_bwd_tables_sorted_scratch_bytes gives
 * the scratch size.  An entry outside its table's range is dropped and flagged (LFFN_STATUS_STRUCTURE).
 */
size_t lffn_gather_bwd_tables_sorted_scratch_bytes(int64_t N, int32_t T, int32_t m, int32_t rows);
int lffn_gather_bwd_tables_sorted(const int32_t *idx, const float *w, const float *dy, float *dtables, int64_t N,
                                  int32_t T, int32_t m, int32_t rows, int32_t d, void *scratch,
                                  size_t scratch_bytes, lffn_stream_t stream);

/*
 * The sorted table gradient for callers that are not allowed to allocate device memory.  (No counterpart in
 * the reference: its scatter-add needs no scratch.)  Such callers exist: a plugin running inside a host
 * that took all device memory into its own pool at start-up (cudaMalloc fails there, or is forbidden), a
 * real-time loop that must not take the allocator's lock.  They cannot hand lffn_gather_bwd_tables_sorted its scratch buffer, so
 * this variant sorts into an array compiled into the library, LFFN_STATIC_SCRATCH_BYTES (32 MiB) long; every
 * GPU that loads the library holds those bytes until the process exits.  Same arguments and bit-identical
 * result.  It calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - Limit: lffn_gather_bwd_tables_sorted_scratch_bytes(N, T, m, rows) <= LFFN_STATIC_SCRATCH_BYTES, about
 *     N*T*m <= 4.1 million entries; larger problems return LFFN_ERR_SCRATCH with the sizes in the message.
 *   - The array's 32 MiB are reserved on a device when the CUDA runtime loads the library's code there, which
 *     (with the runtime's default lazy loading) happens at the first use on that device, not when the shared
 *     library is opened: a host with a fixed pool sees free device memory drop by the size of the library image
 *     on that first use.  The first call of this function on a device also looks up the array's device address
 *     (one runtime query).  So make one warm-up call per device at start-up, outside any stream capture; every
 *     later call allocates nothing and leaves free device memory unchanged.
 *   - All calls on a device share the one array and find the previous call's bytes in it.  Nothing needs
 *     clearing (every word a call reads it has written first), but two calls whose kernels overlap on the
 *     GPU (different streams, or two host threads) race on it: serialise them.
 */
#define LFFN_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
int lffn_gather_bwd_tables_sorted_static(const int32_t *idx, const float *w, const float *dy, float *dtables,
                                         int64_t N, int32_t T, int32_t m, int32_t rows, int32_t d,
                                         lffn_stream_t stream);

/*
 * Whole layer forward on device buffers = LookupFFN._forward without LayerNorm (lookup.py:101-110):
 * hash -> gather -> + bias for tables [t_begin, t_begin + t_count) (`tables` points at the first
 * of those, [t_count * 2^k, d_out]).  idx_ws/w_ws are caller-provided workspaces of
 * N * t_count * m int32 / fp32.
 */
int lffn_layer_fwd(const lffn_hash_desc *desc, const void *x, int32_t x_dtype, int64_t N, int32_t t_begin,
                   int32_t t_count, const void *tables, int32_t table_dtype, int32_t d_out, const float *bias,
                   void *out, int32_t out_dtype, int32_t *idx_ws, float *w_ws, lffn_stream_t stream);

/*
 * The whole feed-forward block of an encoder layer in two kernels = LookupFFN.forward with its LayerNorm
 * (lookup.py:98-110) plus the caller's residual add (layer.py:75-78, inference): LayerNorm inside the hash
 * kernel's load (lffn_hash_fwd_ln), `+ bias` and `+ residual` inside the gather's epilogue
 * (lffn_gather_fwd_residual).  ln_gamma NULL: no LayerNorm; residual NULL: no residual add.
 */
int lffn_layer_fwd_ln_residual(const lffn_hash_desc *desc, const float *ln_gamma, const float *ln_beta, float ln_eps,
                               const void *x, int32_t x_dtype, int64_t N, int32_t t_begin, int32_t t_count,
                               const void *tables, int32_t table_dtype, int32_t d_out, const float *bias,
                               const void *residual, void *out, int32_t out_dtype, int32_t *idx_ws, float *w_ws,
                               lffn_stream_t stream);

/*
 * The same forward for callers that hold HOST buffers (the shape of the reference's CPU
 * inference path, compare.py:23-37): x_host [N, d_in] and out_host [N, d_out] are host pointers
 * (pinned memory makes the copies asynchronous).  Tokens are cut into chunks of chunk_tokens (the first
 * two and the last two chunks half as long, to shorten the copies nothing can overlap) that three internal
 * streams take in turn, so the copy-in of later chunks and the copy-out of earlier ones overlap the kernels.  Parameters
 * (desc->proj_w, proj_bias, tables, bias) stay on the device.  `ws` is a device workspace of
 * lffn_layer_fwd_host_ws_bytes(...) bytes.  Synchronous: returns when out_host is complete.
 */
size_t lffn_layer_fwd_host_ws_bytes(const lffn_hash_desc *desc, int32_t x_dtype, int32_t out_dtype, int32_t d_out,
                                    int64_t chunk_tokens);
int lffn_layer_fwd_host(const lffn_hash_desc *desc, const void *x_host, int32_t x_dtype, int64_t N,
                        const void *tables, int32_t table_dtype, int32_t d_out, const float *bias, void *out_host,
                        int32_t out_dtype, void *ws, size_t ws_bytes, int64_t chunk_tokens, lffn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LOOKUPFFN_H_ */
