/*
 * ptj_b200.h — C ABI of the B200 (sm_100a) implementation of pre-tjax's GPT-2 training operators.
 *
 * Every entry point
 *   - takes plain device pointers, sizes and a CUDA stream handle (void* = cudaStream_t),
 *   - returns 0 (PTJ_OK) or a negative ptj_status; it never throws, never synchronises the device and,
 *     unless stated otherwise, never allocates (scratch buffers are passed in by the caller),
 *   - reads its inputs and writes only its outputs; outputs need no zero-initialisation.
 *
 * "Replaces" comments cite the operator of the reference project (file:line inside pre-tjax) whose role
 * the entry point takes. Element types: `dtype` is PTJ_F32 or PTJ_BF16 for activations; LayerNorm scale/shift,
 * biases, optimizer state and gradients of parameters are always float.
 *
 * Dropout everywhere follows the reference semantics (model_torch_func.py:98-102): in training the value is
 * multiplied by a 0/1 mask with keep probability 1-p and is NOT rescaled; in evaluation it is multiplied by 1-p.
 * Masks come from Philox4x32-10 keyed by `seed`, counter = (element index / 8, stream id): each call serves eight
 * consecutive elements with 16 bits each and an element is dropped when its 16 bits are below floor(p * 65536).
 * Forward and backward regenerate identical masks from (seed, stream id, element index) without storing them.
 *
 * Every `seed` argument (including ptj_dropout_args.seed) is either the seed itself, a value below 2^63, or, with
 * bit 63 set, the device address (in the low 63 bits) of a uint64_t that holds the seed when the kernel runs: see
 * PTJ_SEED_AT. The second form is for callers that record the launches of a training step once (a CUDA graph) and
 * replay them: they rewrite the seed words in device memory between replays instead of re-issuing the launches.
 */
#ifndef PTJ_B200_H_
#define PTJ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  PTJ_OK = 0,
  PTJ_ERR_BAD_SHAPE = -1,   /* a size is non-positive, too large, or violates a divisibility rule      */
  PTJ_ERR_MISALIGNED = -2,  /* a pointer or leading dimension breaks the stated alignment              */
  PTJ_ERR_DTYPE = -3,       /* dtype is not supported by this entry point                              */
  PTJ_ERR_LAUNCH = -4,      /* the CUDA launch (or a driver call preparing it) reported an error       */
  PTJ_ERR_WORKSPACE = -5,   /* the scratch buffer passed in is too small or NULL                       */
  PTJ_ERR_UNSUPPORTED = -6, /* combination of options not implemented                                  */
  PTJ_ERR_DEVICE = -7,      /* current device is not an sm_100 part / driver entry point missing       */
  PTJ_ERR_TIMEOUT = -8,     /* a bounded wait inside a kernel ran out (reported via ptj_last_kernel_fault) */
  PTJ_ERR_TOO_LARGE = -9    /* a size exceeds the fixed capacity of a no-allocation entry point            */
} ptj_status;

enum { PTJ_F32 = 0, PTJ_BF16 = 1 };

/* seed argument that makes a kernel read its seed from the device word at `dev_ptr` (8-byte aligned) */
#define PTJ_SEED_AT(dev_ptr) ((uint64_t)(uintptr_t)(dev_ptr) | ((uint64_t)1 << 63))

/* ---- library ---------------------------------------------------------------------------------------- */
int ptj_version(void);
const char* ptj_status_string(int status);
/* PTJ_OK when the current device has compute capability 10.x, else PTJ_ERR_DEVICE. */
int ptj_device_check(void);
/* Number of kernels this library has launched since load (all entry points, all threads). */
int64_t ptj_launch_count(void);
/* Tensor-core kernels poll their barriers with a bounded number of attempts. When a wait runs out the kernel
 * records a non-zero code in a device word and returns early. This reads and clears that word (synchronises
 * `stream`). 0 means no fault was recorded. */
int ptj_last_kernel_fault(void* stream, unsigned int* code_out);

/* ---- LayerNorm: y = gamma * (x - mean) / std_unbiased + beta, no epsilon ------------------------------ */
/* Replaces t_layernorm_fwd_t (model_triton.py:1625-1637; math model_torch_func.py:104-108). */
int ptj_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y,
                      int64_t rows, int64_t dim, int dtype, void* stream);
/* Replaces t_layernorm_bkwd2_x_t (model_triton.py:1853-1867) and t_layernorm_bkwd2_p_t (:1710-1726) in one
 * pass. dx and/or (dgamma,dbeta) may be NULL to skip that result. dx_add (may be NULL, may alias dx) is added
 * to dx: the gradient that arrives over the residual connection around the normalised branch
 * (model_triton.py:2036, 2190). `scratch` holds per-block partial column sums (needed only when dgamma/dbeta
 * are requested): ptj_layernorm_bwd_scratch_floats(rows, dim) floats.
 * Results are bit-reproducible (two-stage reduction, no atomics). */
size_t ptj_layernorm_bwd_scratch_floats(int64_t rows, int64_t dim);
int ptj_layernorm_bwd(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                      float* dgamma, float* dbeta, float* scratch, size_t scratch_floats, int64_t rows,
                      int64_t dim, int dtype, void* stream);
/* ptj_layernorm_bwd with a second output: dx_dropped = dropout(dx) for the mask stream of site (seed, stream_id) over
 * the contiguous [rows, dim] tensor, i.e. exactly what ptj_dropout(dx, NULL, dx_dropped, ...) would write, without a
 * second pass over dx (the reference runs t_dropout_bkwd as its own kernel, model_triton.py:153). dx must be given;
 * rows must be 16-byte aligned with dim a multiple of the 16-byte vector and at most 8 x 32 vectors
 * (else PTJ_ERR_UNSUPPORTED: call ptj_layernorm_bwd and ptj_dropout).
 * dropped_colsum (float[dim], may be NULL; needs dgamma/dbeta): the column sums of dx_dropped as stored, i.e. the
 * bias gradient of the linear layer whose output went through that dropout (the db of t_linear_bkwd2_p,
 * model_triton.py:423-434, which the reference sums in a pass of its own). */
int ptj_layernorm_bwd_dropout(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                              void* dx_dropped, float* dropped_colsum, float* dgamma, float* dbeta, float* scratch,
                              size_t scratch_floats,
                              int64_t rows, int64_t dim, float p, int train, uint64_t seed, uint32_t stream_id,
                              int dtype, void* stream);

/* LayerNorm backward that needs no scratch buffer from the caller. It has no counterpart in the reference: it
 * exists for callers that cannot allocate device memory themselves, e.g. code running inside a process whose GPU
 * memory was handed out up front to another allocator (cudaMalloc would fail, fragment that pool or stall the
 * device) or a step that must stay off the driver's allocation path. Same arguments and results (bit for bit) as
 * ptj_layernorm_bwd minus scratch / scratch_floats; the partial column sums go to a fixed 4.6 MiB array inside the
 * library that every GPU loading the library holds until the process exits.
 *   - dim <= ptj_layernorm_bwd_noalloc_max_dim() (2048); larger sizes return PTJ_ERR_TOO_LARGE.
 *   - The first call on a device looks up the array's device address (a driver query, done once per device with
 *     that device current); make that first call before any stream capture.
 *   - The array belongs to the CURRENT device: the device that owns `stream` must be current at the call (as for
 *     every entry point that launches on `stream`); with another device current the launch would be handed the
 *     address of that other device's array.
 *   - It calls no cudaMalloc / cudaFree or other allocating routine.
 *   - All calls on a device share the one array, which keeps the last call's contents (nothing in it has to start
 *     at zero: every call overwrites what it reads). Two calls that overlap on the GPU (different streams) race;
 *     order them on one stream or with events. */
size_t ptj_layernorm_bwd_noalloc_max_dim(void);
int ptj_layernorm_bwd_noalloc(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                              float* dgamma, float* dbeta, int64_t rows, int64_t dim, int dtype, void* stream);

/* ---- GELU (tanh form) ------------------------------------------------------------------------------- */
/* Replaces t_gelu_fwd_t (model_triton.py:254-260) and t_gelu_bkwd2_t (:296-304). */
int ptj_gelu_fwd(const void* x, void* y, int64_t n, int dtype, void* stream);
int ptj_gelu_bwd(const void* dy, const void* x_preact, void* dx, int64_t n, int dtype, void* stream);
/* t_gelu_bkwd2_t (model_triton.py:296-304) on a [rows, ld] matrix together with the column sums of its result as
 * stored, colsum float[cols]: the hidden gradient of the FFN and the gradient of its first bias (the db of
 * t_linear_bkwd2_p, :423-434) in one pass. dx may alias dy. scratch: ptj_colsum_scratch_floats(rows, cols) floats.
 * Needs 16-byte aligned pointers, ld and cols multiples of the 16-byte vector and cols <= 8192, else
 * PTJ_ERR_UNSUPPORTED (call ptj_gelu_bwd and ptj_colsum). Bit-reproducible (fixed summation order). */
int ptj_gelu_bwd_colsum(const void* dy, const void* x_preact, void* dx, float* colsum, float* scratch,
                        size_t scratch_floats, int64_t rows, int64_t cols, int64_t ld, int dtype, void* stream);

/* ---- Dropout ---------------------------------------------------------------------------------------- */
/* Replaces t_dropout_fwd_t (model_triton.py:1496-1506) and t_dropout_bkwd2_t (:1562-1572): the backward is the
 * same map applied to the gradient. residual may be NULL; when given, y = residual + dropout(x). */
int ptj_dropout(const void* x, const void* residual, void* y, int64_t n, float p, int train,
                uint64_t seed, uint32_t stream_id, int dtype, void* stream);

/* ---- log-softmax over the last dimension ------------------------------------------------------------- */
/* Replaces t_log_softmax_fwd_t (model_triton.py:62-72) and t_log_softmax_bkwd2_t (:153-164).
 * ld = elements between consecutive rows (>= cols). Rows of any length (chunked online max/sum). */
int ptj_log_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int64_t ld_x, int64_t ld_y,
                        int dtype, void* stream);
int ptj_log_softmax_bwd(const void* dy, const void* x, void* dx, int64_t rows, int64_t cols, int64_t ld,
                        int dtype, void* stream);

/* ---- cross entropy --------------------------------------------------------------------------------- */
/* Replaces t_avg_cross_entropy_loss_bkwd3_t (loss_and_optimizer_triton.py:176-197), t_avg_cross_entropy_loss
 * (:23-32) and accuracy (:199-200). Label 0 is padding: such rows add nothing to the loss, the accuracy or the
 * token count, and get a zero gradient row. A label outside [0, cols) (an id beyond the vocabulary, which the
 * reference would fault on) is treated the same way and is not counted either.
 *   labels      int32[rows]
 *   logits      [rows, ld] (cols valid)
 *   dlogits     same layout, may alias logits (in place), or NULL for forward only
 *   row_stats   float[2*rows] scratch: per-row loss and per-row hit
 *   n_valid     float[1]: number of rows with 0 < label < cols. If count_in_kernel != 0 it is computed here from
 *               labels, otherwise it is read (lets data-parallel callers supply the global count).
 *   out3        float[3]: mean loss, accuracy, n_valid / rows   (deterministic single-block reduction)
 */
int ptj_cross_entropy(const int32_t* labels, const void* logits, void* dlogits, float* row_stats,
                      float* n_valid, int count_in_kernel, float* out3, int64_t rows, int64_t cols,
                      int64_t ld, int dtype, void* stream);

/* Index of the largest of the first `cols` elements of every row (first index on ties) -> out int32[rows].
 * Replaces the torch.argmax over a logits slice in `predict`'s greedy decoding loop
 * (loss_and_optimizer_triton.py:203-212, the argmax at :207). */
int ptj_argmax_rows(const void* x, int32_t* out, int64_t rows, int64_t cols, int64_t ld, int dtype,
                    void* stream);

/* ---- embedding -------------------------------------------------------------------------------------- */
/* Replaces t_embed_fwd + positional add + dropout (model_triton.py:166-167, 2338-2341):
 * y[b,s,:] = dropout(w_emb[ids[b,s],:] * sqrt(dim) + w_pos[s,:]). Weights are `wdtype`, output `dtype`. */
int ptj_embed_fwd(const int32_t* ids, const void* w_emb, const void* w_pos, void* y, int64_t batch,
                  int64_t seq, int64_t dim, int64_t vocab, float p, int train, uint64_t seed,
                  uint32_t stream_id, int wdtype, int dtype, void* stream);
/* Replaces t_embed_bkwd2 / t_indexing_bkwd2 (model_triton.py:183-185, 205-213, 2513-2518) without atomics.
 * dy is the gradient AFTER the embedding dropout (this entry point applies the mask itself).
 *   sorted_pos int32[batch*seq]: token positions (b*seq+s) stably sorted by token id
 *   d_w_emb    float[vocab, dim]: accumulate != 0 adds onto existing contents (tied LM-head gradient)
 *   d_w_pos    float[seq, dim]  : overwritten
 */
int ptj_embed_bwd(const void* dy, const int32_t* ids, const int32_t* sorted_pos, float* d_w_emb,
                  float* d_w_pos, int accumulate, int64_t batch, int64_t seq, int64_t dim, int64_t vocab,
                  float p, int train, uint64_t seed, uint32_t stream_id, int dtype, void* stream);

/* ---- column sums (bias gradients) --------------------------------------------------------------------- */
/* out[c] = sum_r x[r, c]; replaces the dloss_dx.sum(dim=0) of t_linear_bkwd2_p (model_triton.py:423-428).
 * scratch: ptj_colsum_scratch_floats(rows, cols) floats. Deterministic. */
size_t ptj_colsum_scratch_floats(int64_t rows, int64_t cols);
int ptj_colsum(const void* x, float* out, float* scratch, size_t scratch_floats, int64_t rows,
               int64_t cols, int64_t ld, int dtype, void* stream);

/* ---- GEMM ------------------------------------------------------------------------------------------ */
/* C[M,N] = op(A) * op(B) with an elementwise epilogue. Replaces t_matmul_t / the linear variant of t_matmul_k
 * (model_triton.py:314-398) and every torch.matmul / einsum of the training path (t_linear_fwd :306,
 * t_proj_fwd :436, t_proj_bkwd2_p :460-472, t_proj_bkwd2_x :495-508).
 *   a_kmajor != 0: A is stored [M, K] (K contiguous, leading dim lda); else A is stored [K, M] (M contiguous)
 *   b_kmajor != 0: B is stored [N, K] (K contiguous, leading dim ldb); else B is stored [K, N] (N contiguous)
 *   in_dtype   PTJ_BF16: tcgen05 tensor-core kernel (TMA-fed, fp32 accumulate in TMEM); pointers 16-byte aligned,
 *              leading dimensions multiples of 8 elements.
 *              PTJ_F32 : exact-fp32 SIMT kernel, any shape (the "fp32 path").
 *   out_dtype  PTJ_F32 or PTJ_BF16, C row-major with leading dim ldc
 *   epilogue   PTJ_EPI_*; aux / aux_out meaning depends on it (same dtype and ld as C unless noted)
 *   split_k    >1 splits K over that many work items; partial tiles go to `workspace`
 *              (split_k*M*N floats) and are summed in a fixed order (bf16 kernel only; epilogue NONE/ACCUM).
 */
enum {
  PTJ_EPI_NONE = 0,         /* C = acc (+ bias[n] if bias != NULL)                                        */
  PTJ_EPI_GELU = 1,         /* aux_out = acc + bias (pre-activation, may be NULL); C = gelu(acc + bias)   */
  PTJ_EPI_GELU_BWD = 2,     /* C = acc * gelu'(aux[m,n])          (aux = saved pre-activation)            */
  PTJ_EPI_DROPOUT_RESID = 3,/* C = aux[m,n] + dropout(acc + bias) (aux = residual stream)                 */
  PTJ_EPI_ACCUM = 4         /* C += acc (out_dtype float only)                                            */
};
typedef struct {
  float p;            /* dropout probability (PTJ_EPI_DROPOUT_RESID) */
  int train;
  uint64_t seed;
  uint32_t stream_id;
} ptj_dropout_args;
int ptj_gemm(const void* a, const void* b, void* c, const float* bias, const void* aux, void* aux_out,
             int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int a_kmajor,
             int b_kmajor, int in_dtype, int out_dtype, int epilogue, const ptj_dropout_args* dropout,
             int split_k, float* workspace, size_t workspace_floats, void* stream);

/* split_k = PTJ_SPLIT_TAIL lets ptj_gemm even out a bad last round of tiles: a bf16 product on the 256 x 256-tile
 * thread-block-pair kernel whose tile count leaves most of the GPU idle in its last round (96 tiles on 74 pairs) runs
 * as head rows that fill whole rounds plus, in the same launch, the remaining rows split over K; a finishing kernel
 * sums those parts in a fixed order and applies the epilogue. Epilogues PTJ_EPI_NONE (no bias) and
 * PTJ_EPI_DROPOUT_RESID (K-major operands, 16-byte aligned bf16 rows); anything else, or a workspace smaller than
 * ptj_gemm_tail_split_floats(M, N, K) floats, runs unsplit. Head rows are bit-identical to the unsplit product, the
 * rest differs by the summation order. ptj_gemm_tail_split_rows: the first row of the split range (0: no split for
 * this shape). */
#define PTJ_SPLIT_TAIL (-1)
size_t ptj_gemm_tail_split_floats(int64_t M, int64_t N, int64_t K);
int64_t ptj_gemm_tail_split_rows(int64_t M, int64_t N, int64_t K);

/* Two products C_i[M_i, N_i] = op(A_i) op(B_i) (i = 0, 1) in ONE launch: bf16 operands, float32 or bf16 outputs, the
 * same K and the same operand layouts for both, epilogue PTJ_EPI_NONE or (float32 output) PTJ_EPI_ACCUM each, optional
 * K split each (own workspace of split_k * M * N floats). The two may also be row ranges of ONE product, the second
 * split over K, which evens out a last round of tiles that would leave most of the GPU idle. The tiles of both products are dealt to the GPU's thread-block pairs as one list, so two
 * products that would each occupy half of the GPU (the weight gradients of a transformer layer: 36 tiles of 256 x 256
 * each for the two FFN matrices at GPT-2 small) share one round instead of each being split over K and reduced by a
 * second launch. Results are bit-identical to two ptj_gemm calls with the same split_k. Both products must qualify
 * for the thread-block-pair kernel (M, N >= 256 and K >= 2048 or N >= 8192); otherwise PTJ_ERR_UNSUPPORTED is returned
 * and nothing is launched: issue two ptj_gemm calls instead. No counterpart in the reference, whose matmuls are
 * separate launches (model_triton.py:373-398). */
typedef struct ptj_gemm_problem {
  const void* a;
  const void* b;
  void* c;             /* [M, ldc] of out_dtype */
  int64_t M, N, lda, ldb, ldc;
  int out_dtype;       /* PTJ_F32 or PTJ_BF16 */
  int epilogue;        /* PTJ_EPI_NONE or PTJ_EPI_ACCUM (float32 output only) */
  int split_k;
  float* workspace;    /* split_k * M * N floats when split_k > 1, 16-byte aligned */
  size_t workspace_floats;
} ptj_gemm_problem;
int ptj_gemm_grouped2(const ptj_gemm_problem* p0, const ptj_gemm_problem* p1, int64_t K, int a_kmajor, int b_kmajor,
                      void* stream);

/* ---- causal scaled-dot-product attention ----------------------------------------------------------- */
/* Replaces t_scaled_dot_prod_attn_fwd3_t (model_triton.py:706-754) and t_scaled_dot_prod_attn_bkwd3_t
 * (:951-1003): O = dropout(softmax(causal(Q K^T / sqrt(d)))) V with the dropout applied to the probabilities.
 * q, k, v, o (and dq, dk, dv, d_o) are 4-D views [batch, heads, seq, d_head] described by element strides
 * (d_head contiguous), so both the reference's [B,H,3,N,D] tensor and a fused [B*N, H*3*D] projection
 * output are addressed without copies. row_max / row_sum are float[batch*heads*seq] (the reference's acts0 /
 * acts1: running maximum of the scaled scores and sum of exp(score - max)).
 *   dtype PTJ_BF16 with d_head == 64 and seq % 128 == 0 runs the tcgen05 kernels; everything else runs the
 *   exact-fp32 SIMT kernels.
 * Backward recomputes the probabilities; it is deterministic (no atomics).
 *
 * row_kstart (optional, int32[batch, seq]): the first key each query row may attend to, so that row i attends keys
 * [row_kstart[b,i], i]. This is how the masks of the reference's collator (causal x block-diagonal over packed
 * documents x padding, tokenized_dataset.py:110-131, applied by its kernels at model_triton.py:678-681, 917-920) reach
 * the kernels without a dense [B,N,N] tensor: a row of a packed document starts at its document's first token, a
 * padding row gets row_kstart > i and attends nothing (zero output row, row_max 0, row_sum 1, zero gradients).
 * NULL = plain causal attention. Forward and backward of one call must be given the same array.
 */
typedef struct {
  int64_t batch, heads, seq, d_head;
  int64_t q_strides[3], k_strides[3], v_strides[3], o_strides[3]; /* batch, head, row (elements) */
} ptj_attn_shape;
/* Optional: the dropout keep flags of one attention call (probability tensor [B*H, S, S], mask stream of site
 * (seed, stream_id)), computed once and handed to both ptj_attn_fwd and ptj_attn_bwd as `keep_bits`; the kernels then
 * skip their own Philox pass. The flags are the same ones the kernels draw when keep_bits == NULL, so results are
 * bit-identical either way (the reference regenerates its mask in the backward kernel, model_triton.py:688).
 * ptj_attn_keep_bits_bytes: size of the buffer (16-byte aligned), 0 when the shape / dtype does not take the
 * tensor-core path (then pass NULL). */
size_t ptj_attn_keep_bits_bytes(const ptj_attn_shape* shape, int dtype);
int ptj_attn_keep_bits(uint32_t* bits, const ptj_attn_shape* shape, float p, uint64_t seed, uint32_t stream_id,
                       int dtype, void* stream);
int ptj_attn_fwd(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                 const ptj_attn_shape* shape, float p, int train, uint64_t seed, uint32_t stream_id,
                 const uint32_t* keep_bits, const int32_t* row_kstart, int dtype, void* stream);
/* dq/dk/dv use q/k/v strides of `dshape`; d_o and o use o_strides of `shape`.
 * workspace: ptj_attn_bwd_workspace_bytes(shape, dtype) bytes of device memory, 16-byte aligned, contents
 * irrelevant before and after the call (the tensor-core path keeps each KV tile's share of dQ there in fp32 and sums
 * the shares in a fixed order instead of the reference's tl.atomic_add, model_triton.py:938; 0 bytes = not needed,
 * NULL allowed). Too small a workspace returns PTJ_ERR_WORKSPACE. */
size_t ptj_attn_bwd_workspace_bytes(const ptj_attn_shape* shape, int dtype);
int ptj_attn_bwd(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                 const float* row_max, const float* row_sum, void* dq, void* dk, void* dv,
                 const ptj_attn_shape* shape, const ptj_attn_shape* dshape, float p, int train,
                 uint64_t seed, uint32_t stream_id, const uint32_t* keep_bits, const int32_t* row_kstart,
                 void* workspace, size_t workspace_bytes, int dtype, void* stream);

/* ---- optimizer -------------------------------------------------------------------------------------- */
/* sum of squares of a float vector -> out[0] (deterministic two-stage). Replaces grads_l2norm
 * (loss_and_optimizer_triton.py:411-416) on a flat buffer. scratch: ptj_sumsq_scratch_floats(n). */
size_t ptj_sumsq_scratch_floats(int64_t n);
int ptj_sumsq(const float* x, float* out, float* scratch, size_t scratch_floats, int64_t n, void* stream);
/* Replaces adam_w_in_place (loss_and_optimizer_triton.py:376-401) over a flat range, in place:
 *   g' = g * grad_scale * clip,  clip = min(1, max_norm / (sqrt(*sumsq) * grad_scale + 1e-6)) when sumsq != NULL
 *   m = b1 m + (1-b1) g' ; v = b2 v + (1-b2) g'^2 ; p -= lr * ( (m/(1-b1^t)) / (sqrt(v/(1-b2^t)) + eps) + wd_i p )
 * Segments (device arrays): seg_start int64[nseg+1] (ascending element offsets, multiples of 4, seg_start[0]=0,
 * last = n), seg_decay uint8[nseg] says whether weight decay applies to that segment (nseg <= 1024).
 * nseg == 0: wd applies everywhere. sumsq is a device scalar (see ptj_sumsq).
 * shadow (may be NULL): bf16 copy of the updated parameters.
 */
int ptj_adamw(float* p, const float* g, float* m, float* v, void* shadow_bf16, int64_t n,
              const int64_t* seg_start, const uint8_t* seg_decay, int nseg, float lr, float beta1,
              float beta2, float eps, float weight_decay, int64_t t, float grad_scale,
              const float* sumsq, float max_norm, void* stream);
/* dst_bf16[i] = (bf16) src[i] */
int ptj_cast_f32_to_bf16(const float* src, void* dst_bf16, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PTJ_B200_H_ */
