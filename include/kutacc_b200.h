/*
 * kutacc_b200.h -- C ABI of the B200 build of KuTACC's gated-attention path.
 *
 * The entry points in part 1 keep the names, argument order, struct layouts and error behaviour of
 * the reference's public header (include/kutacc.h); a caller compiled against that header links
 * against this library unchanged. Each declaration cites the reference interface it replaces.
 * Part 2 lists additions that the reference does not have (device helpers, error query, a
 * plain-pointer projection entry); they all carry the kutacc_b200_ prefix.
 *
 * Tensors: a kutacc_tensor_h is a pointer to a strided descriptor {dim, data pointer, sizes,
 * strides, dtype} (reference: src/tensor/tensor.h:21-51). The library never owns tensor data.
 * data pointers may be CUDA device pointers (no copies are made) or host pointers (the library
 * stages them through device memory on every call). Strides are in elements for compute
 * operators and in bytes for kutacc_af2_all_gather and kutacc_af2_transpose, as in the reference.
 *
 * Errors: operators return void. A failed check prints one line
 *   "KUTACC_CHECK fail in <func> at <file>:<line> , <message>"
 * on stderr and sets a sticky process-wide flag; while the flag is set every operator returns
 * without touching memory (reference: src/utils/check.h:50-56, src/utils/check.cpp:16).
 */
#ifndef KUTACC_B200_H
#define KUTACC_B200_H

#include <stddef.h>
#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
#include <vector>
extern "C" {
#endif

#define KUTACC_B200_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------- */
/* Part 1: the reference's own interface for this path                                         */
/* ------------------------------------------------------------------------------------------- */

#ifndef KUTACC_OK
#define KUTACC_OK 0
#define KUTACC_ERROR (-1)
#endif

#ifndef KUTACC_H /* the reference header, if included first, already defines these types */

/* replaces include/kutacc.h:32-39 */
typedef struct kutacc_version {
    const char *product_name;
    const char *product_version;
    const char *component_name;
    const char *component_version;
    const char *component_abi_version;
    const char *component_appendinfo;
} kutacc_version_t;

/* replaces include/kutacc.h:49 */
typedef void *kutacc_tensor_h;

/* replaces include/kutacc.h:77-89. Weight matrices are stored W[out][in]; gating_b and output_b
 * are fp32 vectors of nchannels entries. For global attention key_w and value_w are
 * [head_size, nchannels]. */
typedef struct kutacc_af2_attention_weights {
    int64_t nchannels;
    int64_t nheads;
    int64_t head_size;
    kutacc_tensor_h query_w;
    kutacc_tensor_h key_w;
    kutacc_tensor_h value_w;
    kutacc_tensor_h gating_w;
    kutacc_tensor_h gating_b;
    kutacc_tensor_h output_w;
    kutacc_tensor_h output_b;
} kutacc_af2_attention_weights_t;

/* replaces include/kutacc.h:95-104. q, k, v, gate, avg are caller-owned scratch tensors. The
 * reference fills them with its intermediate projections; this library keeps intermediates in its
 * own device workspace and leaves them untouched (handles may be null). */
typedef struct kutacc_af2_attention_inputs {
    int64_t batch;
    int64_t seq_len;
    kutacc_tensor_h q;
    kutacc_tensor_h k;
    kutacc_tensor_h v;
    kutacc_tensor_h gate;
    kutacc_tensor_h avg;
} kutacc_af2_attention_inputs_t;

/* replaces include/kutacc.h:194-202: weights of the transition operator. linear1_w is stored [c_i][c_o],
 * linear2_w [c_o][c_i] (W[out][in]); the biases are fp32 vectors. */
typedef struct kutacc_af2_trans_weights {
    int64_t c_o;
    int64_t c_i;
    kutacc_tensor_h linear1_w;
    kutacc_tensor_h linear1_b;
    kutacc_tensor_h linear2_w;
    kutacc_tensor_h linear2_b;
} kutacc_af2_trans_weights_t;

/* replaces include/kutacc.h:208-214: input_act is [batch, n_res, c_o] bf16 dense; intermediate_act is the
 * reference's [batch, n_res, c_i] scratch, which this library does not write (it may be null). */
typedef struct kutacc_af2_trans_act_inputs {
    int64_t batch;
    int64_t n_res;
    kutacc_tensor_h input_act;
    kutacc_tensor_h intermediate_act;
} kutacc_af2_trans_act_inputs_t;

#endif /* KUTACC_H */

/* replaces include/kutacc.h:47 (src/version/version.cpp:28-35) */
KUTACC_B200_API int kutacc_get_version(kutacc_version_t *version);

/* replaces include/kutacc.h:51-52 (src/comm/kupl.cpp:25-27): process-wide rank bookkeeping */
KUTACC_B200_API extern int64_t world_size;
KUTACC_B200_API extern int64_t rank;

/* replaces include/kutacc.h:55-56 (src/comm/kupl.cpp:50-68). One process per GPU. Builds an NCCL
 * communicator over the ranks; the NCCL unique id is exchanged through a file whose name comes
 * from the environment variable SHMID (as the reference's test runner sets it) or
 * KUTACC_RENDEZVOUS. buffer_size is accepted and recorded; NCCL needs no staging window. */
KUTACC_B200_API void kutacc_comm_init(int64_t world_size_, int64_t rank_, int64_t buffer_size_);
KUTACC_B200_API void kutacc_comm_fini(void);

/* replaces include/kutacc.h:74 (src/comm/all_gather.cpp:21-100). data is [chunk(m), n, len] or
 * [m, chunk(n), len], out is [m, n, len]; len and all strides are BYTES; the sharded axis is
 * dim 1 when data.sizes[0] == out.sizes[0], else dim 0; block(x) = ceil(x / world_size),
 * chunk(x) = min(block(x), x - rank * block(x)). */
KUTACC_B200_API void kutacc_af2_all_gather(kutacc_tensor_h data, kutacc_tensor_h out);

/* replaces include/kutacc.h:58-65 (src/comm/transpose.cpp:21-100): re-shards a byte matrix between "rows
 * split over the ranks" and "columns split over the ranks". data is [chunk(m), n, len] and out [m, chunk(n),
 * len], or data [m, chunk(n), len] and out [chunk(m), n, len]; len and all strides are BYTES; element (i, j)
 * moves from the rank that owns row i to the rank that owns column j. One group of ncclSend/ncclRecv. */
KUTACC_B200_API void kutacc_af2_transpose(kutacc_tensor_h data, kutacc_tensor_h out);

/* replaces include/kutacc.h:297-300 (src/attention/gating_attention.cpp:160-200).
 *   input            [batch*seq_len, nchannels]
 *   bias             [batch, seq_len] additive mask bias (row stride = strides[0])
 *   nonbatched_bias  [nheads, seq_len, seq_len] pair bias, unit key stride; "absent" is a valid
 *                    handle whose sizes[0] == 0
 *   out              [batch, seq_len, nchannels] (row stride = strides[1])
 *   block_size       query tile of the reference's CPU loop; validated (> 0), otherwise a hint
 * dtype of input/bias/nonbatched_bias/weights/out: all bf16, or all fp32 (extension). */
KUTACC_B200_API void kutacc_af2_gating_attention(kutacc_tensor_h input, kutacc_af2_attention_inputs_t *q_based_ptr,
                                                 kutacc_tensor_h bias, kutacc_tensor_h nonbatched_bias,
                                                 kutacc_af2_attention_weights_t *weight_ptr, kutacc_tensor_h out,
                                                 int64_t block_size);

/* replaces include/kutacc.h:305-307 (src/attention/global_attention.cpp:167-205).
 *   q_data [batch, seq_len, 64] bf16 contiguous, q_mask [batch, seq_len, 1] bf16,
 *   out [batch, seq_len, 64]. nchannels must be 64, as in the reference. */
KUTACC_B200_API void kutacc_af2_global_attention(kutacc_af2_attention_inputs_t *q_based_ptr, kutacc_tensor_h q_data,
                                                 kutacc_tensor_h q_mask, kutacc_af2_attention_weights_t *weight_ptr,
                                                 kutacc_tensor_h out);

/* replaces include/kutacc.h:399-400 (src/linear/linear.cpp:21-50):
 * result[m,n] = act[m,k] . weight[n,k]^T + beta * result + bias_data[n]; result is contiguous. */
KUTACC_B200_API void kutacc_af2_linear(kutacc_tensor_h act, kutacc_tensor_h weight, float *bias_data,
                                       kutacc_tensor_h result, int64_t beta);

/* replaces include/kutacc.h:407-408 (src/linear/mm.cpp:94-110). The packed image of an [n,k]
 * weight is the dense row-major [n,k] matrix (n*k elements, the size the reference reports). Takes
 * the element type as uint16_t bit patterns so that the header is plain C. */
KUTACC_B200_API void kutacc_af2_linear_weight_prepack(const uint16_t *weight, uint16_t *result, int64_t n, int64_t k,
                                                      int64_t ldb, int64_t num_threads);

/* replaces include/kutacc.h:321-322 (src/attention/transition.cpp:21-61): out = relu(input_act . linear1_w^T +
 * linear1_b) . linear2_w^T + linear2_b, bf16 with fp32 accumulation and one bf16 rounding of the intermediate
 * and of out; out is [batch, n_res, c_o] dense. */
KUTACC_B200_API void kutacc_af2_transition(kutacc_af2_trans_act_inputs_t *trans_inputs_ptr,
                                           kutacc_af2_trans_weights_t *trans_weights_ptr, kutacc_tensor_h out);

/* Triangle multiplication (replaces include/kutacc.h:154-189, 426-456; src/attention/triangle_multiplication.cpp).
 * The operator is exported as four steps, as in the reference; the caller runs LayerNorm and the permute between
 * them. All tensors bf16, biases fp32. */
typedef struct kutacc_af2_tm_proj_weights {     /* include/kutacc.h:154-162 */
    int64_t c_o;                                /* channels of input_act */
    int64_t c_i;                                /* channels of the projections */
    kutacc_tensor_h proj_w;                     /* [c_i, c_o] */
    kutacc_tensor_h proj_b;                     /* [c_i] fp32 */
    kutacc_tensor_h gate_w;                     /* [c_i, c_o] */
    kutacc_tensor_h gate_b;                     /* [c_i] fp32 */
} kutacc_af2_tm_proj_weights_t;

typedef struct kutacc_af2_tm_act_inputs {       /* include/kutacc.h:168-175 */
    int64_t n_res;
    int64_t n_res_gather;
    kutacc_tensor_h proj_act;                   /* [c_i, n_res, n_res_gather], unit last stride (output) */
    kutacc_tensor_h input_act;                  /* [n_res, n_res_gather, c_o] dense */
    kutacc_tensor_h proj_act_gate;              /* [c_i, n_res, n_res_gather] (output: the gate before the sigmoid) */
} kutacc_af2_tm_act_inputs_t;

typedef struct kutacc_af2_tm_linear_weights {   /* include/kutacc.h:181-189 */
    int64_t c_o;
    int64_t c_i;
    kutacc_tensor_h gating_w;                   /* [c_o, c_o] */
    kutacc_tensor_h gating_b;                   /* [c_o] fp32 */
    kutacc_tensor_h output_proj_w;              /* [c_o, c_i] */
    kutacc_tensor_h output_proj_b;              /* [c_o] fp32 */
} kutacc_af2_tm_linear_weights_t;

/* replaces include/kutacc.h:426-429 (triangle_multiplication.cpp:25-70): proj_act = bf16(input_act . proj_w^T +
 * proj_b), proj_act_gate = bf16(input_act . gate_w^T + gate_b), both stored channel-major, then in place
 * proj_act = bf16((proj_act * mask) * sigmoid(proj_act_gate)); mask [n_res, n_res_gather]. input_prepack is
 * accepted and ignored (the packed image of a matrix is the matrix). */
KUTACC_B200_API void kutacc_af2_triangle_multiplication_calc_proj(kutacc_af2_tm_act_inputs_t *tm_acts_ptr,
                                                                  kutacc_tensor_h mask,
                                                                  kutacc_af2_tm_proj_weights_t *tm_weights_ptr,
                                                                  bool input_prepack);

/* replaces include/kutacc.h:436-439 (triangle_multiplication.cpp:75-104): per channel c of left_proj_act.sizes[0],
 * center[c] = left[c] . right[c]^T (is_incoming false) or right[c]^T . left[c] (is_incoming true), all
 * [c_i, n_res_gather, n_res_gather] with unit last stride. */
KUTACC_B200_API void kutacc_af2_triangle_multiplication_equation(kutacc_tensor_h center_act, kutacc_tensor_h left_proj_act,
                                                                 kutacc_tensor_h right_proj_act, int64_t n_res_gather,
                                                                 bool is_incoming);

/* replaces include/kutacc.h:446-448 (triangle_multiplication.cpp:109-133): gate = input_act . gating_w^T + gating_b
 * and out = center_act . output_proj_w^T + output_proj_b, rows = n_res * n_res_gather; gate, out and center_act are
 * [n_res, n_res_gather, channels] with row stride strides[1]. */
KUTACC_B200_API void kutacc_af2_triangle_multiplication_gate_and_out_linear(
    kutacc_tensor_h gate, kutacc_tensor_h out, kutacc_af2_tm_act_inputs_t *tm_acts_ptr, kutacc_tensor_h center_act,
    kutacc_af2_tm_linear_weights_t *tm_weights_ptr, bool input_prepack);

/* replaces include/kutacc.h:455-456 (triangle_multiplication.cpp:138-158): out = bf16(out * sigmoid(gate)) */
KUTACC_B200_API void kutacc_af2_triangle_multiplication_last(kutacc_tensor_h out, kutacc_tensor_h gate, int64_t n_res,
                                                             int64_t n_res_gather, int64_t c_o);

/* replaces include/kutacc.h:334 (src/normalization/layernorm.cpp:17-20, layernorm_kernel.h:22-53): LayerNorm
 * of ONE row of `size` bf16 channels, out = bf16(fma(fma(x, rstd, -rstd * mean), gamma, beta)) with the
 * reference's shifted-data statistics. Host or device pointers. A launch per row is what this signature
 * implies; use kutacc_b200_layernorm_rows for a matrix. bf16 taken as uint16_t bit patterns. */
KUTACC_B200_API void kutacc_af2_layernorm(uint16_t *data, float *gamma, float *beta, int64_t size, float eps,
                                          uint16_t *out);

/* replaces include/kutacc.h:418 (src/utils/blas.cpp:93-98): 'A' -> m*k, 'B' -> k*n elements */
KUTACC_B200_API size_t kutacc_af2_gemm_pack_get_size(char identifier, char transa, char transb, int m, int n, int k);

/* ------------------------------------------------------------------------------------------- */
/* Part 2: additions (no counterpart in the reference)                                          */
/* ------------------------------------------------------------------------------------------- */

/* dtype tags: 0 and 1 are the reference's (include/kutacc.h:467-471); 2 is new */
#define KUTACC_B200_DTYPE_INT64 0
#define KUTACC_B200_DTYPE_BF16 1
#define KUTACC_B200_DTYPE_FP32 2

/* Plain-C construction of a tensor descriptor (the reference only offers the C++ class
 * kutacc::TensorWrapper). The descriptor copies sizes and strides; data is not owned. */
KUTACC_B200_API kutacc_tensor_h kutacc_b200_tensor_create(void *data, int64_t dim, const int64_t *sizes,
                                                          const int64_t *strides, int dtype);
KUTACC_B200_API void kutacc_b200_tensor_destroy(kutacc_tensor_h t);

/* Sticky error flag: 1 if a check has failed since the last clear. The message of the most recent
 * failure is copied into buf (truncated to cap-1 characters). */
KUTACC_B200_API int kutacc_b200_error_set(void);
KUTACC_B200_API int kutacc_b200_last_error(char *buf, size_t cap);
KUTACC_B200_API void kutacc_b200_clear_error(void);

/* Device selection (default: current CUDA device) and stream (default: the legacy default
 * stream). Operators are synchronous unless kutacc_b200_set_async(1) was called, in which case
 * calls only enqueue work on the stream. A result in HOST memory is then complete after
 * kutacc_b200_synchronize(): kutacc_af2_gating_attention with a large host `out` downloads its rows chunk by chunk
 * on a copy stream of the library and returns while those downloads run, so that the kernels of a following call
 * start beside them (the library orders every later use of its staging pool after them).
 * The library has ONE workspace and ONE staging pool, handed out from their start on every call; only the
 * order of work on a stream protects them. In enqueue-only mode a caller that switches streams between calls
 * must therefore order the streams itself (an event from the old stream that the new one waits for) unless the
 * second call uses neither pool. Calls that use neither: kutacc_af2_all_gather on device tensors whose per-rank
 * rows form one dense slab of the output (it gathers in place), and kutacc_b200_global_attention_noalloc. Every
 * other operator uses the workspace. */
KUTACC_B200_API void kutacc_b200_set_stream(void *cuda_stream);
KUTACC_B200_API void kutacc_b200_set_async(int enabled);
/* The persistent kernels (projections, attention core) normally fill every SM. A caller that runs a
 * collective on another stream beside them (the output all-gather of one slab of rows while the next
 * slab is computed) can ask them to leave `sms` SMs free, 0..64, so that the collective's CTAs find room
 * at once instead of waiting for the persistent CTAs to finish. Default 0. */
KUTACC_B200_API void kutacc_b200_set_sm_margin(int sms);
/* The pair bias of the NEXT kutacc_af2_gating_attention call (or its LayerNorm-fused form) is still being produced on
 * another stream, an all-gather of its row blocks for instance: `cuda_event` (a cudaEvent_t recorded there) is what
 * the call waits for, on the runtime stream, between its projections and its attention kernel, so the projections
 * run beside that work. The event is used by one call and then forgotten; pass NULL to clear it. */
KUTACC_B200_API void kutacc_b200_set_pair_bias_event(void *cuda_event);
KUTACC_B200_API void kutacc_b200_synchronize(void);

/* Device memory helpers for callers without a CUDA runtime of their own. */
KUTACC_B200_API void *kutacc_b200_device_malloc(size_t bytes);
KUTACC_B200_API void kutacc_b200_device_free(void *p);
KUTACC_B200_API void kutacc_b200_memcpy_h2d(void *dst, const void *src, size_t bytes);
KUTACC_B200_API void kutacc_b200_memcpy_d2h(void *dst, const void *src, size_t bytes);

/* Bytes of device workspace currently held by the library (grow-only pool), and release. */
KUTACC_B200_API size_t kutacc_b200_workspace_bytes(void);
KUTACC_B200_API void kutacc_b200_release_workspace(void);

/* Number of kernels the library has launched since load (all operators). */
KUTACC_B200_API uint64_t kutacc_b200_launch_count(void);

/* Per-kernel timing for benchmarks: while enabled, every kernel launch is bracketed by CUDA
 * events. kutacc_b200_profile_read synchronises, writes up to cap durations (ms) in launch order
 * and their names joined by ';' into names, clears the record and returns the count. */
KUTACC_B200_API void kutacc_b200_set_profile(int enabled);
KUTACC_B200_API int kutacc_b200_profile_read(char *names, size_t names_cap, float *ms, int cap);

/* Communicator set-up for callers that can already broadcast 128 bytes between ranks (for
 * example through torch.distributed): rank 0 asks for an id, every rank passes the same id. */
KUTACC_B200_API void kutacc_b200_comm_unique_id(void *id128);
KUTACC_B200_API void kutacc_b200_comm_init_with_id(int64_t world_size_, int64_t rank_, const void *id128);

/* Global attention for callers that must not allocate device memory inside the call (a server whose
 * own pool already owns all of HBM, a loop that cannot take the implicit synchronisation of
 * cudaMalloc/cudaFree, a process under a fixed memory quota). It has no counterpart in the reference.
 * Same arithmetic as kutacc_af2_global_attention; every pointer is a device pointer owned by the caller
 * (q_data [batch, seq_len, 64] bf16 contiguous, q_mask [batch, seq_len] bf16, weights as for the operator
 * above, biases fp32, out [batch, seq_len, 64] bf16 with row stride out_row_stride elements; q_data, out and the
 * five weights 16-byte aligned, or the call is refused); work is
 * enqueued on cuda_stream and the call returns without synchronising. Its scratch is a 4 MiB array
 * inside the library image, resident on every GPU that loads the library until the process exits;
 * shapes that need more (batch * row-splits beyond about 7000) are refused with an error. The first
 * call on a device looks up the array's device address: make it outside of stream capture. Calls share
 * the array, so two calls that overlap on the GPU race. Returns 0, or -1 after reporting an error. */
KUTACC_B200_API int kutacc_b200_global_attention_noalloc(const void *q_data, const void *q_mask, const void *query_w,
                                                         const void *key_w, const void *value_w, const void *gating_w,
                                                         const float *gating_b, const void *output_w,
                                                         const float *output_b, void *out, int64_t out_row_stride,
                                                         int64_t batch, int64_t seq_len, int64_t nheads,
                                                         int64_t head_size, void *cuda_stream);

/* Self-test of the failure-detection path: launches a one-warp kernel that waits, for at most
 * limit_microseconds (1..100000), on a barrier nothing arrives on. The wait gives up, the kernel returns
 * normally, and the usual error convention reports "a device-side wait ran out of time" at the next
 * synchronisation (at once in synchronous mode). Returns 0 when the kernel was launched. No GPU fault is
 * involved; the context stays usable. */
KUTACC_B200_API int kutacc_b200_selftest_wait_timeout(int64_t limit_microseconds);

/* Pair-bias projection written directly in the layout the attention operator consumes:
 * nb[h, q, k] = z[q, k, :] . wb[h, :]   with z [rows, n_k, c_z], wb [nheads, c_z], nb
 * [nheads, rows, n_k] (row stride of head h = nb_head_stride elements). Same arithmetic as
 * kutacc_af2_linear on z viewed [rows*n_k, c_z] followed by the caller's permute. dtype bf16/fp32.
 * nb's strides may place the heads of a row next to each other (a [rows, nheads, n_k] storage seen as
 * [nheads, rows, n_k]: strides {n_k, nheads * n_k, 1}; bf16, c_z 64 or 128): the rows one rank projects are then one
 * dense block, which kutacc_af2_all_gather gathers in place. kutacc_af2_gating_attention takes such a pair bias too. */
KUTACC_B200_API void kutacc_b200_pair_bias(kutacc_tensor_h z, kutacc_tensor_h wb, kutacc_tensor_h nb);

/* LayerNorm fused in front of the two projections of the attention path (no counterpart in the reference, whose
 * callers run kutacc_af2_layernorm row by row first, include/kutacc.h:334, and pass the normalised tensor on).
 * Both take the LayerNorm's fp32 gamma and beta (one value per channel, host or device) and eps, and compute what the
 * unfused sequence computes, up to bf16 rounding: the normalisation is folded into the projection weights and
 * applied in the projection's epilogue from per-row statistics, so the normalised activations are never stored.
 *   kutacc_b200_gating_attention_ln : kutacc_af2_gating_attention(LayerNorm(input), ...), bf16
 *   kutacc_b200_pair_bias_ln        : kutacc_b200_pair_bias(LayerNorm(z), wb, nb), bf16 */
KUTACC_B200_API void kutacc_b200_gating_attention_ln(kutacc_tensor_h input, kutacc_af2_attention_inputs_t *q_based_ptr,
                                                     kutacc_tensor_h bias, kutacc_tensor_h nonbatched_bias,
                                                     kutacc_af2_attention_weights_t *weight_ptr, const float *ln_gamma,
                                                     const float *ln_beta, float eps, kutacc_tensor_h out,
                                                     int64_t block_size);
KUTACC_B200_API void kutacc_b200_pair_bias_ln(kutacc_tensor_h z, const float *ln_gamma, const float *ln_beta, float eps,
                                              kutacc_tensor_h wb, kutacc_tensor_h nb);

/* The same LayerNorm over every row of a [rows, size] bf16 matrix in one launch (the loop over rows that the
 * reference leaves to its caller). Strides in elements, row_stride and out_row_stride >= size; out may alias
 * data. Host or device pointers. */
KUTACC_B200_API void kutacc_b200_layernorm_rows(const void *data, const float *gamma, const float *beta, int64_t rows,
                                                int64_t size, int64_t row_stride, int64_t out_row_stride, float eps,
                                                void *out);

#ifdef __cplusplus
} /* extern "C" */

#ifndef KUTACC_H
namespace kutacc {
/* replaces include/kutacc.h:467-471; kFP32 is an addition (the reference tags fp32 buffers kBF16
 * or passes raw float pointers). */
typedef enum TensorDataType { kInt64 = 0, kBF16 = 1, kFP32 = 2, kNumTypes } DType;

/* replaces include/kutacc.h:484-497 (src/tensor/tensor.cpp:20-30,89-92): owns the descriptor, not
 * the data. Same constructor signature, so the mangled symbols match the reference's. */
struct KUTACC_B200_API TensorWrapper {
private:
    kutacc_tensor_h tensor_;

public:
    TensorWrapper(void *data_ptr, std::vector<int64_t> &&sizes, std::vector<int64_t> &&strides, int64_t dim,
                  DType dtype);
    TensorWrapper();
    kutacc_tensor_h get_tensor() { return tensor_; }
    ~TensorWrapper();
};
}  // namespace kutacc
#endif /* KUTACC_H */
#endif /* __cplusplus */

#endif /* KUTACC_B200_H */
