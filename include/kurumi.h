/* kurumi C ABI, as exported by libkurumi_cuda.so: the graph-builder / eval surface a kurumi
 * front end binds, restricted to the ops the CUDA backend evaluates, plus the backend kind
 * KU_CUDA. Every prototype below has the same name, argument order and error behaviour as the
 * reference header kurumi/include/kurumi.h (line numbers cited per group), so an existing
 * binding (cffi / cbindgen / ctypes) keeps working unchanged.
 *
 * Build a graph of nodes (each builder returns a node id; KU_ERR on error, then
 * ku_last_error() gives the message), create a backend once, evaluate. Handles are opaque and
 * freed by their matching ku_*_free. Not thread-safe per handle. Tensor bytes are
 * little-endian, row-major. */
#ifndef KURUMI_H
#define KURUMI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KU_ERR 0xFFFFFFFFu /* kurumi.h:25 */

/* dtype tags, kurumi.h:29-34 (index = kurumi's DType declaration order) */
typedef enum {
  KU_BOOL = 0, KU_U8, KU_U16, KU_U32, KU_U64,
  KU_I8, KU_I16, KU_I32, KU_I64,
  KU_F8E4M3, KU_F8E5M2, KU_F16, KU_BF16, KU_F32, KU_F64,
  KU_C64, KU_C128
} KuDType;

/* backend kinds, kurumi.h:38 has {KU_CPU, KU_METAL}; KU_CUDA is the value this library adds.
 * libkurumi_cuda.so creates only KU_CUDA: any other kind returns NULL with an error message
 * (there is no CPU evaluator inside this library). */
typedef enum { KU_CPU = 0, KU_METAL = 1, KU_CUDA = 2 } KuBackendKind;

typedef struct KuGraph KuGraph;     /* kurumi.h:40-45 */
typedef struct KuTensor KuTensor;
typedef struct KuFeeds KuFeeds;
typedef struct KuBackend KuBackend;
typedef struct KuRunnable KuRunnable; /* a rebuilt graph blob with its entries */
typedef uint32_t KuNode;            /* kurumi.h:47 */

const char *ku_last_error(void);    /* kurumi.h:51 */

/* graph lifecycle and leaves, kurumi.h:54-60 */
KuGraph *ku_graph_new(void);
void ku_graph_free(KuGraph *g);
KuNode ku_input(KuGraph *g, const size_t *shape, size_t rank, uint32_t dtype);
KuNode ku_constant_f32(KuGraph *g, const float *data, size_t len, const size_t *shape, size_t rank);
KuNode ku_constant(KuGraph *g, uint32_t dtype, const uint8_t *data, size_t nbytes, const size_t *shape, size_t rank);
KuNode ku_scalar(KuGraph *g, KuNode like, float v);

/* two-operand builders, kurumi.h:63-84 */
KuNode ku_add(KuGraph *g, KuNode a, KuNode b);
KuNode ku_sub(KuGraph *g, KuNode a, KuNode b);
KuNode ku_mul(KuGraph *g, KuNode a, KuNode b);
KuNode ku_div(KuGraph *g, KuNode a, KuNode b);
KuNode ku_max(KuGraph *g, KuNode a, KuNode b);
KuNode ku_min(KuGraph *g, KuNode a, KuNode b);
KuNode ku_idiv(KuGraph *g, KuNode a, KuNode b);
KuNode ku_and(KuGraph *g, KuNode a, KuNode b);
KuNode ku_or(KuGraph *g, KuNode a, KuNode b);
KuNode ku_xor(KuGraph *g, KuNode a, KuNode b);
KuNode ku_shl(KuGraph *g, KuNode a, KuNode b);
KuNode ku_shr(KuGraph *g, KuNode a, KuNode b);
KuNode ku_lt(KuGraph *g, KuNode a, KuNode b);
KuNode ku_eq(KuGraph *g, KuNode a, KuNode b);
KuNode ku_le(KuGraph *g, KuNode a, KuNode b);
KuNode ku_gt(KuGraph *g, KuNode a, KuNode b);
KuNode ku_ge(KuGraph *g, KuNode a, KuNode b);
KuNode ku_ne(KuGraph *g, KuNode a, KuNode b);

/* unary builders, kurumi.h:102-150 */
KuNode ku_neg(KuGraph *g, KuNode x);
KuNode ku_recip(KuGraph *g, KuNode x);
KuNode ku_sqrt(KuGraph *g, KuNode x);
KuNode ku_square(KuGraph *g, KuNode x);
KuNode ku_abs(KuGraph *g, KuNode x);
KuNode ku_floor(KuGraph *g, KuNode x);
KuNode ku_exp(KuGraph *g, KuNode x);
KuNode ku_exp2(KuGraph *g, KuNode x);
KuNode ku_ln(KuGraph *g, KuNode x);
KuNode ku_log2(KuGraph *g, KuNode x);
KuNode ku_sin(KuGraph *g, KuNode x);
KuNode ku_cos(KuGraph *g, KuNode x);
KuNode ku_relu(KuGraph *g, KuNode x);
KuNode ku_gelu(KuGraph *g, KuNode x);
KuNode ku_silu(KuGraph *g, KuNode x);
KuNode ku_sigmoid(KuGraph *g, KuNode x);
KuNode ku_tanh(KuGraph *g, KuNode x);
KuNode ku_logical_not(KuGraph *g, KuNode x);
KuNode ku_detach(KuGraph *g, KuNode x);                       /* kurumi.h:289 */

/* reductions and axis ops, kurumi.h:186-199,217 */
KuNode ku_sum(KuGraph *g, KuNode x, size_t axis);
KuNode ku_prod(KuGraph *g, KuNode x, size_t axis);
KuNode ku_mean(KuGraph *g, KuNode x, size_t axis);
KuNode ku_reduce_max(KuGraph *g, KuNode x, size_t axis);
KuNode ku_reduce_min(KuGraph *g, KuNode x, size_t axis);
KuNode ku_softmax(KuGraph *g, KuNode x, size_t axis);
/* indexing along one axis, kurumi.h:245-253. Gathers clamp out-of-range indices, scatters drop them; updates fold into a
 * copy of the operand in index order; scatter combine: 0 = set, 1 = add, 2 = max, 3 = min. sort = gather_along(x, argsort(x)). */
KuNode ku_gather(KuGraph *g, KuNode x, KuNode idx, size_t axis);
KuNode ku_gather_along(KuGraph *g, KuNode x, KuNode idx, size_t axis);
KuNode ku_take_along_dim(KuGraph *g, KuNode x, KuNode idx, size_t axis);
KuNode ku_sort(KuGraph *g, KuNode x, size_t axis, uint32_t descending);
KuNode ku_argsort(KuGraph *g, KuNode x, size_t axis, uint32_t descending);
KuNode ku_scatter(KuGraph *g, KuNode operand, KuNode indices, KuNode updates, size_t axis, uint32_t combine);
KuNode ku_scatter_along(KuGraph *g, KuNode operand, KuNode indices, KuNode updates, size_t axis, uint32_t combine);
KuNode ku_argmax(KuGraph *g, KuNode x, size_t axis); /* kurumi.h:193-194: I64 index of the first maximum / minimum */
KuNode ku_argmin(KuGraph *g, KuNode x, size_t axis);
KuNode ku_rmsnorm(KuGraph *g, KuNode x, size_t axis, float eps); /* kurumi.h:302 */
KuNode ku_clamp_min(KuGraph *g, KuNode x, float v);

/* contraction, kurumi.h:221-224 */
KuNode ku_matmul(KuGraph *g, KuNode a, KuNode b);
KuNode ku_dot_general(KuGraph *g, KuNode a, KuNode b, const size_t *lc, size_t nlc, const size_t *rc, size_t nrc,
                      const size_t *lb, size_t nlb, const size_t *rb, size_t nrb);

KuNode ku_where(KuGraph *g, KuNode cond, KuNode a, KuNode b);   /* kurumi.h:244 */

/* movement, kurumi.h:269-286 */
KuNode ku_reshape(KuGraph *g, KuNode x, const size_t *shape, size_t rank);
KuNode ku_expand(KuGraph *g, KuNode x, const size_t *shape, size_t rank);
KuNode ku_permute(KuGraph *g, KuNode x, const size_t *perm, size_t rank);
KuNode ku_transpose(KuGraph *g, KuNode x, size_t i, size_t j);
KuNode ku_flip(KuGraph *g, KuNode x, const size_t *axes, size_t n);
KuNode ku_slice(KuGraph *g, KuNode x, const size_t *ranges, size_t rank);      /* 2*rank (start,end) */
KuNode ku_slice_step(KuGraph *g, KuNode x, const size_t *ranges, size_t rank); /* 3*rank (start,end,step) */
KuNode ku_pad(KuGraph *g, KuNode x, const size_t *pads, size_t rank);          /* 2*rank (lo,hi), value 0 */
KuNode ku_broadcast_to(KuGraph *g, KuNode x, const size_t *shape, size_t rank);

/* generation and casts, kurumi.h:290-292 */
KuNode ku_iota(KuGraph *g, const size_t *shape, size_t rank, size_t axis, uint32_t dtype);
KuNode ku_cast(KuGraph *g, KuNode x, uint32_t dtype);
KuNode ku_bitcast(KuGraph *g, KuNode x, uint32_t dtype);

KuNode ku_sdpa(KuGraph *g, KuNode q, KuNode k, KuNode v, uint32_t causal);      /* kurumi.h:343 */

/* rng, kurumi.h:346-353 */
KuNode ku_rand_uniform(KuGraph *g, const size_t *shape, size_t rank, uint64_t seed);
KuNode ku_randn(KuGraph *g, const size_t *shape, size_t rank, uint64_t seed);
KuNode ku_rand_range(KuGraph *g, const size_t *shape, size_t rank, uint64_t seed, float lo, float hi);
KuNode ku_rand_uniform_keyed(KuGraph *g, const size_t *shape, size_t rank, KuNode seed);

/* backend + eval, kurumi.h:381-388 */
KuBackend *ku_backend_new(uint32_t kind); /* NULL if unavailable */
void ku_backend_free(KuBackend *b);
KuTensor *ku_eval(KuGraph *g, KuNode node, const KuBackend *backend);
KuTensor *ku_eval_with(KuGraph *g, KuNode node, const KuBackend *backend, const KuFeeds *feeds);
int32_t ku_eval_many(KuGraph *g, const KuNode *ids, size_t n, const KuBackend *backend, const KuFeeds *feeds,
                     KuTensor **out); /* 0 ok, -1 err */

/* weight-only quantised matmul, kurumi.h:225-234: act[M,K] x dequant(qweight)[N,K]^T -> [M,N] in act's dtype.
 * qweight is a KU_U8-packed tensor [N, K*bits/8], scales / mins are KU_F16 [N, K/group_size]; mins = KU_ERR for
 * symmetric. ku_quantize writes out_packed (rows*cols*bits/8 bytes), out_scales (rows*cols/group_size f16 bit
 * patterns) and out_mins (same count, or NULL when symmetric != 0); bits is 2, 4 or 8; bad arguments leave the
 * outputs untouched and set ku_last_error. */
KuNode ku_quant_matmul(KuGraph *g, KuNode act, KuNode qweight, KuNode scales, KuNode mins, uint8_t bits,
                       size_t group_size);
void ku_quantize(const float *w, size_t rows, size_t cols, uint8_t bits, size_t group_size, uint32_t symmetric,
                 uint8_t *out_packed, uint16_t *out_scales, uint16_t *out_mins);

/* passes and inspection, kurumi.h:395-405 */
KuNode ku_amp(KuGraph *g, KuNode root); /* mixed precision (f16 matmuls) */
size_t ku_node_count(const KuGraph *g, KuNode root);
size_t ku_dump(const KuGraph *g, KuNode root, uint8_t *out, size_t cap);
size_t ku_node_rank(const KuGraph *g, KuNode node);          /* SIZE_MAX on error */
void ku_node_shape(const KuGraph *g, KuNode node, size_t *out);
uint32_t ku_node_dtype(const KuGraph *g, KuNode node);       /* KU_ERR on error */

/* runnable-graph blobs (KGPH v2, the graph section of a `.hodu` artifact), kurumi.h:407-455: serialize a
 * graph with its output nodes and input bindings (node, role 0 = weight / 1 = runtime feed, name), and
 * rebuild it elsewhere. Size-then-write: cap = 0 with out = NULL returns the length; 0 on error. Blobs
 * whose nodes are outside this library's primitive set are refused by ku_graph_deserialize (NULL). */
size_t ku_graph_serialize(const KuGraph *g, const KuNode *outputs, size_t n_out, const KuNode *in_nodes,
                          const uint8_t *in_roles, const char *const *in_names, size_t n_in, uint8_t *out, size_t cap);
size_t ku_graph_serialize_reachable(const KuGraph *g, const KuNode *outputs, size_t n_out, const KuNode *in_nodes,
                                    const uint8_t *in_roles, const char *const *in_names, size_t n_in, uint8_t *out,
                                    size_t cap);
size_t ku_graph_serialize_multi(const KuGraph *g, size_t n_entries, const char *const *names,
                                const uint32_t *out_counts, const KuNode *outputs, const uint32_t *in_counts,
                                const KuNode *in_nodes, const uint8_t *in_roles, const char *const *in_names,
                                uint8_t *out, size_t cap);
KuRunnable *ku_graph_deserialize(const uint8_t *bytes, size_t len); /* NULL on a malformed or entry-less blob */
KuGraph *ku_runnable_take_graph(KuRunnable *h);                     /* call once; free with ku_graph_free */
size_t ku_runnable_output_count(const KuRunnable *h);               /* the non-entry accessors expose entry 0 */
KuNode ku_runnable_output(const KuRunnable *h, size_t i);
size_t ku_runnable_input_count(const KuRunnable *h);
KuNode ku_runnable_input_node(const KuRunnable *h, size_t i);
uint32_t ku_runnable_input_role(const KuRunnable *h, size_t i);
size_t ku_runnable_input_name(const KuRunnable *h, size_t i, uint8_t *out, size_t cap); /* UTF-8, no NUL; returns the full length */
size_t ku_runnable_entry_count(const KuRunnable *h);
size_t ku_runnable_entry_name(const KuRunnable *h, size_t i, uint8_t *out, size_t cap);
size_t ku_runnable_entry_output_count(const KuRunnable *h, size_t i);
KuNode ku_runnable_entry_output(const KuRunnable *h, size_t i, size_t j);
size_t ku_runnable_entry_input_count(const KuRunnable *h, size_t i);
KuNode ku_runnable_entry_input_node(const KuRunnable *h, size_t i, size_t j);
uint32_t ku_runnable_entry_input_role(const KuRunnable *h, size_t i, size_t j);
size_t ku_runnable_entry_input_name(const KuRunnable *h, size_t i, size_t j, uint8_t *out, size_t cap);
void ku_runnable_free(KuRunnable *h);

/* plan replay, kurumi.h:455-458 (kurumi/src/capi/eval.rs:152-182): compile once, run per feeds; constants are never
 * re-copied. The reference compiles for its f32 fused CPU path and returns NULL off it; this library compiles the
 * device program (kernels generated and built ahead of the first run) on a CUDA backend of its own on device 0,
 * shared by all plans, and returns NULL only for a graph no kernel can evaluate. ku_plan_run takes the same graph. */
typedef struct KuPlan KuPlan;
KuPlan *ku_plan_compile(const KuGraph *g, KuNode node);
KuTensor *ku_plan_run(const KuPlan *p, const KuGraph *g, const KuFeeds *feeds);
void ku_plan_free(KuPlan *p);

/* feeds, kurumi.h:461-463 */
KuFeeds *ku_feeds_new(void);
void ku_feeds_free(KuFeeds *f);
void ku_feeds_set(KuFeeds *f, KuNode node, const KuTensor *tensor); /* copies the tensor */

/* tensors, kurumi.h:466-479 */
KuTensor *ku_tensor_f32(const float *data, size_t len, const size_t *shape, size_t rank);
KuTensor *ku_tensor_new(uint32_t dtype, const uint8_t *data, size_t nbytes, const size_t *shape, size_t rank);
void ku_tensor_free(KuTensor *t);
size_t ku_tensor_rank(const KuTensor *t);
void ku_tensor_shape(const KuTensor *t, size_t *out);
size_t ku_tensor_len(const KuTensor *t);
uint32_t ku_tensor_dtype(const KuTensor *t);
ptrdiff_t ku_tensor_data_f32(const KuTensor *t, float *out, size_t cap);
size_t ku_tensor_nbytes(const KuTensor *t);
void ku_tensor_bytes(const KuTensor *t, uint8_t *out);

#ifdef __cplusplus
}
#endif
#endif /* KURUMI_H */
