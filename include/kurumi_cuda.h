/* Extensions of the kurumi C ABI that only the CUDA library exports: device-resident tensors and
 * evaluation (so a caller can keep weights and activations in HBM between evals), the backend's
 * stream, timing and launch statistics, and the mixed-precision pass with a target dtype.
 * None of these has a counterpart in the reference header kurumi/include/kurumi.h; the closest
 * reference behaviour is cited per entry. Same conventions as kurumi.h: opaque handles, NULL / -1
 * / KU_ERR on error with the message in ku_last_error(), not thread-safe per handle. */
#ifndef KURUMI_CUDA_H
#define KURUMI_CUDA_H

#include "kurumi.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct KuDevTensor KuDevTensor;
typedef struct KuDevFeeds KuDevFeeds;

/* A CUDA backend on a chosen device of this process (ku_backend_new(KU_CUDA) uses device 0).
 * Fails (NULL) when no sm_100 device is visible: there is no CPU fallback. */
KuBackend *ku_cuda_backend_new(int32_t device);

/* Host -> device copy of a tensor into a new device tensor (stream-ordered on the backend's
 * stream). ku_cuda_upload_bytes reads `nbytes` from the caller's buffer, which must stay valid
 * until ku_cuda_sync when it is pinned memory. Reference analogue: the Metal backend's const
 * upload, kurumi_metal/src/backend/eval_walk.rs:99-114. */
KuDevTensor *ku_cuda_upload(const KuBackend *b, const KuTensor *t);
KuDevTensor *ku_cuda_upload_bytes(const KuBackend *b, uint32_t dtype, const void *data, size_t nbytes, const size_t *shape, size_t rank);
/* Device -> host: a new KuTensor, or raw bytes into `out` (>= ku_cuda_dev_nbytes). Both wait for the result. */
KuTensor *ku_cuda_download(const KuBackend *b, const KuDevTensor *t);
int32_t ku_cuda_download_bytes(const KuBackend *b, const KuDevTensor *t, void *out, size_t cap);
void ku_cuda_dev_free(const KuBackend *b, KuDevTensor *t);
void *ku_cuda_dev_ptr(const KuDevTensor *t);
size_t ku_cuda_dev_nbytes(const KuDevTensor *t);
size_t ku_cuda_dev_rank(const KuDevTensor *t);
void ku_cuda_dev_shape(const KuDevTensor *t, size_t *out);
uint32_t ku_cuda_dev_dtype(const KuDevTensor *t);

/* Feeds that already live on the device (the tensor is borrowed, not copied). */
KuDevFeeds *ku_cuda_dev_feeds_new(void);
void ku_cuda_dev_feeds_free(KuDevFeeds *f);
void ku_cuda_dev_feeds_set(KuDevFeeds *f, KuNode node, const KuDevTensor *t);

/* ku_eval_many (kurumi.h:387) with device-resident outputs: evaluates ids[0..n] in one shared
 * pass and writes a new KuDevTensor per id into out. `feeds` and `dev_feeds` may each be NULL.
 * Asynchronous: returns once the work is queued on the backend's stream. 0 ok, -1 error. */
int32_t ku_cuda_eval_device(KuGraph *g, const KuNode *ids, size_t n, const KuBackend *b, const KuFeeds *feeds,
                            const KuDevFeeds *dev_feeds, KuDevTensor **out);

int32_t ku_cuda_sync(const KuBackend *b);        /* wait for the backend's stream */
void *ku_cuda_stream(const KuBackend *b);        /* the cudaStream_t every launch of this backend goes to */
int32_t ku_cuda_device(const KuBackend *b);

/* Counters since backend creation, in this order: kernel launches, NVRTC compiles, NVRTC cache
 * hits, host->device bytes, device->host bytes, device allocations, pool hits. Returns how many
 * were written. Reference analogue: KURUMI_PHASE statistics, kurumi_metal/src/backend.rs:68-90. */
size_t ku_cuda_stats(const KuBackend *b, uint64_t *out, size_t cap);
/* Per-kernel-family device time, measured with CUDA events around every launch while enabled.
 * ku_cuda_profile_take writes a text table ("family launches ms algo_bytes flops" per line) into
 * out (no NUL), returns its full length, and resets the accumulators. Reference analogue:
 * KURUMI_GPUTIME, kurumi_metal/src/context/encoder.rs:44-47. */
void ku_cuda_profile_enable(const KuBackend *b, uint32_t on);
size_t ku_cuda_profile_take(const KuBackend *b, uint8_t *out, size_t cap);

/* ku_amp (kurumi.h:395) with a target dtype: KU_F16 is the reference pass; KU_BF16 the same
 * rewrite in bf16; KU_F8E4M3 quantises both operands of every contraction through
 * cast(cast(x, F8E4M3), dtype) so the backend can feed fp8 to the tensor cores. */
KuNode ku_cuda_amp_to(KuGraph *g, KuNode root, uint32_t dtype);

/* The explicit forms of ku_sdpa (kurumi.h:343), which picks between them by the size of the score
 * buffer: the fused primitive Op::Sdpa and the dot + softmax decomposition. They are public in the
 * Rust API (kurumi_core/src/graph/ops/nn/attention.rs:97-133) but absent from the reference's C header. */
KuNode ku_sdpa_fused(KuGraph *g, KuNode q, KuNode k, KuNode v, uint32_t causal);
KuNode ku_sdpa_decomposed(KuGraph *g, KuNode q, KuNode k, KuNode v, uint32_t causal);

/* Softmax over strided lines on raw device pointers: out[i * len + j] = softmax over j of
 * (in[j * ld + i] + bias[j]) for i < lines, j < len, f32; bias may be NULL. It is the kernel the
 * graph path runs for a softmax consumed through a transpose view (Op::Softmax, kurumi_core/src/
 * graph/op.rs:48-51, oracle kurumi_core/src/interp/nn.rs:35-69), callable without recording a
 * graph. Queued on the backend's stream; scratch comes from the backend's device pool. 0 ok, -1 error. */
int32_t ku_cuda_softmax_lines_f32(const KuBackend *b, const float *in, const float *bias, float *out, size_t lines, size_t len, size_t ld);

/* The same softmax for callers that must not allocate device memory when they call it: a
 * latency-critical loop that cannot take the device-wide synchronisation cudaMalloc / cudaFree may
 * imply, a host application that owns all of HBM through its own arena, or code running where the
 * CUDA allocator must not be entered (another library's allocation hook). No counterpart in the reference:
 * kurumi has no device entry point of this kind. The scratch is a fixed 8 MiB array in the library's device
 * image (every GPU that loads the library holds it until exit), so the call is rejected with -1 when
 * lines * ceil(len / 128) * 8 + lines * 4 bytes exceed 8 MiB (for example 8192 lines of 8192 fit,
 * 16384 lines of 16384 do not), and, like the entry above, for lines longer than 65535 * 64 positions.
 * Runs on `stream`, a cudaStream_t that must belong to the device that is current when the call is made (the
 * scratch address is looked up for the current device; the call does not check whose stream it was given).
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and, with the
 * runtime's lazy loading, is also when the kernels and the array are placed on that GPU: make one small real
 * call per device (a few lines, so that all three kernels load) at start-up, before HBM is handed away and
 * before any stream capture begins; later calls neither allocate nor load. All calls share the one array:
 * nothing in it needs clearing between calls, but two calls whose kernels can overlap on the GPU
 * (different streams, no dependency) race on it. No cudaMalloc / cudaFree. */
int32_t ku_cuda_softmax_lines_f32_noalloc(const float *in, const float *bias, float *out, size_t lines, size_t len, size_t ld, void *stream);

/* Everything the backend caches for a graph - compiled programs with their scratch buffers, uploaded constants,
 * chunk pipelines with their device buffers - lives until the backend is freed or until this call; call it before
 * ku_graph_free in a process that records many graphs. Reference analogue: the Metal backend's per-graph caches,
 * kurumi_metal/src/backend.rs:95-109, which die with the backend. */
void ku_cuda_release_graph(const KuBackend *b, const KuGraph *g);

/* Assembly of a row-sharded result over NCCL (NVLink / NVSwitch), one process per GPU: rank 0 makes a 128-byte id
 * (ku_cuda_comm_unique_id) and hands it to the other ranks by any host channel; every rank then calls
 * ku_cuda_comm_init (collective) on its backend. ku_cuda_all_gather_rows returns, on every rank, a new device tensor
 * [world * rows, ...] holding the ranks' shards in rank order; it is queued on the backend's stream. Shards must have
 * the same shape on every rank. The sharded evaluation itself needs no exchange (each rank evaluates the part graph of
 * ku_graph_row_split on its slices); this is only for callers that want the whole result on one device. 0 / non-NULL
 * ok, -1 / NULL error. No counterpart in the reference, which is single-device (kurumi_core/src/backend.rs:14-31). */
int32_t ku_cuda_comm_unique_id(uint8_t *out128);
int32_t ku_cuda_comm_init(const KuBackend *b, const uint8_t *id128, int32_t rank, int32_t world);
void ku_cuda_comm_free(const KuBackend *b);
KuDevTensor *ku_cuda_all_gather_rows(const KuBackend *b, const KuDevTensor *shard);

/* Row splitting: a new graph whose root yields rows [c, c + 1) * rows / parts (axis 0) of `root`, for any part c, given
 * the matching slice of every input the root depends on row-wise and all of the others. Writes the part graph's root
 * to *part_root, the number of Input nodes in the root's cone to *n_inputs and, for the first `cap` of them, the
 * original node, the part graph's node and the axis to slice (-1: the part needs the whole tensor). NULL with a reason
 * in ku_last_error() when the evaluation does not separate by rows (a reduction or softmax along the split axis,
 * attention split over its queries, ...) or the extents do not divide. Free the result with ku_graph_free. The CUDA
 * backend uses the same analysis inside ku_eval_with to pipeline large host-buffer evaluations, and callers use it to
 * shard one evaluation over several GPUs. The reference evaluates a graph in one piece on one device
 * (kurumi_core/src/backend.rs:14-31): no counterpart. Pure graph code: the test oracle exports it too. */
KuGraph *ku_graph_row_split(const KuGraph *g, KuNode root, size_t parts, KuNode *part_root, KuNode *orig_inputs, KuNode *part_inputs, int32_t *axes, size_t cap,
                            size_t *n_inputs);

/* Compile every kernel the evaluation of ids[0..n] needs to an sm_100a cubin, without a GPU.
 * Writes the kernel family of each launch, one per line, into out (no NUL); returns the full
 * length, or (size_t)-1 on error. */
size_t ku_cuda_compile_check(KuGraph *g, const KuNode *ids, size_t n, uint8_t *out, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* KURUMI_CUDA_H */
