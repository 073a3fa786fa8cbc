/*
 * spdnn_b200 -- C ABI of the B200 (sm_100a) sparse-DNN inference path
 *     Y_{l+1} = min(clip, ReLU(Y_l W_l + bias)),  l = 0 .. L-1
 * with Y a batch x N activation matrix and every W_l an N x N sparse matrix
 * (Graph Challenge networks: 32 non-zeros per column, all 0.0625).
 *
 * It replaces, behind plain pointers and sizes, the GPU execution functions of the
 * reference (paths relative to the reference's project root):
 *   ftxj::test_benchmark_graph_challenge            src/microbenchmark/header.h:16-19,
 *                                                   defined src/microbenchmark/all_network.cu:207-526
 *                                                   (64-bit/streaming variant src/microbenchmark/out_memory.cu:208)
 *   ftxj::test_benchmark_multi_gpu_graph_challenge  src/microbenchmark/multi_gpu/header.h:5-14,
 *                                                   defined src/microbenchmark/multi_gpu/multi_gpu.cu:207
 * and the CUDA plumbing they use (ftxj::GpuEnv, src/gpu_lib/gpu_env.h:11-89; Safe_Call,
 * src/gpu_lib/gpu_runtime.h:6-17).  Those functions take the output of the reference's
 * inspector, which carries no sparsity pattern beyond its block assumptions, so the seam
 * here is one step earlier: the data the drivers load -- one COO/CSC matrix per layer
 * (src/utils/matrix.h:255-282) and the input images (src/network.cpp:33-54).
 *
 * Conventions: every function returns SPDNN_OK (0) or a negative status and never exits
 * the process (the reference's Safe_Call does); spdnn_last_error() gives the message.
 * Host buffers that describe LAYERS are borrowed for the duration of the call.  Host buffers that hold
 * INPUT images are copied with cudaMemcpyAsync on the context's stream: from pageable memory the
 * copy has read the buffer when the call returns, from page-locked (pinned) memory it may still be
 * reading it, so keep a pinned input buffer unchanged until the next call that waits for the stream
 * (spdnn_infer, spdnn_sync, spdnn_get_*) has returned.  All device memory belongs to
 * the context and is released by spdnn_destroy().  One context drives one GPU; different
 * contexts may be used from different host threads concurrently (no mutable state is shared
 * between contexts), one context must not be used by two threads at once.
 */
#ifndef SPDNN_B200_H
#define SPDNN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct spdnn spdnn_t;

enum {
    SPDNN_OK = 0,
    SPDNN_ERR_ARG = -1,      /* bad argument (shape, range, null pointer, order of calls) */
    SPDNN_ERR_CUDA = -2,     /* a CUDA runtime call failed; message holds the CUDA error */
    SPDNN_ERR_MEMORY = -3,   /* host or device allocation failed */
    SPDNN_ERR_STATE = -4,    /* call made before its prerequisites (layers/input missing) */
    SPDNN_ERR_DEVICE = -5,   /* a kernel reported an internal inconsistency */
    SPDNN_ERR_LIMIT = -6     /* a fixed capacity of the library was exceeded */
};

/* Largest number of images one spdnn_layer_static call accepts (its scratch is a fixed array). */
#define SPDNN_STATIC_MAX_IMAGES 2097152

/* Filled by spdnn_infer / spdnn_sync. */
typedef struct spdnn_stats {
    int32_t layers;             /* layers executed */
    int32_t batch;              /* images the input held */
    int64_t survivors;          /* images alive after the last layer */
    float prepare_ms;           /* device time of the input layout conversion of the last set_input */
    float infer_ms;             /* device time of the layer loop incl. on-device compaction (CUDA events) */
    double algorithmic_bytes;   /* sum over layers of 4N(live_in + live_out) + bytes of W_l as CSC */
    int64_t kernel_launches;    /* kernels of this library launched by the last infer (+ last set_input) */
    int32_t loop_launches;      /* of those, launches of the layer loop (1 per layer, or 1 per chunk of layers) */
    int32_t resident_group;     /* images per block of the shared-memory-resident kernel, 0 = per-layer kernel */
} spdnn_stats_t;

/* Replaces GpuEnv::GpuEnv(gpu_id) + the allocations of all_network.cu:283-303.
 * clip is 32 in the reference (all_network.cu:8-10). */
int spdnn_create(spdnn_t **ctx, int device, int neurons, int layers, float bias, float clip);

/* Layer `layer` (0-based) as CSC: column c = output neuron c holds input neurons
 * row_idx[col_ptr[c] .. col_ptr[c+1]) with weights val[...] (val == NULL: every weight is
 * 0.0625, the constant the reference's inspector assumes, src/inspector/matrix_block_container.h:218).
 * Rows of a column may come in any order; they are summed in ascending row order, the
 * order of the reference's CPU loop (src/utils/cpu_spmm.h:12-43).  Replaces the per-layer
 * upload all_network.cu:296-303 and the inspector pass src/network.cpp:97-121. */
int spdnn_set_layer_csc(spdnn_t *ctx, int layer, const int32_t *col_ptr, const int32_t *row_idx, const float *val);

/* Same layer given as the triplets of the reference's layer file: line `a b v` means
 * W[a][b] = v, a = input neuron, b = output neuron, index_base = 1 in the files
 * (src/utils/matrix.h:255-282 with T == false). */
int spdnn_set_layer_coo(spdnn_t *ctx, int layer, int64_t nnz, const int32_t *in_neuron, const int32_t *out_neuron,
                        const float *val, int index_base);

/* Layer `layer` is the same matrix as `other_layer`, which was set before: both share one device
 * copy and the host-side preparation is not repeated.  (spdnn_set_layer_csc finds equal layers by
 * content as well, but only after canonicalising the new one.)  The reference uploads every layer
 * separately (all_network.cu:296-303); networks whose layers repeat with a short period -- its
 * stride table all_network.cu:316-327 cycles -- make this the cheap way to declare 1920 of them. */
int spdnn_set_layer_same_as(spdnn_t *ctx, int layer, int other_layer);

/* Input images, dense batch x N row-major fp32 in HOST memory (the reference's `input`
 * vectors flattened, all_network.cu:240-248, 283-284).  Image i gets the global number
 * first_global_id + i.  Replaces the H2D upload of A_d. */
int spdnn_set_input_dense(spdnn_t *ctx, const float *y0, int batch, int first_global_id);

/* Same, from a DEVICE buffer on the context's GPU (inputs already resident in HBM).  The buffer
 * may be read in place by the inference pass that follows (when its first launch can take a
 * row-major matrix; otherwise it is converted to the internal layout here): keep it unchanged
 * until that pass has finished (spdnn_infer returned, or spdnn_sync after spdnn_infer_async).
 * It is never written. */
int spdnn_set_input_dense_device(spdnn_t *ctx, const float *y0_dev, int batch, int first_global_id);

/* Input images as the triplets of the reference's input file: `img neuron val`
 * (src/network.cpp:33-54; index_base = 1 in the file).  img is relative to this shard:
 * img - index_base in [0, batch). */
int spdnn_set_input_coo(spdnn_t *ctx, int64_t nnz, const int32_t *img, const int32_t *neuron, const float *val,
                        int batch, int first_global_id, int index_base);

/* Input images as a bit matrix in HOST memory: image i is row i of `row_bytes` bytes, bit (n & 7) of byte
 * n >> 3 set = neuron n of the image is 1.0, clear = 0.0 (numpy: packbits(y0 != 0, axis=1, bitorder="little")).
 * row_bytes is a multiple of 4 and at least ceil(neurons / 8).  The challenge's inputs are binary -- every
 * entry of the reference's input file carries the value 1 (src/network.cpp:49-51 logs anything else) -- so this
 * is the same information as spdnn_set_input_coo's triplets or spdnn_set_input_dense's matrix in 1/32 of the
 * dense bytes; it replaces the same H2D upload of A_d (all_network.cu:283-284).  The _device form takes the
 * matrix from a 4-byte aligned buffer on the context's GPU. */
int spdnn_set_input_bits(spdnn_t *ctx, const uint8_t *bits, int64_t row_bytes, int batch, int first_global_id);
int spdnn_set_input_bits_device(spdnn_t *ctx, const uint8_t *bits_dev, int64_t row_bytes, int batch, int first_global_id);

/* The layer loop of all_network.cu:333-519: all layers on the images of the last
 * set_input, with dead images removed on the device after every layer.  Blocks until the
 * result is on the device and fills *stats (may be NULL).  Consumes the input. */
int spdnn_infer(spdnn_t *ctx, spdnn_stats_t *stats);

/* Asynchronous form: enqueue on the context's stream and return; spdnn_sync waits and
 * fills the statistics.  A set_input call made while a pass is in flight does not wait: the
 * new input is ordered behind that pass on the stream and the pass's unfetched results are
 * dropped, so passes can be queued back to back and only the last one synchronised. */
int spdnn_infer_async(spdnn_t *ctx);
int spdnn_sync(spdnn_t *ctx, spdnn_stats_t *stats);

/* Use the caller's CUDA stream (a cudaStream_t passed as void*) for everything the context
 * enqueues from now on; NULL restores the context's own stream.  Replaces
 * GpuEnv::get_stream (gpu_env.h:85-87). */
int spdnn_set_stream(spdnn_t *ctx, void *cuda_stream);

/* live[l] = images alive after layer l: the numbers of the reference's
 * "layer l, batch = k" lines (all_network.cu:508).  capacity >= layers. */
int spdnn_get_layer_live(spdnn_t *ctx, int32_t *live, int capacity);

/* Ascending global image numbers alive after the last layer (the challenge's category
 * list; the reference prints only the count). */
int spdnn_get_categories(spdnn_t *ctx, int32_t *ids, int capacity, int *count);

/* Final activations of the survivors, count x N row-major fp32 in host memory, rows in the
 * order of spdnn_get_categories (the reference copies C back at all_network.cu:521). */
int spdnn_get_activations(spdnn_t *ctx, float *y, int64_t capacity_rows);

/* How the library stored layer `layer`: classes = number of distinct columns (columns with
 * identical rows and weights are computed once), k = padded non-zeros per column,
 * uniform = 1 when all weights are one power-of-two constant.  Any pointer may be NULL. */
int spdnn_get_layer_info(spdnn_t *ctx, int layer, int *classes, int *k, int *uniform);

/* The layer preparation alone, on the host, without a context or a GPU: how a CSC layer of
 * `neurons` columns would be stored (same outputs as spdnn_get_layer_info).  Returns
 * SPDNN_ERR_ARG for a malformed layer.  It takes the place of running the reference's
 * inspector stand-alone (src/main.cpp:57-92). */
int spdnn_inspect_layer_csc(int neurons, const int32_t *col_ptr, const int32_t *row_idx, const float *val,
                            int *classes, int *k, int *uniform);

/* The analysis of a whole network, on the host, without a context or a GPU: for every layer the
 * number of classes when it is expressed in the value ids of the layer before it, the number of
 * value ids it reads (v_in[l] == classes[l-1], or `neurons` where the layer before has no
 * repeated columns) and the table form the resident kernel would use (0 = K gathers per class,
 * 1 = alternating pair).  Layer l is given as CSC through col_ptr[l], row_idx[l], val[l]
 * (val or val[l] may be NULL: all weights 0.0625).  Output arrays hold `layers` entries and
 * may be NULL. */
int spdnn_inspect_network_csc(int neurons, int layers, const int32_t *const *col_ptr, const int32_t *const *row_idx,
                              const float *const *val, int32_t *classes, int32_t *v_in, int32_t *form);

/* One layer, for callers that cannot allocate device memory when they run it (a plugin inside
 * another runtime's memory pool, a callback where cudaMalloc's implicit synchronisation is
 * forbidden, a process whose footprint is frozen after start-up).  This entry point has no
 * counterpart in the reference; it runs the same layer arithmetic as spdnn_infer on buffers
 * the caller owns and keeps its own scratch (survivor ballots, block counters) in a fixed
 * array inside the loaded module, so it calls no cudaMalloc / cudaFree and needs no context.
 *
 *   yin, yout      device, tile layout: tile t holds images 32t..32t+31 as [neurons + 1][32]
 *                  floats (row r = neuron r for the 32 images, row `neurons` = zeros, used
 *                  as padding target); yout must not alias yin
 *   live_in        images to process; image j is read from position in_positions[j] of yin
 *                  (device array, or NULL for j) and written to position j of yout
 *   off            device [neurons][k]: for output neuron c the k input rows times 32,
 *                  ascending; pad short columns with neurons * 32.  k: multiple of 4
 *   vals           device [neurons][k] weights, or NULL: every weight is w (a power of two)
 *   survivors      device out, capacity live_in: ascending positions in yout of the images
 *                  with a non-zero activation; survivor_count: device out, their number
 *   cuda_stream    cudaStream_t as void* (NULL = default stream); the call only enqueues
 *   err, err_len   optional host buffer that receives the message of a failure
 *
 * What a caller that chains calls must know: positions live_in .. 32 * ceil(live_in / 32) - 1 of yout (the
 * unused lanes of the last tile) are overwritten with a copy of that tile's first image; row `neurons`
 * of yout is never written, so a buffer that is fed back as yin must have that row zeroed once by its
 * owner; live_in == 0 is valid (survivor_count becomes 0, nothing else is written).
 *
 * Limits: neurons < 2^26; at most SPDNN_STATIC_MAX_IMAGES images per call (SPDNN_ERR_LIMIT beyond that: split
 * the batch).  The scratch array (about 264 KB) is held by every GPU that loads the library
 * until the process exits and is shared by all calls on that GPU: calls that overlap on the
 * device race, so keep them on one stream or order them with events.  The first call on a
 * device also looks up the array's device address and the launch shape; make that call
 * before any stream capture. */
int spdnn_layer_static(const float *yin, float *yout, int neurons, int live_in, const int32_t *in_positions,
                       const int32_t *off, const float *vals, int k, float w, float bias, float clip,
                       int32_t *survivors, int32_t *survivor_count, void *cuda_stream, char *err, int err_len);

const char *spdnn_last_error(const spdnn_t *ctx);
void spdnn_destroy(spdnn_t *ctx);

/* Library version string. */
const char *spdnn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SPDNN_B200_H */
