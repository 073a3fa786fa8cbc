// C ABI of the sm_100a sparse-DNN inference path (declarations: include/spdnn_b200.h).
//
// Host side of what the reference does in ftxj::test_benchmark_graph_challenge
// (src/microbenchmark/all_network.cu:207-526): own the device buffers, upload layers and
// inputs, run the layer loop, hand back survivors.  Differences that matter to a caller:
// errors come back as status codes instead of exit() (src/gpu_lib/gpu_runtime.h:6-17), the
// layer loop has no host round-trip (the reference synchronises and copies active[] every
// layer, all_network.cu:444-510) and is replayed from one CUDA graph, and everything
// allocated is freed by spdnn_destroy.
#include "../../include/spdnn_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "layer_inspect.h"
#include "spdnn_kernels.cuh"
#include "spdnn_alt2.cuh"
#include "spdnn_bits.cuh"
#include "spdnn_front.cuh"
#include "spdnn_resident.cuh"

using namespace spdnn_impl;

namespace {

// Device copy of one layer's tables for the per-layer kernel, plus the canonical host form
// the resident kernel's tables are derived from when the whole network is known.
struct DevLayer {
    int32_t *off = nullptr;
    float *vals = nullptr;
    int32_t *mem_ptr = nullptr;
    int32_t *mem = nullptr;
    int classes = 0, k = 0;
    bool uniform = false, identity_members = false;
    float w = 0.0f;
    int64_t nnz = 0;
    uint64_t h1 = 0, h2 = 0;
    int device = 0;
    std::shared_ptr<HostLayer> host;      // null when the host copy was not kept (resident kernel unavailable)
    // Streamed layer (the device budget for weights was used up when it was set): the four tables live in ONE
    // block of page-locked host memory, [off][vals][mem_ptr][mem], and are copied into one of two device slots
    // while the layer before runs; off/vals/mem_ptr/mem above stay null.
    unsigned char *pinned = nullptr;
    size_t pinned_bytes = 0, o_vals = 0, o_mem_ptr = 0, o_mem = 0;
    ~DevLayer() {
        cudaSetDevice(device);
        cudaFree(off); cudaFree(vals); cudaFree(mem_ptr); cudaFree(mem);
        if (pinned) cudaFreeHost(pinned);
    }
};

// Device copy of one layer's tables for the resident kernel.  They depend on the layer AND on
// the classes of the layer before it (its value ids).
struct DevRes {
    int32_t *blob = nullptr, *rep = nullptr, *mem_ptr = nullptr, *mem = nullptr;
    int blob_bytes = 0, o_vals = 0, classes = 0, k = 0, v_in = 0, mode = 0;
    bool uniform = false;
    float w = 0.0f;
    std::vector<int32_t> class_of;        // value ids this layer hands to the next one
    uint64_t partition_hash = 0;
    int device = 0;
    ~DevRes() {
        cudaSetDevice(device);
        cudaFree(blob); cudaFree(rep); cudaFree(mem_ptr); cudaFree(mem);
    }
};

}  // namespace

struct spdnn {
    int device = 0, n = 0, layers = 0;
    float bias = 0.0f, clip = 32.0f;
    int sm_count = 0;
    cudaStream_t own_stream = nullptr, stream = nullptr;
    cudaEvent_t ev_prep0 = nullptr, ev_prep1 = nullptr, ev_inf0 = nullptr, ev_inf1 = nullptr;

    std::vector<std::shared_ptr<DevLayer>> layer;
    std::unordered_map<uint64_t, std::weak_ptr<DevLayer>> shared;   // content hash -> layer
    std::vector<std::shared_ptr<DevRes>> res;                        // per layer, built when the graph is
    std::unordered_map<uint64_t, std::weak_ptr<DevRes>> res_shared;  // (layer, input partition) -> tables
    size_t host_bytes = 0, host_budget = (size_t)16 << 30;           // canonical layers kept on the host
    // Out-of-core weights: per-layer tables beyond weight_budget bytes of device memory stay in page-locked host
    // memory and are streamed through two device slots by a copy stream, double-buffered against the layer loop
    // (what the reference's out_memory.cu:315-329, 368-388 does with its second stream).
    size_t weight_bytes = 0, weight_budget = ~(size_t)0;             // SPDNN_WEIGHT_BUDGET_MB
    unsigned char *wslot[2] = {nullptr, nullptr};
    size_t wslot_bytes = 0;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_ready[2] = {nullptr, nullptr}, ev_free[2] = {nullptr, nullptr};
    int streamed_launches = 0;         // of the captured schedule

    long long tile_stride = 0;
    int tiles_cap = 0;
    float *y[2] = {nullptr, nullptr};
    LoopCtl *ctl = nullptr;            // one record per launch boundary (at most layers + 1)
    int32_t *died_at = nullptr;        // [layers] images that died in each layer
    ResLayer *res_table = nullptr;     // [layers] tables of the resident kernel
    bool resident = true;              // use the shared-memory-resident kernel where a chunk fits
    bool reps_only = true;             // SPDNN_REPS_ONLY=0: every launch writes all N rows
    bool exact_shortcut = false;       // SPDNN_EXACT_SHORTCUT=1: exact-sum shortcut of the ALT2 float form (off: saturated tiles leave the
                                       // float form anyway, and elsewhere its test costs more than it saves -- measured)
    bool bit_form = true;              // SPDNN_BIT_FORM=0 disables the bit form of saturated activations (ALT2)
    int table_ring_max = 2;            // SPDNN_TABLE_RING=2|4: most staged groups of ALT2 tables in flight or in use
    int word_ring_max = 33;            // SPDNN_WORD_RING: most word buffers of the bit form (layers per group + 1)
    int table_group_max = 32;          // SPDNN_TABLE_GROUP=1..32: most layers one bulk copy brings
    std::vector<unsigned char *> streams;   // packed ALT2 table streams of the captured schedule (one per chunk)
    bool print_schedule = false;       // SPDNN_PRINT_SCHEDULE=1: one line per launch when the graph is built
    bool resident_always = false;      // ... even for a lone layer that the per-layer kernel would serve better
    int res_ti_max = 32;               // largest group of images per block to try
    int res_ipt_max = 8;               // most images per thread to try
    int last_group = 0;                // group size of the last captured schedule's resident launches
    int smem_optin = 0;                // shared memory one block may opt in to
    bool stage_tables = true;          // bring the per-layer tables into shared memory with bulk copies
    int chunk_first = 8, chunk_max = 2048, chunk_growth = 4;      // SPDNN_CHUNK_FIRST / _MAX / _GROWTH
    std::vector<int> chunk_list;       // SPDNN_CHUNKS=a,b,c,...: lengths of the first resident chunks of a pass, in order
    bool chunk_growth_set = false;     // SPDNN_CHUNK_GROWTH was given: it applies to every chunk
    int chunk_growth_generic = 2;      // GENERIC chunks grow more slowly: a tile that is not saturated when its chunk starts
                                       // stays in the float form to the chunk's end, and that form costs 32 gathers per output
    int nsteps = 0;                    // launches of the last captured schedule
    std::vector<int32_t> host_died, host_live;
    int32_t *slot = nullptr;
    uint32_t *mask = nullptr;
    unsigned char *tile_done = nullptr;   // [tiles] verdict of the bits_kernel pre-pass of an ALT2 chunk
    // Binary inputs (spdnn_front.cuh): the input as one word per (tile, neuron); in_flag is raised on the device
    // while an input is converted when it holds a value other than 0 and 1, and picks the variant of the first
    // layer's launches; has_floats marks the tiles whose float form was written.
    uint32_t *xw = nullptr;
    int nw = 0;
    int32_t *in_flag = nullptr;
    unsigned char *has_floats = nullptr;
    bool binary_front = true;          // SPDNN_BINARY_FRONT=0: inputs are always converted to float tiles
    bool count_front = true;           // SPDNN_COUNT_FRONT=0: layer 0 of a binary input always gathers per image
    bool bits_prepass = true;          // SPDNN_BITS_KERNEL=0: ALT2 chunks of wide layers run without the pre-pass
    bool bits_first_chunk = false;     // SPDNN_BITS_FIRST=1: also before the first resident chunk of a pass
    bool bits_small = false;           // SPDNN_BITS_SMALL=1: the pre-pass also for chunks whose layers have at most 64 classes
                                       // (one warp per 32 images)
    bool table_cache = true;           // SPDNN_TABLE_CACHE=0: the pre-pass always streams its layer records
    bool two_blocks = true;            // SPDNN_TWO_BLOCKS=0: ALT2 chunks keep the largest group of images per block even where it leaves one block per SM
    int alt2_threads = 0;              // SPDNN_ALT2_THREADS=256|512: block size of ALT2 chunks with 4 images per thread (0: by shared memory)
    int bits_threads = 0;              // SPDNN_BITS_THREADS: threads per block of the pre-pass (0: by the classes)
    int extra_launches = 0;            // pre-pass launches of the captured schedule
    int graph_extra[2] = {0, 0};
    int32_t *ids[2] = {nullptr, nullptr};
    unsigned int *counter = nullptr;   // [0] blocks finished, [1] next work item
    int32_t *status = nullptr;

    void *stage = nullptr;             // device staging for host inputs / outputs
    size_t stage_bytes = 0;
    size_t stage_chunk = (size_t)512 << 20;   // SPDNN_STAGE_KB: most bytes of a host input staged per copy

    int batch = 0, first_id = 0;
    bool input_ready = false, result_ready = false, in_flight = false, prep_timed = false;
    // One captured pass per kind of input: [0] the input is in tiles (y[0]); [1] the first launch reads the
    // caller's row-major matrix in place (only when that launch is a resident chunk; else null).
    cudaGraphExec_t graph_exec[2] = {nullptr, nullptr};
    int graph_steps[2] = {0, 0}, graph_group[2] = {0, 0};
    bool graph_dirty = true;
    bool alt2_small_blocks = true;     // SPDNN_ALT2_SMALL_BLOCKS=0: 256-thread blocks also for layers of <= 64 classes
    bool lazy_expand = true;           // SPDNN_LAZY_EXPAND=0: the last launch of a pass writes all member rows itself
    int expand_layer_of_plan = -1;     // set by enqueue_layers
    int graph_expand_layer[2] = {-1, -1};   // per captured pass: the layer whose classes spdnn_get_activations must
                                            // still expand to all member rows (-1: the tiles are complete)
    bool final_needs_expand = false;   // ... pending for the pass that ran last
    int final_expand_layer = -1;
    bool dense_direct = false;         // SPDNN_DENSE_DIRECT=1: let the first launch read a dense input in place where
                                       // it can (measured slower than the layout pass + per-layer kernel at N = 1024)
    const float **dense_cell = nullptr;     // device: address of the row-major input of the pass being set up
    const float *dense_src = nullptr;       // ... as set by the last spdnn_set_input_dense* (null: converted to tiles)
    int input_kind = 0;
    int cpi_override = 0, grid_override = 0;

    std::vector<LoopCtl> host_ctl;
    spdnn_stats_t stats{};
    int64_t prep_launches = 0;
    std::string err;
};

namespace {

int fail(spdnn *c, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (c) c->err = buf;
    return code;
}

#define CK(call)                                                                                      \
    do {                                                                                              \
        cudaError_t e__ = (call);                                                                     \
        if (e__ != cudaSuccess)                                                                       \
            return fail(c, SPDNN_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__),   \
                        __FILE__, __LINE__);                                                          \
    } while (0)

int free_buffers(spdnn *c) {
    cudaFree(c->y[0]); cudaFree(c->y[1]); cudaFree(c->slot); cudaFree(c->mask); cudaFree(c->tile_done);
    cudaFree(c->ids[0]); cudaFree(c->ids[1]); cudaFree(c->xw); cudaFree(c->has_floats);
    c->y[0] = c->y[1] = nullptr; c->slot = nullptr; c->mask = nullptr; c->ids[0] = c->ids[1] = nullptr;
    c->tile_done = nullptr; c->xw = nullptr; c->has_floats = nullptr;
    c->tiles_cap = 0;
    return SPDNN_OK;
}

int ensure_capacity(spdnn *c, int batch) {
    const int tiles = (batch + 31) / 32;
    if (tiles <= c->tiles_cap) return SPDNN_OK;
    free_buffers(c);
    c->graph_dirty = true;
    const size_t ybytes = (size_t)tiles * (size_t)c->tile_stride * sizeof(float);
    for (int i = 0; i < 2; ++i) {
        CK(cudaMalloc(&c->y[i], ybytes));
        CK(cudaMemsetAsync(c->y[i], 0, ybytes, c->stream));      // incl. the permanent zero row of every tile
        CK(cudaMalloc(&c->ids[i], sizeof(int32_t) * (size_t)tiles * 32));
    }
    CK(cudaMalloc(&c->slot, sizeof(int32_t) * (size_t)tiles * 32));
    CK(cudaMalloc(&c->mask, sizeof(uint32_t) * (size_t)tiles));
    CK(cudaMemsetAsync(c->mask, 0, sizeof(uint32_t) * (size_t)tiles, c->stream));
    CK(cudaMalloc(&c->tile_done, (size_t)tiles));
    CK(cudaMemsetAsync(c->tile_done, 0, (size_t)tiles, c->stream));
    CK(cudaMalloc(&c->xw, sizeof(uint32_t) * (size_t)tiles * c->nw));
    CK(cudaMemsetAsync(c->xw, 0, sizeof(uint32_t) * (size_t)tiles * c->nw, c->stream));     // incl. the zero words behind the neurons
    CK(cudaMalloc(&c->has_floats, (size_t)tiles));
    CK(cudaMemsetAsync(c->has_floats, 0, (size_t)tiles, c->stream));
    c->tiles_cap = tiles;
    return SPDNN_OK;
}

int ensure_stage(spdnn *c, size_t bytes) {
    if (bytes <= c->stage_bytes) return SPDNN_OK;
    CK(cudaStreamSynchronize(c->stream));
    cudaFree(c->stage);
    c->stage = nullptr; c->stage_bytes = 0;
    CK(cudaMalloc(&c->stage, bytes));
    c->stage_bytes = bytes;
    return SPDNN_OK;
}

int begin_input(spdnn *c, int batch, int first_global_id) {
    if (batch < 0) return fail(c, SPDNN_ERR_ARG, "batch must be >= 0");
    if ((long long)first_global_id + batch > 0x7fffffffLL || first_global_id < 0)
        return fail(c, SPDNN_ERR_ARG, "global image numbers must fit in int32");
    // A pass still in flight is not waited for: the new input is ordered behind it on the stream
    // and its results, which nobody fetched, are dropped.
    c->in_flight = false;
    int rc = ensure_capacity(c, batch > 0 ? batch : 1);
    if (rc) return rc;
    c->batch = batch;
    c->first_id = first_global_id;
    c->input_ready = false;
    c->result_ready = false;
    c->prep_launches = 0;
    c->dense_src = nullptr;
    c->input_kind = 0;
    CK(cudaEventRecord(c->ev_prep0, c->stream));
    // the input counts as binary until a conversion kernel sees another value; with the binary front
    // switched off every input takes the float path
    CK(cudaMemsetAsync(c->in_flag, c->binary_front ? 0 : 1, 1, c->stream));
    CK(cudaMemsetAsync(c->has_floats, 0, (size_t)((batch + 31) / 32 > 0 ? (batch + 31) / 32 : 1), c->stream));
    return SPDNN_OK;
}

// An input that turned out not to be binary after some of its tiles were converted as words only: their
// float form is rebuilt from the words (those tiles held zeros and ones).
int repair_float_tiles(spdnn *c) {
    const int tiles = (c->batch + 31) / 32;
    if (!c->binary_front || tiles == 0) return SPDNN_OK;
    const long long warps = (long long)tiles * c->n;
    const int grid = (int)std::min<long long>((warps + 7) / 8, (long long)c->sm_count * 32);
    words_to_tiles_kernel<<<std::max(1, grid), 256, 0, c->stream>>>(c->xw, c->nw, c->n, tiles, c->y[0], c->tile_stride, c->has_floats,
                                                                     c->in_flag, 1);
    CK(cudaGetLastError());
    c->prep_launches += 1;
    return SPDNN_OK;
}

int end_input(spdnn *c) {
    init_loop_kernel<<<std::max(1, std::min(1024, (c->batch + 255) / 256)), 256, 0, c->stream>>>(
        c->ctl, c->ids[0], c->batch, c->first_id, c->died_at, c->layers, c->dense_cell, c->dense_src);
    CK(cudaGetLastError());
    c->prep_launches += 1;
    CK(cudaEventRecord(c->ev_prep1, c->stream));
    c->prep_timed = true;
    c->input_ready = true;
    return SPDNN_OK;
}

int convert_dense_device(spdnn *c, const float *dev_rows, int rows, int first_tile) {
    // rows is a multiple of 32 except for the last chunk
    const dim3 block(32, 8);
    if (rows <= 0) return SPDNN_OK;
    const long long items = (long long)((rows + 31) / 32) * ((c->n + kLayoutCols - 1) / kLayoutCols);
    const int grid = (int)std::min<long long>(items, (long long)c->sm_count * 32);
    if (c->binary_front) {
        // words first (this raises the flag when a value is neither 0 nor 1); the float tiles only once the flag is up
        const dim3 wgrid((rows + 31) / 32, (c->n + 1023) / 1024);
        dense_to_words_kernel<<<wgrid, block, 0, c->stream>>>(dev_rows, c->n, rows, c->xw, c->nw, first_tile, c->in_flag);
        CK(cudaGetLastError());
        c->prep_launches += 1;
    }
    dense_to_tiles_kernel<<<grid, block, 0, c->stream>>>(dev_rows, c->y[0], c->n, rows, c->tile_stride, first_tile,
                                                         c->binary_front ? c->in_flag : nullptr, c->has_floats);
    CK(cudaGetLastError());
    c->prep_launches += 1;
    return SPDNN_OK;
}

template <int KT, bool UNIFORM>
int launch_layer_t(spdnn *c, const LayerDesc &d, const LayerArgs &a, int grid) {
    if (a.xw != nullptr) layer_kernel<KT, UNIFORM, true><<<grid, kThreads, 0, c->stream>>>(d, a);      // input as words
    else layer_kernel<KT, UNIFORM, false><<<grid, kThreads, 0, c->stream>>>(d, a);
    CK(cudaGetLastError());
    return SPDNN_OK;
}

int launch_layer(spdnn *c, const LayerDesc &d, const LayerArgs &a, int grid, bool uniform) {
    if (d.k == 32) return uniform ? launch_layer_t<32, true>(c, d, a, grid) : launch_layer_t<32, false>(c, d, a, grid);
    return uniform ? launch_layer_t<0, true>(c, d, a, grid) : launch_layer_t<0, false>(c, d, a, grid);
}

template <int KT, bool UNIFORM>
int blocks_per_sm_t() {
    int b = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, layer_kernel<KT, UNIFORM>, kThreads, 0) != cudaSuccess) b = 1;
    return b > 0 ? b : 1;
}

int blocks_per_sm(int k, bool uniform) {
    if (k == 32) return uniform ? blocks_per_sm_t<32, true>() : blocks_per_sm_t<32, false>();
    return uniform ? blocks_per_sm_t<0, true>() : blocks_per_sm_t<0, false>();
}

// Opts a kernel in to the largest dynamic shared memory the device allows beside the kernel's own static
// shared memory.  Called at every captured launch (a handful per graph build): the attribute is per device,
// and a "done" flag shared between contexts would be a data race between host threads.
template <typename Kernel>
int allow_max_dynamic_smem(spdnn *c, Kernel kernel) {
    cudaFuncAttributes fa;
    CK(cudaFuncGetAttributes(&fa, kernel));
    CK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, c->smem_optin - (int)fa.sharedSizeBytes));
    return SPDNN_OK;
}

template <int TI, int IPT, int KT, bool UNIFORM, bool STAGED>
int launch_resident_t(spdnn *c, const ResArgs &a, int grid, size_t smem) {
    if (int rc = allow_max_dynamic_smem(c, resident_kernel<TI, IPT, KT, UNIFORM, STAGED>)) return rc;
    resident_kernel<TI, IPT, KT, UNIFORM, STAGED><<<grid, SPDNN_GENERIC_THREADS, smem, c->stream>>>(a);
    CK(cudaGetLastError());
    return SPDNN_OK;
}

template <int TI, int IPT, int KT, bool STAGED, int NT>
int launch_alt2_t(spdnn *c, const ResArgs &a, int grid, size_t smem) {
    if (int rc = allow_max_dynamic_smem(c, alt2_kernel<TI, IPT, KT, STAGED, NT>)) return rc;
    alt2_kernel<TI, IPT, KT, STAGED, NT><<<grid, NT, smem, c->stream>>>(a);
    CK(cudaGetLastError());
    return SPDNN_OK;
}

// ALT2 form (always a uniform weight): group sizes 32/16 with 8 images per thread, 16/8/4 with 4.
template <int TI, int IPT, int NT>
int launch_alt2(spdnn *c, const ResArgs &a, int grid, size_t smem, bool k32) {
    const bool staged = a.tring > 0;
    if (k32) return staged ? launch_alt2_t<TI, IPT, 32, true, NT>(c, a, grid, smem) : launch_alt2_t<TI, IPT, 32, false, NT>(c, a, grid, smem);
    return staged ? launch_alt2_t<TI, IPT, 0, true, NT>(c, a, grid, smem) : launch_alt2_t<TI, IPT, 0, false, NT>(c, a, grid, smem);
}

template <int TI>
int launch_generic(spdnn *c, const ResArgs &a, int grid, size_t smem, bool k32, bool uniform) {
    const bool staged = a.table_bytes > 0;
    if (k32) {
        if (uniform) return staged ? launch_resident_t<TI, 4, 32, true, true>(c, a, grid, smem)
                                   : launch_resident_t<TI, 4, 32, true, false>(c, a, grid, smem);
        return staged ? launch_resident_t<TI, 4, 32, false, true>(c, a, grid, smem)
                      : launch_resident_t<TI, 4, 32, false, false>(c, a, grid, smem);
    }
    if (uniform) return staged ? launch_resident_t<TI, 4, 0, true, true>(c, a, grid, smem)
                               : launch_resident_t<TI, 4, 0, true, false>(c, a, grid, smem);
    return staged ? launch_resident_t<TI, 4, 0, false, true>(c, a, grid, smem)
                  : launch_resident_t<TI, 4, 0, false, false>(c, a, grid, smem);
}

int launch_resident(spdnn *c, int ti, int ipt, const ResArgs &a, int grid, size_t smem, int mode, bool k32, bool uniform) {
    if (mode == kResAlt2) {
        // layers of at most 64 classes: blocks of 128 threads (one warp does the bit form; twice the blocks per SM)
        if (ipt == 8 && ti == 32 && !a.bit_multi && c->alt2_small_blocks) return launch_alt2<32, 8, 128>(c, a, grid, smem, k32);
        if (ipt == 8) return ti == 32 ? launch_alt2<32, 8, kThreads>(c, a, grid, smem, k32) : launch_alt2<16, 8, kThreads>(c, a, grid, smem, k32);
        // one block per SM by its shared memory: 512 threads
        const bool wide = c->alt2_threads != 256 && smem * 2 + 4096 > (size_t)c->smem_optin;
        if (wide)
            switch (ti) {
                case 16: return launch_alt2<16, 4, 512>(c, a, grid, smem, k32);
                case 8: return launch_alt2<8, 4, 512>(c, a, grid, smem, k32);
                default: return launch_alt2<4, 4, 512>(c, a, grid, smem, k32);
            }
        switch (ti) {
            case 16: return launch_alt2<16, 4, kThreads>(c, a, grid, smem, k32);
            case 8: return launch_alt2<8, 4, kThreads>(c, a, grid, smem, k32);
            default: return launch_alt2<4, 4, kThreads>(c, a, grid, smem, k32);
        }
    }
    switch (ti) {
        case 16: return launch_generic<16>(c, a, grid, smem, k32, uniform);
        case 8: return launch_generic<8>(c, a, grid, smem, k32, uniform);
        default: return launch_generic<4>(c, a, grid, smem, k32, uniform);
    }
}

template <typename T>
int upload_vec(spdnn *c, T **dst, const std::vector<T> &v) {
    if (v.empty()) return SPDNN_OK;
    CK(cudaMalloc(dst, sizeof(T) * v.size()));
    CK(cudaMemcpyAsync(*dst, v.data(), sizeof(T) * v.size(), cudaMemcpyHostToDevice, c->stream));
    return SPDNN_OK;
}

// Builds (outside stream capture) the resident kernel's tables for every layer whose
// canonical form is on the host, walking the network front to back because a layer's tables
// are written in the value ids the layer before it produces.
int prepare_resident(spdnn *c) {
    for (auto &r : c->res) r.reset();
    if (!c->resident) return SPDNN_OK;
    const int32_t *vid = nullptr;      // value ids of the current layer's input (null: the neurons themselves)
    int v_in = c->n;
    uint64_t in_hash = 0;
    for (int l = 0; l < c->layers; ++l) {
        const DevLayer &L = *c->layer[l];
        if (!L.host) { vid = nullptr; v_in = c->n; in_hash = 0; continue; }
        const uint64_t key = mix64(L.h1 ^ mix64(in_hash + 0x1234567ull));
        std::shared_ptr<DevRes> R;
        auto it = c->res_shared.find(key);
        if (it != c->res_shared.end()) R = it->second.lock();
        if (!R) {
            ResidentTables t;
            try {
                build_resident_tables(*L.host, vid, v_in, t);
            } catch (const std::bad_alloc &) {
                return fail(c, SPDNN_ERR_MEMORY, "out of host memory preparing layer %d", l);
            }
            R = std::make_shared<DevRes>();
            R->device = c->device;
            t.blob.resize((t.blob.size() + 3) / 4 * 4, 0);       // bulk copies move multiples of 16 bytes
            R->blob_bytes = (int)(t.blob.size() * 4);
            R->o_vals = t.o_vals; R->classes = t.classes; R->k = L.k; R->v_in = t.v_in; R->mode = t.mode;
            R->uniform = L.uniform; R->w = L.w;
            int rc = upload_vec(c, &R->blob, t.blob);
            if (!rc) rc = upload_vec(c, &R->rep, t.rep);
            if (!rc) rc = upload_vec(c, &R->mem_ptr, t.mem_ptr);
            if (!rc) rc = upload_vec(c, &R->mem, t.mem);
            if (rc) return rc;
            CK(cudaStreamSynchronize(c->stream));
            R->class_of.swap(t.class_of);
            R->partition_hash = t.partition_hash;
            c->res_shared[key] = R;
        }
        c->res[l] = R;
        if (R->classes < c->n) { vid = R->class_of.data(); v_in = R->classes; in_hash = R->partition_hash; }
        else { vid = nullptr; v_in = c->n; in_hash = 0; }
    }
    std::vector<ResLayer> t(c->layers);
    for (int l = 0; l < c->layers; ++l) {
        ResLayer e{};
        if (c->res[l]) {
            const DevRes &R = *c->res[l];
            e.blob = R.blob; e.rep = R.rep; e.mem_ptr = R.mem_ptr; e.mem = R.mem;
            e.blob_bytes = R.blob_bytes; e.o_vals = R.o_vals; e.classes = R.classes; e.k = R.k; e.v_in = R.v_in; e.w = R.w;
        }
        t[l] = e;
    }
    CK(cudaMemcpyAsync(c->res_table, t.data(), sizeof(ResLayer) * t.size(), cudaMemcpyHostToDevice, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return SPDNN_OK;
}

// Rows one activation buffer needs for layer l inside a resident chunk.
inline int resident_rows(const DevRes &R) { return ((std::max(R.v_in, R.classes) + 1) & ~1) + 2; }

// Dynamic shared memory of a resident block.  GENERIC chunks: two activation buffers and two
// staged tables.  ALT2 chunks: two activation buffers, `tring` groups of 1 << gshift layer records
// of `stride` bytes (the word buffers of the bit form live in the activation buffer that is free).
inline size_t resident_smem_bytes(int ti, int rows, int table) { return 2 * (size_t)rows * ti * 4 + 2 * (size_t)table; }
inline size_t alt2_smem_bytes(int ti, int rows, int stride, int gshift, int tring) {
    return 2 * (size_t)rows * ti * 4 + (size_t)tring * ((size_t)stride << gshift);
}

// Enqueues the whole network: chunks of layers through the resident kernel where a group of
// images fits in shared memory (chunk lengths chunk_first, x chunk_growth, ... up to chunk_max: short while
// images still die, long once the survivors are stable), one launch per layer otherwise.
struct Step {
    int first = 0, count = 1;      // layers [first, first + count)
    int ti = 0, ipt = 4;           // resident chunk: images per block / per thread; ti == 0: per-layer kernel
    int rows = 0, table = 0;       // resident chunk: rows of one activation buffer, bytes per staged table
    // ALT2 chunk (alt2_kernel): packed table stream and its staging, word buffers of the bit form
    int stride = 0, gshift = 0, tring = 0, wring = 2, rows_w = 0, max_classes = 0;
    unsigned char *stream = nullptr;
    bool dense = false;            // resident chunk that reads the caller's row-major input in place
    // bits_kernel pre-pass of an ALT2 chunk (0 threads: none): its own staging of the packed stream
    int bits_threads = 0, bits_gshift = 0, bits_tring = 0, wwords = 0;
    // ... with the chunk's distinct records cached in shared memory (cache_records > 0)
    unsigned char *cache = nullptr;
    unsigned short *rec_of = nullptr;
    int cache_records = 0;
};

// The launches of one pass, front to back.
// dense_first: the pass starts from the caller's row-major input; its first launch is then a resident
// chunk wherever one fits (Step::dense), because loading the rows into shared memory also does the change
// of layout.
std::vector<Step> plan_steps(spdnn *c, bool dense_first) {
    std::vector<Step> plan;
    int l = 0, chunk = c->chunk_list.empty() ? c->chunk_first : c->chunk_list[0];
    int resident_chunks = 0;       // resident chunks planned so far
    int alt2_chunks = 0;           // ALT2 chunks planned so far
    int generic_chunks = 0;        // GENERIC chunks planned so far
    while (l < c->layers) {
        Step st;
        st.first = l;
        if (c->res[l]) {
            const DevRes &R0 = *c->res[l];
            const bool k32 = (R0.k == 32);
            auto fits = [&](int t_i, int r, int table) {
                return resident_smem_bytes(t_i, r, table) + 2048 <= (size_t)c->smem_optin;
            };
            int rows = resident_rows(R0), ti = 0, ipt = 4;
            // (images per block, images per thread) in order of preference; a form that would leave
            // most threads without a class (under half of what one pass of the block covers) is skipped
            static const int kAlt2[][2] = {{32, 8}, {16, 4}, {16, 8}, {8, 4}, {4, 4}};
            static const int kGeneric[][2] = {{16, 4}, {8, 4}, {4, 4}};
            const int (*cand)[2] = R0.mode == kResAlt2 ? kAlt2 : kGeneric;
            const int ncand = R0.mode == kResAlt2 ? 5 : 3;
            // First launch of a pass that reads the input in place.  A layer that reads all N rows to compute
            // few classes is mostly loading: it pays only with several blocks of at least 8 images per SM, so
            // that one block's loads overlap another's arithmetic -- it takes the largest group that leaves
            // room for three blocks, and if there is none this kind of pass is not built.  Any other first
            // chunk keeps the group size that suits its arithmetic.
            const bool dense_wanted = (l == 0 && dense_first);
            const bool wide_few = (R0.v_in == c->n && R0.classes * 2 <= c->n);
            bool dense_here = false;
            for (int pass = (dense_wanted && wide_few) ? 0 : 1; pass < 2 && !ti; ++pass)
                for (int q = 0; q < ncand; ++q) {
                    const int t_i = cand[q][0], i_pt = cand[q][1];
                    if (t_i > c->res_ti_max || i_pt > c->res_ipt_max || !fits(t_i, rows, 0)) continue;
                    if (i_pt == 8 && R0.classes * 2 < kThreads * i_pt / t_i) continue;
                    if (pass == 0 && (t_i < 8 || resident_smem_bytes(t_i, rows, 0) * 3 > (size_t)c->smem_optin)) continue;
                    ti = t_i; ipt = i_pt;
                    dense_here = dense_wanted && (pass == 0 || !wide_few);
                    break;
                }
            if (ti) {
                // extend while the layers are of one kernel variant and the group still fits
                int f = 1, blob = R0.blob_bytes, maxc = R0.classes;
                while (f < chunk && l + f < c->layers && c->res[l + f]) {
                    const DevRes &M = *c->res[l + f];
                    if (M.mode != R0.mode || M.uniform != R0.uniform || (M.k == 32) != k32) break;
                    const int r2 = std::max(rows, resident_rows(M));
                    if (!fits(ti, r2, 0)) break;
                    rows = r2;
                    blob = std::max(blob, M.blob_bytes);
                    maxc = std::max(maxc, M.classes);
                    ++f;
                }
                int tb = (blob + 127) / 128 * 128;
                if (!(c->stage_tables && fits(ti, rows, tb))) tb = 0;
                if (R0.mode == kResAlt2) {
                    // packed stream: groups of up to 32 layers per bulk copy (what a group costs besides its
                    // layers -- waiting for the copy, checking the result -- is spread over them), the next group
                    // on its way while one is applied, as many word buffers as a group has layers plus the one
                    // it starts from -- whatever of that fits
                    st.max_classes = maxc;
                    st.stride = alt2_stream_stride(maxc);
                    st.rows_w = std::max(rows, 32);
                    // staging may take a quarter of the shared memory at most, so that the blocks per SM stay
                    // what the activations allow; word buffers of the bit form: as many as one activation buffer
                    // holds, 33 at most (under two the chunk runs without the bit form)
                    auto stage = [&](int t_i, size_t limit) {
                        st.tring = 0; st.gshift = 0;
                        st.wring = (int)std::min<size_t>((size_t)c->word_ring_max, ((size_t)rows * t_i * 4) / ((size_t)st.rows_w * 4));
                        if (c->stage_tables)
                            for (int gs = 5; gs >= 0 && !st.tring; --gs)
                                for (int tr = 4; tr >= 2 && !st.tring; tr /= 2)
                                    if ((1 << gs) <= c->table_group_max && ((1 << gs) < 2 * f || gs == 0) && tr <= c->table_ring_max &&
                                        alt2_smem_bytes(t_i, rows, st.stride, gs, tr) + 2048 <= limit &&
                                        (size_t)tr * ((size_t)st.stride << gs) <= (size_t)c->smem_optin / 4) { st.gshift = gs; st.tring = tr; }
                        return alt2_smem_bytes(t_i, rows, st.stride, st.gshift, st.tring);
                    };
                    const size_t need = stage(ti, (size_t)c->smem_optin);
                    // A block that has an SM to itself cannot hide the loading and storing of its rows, nor the tail of a
                    // layer, behind another block's arithmetic: where half the images per block (and tables staged at
                    // least four layers at a time) let two blocks share an SM, that is faster (measured at 16384 neurons).
                    if (c->two_blocks && ipt == 4 && ti >= 8 && ti / 2 <= c->res_ti_max && need * 2 + 4096 > (size_t)c->smem_optin) {
                        const size_t half = stage(ti / 2, ((size_t)c->smem_optin - 4096) / 2);
                        if (st.tring > 0 && st.gshift >= 2 && half * 2 + 4096 <= (size_t)c->smem_optin) ti /= 2;
                        else stage(ti, (size_t)c->smem_optin);
                    }
                    // Pre-pass for tiles that are saturated already (bits_kernel): layers of more than one pass of 64
                    // classes, where the float buffers leave this kernel's own bit form few images per block.  Not
                    // before the first two chunks of a pass: the challenge networks saturate around layer 30, and a
                    // tile that is not saturated costs the pre-pass a read of all its rows for nothing.
                    const int rows_max = std::max(rows, maxc);
                    if (c->bits_prepass && c->bit_form && c->clip > 0.0f && (maxc > 64 || c->bits_small) && rows_max <= 16383 &&
                        (alt2_chunks > 1 || c->bits_first_chunk)) {
                        st.wwords = (rows_max + 63) / 64 * 64;
                        const int passes = (maxc + 63) / 64;
                        int nt = c->bits_threads > 0 ? c->bits_threads : 32 * ((passes + 1) / 2);
                        st.bits_threads = std::max(maxc > 64 ? 128 : 32, std::min(kBitsMaxThreads, (nt + 31) / 32 * 32));
                        // table staging: groups of about 16 KB, four in flight when a group is one layer
                        st.bits_gshift = 0; st.bits_tring = 0;
                        if (c->stage_tables) {
                            while (st.bits_gshift < 5 && ((size_t)st.stride << (st.bits_gshift + 1)) <= (size_t)20 << 10 &&
                                   (1 << (st.bits_gshift + 1)) <= c->table_group_max) ++st.bits_gshift;
                            st.bits_tring = st.bits_gshift == 0 ? 4 : 2;
                            if (c->table_ring_max < st.bits_tring) st.bits_tring = 2;
                            if ((size_t)st.wwords * 8 + (size_t)st.bits_tring * ((size_t)st.stride << st.bits_gshift) + 2048 > (size_t)c->smem_optin)
                                st.bits_tring = 0;
                        }
                    }
                }
                if (R0.mode == kResGeneric) {
                    // count_kernel pre-pass for tiles that are saturated already: uniform weight, 32 entries per class
                    // (its adder tree is built for 32), the two word buffers in shared memory
                    bool k32_all = k32 && R0.uniform;
                    for (int q = 0; q < f && k32_all; ++q) k32_all = c->res[l + q]->k == 32 && c->res[l + q]->uniform;
                    const int words = (rows + 63) / 64 * 64;
                    if (c->bits_prepass && c->bit_form && c->clip > 0.0f && k32_all && (generic_chunks > 0 || c->bits_first_chunk) &&
                        (size_t)words * 8 + 2048 <= (size_t)c->smem_optin) {
                        st.wwords = words;
                        const int passes = (maxc + 31) / 32;
                        const int nt = c->bits_threads > 0 ? c->bits_threads : 32 * ((passes + 1) / 2);
                        st.bits_threads = std::max(128, std::min(kBitsMaxThreads, (nt + 31) / 32 * 32));
                    }
                }
                // A lone layer that reads all N rows of every image but computes few classes from
                // them (the first layer of a network with repeated columns) gains nothing from
                // staging the rows in shared memory: gather straight from global memory instead.
                const bool lone_wide = (f == 1 && R0.v_in == c->n && R0.classes * 2 <= c->n && !c->resident_always) && !dense_here;
                if (!lone_wide && ti) {
                    st.count = f; st.ti = ti; st.ipt = ipt; st.rows = rows; st.table = tb;
                    st.dense = dense_here;
                }
            }
        }
        if (st.ti) {
            ++resident_chunks;
            if (resident_chunks < (int)c->chunk_list.size()) chunk = c->chunk_list[resident_chunks];
            // A chunk with a bits_kernel pre-pass runs its saturated tiles at a fraction of the float form's cost and
            // dead images cost it nothing, so such chunks can be long.  But a tile that is NOT saturated when the chunk
            // starts is the float form's for the whole chunk (at 65536 neurons about 1.4 us per layer and tile against
            // 0.3): the first chunk with a pre-pass is as short as the chunk before it, and only the one after it takes
            // the rest of the network -- a tile that saturates a few layers late then costs tens of layers, not
            // thousands (measured: one such tile among 7500 images made a pass 2.6 ms longer).
            else if ((st.max_classes > 64 || c->bits_small) && st.max_classes > 0 && alt2_chunks >= 1 && c->bits_prepass && c->bit_form && c->clip > 0.0f && !c->chunk_growth_set)
                chunk = alt2_chunks >= 2 ? c->chunk_max : chunk;
            else chunk = std::min(chunk * (st.max_classes > 0 ? c->chunk_growth : c->chunk_growth_generic), c->chunk_max);
        }
        if (st.ti && st.max_classes > 0) ++alt2_chunks;
        if (st.ti && st.max_classes == 0) ++generic_chunks;
        if (!st.ti) st.bits_threads = 0;
        plan.push_back(st);
        l += st.count;
    }
    return plan;
}

// Enqueues the whole network: chunks of layers through the resident kernel where a group of
// images fits in shared memory (chunk lengths chunk_first, x chunk_growth, ... up to chunk_max: short while
// images still die, long once the survivors are stable), one launch per layer otherwise.  A
// launch that is followed by a resident chunk writes only the one row per class that chunk
// will read.
//
// gated: the pass may start from a binary input kept as words (spdnn_front.cuh).  The launches of the first
// layer then exist twice, one variant per value of the flag that the input conversion leaves on the device
// (0: binary, read the words; 1: read the float tiles), and each checks the flag at entry:
//   kFrontWords   layer 0 runs in the per-layer kernel, whose BITS variant gathers from the words;
//   kFrontExpand  the pass starts with a resident chunk: the words are expanded to float tiles first.
enum { kFrontNone = 0, kFrontWords = 1, kFrontExpand = 3 };

int enqueue_layers(spdnn *c, const std::vector<Step> &plan, bool gated) {
    c->last_group = 0;
    c->extra_launches = 0;
    c->streamed_launches = 0;
    int front = kFrontNone;
    if (gated) {
        if (plan[0].ti == 0) {
            front = kFrontWords;
        } else {
            front = kFrontExpand;
            const long long warps = (long long)c->tiles_cap * c->n;
            const int grid = (int)std::min<long long>((warps + 7) / 8, (long long)c->sm_count * 32);
            words_to_tiles_kernel<<<std::max(1, grid), 256, 0, c->stream>>>(c->xw, c->nw, c->n, c->tiles_cap, c->y[0], c->tile_stride,
                                                                             nullptr, c->in_flag, 0);
            CK(cudaGetLastError());
            c->extra_launches += 1;
            if (c->print_schedule) fprintf(stderr, "[spdnn] binary inputs: words expanded to float tiles before step 0\n");
        }
    }
    for (size_t step = 0; step < plan.size(); ++step) {
        const Step &st = plan[step];
        const int l = st.first;
        const DevLayer &L = *c->layer[l];
        const float *yin = c->y[step & 1];
        float *yout = c->y[(step & 1) ^ 1];
        const bool next_resident = c->reps_only && step + 1 < plan.size() && plan[step + 1].ti != 0;
        // The last launch of a pass stores one row per class too when it is a resident chunk: the categories
        // and survivor counts need no more, and spdnn_get_activations expands the classes when it is called.
        const int last_layer = st.first + st.count - 1;
        const bool lazy_last = c->lazy_expand && c->reps_only && step + 1 == plan.size() && st.ti != 0 && c->res[last_layer] &&
                               c->res[last_layer]->mem_ptr != nullptr;
        if (step + 1 == plan.size()) c->expand_layer_of_plan = lazy_last ? last_layer : -1;
        if (st.ti) {
            const DevRes &R0 = *c->res[l];
            ResArgs a;
            a.yin = yin; a.yout = yout; a.tile_stride = c->tile_stride;
            a.ctl_in = c->ctl + step; a.ctl_out = c->ctl + step + 1;
            a.slot = c->slot; a.mask = c->mask; a.ids0 = c->ids[0]; a.ids1 = c->ids[1];
            a.counter = c->counter; a.work = c->counter + 1; a.status = c->status;
            a.layers = c->res_table + l; a.died_at = c->died_at + l; a.nlayers = st.count;
            a.buf_rows = st.rows; a.table_bytes = st.table;
            a.dense_in = st.dense ? c->dense_cell : nullptr;
            a.sm_count = c->sm_count;
            a.stream = st.stream; a.stream_stride = st.stride; a.tgroup_shift = st.gshift; a.tring = st.tring;
            a.wring = st.wring; a.rows_w = st.rows_w; a.bit_multi = st.max_classes > 64 ? 1 : 0;
            a.n = c->n; a.bias = c->bias; a.clip = c->clip;
            a.reps_only = (next_resident || lazy_last) ? 1 : 0;
            a.exact_ok = (l > 0 && c->clip <= 1024.0f && c->exact_shortcut) ? 1 : 0;
            const int grid = std::max(1, (c->tiles_cap * 32 + st.ti - 1) / st.ti);
            const bool alt2 = (R0.mode == kResAlt2);
            const size_t smem = alt2 ? alt2_smem_bytes(st.ti, st.rows, st.stride, st.gshift, st.tring)
                                     : resident_smem_bytes(st.ti, st.rows, st.table);
            a.bit_ok = (alt2 && c->bit_form && c->clip > 0.0f && st.wring >= 2) ? 1 : 0;
            a.tile_done = nullptr; a.wwords = 0;
            a.cache = nullptr; a.rec_of = nullptr; a.cache_records = 0;
            a.gate = nullptr; a.gate_want = 0;
            if (alt2 && st.bits_threads > 0) {
                // pre-pass: tiles of 32 images that are saturated already run the whole chunk as words
                ResArgs b = a;                 // (gated like the launch it prepares)
                b.tile_done = c->tile_done; b.wwords = st.wwords;
                b.tgroup_shift = st.bits_gshift; b.tring = st.bits_tring;
                b.cache = st.cache; b.rec_of = st.rec_of; b.cache_records = st.cache_records;
                size_t bsmem = (size_t)st.wwords * 8 + (size_t)st.bits_tring * ((size_t)st.stride << st.bits_gshift);
                if (st.cache_records > 0) {
                    // two word buffers, the records, the layer -> record map, a copy of a segment's input words
                    bsmem = (size_t)st.wwords * 12 + (size_t)st.cache_records * st.stride + ((size_t)st.count * 2 + 15) / 16 * 16;
                    if (int rc = allow_max_dynamic_smem(c, bits_kernel<kBitsCached>)) return rc;
                    bits_kernel<kBitsCached><<<c->tiles_cap, st.bits_threads, bsmem, c->stream>>>(b);
                } else if (st.bits_tring > 0) {
                    if (int rc = allow_max_dynamic_smem(c, bits_kernel<kBitsRing>)) return rc;
                    bits_kernel<kBitsRing><<<c->tiles_cap, st.bits_threads, bsmem, c->stream>>>(b);
                } else {
                    if (int rc = allow_max_dynamic_smem(c, bits_kernel<kBitsGlobal>)) return rc;
                    bits_kernel<kBitsGlobal><<<c->tiles_cap, st.bits_threads, bsmem, c->stream>>>(b);
                }
                CK(cudaGetLastError());
                c->extra_launches += 1;
                a.tile_done = c->tile_done;
                if (c->print_schedule)
                    fprintf(stderr, "[spdnn] step %zu: pre-pass for saturated tiles, layers %d..%d  %d threads per 32 images  %d words  smem %zu B  tables %s (%d layers per copy, %d in flight; %d distinct records cached)\n",
                            step, l, l + st.count - 1, st.bits_threads, st.wwords, bsmem, st.cache_records ? "cached" : st.bits_tring ? "staged" : "global",
                            1 << st.bits_gshift, st.bits_tring, st.cache_records);
            }
            if (!alt2 && st.bits_threads > 0) {
                // pre-pass: saturated tiles of 32 images run the whole chunk as words, a class's output decided by the
                // count of its clip-valued inputs
                ResArgs b = a;
                b.tile_done = c->tile_done; b.wwords = st.wwords;
                const size_t bsmem = (size_t)st.wwords * 8;
                if (int rc = allow_max_dynamic_smem(c, count_kernel)) return rc;
                count_kernel<<<c->tiles_cap, st.bits_threads, bsmem, c->stream>>>(b);
                CK(cudaGetLastError());
                c->extra_launches += 1;
                a.tile_done = c->tile_done;
                if (c->print_schedule)
                    fprintf(stderr, "[spdnn] step %zu: pre-pass for saturated tiles (count form), layers %d..%d  %d threads per 32 images  %d words  smem %zu B\n",
                            step, l, l + st.count - 1, st.bits_threads, st.wwords, bsmem);
            }
            int rc = launch_resident(c, st.ti, st.ipt, a, grid, smem, R0.mode, R0.k == 32, R0.uniform);
            if (rc) return rc;
            c->last_group = st.ti;
            char tables_txt[96];
            if (alt2 && st.tring) snprintf(tables_txt, sizeof tables_txt, "staged (%d layers per copy, %d copies in flight), %d word buffers", 1 << st.gshift, st.tring, st.wring);
            else if (alt2) snprintf(tables_txt, sizeof tables_txt, "global, %d word buffers", st.wring);
            else snprintf(tables_txt, sizeof tables_txt, "%s", st.table ? "staged" : "global");
            if (c->print_schedule)
                fprintf(stderr, "[spdnn] step %zu: resident layers %d..%d  group %d images (%d per thread)  %s  rows %d (v_in %d, classes %d)  smem %zu B  tables %s%s\n",
                        step, l, l + st.count - 1, st.ti, st.ipt, R0.mode == kResAlt2 ? "ALT2" : "GENERIC", st.rows, R0.v_in,
                        R0.classes, smem, tables_txt, next_resident ? "  writes representatives only" : "");
            if (c->print_schedule && st.dense) fprintf(stderr, "[spdnn]         reads the row-major input in place\n");
        } else {
            LayerDesc d;
            d.off = L.off; d.vals = L.vals;
            d.mem_ptr = L.identity_members ? nullptr : L.mem_ptr;
            d.mem = L.mem;
            int wslot = -1;
            if (L.pinned) {
                // Streamed layer: its tables travel on the copy stream into the slot that the streamed launch before
                // the last one has left, while the launches in between run (in the captured graph: the copy depends
                // on that launch and on the copy before it, this launch on the copy).
                wslot = c->streamed_launches & 1;
                if (c->streamed_launches == 0) {
                    CK(cudaEventRecord(c->ev_fork, c->stream));
                    CK(cudaStreamWaitEvent(c->copy_stream, c->ev_fork, 0));
                }
                if (c->streamed_launches >= 2) CK(cudaStreamWaitEvent(c->copy_stream, c->ev_free[wslot], 0));
                CK(cudaMemcpyAsync(c->wslot[wslot], L.pinned, L.pinned_bytes, cudaMemcpyHostToDevice, c->copy_stream));
                CK(cudaEventRecord(c->ev_ready[wslot], c->copy_stream));
                CK(cudaStreamWaitEvent(c->stream, c->ev_ready[wslot], 0));
                unsigned char *base = c->wslot[wslot];
                d.off = reinterpret_cast<const int32_t *>(base);
                d.vals = L.uniform ? nullptr : reinterpret_cast<const float *>(base + L.o_vals);
                d.mem_ptr = L.identity_members ? nullptr : reinterpret_cast<const int32_t *>(base + L.o_mem_ptr);
                d.mem = reinterpret_cast<const int32_t *>(base + L.o_mem);
                c->streamed_launches += 1;
            }
            d.classes = L.classes; d.k = L.k; d.w = L.w;
            // Work item = (tile, block of classes).  Without duplicate columns every input row is
            // used by ~K classes: keep a whole tile in one block when it fits the L1 so those
            // re-reads hit there; otherwise small items for balance.
            int cpi = 16;
            if (L.identity_members && (size_t)c->tile_stride * 4 <= (size_t)160 * 1024) cpi = L.classes;
            if (c->cpi_override > 0) cpi = c->cpi_override;
            d.classes_per_item = std::max(1, std::min(cpi, L.classes));
            LayerArgs a;
            a.yin = yin; a.yout = yout;
            a.tile_stride = c->tile_stride;
            a.ctl_in = c->ctl + step; a.ctl_out = c->ctl + step + 1;
            a.slot = c->slot; a.mask = c->mask; a.ids0 = c->ids[0]; a.ids1 = c->ids[1];
            a.counter = c->counter; a.work = c->counter + 1; a.status = c->status;
            a.died_at = c->died_at + l;
            // one row per class suffices only when the chunk that follows reads through the representatives of
            // this layer's classes; a layer whose canonical form was not kept on the host (budget) has no
            // resident tables, the next layer then reads all N rows
            const bool next_reads_reps = next_resident && c->res[l] && l + 1 < c->layers && c->res[l + 1] &&
                                         c->res[l + 1]->rep != nullptr;
            a.first_member_only = (next_reads_reps && !L.identity_members) ? 1 : 0;
            a.bias = c->bias; a.clip = c->clip;
            a.xw = nullptr; a.nw = 0; a.gate = nullptr; a.gate_want = 0;
            const long long ncb = (L.classes + d.classes_per_item - 1) / d.classes_per_item;
            if ((long long)c->tiles_cap * ncb >= 0xffffffffLL) return fail(c, SPDNN_ERR_LIMIT, "batch too large for one launch");
            int grid = c->grid_override > 0 ? c->grid_override : c->sm_count * blocks_per_sm(L.k, L.uniform);
            if (step == 0 && front == kFrontWords) {
                {
                    LayerArgs w = a;           // binary inputs: gather from the words
                    w.xw = c->xw; w.nw = c->nw; w.gate = c->in_flag; w.gate_want = 0;
                    const bool by_count = L.uniform && L.k == 32 && c->count_front;
                    if (by_count) {
                        // uniform weight, 32 entries per class: bit-sliced counts of 32 images at once
                        int bps = 0;
                        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, front_count_kernel, kThreads, 0) != cudaSuccess || bps < 1) bps = 1;
                        const long long fitems = (long long)c->tiles_cap * ((L.classes + kFrontClassesPerItem - 1) / kFrontClassesPerItem);
                        if (fitems >= 0xffffffffLL) return fail(c, SPDNN_ERR_LIMIT, "batch too large for one launch");
                        front_count_kernel<<<c->sm_count * bps, kThreads, 0, c->stream>>>(d, w);
                        CK(cudaGetLastError());
                    } else {
                        int rc = launch_layer(c, d, w, grid, L.uniform);
                        if (rc) return rc;
                    }
                    c->extra_launches += 1;
                    if (c->print_schedule)
                        fprintf(stderr, "[spdnn] step 0, binary inputs: %s on the input words\n", by_count ? "counting kernel" : "per-layer kernel");
                }
                a.gate = c->in_flag; a.gate_want = 1;
            }
            int rc = launch_layer(c, d, a, grid, L.uniform);
            if (rc) return rc;
            if (wslot >= 0) CK(cudaEventRecord(c->ev_free[wslot], c->stream));
            if (c->print_schedule)
                fprintf(stderr, "[spdnn] step %zu: per-layer kernel, layer %d  classes %d  k %d  grid %d%s%s\n", step, l, L.classes, L.k,
                        grid, a.first_member_only ? "  writes representatives only" : "",
                        wslot >= 0 ? "  tables streamed from host memory" : "");
        }
    }
    c->nsteps = (int)plan.size();
    finalize_ids_kernel<<<std::max(1, std::min(c->tiles_cap, 4 * c->sm_count)), 256, 0, c->stream>>>(c->ctl + c->nsteps, c->slot,
                                                                                             c->ids[0], c->ids[1]);
    CK(cudaGetLastError());
    return SPDNN_OK;
}

// Captures the launches of one pass for one kind of input (0: tiles, 1: row-major read in place).
int build_graph_kind(spdnn *c, int kind) {
    std::vector<Step> plan = plan_steps(c, kind == 1);
    if (kind == 1 && !(plan[0].ti && plan[0].dense)) return SPDNN_OK;      // no resident first launch: kind 0 serves
    // outside the capture: the packed table stream of every ALT2 chunk
    for (Step &st : plan) {
        if (!st.ti || c->res[st.first]->mode != kResAlt2) continue;
        if (st.rows > 16383) return fail(c, SPDNN_ERR_LIMIT, "layer %d: %d rows do not fit a packed table entry", st.first, st.rows);
        CK(cudaMalloc(&st.stream, (size_t)st.count * st.stride));
        c->streams.push_back(st.stream);
        alt2_pack_kernel<<<st.count, 256, 0, c->stream>>>(c->res_table + st.first, st.stride, st.stream, c->bias, c->clip);
        CK(cudaGetLastError());
        if (st.bits_threads > 0 && c->table_cache && c->stage_tables) {
            // Layers with the same tables (same matrix, same value ids going in) share one record.  When the chunk's
            // distinct records fit beside the word buffers, the pre-pass keeps them all in shared memory.
            std::unordered_map<const DevRes *, int> seen;
            std::vector<unsigned short> rec_of(st.count);
            std::vector<int> first_layer;
            for (int q = 0; q < st.count; ++q) {
                const DevRes *r = c->res[st.first + q].get();
                auto it = seen.find(r);
                if (it == seen.end()) {
                    it = seen.emplace(r, (int)first_layer.size()).first;
                    first_layer.push_back(q);
                }
                rec_of[q] = (unsigned short)std::min(it->second, 65535);
            }
            const size_t d = first_layer.size();
            const size_t rec_bytes = ((size_t)st.count * 2 + 15) / 16 * 16;
            if (d <= 65535 && d * st.stride < ((size_t)1 << 20) &&
                (size_t)st.wwords * 12 + d * st.stride + rec_bytes + 2048 <= (size_t)c->smem_optin) {
                CK(cudaMalloc(&st.cache, d * st.stride));
                c->streams.push_back(st.cache);
                unsigned char *rec_dev = nullptr;
                CK(cudaMalloc(&rec_dev, rec_bytes));
                c->streams.push_back(rec_dev);
                st.rec_of = reinterpret_cast<unsigned short *>(rec_dev);
                for (size_t q = 0; q < d; ++q)
                    CK(cudaMemcpyAsync(st.cache + q * st.stride, st.stream + (size_t)first_layer[q] * st.stride, st.stride,
                                       cudaMemcpyDeviceToDevice, c->stream));
                CK(cudaMemcpyAsync(rec_dev, rec_of.data(), (size_t)st.count * 2, cudaMemcpyHostToDevice, c->stream));
                CK(cudaStreamSynchronize(c->stream));          // rec_of is a local
                st.cache_records = (int)d;
            }
        }
    }
    CK(cudaStreamSynchronize(c->stream));
    cudaGraph_t g = nullptr;
    CK(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_layers(c, plan, kind == 0 && c->binary_front);
    cudaError_t e = cudaStreamEndCapture(c->stream, &g);
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return fail(c, SPDNN_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&c->graph_exec[kind], g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(c, SPDNN_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
    c->graph_steps[kind] = c->nsteps;
    c->graph_extra[kind] = c->extra_launches;
    c->graph_group[kind] = c->last_group;
    c->graph_expand_layer[kind] = c->expand_layer_of_plan;
    return SPDNN_OK;
}

int build_graph(spdnn *c) {
    for (int kind = 0; kind < 2; ++kind)
        if (c->graph_exec[kind]) { cudaGraphExecDestroy(c->graph_exec[kind]); c->graph_exec[kind] = nullptr; }
    for (unsigned char *p : c->streams) cudaFree(p);
    c->streams.clear();
    int rc = prepare_resident(c);
    if (rc) return rc;
    {
        // device slots of the streamed layers: two, each as large as the largest of them
        size_t need = 0;
        for (auto &L : c->layer) need = std::max(need, L->pinned_bytes);
        if (need > c->wslot_bytes) {
            CK(cudaStreamSynchronize(c->stream));
            for (int i = 0; i < 2; ++i) {
                cudaFree(c->wslot[i]);
                c->wslot[i] = nullptr;
                CK(cudaMalloc(&c->wslot[i], need));
            }
            c->wslot_bytes = need;
        }
    }
    rc = build_graph_kind(c, 0);
    if (rc) return rc;
    if (c->dense_direct && c->resident) {
        rc = build_graph_kind(c, 1);
        if (rc) return rc;
    }
    c->graph_dirty = false;
    return SPDNN_OK;
}

// Builds the graphs if every layer has been set; returns false (without an error) when it cannot yet.
bool graphs_ready(spdnn *c) {
    if (!c->graph_dirty) return true;
    for (int l = 0; l < c->layers; ++l)
        if (!c->layer[l]) return false;
    return build_graph(c) == SPDNN_OK;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) { cudaGetDevice(&prev); cudaSetDevice(dev); }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

}  // namespace

extern "C" {

const char *spdnn_version(void) { return "spdnn_b200 0.1 (sm_100a)"; }

const char *spdnn_last_error(const spdnn_t *c) { return c ? c->err.c_str() : "null context"; }

int spdnn_create(spdnn_t **out, int device, int neurons, int layers, float bias, float clip) {
    if (!out) return SPDNN_ERR_ARG;
    *out = nullptr;
    spdnn *c = new (std::nothrow) spdnn();
    if (!c) return SPDNN_ERR_MEMORY;
    *out = c;   // returned even on failure so that the caller can read the message; destroy it either way
    if (neurons <= 0 || neurons > (1 << 26)) return fail(c, SPDNN_ERR_ARG, "neurons must be in [1, 2^26]");
    if (layers <= 0) return fail(c, SPDNN_ERR_ARG, "layers must be positive");
    if (!(clip > 0.0f)) return fail(c, SPDNN_ERR_ARG, "clip must be positive");
    int count = 0;
    CK(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return fail(c, SPDNN_ERR_ARG, "device %d not present (%d devices)", device, count);
    c->device = device; c->n = neurons; c->layers = layers; c->bias = bias; c->clip = clip;
    c->tile_stride = ((long long)neurons + 1) * 32;
    c->nw = front_words_per_tile(neurons);
    DeviceGuard guard(device);
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, device));
    c->sm_count = prop.multiProcessorCount;
    CK(cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking));
    c->stream = c->own_stream;
    CK(cudaEventCreate(&c->ev_prep0)); CK(cudaEventCreate(&c->ev_prep1));
    CK(cudaEventCreate(&c->ev_inf0)); CK(cudaEventCreate(&c->ev_inf1));
    CK(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
    CK(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
    for (int i = 0; i < 2; ++i) {
        CK(cudaEventCreateWithFlags(&c->ev_ready[i], cudaEventDisableTiming));
        CK(cudaEventCreateWithFlags(&c->ev_free[i], cudaEventDisableTiming));
    }
    c->layer.resize(layers);
    CK(cudaMalloc(&c->ctl, sizeof(LoopCtl) * (size_t)(layers + 1)));
    CK(cudaMemset(c->ctl, 0, sizeof(LoopCtl) * (size_t)(layers + 1)));
    CK(cudaMalloc(&c->counter, 2 * sizeof(unsigned int)));
    CK(cudaMemset(c->counter, 0, 2 * sizeof(unsigned int)));
    CK(cudaMalloc(&c->status, sizeof(int32_t)));
    CK(cudaMalloc(&c->dense_cell, sizeof(const float *)));
    CK(cudaMemset(c->dense_cell, 0, sizeof(const float *)));
    CK(cudaMemset(c->status, 0, sizeof(int32_t)));
    CK(cudaMalloc(&c->in_flag, sizeof(int32_t)));
    CK(cudaMemset(c->in_flag, 0, sizeof(int32_t)));
    CK(cudaMalloc(&c->died_at, sizeof(int32_t) * (size_t)layers));
    CK(cudaMemset(c->died_at, 0, sizeof(int32_t) * (size_t)layers));
    CK(cudaMalloc(&c->res_table, sizeof(ResLayer) * (size_t)layers));
    c->host_ctl.resize(layers + 1);
    c->host_died.assign(layers, 0);
    c->host_live.assign(layers, 0);
    {
        int optin = 0;
        CK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        c->smem_optin = optin;
        if (const char *e = getenv("SPDNN_RESIDENT")) { c->resident = atoi(e) != 0; c->resident_always = atoi(e) > 1; }
        if (const char *e = getenv("SPDNN_RESIDENT_TI")) {
            const int ti = atoi(e);
            if (ti == 32 || ti == 16 || ti == 8 || ti == 4) c->res_ti_max = ti;
        }
        if (const char *e = getenv("SPDNN_RESIDENT_IPT")) c->res_ipt_max = atoi(e) >= 8 ? 8 : 4;
        if (const char *e = getenv("SPDNN_STAGE_TABLES")) c->stage_tables = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_PRINT_SCHEDULE")) c->print_schedule = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_EXACT_SHORTCUT")) c->exact_shortcut = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_BIT_FORM")) c->bit_form = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_STAGE_KB")) c->stage_chunk = (size_t)std::max(1, atoi(e)) << 10;
        if (const char *e = getenv("SPDNN_BINARY_FRONT")) c->binary_front = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_COUNT_FRONT")) c->count_front = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_BITS_KERNEL")) c->bits_prepass = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_BITS_FIRST")) c->bits_first_chunk = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_TWO_BLOCKS")) c->two_blocks = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_TABLE_CACHE")) c->table_cache = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_BITS_SMALL")) c->bits_small = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_ALT2_THREADS")) c->alt2_threads = atoi(e) == 512 ? 512 : atoi(e) == 256 ? 256 : 0;
        if (const char *e = getenv("SPDNN_BITS_THREADS")) c->bits_threads = std::max(0, std::min(kBitsMaxThreads, atoi(e)));
        if (const char *e = getenv("SPDNN_LAZY_EXPAND")) c->lazy_expand = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_ALT2_SMALL_BLOCKS")) c->alt2_small_blocks = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_DENSE_DIRECT")) c->dense_direct = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_TABLE_RING")) c->table_ring_max = atoi(e) >= 4 ? 4 : 2;
        if (const char *e = getenv("SPDNN_WORD_RING")) c->word_ring_max = std::max(2, std::min(33, atoi(e)));
        if (const char *e = getenv("SPDNN_TABLE_GROUP")) c->table_group_max = std::max(1, std::min(32, atoi(e)));
        if (const char *e = getenv("SPDNN_REPS_ONLY")) c->reps_only = atoi(e) != 0;
        if (const char *e = getenv("SPDNN_CHUNK_FIRST")) c->chunk_first = std::max(1, atoi(e));
        if (const char *e = getenv("SPDNN_CHUNK_MAX")) c->chunk_max = std::max(1, atoi(e));
        if (const char *e = getenv("SPDNN_CHUNKS")) {
            for (const char *q = e; *q;) {
                char *end = nullptr;
                const long v = strtol(q, &end, 10);
                if (end == q) break;
                if (v > 0) c->chunk_list.push_back((int)std::min<long>(v, 1 << 20));
                q = (*end == ',') ? end + 1 : end;
            }
        }
        if (const char *e = getenv("SPDNN_CHUNK_GROWTH")) {
            c->chunk_growth = c->chunk_growth_generic = std::max(1, std::min(64, atoi(e)));
            c->chunk_growth_set = true;
        }
        if (const char *e = getenv("SPDNN_HOST_BUDGET_MB")) c->host_budget = (size_t)atoll(e) << 20;
        if (const char *e = getenv("SPDNN_WEIGHT_BUDGET_MB")) c->weight_budget = (size_t)atoll(e) << 20;
    }
    c->res.resize(layers);
    return SPDNN_OK;
}

void spdnn_destroy(spdnn_t *c) {
    if (!c) return;
    DeviceGuard guard(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (int kind = 0; kind < 2; ++kind)
        if (c->graph_exec[kind]) cudaGraphExecDestroy(c->graph_exec[kind]);
    cudaFree(c->dense_cell);
    free_buffers(c);
    cudaFree(c->ctl); cudaFree(c->counter); cudaFree(c->status); cudaFree(c->stage); cudaFree(c->in_flag);
    cudaFree(c->died_at); cudaFree(c->res_table);
    for (unsigned char *p : c->streams) cudaFree(p);
    c->layer.clear();
    if (c->ev_prep0) cudaEventDestroy(c->ev_prep0);
    if (c->ev_prep1) cudaEventDestroy(c->ev_prep1);
    if (c->ev_inf0) cudaEventDestroy(c->ev_inf0);
    if (c->ev_inf1) cudaEventDestroy(c->ev_inf1);
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    for (int i = 0; i < 2; ++i) {
        if (c->ev_ready[i]) cudaEventDestroy(c->ev_ready[i]);
        if (c->ev_free[i]) cudaEventDestroy(c->ev_free[i]);
        cudaFree(c->wslot[i]);
    }
    delete c;
}

int spdnn_set_stream(spdnn_t *c, void *cuda_stream) {
    if (!c) return SPDNN_ERR_ARG;
    DeviceGuard guard(c->device);
    if (c->in_flight) {
        int rc = spdnn_sync(c, nullptr);
        if (rc) return rc;
    }
    CK(cudaStreamSynchronize(c->stream));
    c->stream = cuda_stream ? (cudaStream_t)cuda_stream : c->own_stream;
    c->graph_dirty = true;    // the graph is re-captured on the stream it will be launched on
    return SPDNN_OK;
}

int spdnn_set_layer_csc(spdnn_t *c, int layer, const int32_t *col_ptr, const int32_t *row_idx, const float *val) {
    if (!c) return SPDNN_ERR_ARG;
    if (layer < 0 || layer >= c->layers) return fail(c, SPDNN_ERR_ARG, "layer %d out of range [0, %d)", layer, c->layers);
    if (!col_ptr || !row_idx) return fail(c, SPDNN_ERR_ARG, "col_ptr and row_idx must not be null");
    DeviceGuard guard(c->device);
    if (c->in_flight) {
        int rc = spdnn_sync(c, nullptr);
        if (rc) return rc;
    }
    auto host = std::make_shared<HostLayer>();
    PerLayerTables p;
    std::string why;
    try {
        why = canonicalize_layer(c->n, col_ptr, row_idx, val, *host);
        if (!why.empty()) return fail(c, SPDNN_ERR_ARG, "layer %d: %s", layer, why.c_str());
        c->graph_dirty = true;
        // equal layers share one device copy
        auto it = c->shared.find(host->hash1);
        if (it != c->shared.end()) {
            if (auto sp = it->second.lock()) {
                if (sp->h2 == host->hash2 && sp->k == host->k && sp->nnz == host->nnz) {
                    c->layer[layer] = sp;
                    return SPDNN_OK;
                }
            }
        }
        build_per_layer_tables(*host, p);
    } catch (const std::bad_alloc &) {
        return fail(c, SPDNN_ERR_MEMORY, "out of host memory preparing layer %d", layer);
    }
    auto L = std::make_shared<DevLayer>();
    L->device = c->device;
    L->classes = p.classes; L->k = host->k; L->uniform = host->uniform; L->identity_members = p.identity_members;
    L->w = host->w; L->nnz = host->nnz; L->h1 = host->hash1; L->h2 = host->hash2;
    const size_t table_bytes = 4 * (std::max<size_t>(p.off.size(), 4) + (host->uniform ? 0 : std::max<size_t>(p.vals.size(), 4)) +
                                    p.mem_ptr.size() + std::max<size_t>(p.mem.size(), 1));
    if (c->weight_bytes + table_bytes > c->weight_budget) {
        // over the device budget: keep the tables in page-locked host memory, streamed in by the layer loop
        const size_t off_b = (4 * std::max<size_t>(p.off.size(), 4) + 15) / 16 * 16;
        const size_t val_b = host->uniform ? 0 : (4 * std::max<size_t>(p.vals.size(), 4) + 15) / 16 * 16;
        const size_t mp_b = (4 * p.mem_ptr.size() + 15) / 16 * 16, mem_b = (4 * std::max<size_t>(p.mem.size(), 1) + 15) / 16 * 16;
        L->o_vals = off_b; L->o_mem_ptr = off_b + val_b; L->o_mem = L->o_mem_ptr + mp_b;
        L->pinned_bytes = L->o_mem + mem_b;
        if (cudaMallocHost(&L->pinned, L->pinned_bytes) != cudaSuccess) {
            cudaGetLastError();
            return fail(c, SPDNN_ERR_MEMORY, "out of page-locked host memory for streamed layer %d", layer);
        }
        memset(L->pinned, 0, L->pinned_bytes);
        memcpy(L->pinned, p.off.data(), 4 * p.off.size());
        if (!host->uniform) memcpy(L->pinned + L->o_vals, p.vals.data(), 4 * p.vals.size());
        memcpy(L->pinned + L->o_mem_ptr, p.mem_ptr.data(), 4 * p.mem_ptr.size());
        memcpy(L->pinned + L->o_mem, p.mem.data(), 4 * p.mem.size());
        c->layer[layer] = L;               // no canonical host copy: a streamed layer runs in the per-layer kernel
        c->shared[host->hash1] = L;
        return SPDNN_OK;
    }
    c->weight_bytes += table_bytes;
    CK(cudaMalloc(&L->off, sizeof(int32_t) * std::max<size_t>(p.off.size(), 4)));
    CK(cudaMemcpyAsync(L->off, p.off.data(), sizeof(int32_t) * p.off.size(), cudaMemcpyHostToDevice, c->stream));
    if (!host->uniform) {
        CK(cudaMalloc(&L->vals, sizeof(float) * std::max<size_t>(p.vals.size(), 4)));
        CK(cudaMemcpyAsync(L->vals, p.vals.data(), sizeof(float) * p.vals.size(), cudaMemcpyHostToDevice, c->stream));
    }
    CK(cudaMalloc(&L->mem_ptr, sizeof(int32_t) * p.mem_ptr.size()));
    CK(cudaMemcpyAsync(L->mem_ptr, p.mem_ptr.data(), sizeof(int32_t) * p.mem_ptr.size(), cudaMemcpyHostToDevice, c->stream));
    CK(cudaMalloc(&L->mem, sizeof(int32_t) * std::max<size_t>(p.mem.size(), 1)));
    CK(cudaMemcpyAsync(L->mem, p.mem.data(), sizeof(int32_t) * p.mem.size(), cudaMemcpyHostToDevice, c->stream));
    CK(cudaStreamSynchronize(c->stream));     // p's host vectors die with this call
    // the canonical form stays on the host (within a budget) for the resident kernel's tables
    if (c->resident) {
        if (host->uniform) std::vector<float>().swap(host->vals);
        const size_t bytes = host->rows.size() * 4 + host->vals.size() * 4;
        if (c->host_bytes + bytes <= c->host_budget) {
            c->host_bytes += bytes;
            L->host = host;
        }
    }
    c->layer[layer] = L;
    c->shared[host->hash1] = L;
    return SPDNN_OK;
}

int spdnn_set_layer_same_as(spdnn_t *c, int layer, int other_layer) {
    if (!c) return SPDNN_ERR_ARG;
    if (layer < 0 || layer >= c->layers || other_layer < 0 || other_layer >= c->layers)
        return fail(c, SPDNN_ERR_ARG, "layer %d or %d out of range [0, %d)", layer, other_layer, c->layers);
    if (!c->layer[other_layer]) return fail(c, SPDNN_ERR_STATE, "layer %d was never set", other_layer);
    DeviceGuard guard(c->device);
    if (c->in_flight) {
        int rc = spdnn_sync(c, nullptr);
        if (rc) return rc;
    }
    c->layer[layer] = c->layer[other_layer];
    c->graph_dirty = true;
    return SPDNN_OK;
}

int spdnn_set_layer_coo(spdnn_t *c, int layer, int64_t nnz, const int32_t *in_neuron, const int32_t *out_neuron,
                        const float *val, int index_base) {
    if (!c) return SPDNN_ERR_ARG;
    if (nnz < 0 || nnz > 0x7fffffffLL) return fail(c, SPDNN_ERR_ARG, "nnz out of range");
    if (nnz && (!in_neuron || !out_neuron)) return fail(c, SPDNN_ERR_ARG, "triplet arrays must not be null");
    const int n = c->n;
    try {
        std::vector<int32_t> col_ptr((size_t)n + 1, 0), rows((size_t)nnz);
        std::vector<float> vals(val ? (size_t)nnz : 0);
        for (int64_t i = 0; i < nnz; ++i) {
            const int64_t b = (int64_t)out_neuron[i] - index_base, a = (int64_t)in_neuron[i] - index_base;
            if (b < 0 || b >= n || a < 0 || a >= n)
                return fail(c, SPDNN_ERR_ARG, "layer %d: triplet %lld (%d, %d) out of range", layer, (long long)i,
                            in_neuron[i], out_neuron[i]);
            col_ptr[b + 1]++;
        }
        for (int i = 0; i < n; ++i) col_ptr[i + 1] += col_ptr[i];
        std::vector<int32_t> fill(col_ptr.begin(), col_ptr.end() - 1);
        for (int64_t i = 0; i < nnz; ++i) {
            const int b = out_neuron[i] - index_base;
            const int p = fill[b]++;
            rows[p] = in_neuron[i] - index_base;
            if (val) vals[p] = val[i];
        }
        return spdnn_set_layer_csc(c, layer, col_ptr.data(), rows.data(), val ? vals.data() : nullptr);
    } catch (const std::bad_alloc &) {
        return fail(c, SPDNN_ERR_MEMORY, "out of host memory converting layer %d", layer);
    }
}

int spdnn_set_input_dense_device(spdnn_t *c, const float *y0_dev, int batch, int first_global_id) {
    if (!c) return SPDNN_ERR_ARG;
    if (!y0_dev && batch > 0) return fail(c, SPDNN_ERR_ARG, "input pointer is null");
    DeviceGuard guard(c->device);
    int rc = begin_input(c, batch, first_global_id);
    if (rc) return rc;
    if (batch > 0 && c->dense_direct && graphs_ready(c) && c->graph_exec[1]) {
        c->dense_src = y0_dev;       // read in place by the first launch of the pass
        c->input_kind = 1;
        return end_input(c);
    }
    rc = convert_dense_device(c, y0_dev, batch, 0);
    if (rc) return rc;
    rc = repair_float_tiles(c);
    if (rc) return rc;
    return end_input(c);
}

int spdnn_set_input_dense(spdnn_t *c, const float *y0, int batch, int first_global_id) {
    if (!c) return SPDNN_ERR_ARG;
    if (!y0 && batch > 0) return fail(c, SPDNN_ERR_ARG, "input pointer is null");
    DeviceGuard guard(c->device);
    int rc = begin_input(c, batch, first_global_id);
    if (rc) return rc;
    const size_t row_bytes = sizeof(float) * (size_t)c->n;
    if (batch > 0 && c->dense_direct && (size_t)batch * row_bytes <= ((size_t)1 << 30) && graphs_ready(c) && c->graph_exec[1]) {
        // one copy into the staging buffer, which the first launch of the pass reads in place
        rc = ensure_stage(c, (size_t)batch * row_bytes);
        if (rc) return rc;
        CK(cudaMemcpyAsync(c->stage, y0, (size_t)batch * row_bytes, cudaMemcpyHostToDevice, c->stream));
        c->dense_src = (const float *)c->stage;
        c->input_kind = 1;
        return end_input(c);
    }
    // staged through a device buffer in chunks of whole tiles
    size_t chunk_rows = std::max<size_t>(32, c->stage_chunk / row_bytes / 32 * 32);
    chunk_rows = std::min<size_t>(chunk_rows, (size_t)(batch + 31) / 32 * 32);
    if (batch > 0) {
        rc = ensure_stage(c, chunk_rows * row_bytes);
        if (rc) return rc;
    }
    for (size_t r0 = 0; r0 < (size_t)batch; r0 += chunk_rows) {
        const size_t rows = std::min(chunk_rows, (size_t)batch - r0);
        CK(cudaMemcpyAsync(c->stage, y0 + r0 * c->n, rows * row_bytes, cudaMemcpyHostToDevice, c->stream));
        rc = convert_dense_device(c, (const float *)c->stage, (int)rows, (int)(r0 / 32));
        if (rc) return rc;
    }
    rc = repair_float_tiles(c);
    if (rc) return rc;
    return end_input(c);
}

int spdnn_set_input_coo(spdnn_t *c, int64_t nnz, const int32_t *img, const int32_t *neuron, const float *val,
                        int batch, int first_global_id, int index_base) {
    if (!c) return SPDNN_ERR_ARG;
    if (nnz < 0) return fail(c, SPDNN_ERR_ARG, "nnz must be >= 0");
    if (nnz && (!img || !neuron)) return fail(c, SPDNN_ERR_ARG, "triplet arrays must not be null");
    DeviceGuard guard(c->device);
    int rc = begin_input(c, batch, first_global_id);
    if (rc) return rc;
    const int tiles = (batch + 31) / 32;
    // Triplets without values are ones: a binary input, kept as words only.  With values both forms are built
    // (the words' flag tells the pass which one to read).
    const bool words = c->binary_front, floats = !c->binary_front || val != nullptr;
    if (tiles && floats) {
        CK(cudaMemsetAsync(c->y[0], 0, sizeof(float) * (size_t)tiles * c->tile_stride, c->stream));
        CK(cudaMemsetAsync(c->has_floats, 1, (size_t)tiles, c->stream));
    }
    if (tiles && words) CK(cudaMemsetAsync(c->xw, 0, sizeof(uint32_t) * (size_t)tiles * c->nw, c->stream));
    const int64_t chunk = std::min<int64_t>(std::max<int64_t>(nnz, 1), (int64_t)32 << 20);
    const size_t per = val ? 12 : 8;
    if (nnz) {
        rc = ensure_stage(c, (size_t)chunk * per);
        if (rc) return rc;
    }
    for (int64_t s = 0; s < nnz; s += chunk) {
        const int64_t m = std::min(chunk, nnz - s);
        int32_t *d_img = (int32_t *)c->stage, *d_neu = d_img + chunk;
        float *d_val = val ? (float *)(d_neu + chunk) : nullptr;
        CK(cudaMemcpyAsync(d_img, img + s, sizeof(int32_t) * (size_t)m, cudaMemcpyHostToDevice, c->stream));
        CK(cudaMemcpyAsync(d_neu, neuron + s, sizeof(int32_t) * (size_t)m, cudaMemcpyHostToDevice, c->stream));
        if (val) CK(cudaMemcpyAsync(d_val, val + s, sizeof(float) * (size_t)m, cudaMemcpyHostToDevice, c->stream));
        const int grid = (int)std::min<int64_t>((m + 255) / 256, (int64_t)c->sm_count * 16);
        if (words) {
            coo_to_words_kernel<<<grid, 256, 0, c->stream>>>(d_img, d_neu, d_val, m, index_base, c->n, batch, c->xw, c->nw,
                                                             c->in_flag, c->status);
            CK(cudaGetLastError());
            c->prep_launches += 1;
        }
        if (floats) {
            coo_to_tiles_kernel<<<grid, 256, 0, c->stream>>>(d_img, d_neu, d_val, m, index_base, c->n, batch, c->y[0],
                                                             c->tile_stride, c->status);
            CK(cudaGetLastError());
            c->prep_launches += 1;
        }
    }
    return end_input(c);
}

// Packed rows on the device -> words; with the binary front switched off, on to float tiles.
static int convert_bits_device(spdnn *c, const uint32_t *dev_rows, long long row_words, int rows, int first_tile) {
    if (rows <= 0) return SPDNN_OK;
    const long long warps = (long long)((rows + 31) / 32) * ((c->n + 31) / 32);
    const int grid = (int)std::min<long long>((warps + 7) / 8, (long long)c->sm_count * 32);
    rows_to_words_kernel<<<std::max(1, grid), 256, 0, c->stream>>>(dev_rows, row_words, c->n, rows, c->xw, c->nw, first_tile);
    CK(cudaGetLastError());
    c->prep_launches += 1;
    return SPDNN_OK;
}

static int finish_bits_input(spdnn *c) {
    if (!c->binary_front && c->batch > 0) {
        // every pass reads float tiles: expand the words (the flag is 1 for the whole life of such a context)
        const int tiles = (c->batch + 31) / 32;
        const long long warps = (long long)tiles * c->n;
        const int grid = (int)std::min<long long>((warps + 7) / 8, (long long)c->sm_count * 32);
        words_to_tiles_kernel<<<std::max(1, grid), 256, 0, c->stream>>>(c->xw, c->nw, c->n, tiles, c->y[0], c->tile_stride, nullptr,
                                                                         c->in_flag, 1);
        CK(cudaGetLastError());
        c->prep_launches += 1;
    }
    return end_input(c);
}

int spdnn_set_input_bits_device(spdnn_t *c, const uint8_t *bits_dev, int64_t row_bytes, int batch, int first_global_id) {
    if (!c) return SPDNN_ERR_ARG;
    if (!bits_dev && batch > 0) return fail(c, SPDNN_ERR_ARG, "input pointer is null");
    if (row_bytes < (c->n + 7) / 8 || (row_bytes & 3) || (reinterpret_cast<size_t>(bits_dev) & 3))
        return fail(c, SPDNN_ERR_ARG, "row_bytes must be a multiple of 4 and at least ceil(neurons / 8); the buffer 4-byte aligned");
    DeviceGuard guard(c->device);
    int rc = begin_input(c, batch, first_global_id);
    if (rc) return rc;
    rc = convert_bits_device(c, reinterpret_cast<const uint32_t *>(bits_dev), row_bytes / 4, batch, 0);
    if (rc) return rc;
    return finish_bits_input(c);
}

int spdnn_set_input_bits(spdnn_t *c, const uint8_t *bits, int64_t row_bytes, int batch, int first_global_id) {
    if (!c) return SPDNN_ERR_ARG;
    if (!bits && batch > 0) return fail(c, SPDNN_ERR_ARG, "input pointer is null");
    if (row_bytes < (c->n + 7) / 8 || (row_bytes & 3))
        return fail(c, SPDNN_ERR_ARG, "row_bytes must be a multiple of 4 and at least ceil(neurons / 8)");
    DeviceGuard guard(c->device);
    int rc = begin_input(c, batch, first_global_id);
    if (rc) return rc;
    // staged through a device buffer in chunks of whole tiles
    size_t chunk_rows = std::max<size_t>(32, c->stage_chunk / 2 / (size_t)row_bytes / 32 * 32);
    chunk_rows = std::min<size_t>(chunk_rows, (size_t)(batch + 31) / 32 * 32);
    if (batch > 0) {
        rc = ensure_stage(c, chunk_rows * (size_t)row_bytes);
        if (rc) return rc;
    }
    for (size_t r0 = 0; r0 < (size_t)batch; r0 += chunk_rows) {
        const size_t rows = std::min(chunk_rows, (size_t)batch - r0);
        CK(cudaMemcpyAsync(c->stage, bits + r0 * (size_t)row_bytes, rows * (size_t)row_bytes, cudaMemcpyHostToDevice, c->stream));
        rc = convert_bits_device(c, (const uint32_t *)c->stage, row_bytes / 4, (int)rows, (int)(r0 / 32));
        if (rc) return rc;
    }
    return finish_bits_input(c);
}

int spdnn_infer_async(spdnn_t *c) {
    if (!c) return SPDNN_ERR_ARG;
    if (!c->input_ready) return fail(c, SPDNN_ERR_STATE, "no input set (or the last input was already consumed)");
    for (int l = 0; l < c->layers; ++l)
        if (!c->layer[l]) return fail(c, SPDNN_ERR_STATE, "layer %d was never set", l);
    DeviceGuard guard(c->device);
    if (c->graph_dirty) {
        int rc = build_graph(c);
        if (rc) return rc;
    }
    CK(cudaEventRecord(c->ev_inf0, c->stream));
    if (c->input_kind == 1 && !c->graph_exec[1])
        return fail(c, SPDNN_ERR_STATE, "the network changed after the input was set: set the input again");
    c->nsteps = c->graph_steps[c->input_kind];
    c->extra_launches = c->graph_extra[c->input_kind];
    c->last_group = c->graph_group[c->input_kind];
    c->final_expand_layer = c->graph_expand_layer[c->input_kind];
    c->final_needs_expand = c->final_expand_layer >= 0;
    CK(cudaGraphLaunch(c->graph_exec[c->input_kind], c->stream));
    CK(cudaEventRecord(c->ev_inf1, c->stream));
    c->input_ready = false;
    c->in_flight = true;
    return SPDNN_OK;
}

int spdnn_sync(spdnn_t *c, spdnn_stats_t *stats) {
    if (!c) return SPDNN_ERR_ARG;
    DeviceGuard guard(c->device);
    if (c->in_flight) {
        CK(cudaMemcpyAsync(c->host_ctl.data(), c->ctl, sizeof(LoopCtl) * (size_t)(c->nsteps + 1), cudaMemcpyDeviceToHost,
                           c->stream));
        CK(cudaMemcpyAsync(c->host_died.data(), c->died_at, sizeof(int32_t) * (size_t)c->layers, cudaMemcpyDeviceToHost,
                           c->stream));
        int32_t st = 0;
        CK(cudaMemcpyAsync(&st, c->status, sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
        CK(cudaStreamSynchronize(c->stream));
        c->in_flight = false;
        if (st != 0) {
            cudaMemsetAsync(c->status, 0, sizeof(int32_t), c->stream);
            return fail(c, SPDNN_ERR_DEVICE, "device-side check failed (code %d: %s)", st,
                        st == 3 ? "input triplet out of range"
                                : st == 4 ? "a table copy into shared memory did not complete within the wait limit"
                                          : "survivor count inconsistent");
        }
        spdnn_stats_t s{};
        s.layers = c->layers; s.batch = c->batch;
        s.survivors = c->host_ctl[c->nsteps].live;
        {
            long long live = c->batch;
            for (int l = 0; l < c->layers; ++l) {
                live -= c->host_died[l];
                c->host_live[l] = (int32_t)live;
            }
            if (live != s.survivors) {
                return fail(c, SPDNN_ERR_DEVICE, "survivor bookkeeping inconsistent (%lld by layer, %lld final)", live,
                            (long long)s.survivors);
            }
        }
        CK(cudaEventElapsedTime(&s.infer_ms, c->ev_inf0, c->ev_inf1));
        if (c->prep_timed) CK(cudaEventElapsedTime(&s.prepare_ms, c->ev_prep0, c->ev_prep1));
        double bytes = 0.0;
        for (int l = 0; l < c->layers; ++l) {
            const double live_in = l ? (double)c->host_live[l - 1] : (double)c->batch;
            bytes += 4.0 * c->n * (live_in + (double)c->host_live[l]);
            bytes += 4.0 * (c->n + 1) + 8.0 * (double)c->layer[l]->nnz;
        }
        s.algorithmic_bytes = bytes;
        s.kernel_launches = c->nsteps + c->extra_launches + 1 + c->prep_launches;      // + finalize_ids_kernel
        s.loop_launches = c->nsteps;
        s.resident_group = c->last_group;
        c->stats = s;
        c->result_ready = true;
    }
    if (stats) *stats = c->stats;
    return SPDNN_OK;
}

int spdnn_infer(spdnn_t *c, spdnn_stats_t *stats) {
    int rc = spdnn_infer_async(c);
    if (rc) return rc;
    return spdnn_sync(c, stats);
}

int spdnn_get_layer_live(spdnn_t *c, int32_t *live, int capacity) {
    if (!c || !live) return SPDNN_ERR_ARG;
    if (c->in_flight) { int rc = spdnn_sync(c, nullptr); if (rc) return rc; }
    if (!c->result_ready) return fail(c, SPDNN_ERR_STATE, "no result: call spdnn_infer first");
    if (capacity < c->layers) return fail(c, SPDNN_ERR_ARG, "capacity %d < layers %d", capacity, c->layers);
    for (int l = 0; l < c->layers; ++l) live[l] = c->host_live[l];
    return SPDNN_OK;
}

int spdnn_get_categories(spdnn_t *c, int32_t *ids, int capacity, int *count) {
    if (!c || !count) return SPDNN_ERR_ARG;
    if (c->in_flight) { int rc = spdnn_sync(c, nullptr); if (rc) return rc; }
    if (!c->result_ready) return fail(c, SPDNN_ERR_STATE, "no result: call spdnn_infer first");
    const LoopCtl fin = c->host_ctl[c->nsteps];
    *count = fin.live;
    if (fin.live == 0) return SPDNN_OK;
    if (!ids || capacity < fin.live) return fail(c, SPDNN_ERR_ARG, "capacity %d < survivors %d", capacity, fin.live);
    DeviceGuard guard(c->device);
    CK(cudaMemcpyAsync(ids, c->ids[fin.ids_buf], sizeof(int32_t) * (size_t)fin.live, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return SPDNN_OK;
}

int spdnn_get_activations(spdnn_t *c, float *y, int64_t capacity_rows) {
    if (!c) return SPDNN_ERR_ARG;
    if (c->in_flight) { int rc = spdnn_sync(c, nullptr); if (rc) return rc; }
    if (!c->result_ready) return fail(c, SPDNN_ERR_STATE, "no result: call spdnn_infer first");
    const int live = c->host_ctl[c->nsteps].live;
    if (live == 0) return SPDNN_OK;
    if (!y || capacity_rows < live) return fail(c, SPDNN_ERR_ARG, "capacity %lld < survivors %d", (long long)capacity_rows, live);
    DeviceGuard guard(c->device);
    const size_t row_bytes = sizeof(float) * (size_t)c->n;
    size_t chunk_rows = std::max<size_t>(32, c->stage_chunk / row_bytes / 32 * 32);
    chunk_rows = std::min<size_t>(chunk_rows, (size_t)(live + 31) / 32 * 32);
    int rc = ensure_stage(c, chunk_rows * row_bytes);
    if (rc) return rc;
    float *fin = c->y[c->nsteps & 1];
    if (c->final_needs_expand) {
        // the last launch stored one row per class: copy it to the other members in every tile it wrote
        const DevRes &R = *c->res[c->final_expand_layer];
        const int tiles = (c->host_ctl[c->nsteps - 1].live + 31) / 32;
        const long long warps = (long long)tiles * R.classes;
        const int grid = (int)std::min<long long>((warps + 7) / 8, (long long)c->sm_count * 16);
        expand_members_kernel<<<std::max(1, grid), 256, 0, c->stream>>>(fin, c->tile_stride, tiles, R.mem_ptr, R.mem, R.classes);
        CK(cudaGetLastError());
        c->final_needs_expand = false;
    }
    // the kernel indexes images from 0; a chunk is selected by offsetting the output pointer
    // and launching only its tile rows
    for (size_t r0 = 0; r0 < (size_t)live; r0 += chunk_rows) {
        const size_t rows = std::min(chunk_rows, (size_t)live - r0);
        const dim3 block(32, 8), grid((unsigned)((rows + 31) / 32), (c->n + 31) / 32);
        tiles_to_dense_kernel<<<grid, block, 0, c->stream>>>(fin, c->tile_stride, c->ctl + c->nsteps, c->slot, c->n,
                                                            (float *)c->stage, (int)r0);
        CK(cudaGetLastError());
        CK(cudaMemcpyAsync(y + r0 * c->n, c->stage, rows * row_bytes, cudaMemcpyDeviceToHost, c->stream));
    }
    CK(cudaStreamSynchronize(c->stream));
    return SPDNN_OK;
}

int spdnn_get_layer_info(spdnn_t *c, int layer, int *classes, int *k, int *uniform) {
    if (!c) return SPDNN_ERR_ARG;
    if (layer < 0 || layer >= c->layers) return fail(c, SPDNN_ERR_ARG, "layer %d out of range", layer);
    if (!c->layer[layer]) return fail(c, SPDNN_ERR_STATE, "layer %d was never set", layer);
    if (classes) *classes = c->layer[layer]->classes;
    if (k) *k = c->layer[layer]->k;
    if (uniform) *uniform = c->layer[layer]->uniform ? 1 : 0;
    return SPDNN_OK;
}

int spdnn_inspect_layer_csc(int neurons, const int32_t *col_ptr, const int32_t *row_idx, const float *val,
                            int *classes, int *k, int *uniform) {
    HostLayer h;
    PerLayerTables p;
    try {
        if (!canonicalize_layer(neurons, col_ptr, row_idx, val, h).empty()) return SPDNN_ERR_ARG;
        build_per_layer_tables(h, p);
    } catch (const std::bad_alloc &) {
        return SPDNN_ERR_MEMORY;
    }
    if (classes) *classes = p.classes;
    if (k) *k = h.k;
    if (uniform) *uniform = h.uniform ? 1 : 0;
    return SPDNN_OK;
}

int spdnn_inspect_network_csc(int neurons, int layers, const int32_t *const *col_ptr, const int32_t *const *row_idx,
                              const float *const *val, int32_t *classes, int32_t *v_in, int32_t *form) {
    if (layers < 0 || !col_ptr || !row_idx) return SPDNN_ERR_ARG;
    try {
        std::vector<int32_t> vid;          // value ids of the current layer's input (empty: the neurons themselves)
        int vin = neurons;
        for (int l = 0; l < layers; ++l) {
            HostLayer h;
            if (!canonicalize_layer(neurons, col_ptr[l], row_idx[l], val ? val[l] : nullptr, h).empty()) return SPDNN_ERR_ARG;
            ResidentTables t;
            build_resident_tables(h, vid.empty() ? nullptr : vid.data(), vin, t);
            if (classes) classes[l] = t.classes;
            if (v_in) v_in[l] = t.v_in;
            if (form) form[l] = t.mode;
            if (t.classes < neurons) { vid.swap(t.class_of); vin = t.classes; }
            else { vid.clear(); vin = neurons; }
        }
    } catch (const std::bad_alloc &) {
        return SPDNN_ERR_MEMORY;
    }
    return SPDNN_OK;
}

}  // extern "C"
