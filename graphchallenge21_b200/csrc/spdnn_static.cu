// spdnn_layer_static: one layer of the inference loop for callers that cannot allocate.
//
// Some hosts of this library may not call cudaMalloc at the point where they run a layer: a
// plugin running inside another runtime's memory pool that has handed out the whole device,
// a callback on a latency-critical path where an allocation (an implicit device
// synchronisation) is forbidden, or a process that has dropped the right to grow its
// footprint after start-up.  Everything else in this library keeps its work buffers in
// context-owned device memory; this entry point instead keeps the scratch of the layer
// kernel -- the per-tile survivor ballots and the two block counters -- in a fixed array that
// is part of the loaded module.  The caller passes inputs and outputs; nothing is allocated
// or freed here, by the CUDA runtime or otherwise.
//
// The price: the array is sized for at most SPDNN_STATIC_MAX_IMAGES images per call, every
// GPU that loads the library holds it (264 KB) until the process exits, and all calls on one
// GPU share it, so two calls must not overlap on the device (put them on one stream or order
// them with events) -- overlapping calls race on the ballots and counters.
#include "../../include/spdnn_b200.h"

#include <cstdio>
#include <mutex>

#include "spdnn_kernels.cuh"

using namespace spdnn_impl;

namespace {

constexpr int kMaxTiles = SPDNN_STATIC_MAX_IMAGES / 32;

struct StaticScratch {
    unsigned int counter;          // blocks finished
    unsigned int work;             // next work item
    unsigned int pad[62];
    uint32_t mask[kMaxTiles];      // ballot of alive lanes per output tile
};

// In host code this name is only a handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

struct StaticArgs {
    const float *yin;
    float *yout;
    long long tile_stride;
    const int32_t *in_positions;   // nullptr: image j sits at position j of yin
    const int32_t *off;
    const float *vals;
    int32_t *survivors;
    int32_t *survivor_count;
    StaticScratch *scratch;
    int neurons, k, live_in, classes_per_item;
    float w, bias, clip;
};

// Same arithmetic as layer_kernel (class_sum, relu_clip); differs in where the scratch lives
// and in the tail, which always writes the survivor positions and their count.
template <int KT, bool UNIFORM>
__global__ void __launch_bounds__(kThreads, SPDNN_MIN_BLOCKS) layer_static_kernel(const StaticArgs a) {
    __shared__ unsigned int s_mask, s_item;
    __shared__ int s_last, s_warp[kWarps], s_total;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    StaticScratch *sc = a.scratch;
    LayerDesc d;
    d.off = a.off; d.vals = a.vals; d.mem_ptr = nullptr; d.mem = nullptr;
    d.classes = a.neurons; d.k = a.k; d.w = a.w; d.classes_per_item = a.classes_per_item;
    const int ntiles = (a.live_in + 31) >> 5;
    const int cpi = a.classes_per_item;
    const int ncb = (a.neurons + cpi - 1) / cpi;
    const unsigned int items = (unsigned int)ntiles * (unsigned int)ncb;
    const int per_warp = (cpi + kWarps - 1) / kWarps;
    for (;;) {
        if (tid == 0) { s_item = atomicAdd(&sc->work, 1u); s_mask = 0u; }
        __syncthreads();
        const unsigned int item = s_item;
        if (item >= items) break;
        const int tile = (int)(item / (unsigned int)ncb);
        const int cb = (int)(item - (unsigned int)tile * (unsigned int)ncb);
        const int j = tile * 32 + lane;
        const bool valid = j < a.live_in;
        const int jj = valid ? j : tile * 32;
        const int src = a.in_positions ? __ldg(a.in_positions + jj) : jj;
        const float *__restrict__ yin = a.yin + (size_t)(src >> 5) * a.tile_stride + (src & 31);
        float *__restrict__ yout = a.yout + (size_t)tile * a.tile_stride + lane;
        bool any = false;
        const int u_end = min(a.neurons, (cb + 1) * cpi);
        const int u0 = cb * cpi + warp * per_warp, u1 = min(u0 + per_warp, u_end);
        for (int u = u0; u < u1; ++u) {
            const float y = relu_clip(__fadd_rn(class_sum<KT, UNIFORM>(d, u, yin), a.bias), a.clip);
            any |= (y != 0.0f);
            yout[(size_t)u * 32] = y;
        }
        const unsigned int m = __ballot_sync(0xffffffffu, any && valid);
        if (lane == 0 && m) atomicOr(&s_mask, m);
        __syncthreads();
        if (tid == 0 && s_mask) atomicOr(&sc->mask[tile], s_mask);
    }
    if (tid == 0) {
        __threadfence();
        s_last = (atomicAdd(&sc->counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // last block: prefix sum over the ballots -> ascending survivor positions
    const int per = (ntiles + kThreads - 1) / kThreads;
    const int t0 = min(tid * per, ntiles), t1 = min(t0 + per, ntiles);
    int cnt = 0;
    for (int t = t0; t < t1; ++t) cnt += __popc(__ldcg(&sc->mask[t]));
    int inc = cnt;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, s);
        if (lane >= s) inc += o;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < kWarps ? s_warp[lane] : 0;
#pragma unroll
        for (int s = 1; s < kWarps; s <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, w, s);
            if (lane >= s) w += o;
        }
        if (lane < kWarps) s_warp[lane] = w;
        if (lane == kWarps - 1) s_total = w;
    }
    __syncthreads();
    int base = inc - cnt + (warp ? s_warp[warp - 1] : 0);
    for (int t = t0; t < t1; ++t) {
        uint32_t m = __ldcg(&sc->mask[t]);
        while (m) {
            const int b = __ffs(m) - 1;
            m &= m - 1;
            a.survivors[base++] = t * 32 + b;
        }
        sc->mask[t] = 0u;        // leave the scratch clean for the next call
    }
    if (tid == 0) {
        *a.survivor_count = s_total;
        sc->counter = 0u;
        sc->work = 0u;
    }
}

struct PerDevice {
    StaticScratch *scratch = nullptr;
    int sm_count = 0;
    int blocks_per_sm[4] = {0, 0, 0, 0};
};

std::mutex g_mu;
PerDevice g_dev[64];

int say(char *err, int err_len, int code, const char *msg) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", msg);
    return code;
}

template <int KT, bool UNIFORM>
cudaError_t occupancy(int *b) {
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(b, layer_static_kernel<KT, UNIFORM>, kThreads, 0);
}

}  // namespace

extern "C" int spdnn_layer_static(const float *yin, float *yout, int neurons, int live_in, const int32_t *in_positions,
                                  const int32_t *off, const float *vals, int k, float w, float bias, float clip,
                                  int32_t *survivors, int32_t *survivor_count, void *cuda_stream, char *err,
                                  int err_len) {
    if (!yin || !yout || !off || !survivors || !survivor_count) return say(err, err_len, SPDNN_ERR_ARG, "null device pointer");
    // the padding entry of `off` is neurons * 32 and must fit in int32
    if (neurons <= 0 || neurons >= (1 << 26)) return say(err, err_len, SPDNN_ERR_ARG, "neurons must be in [1, 2^26)");
    if (k <= 0 || (k & 3)) return say(err, err_len, SPDNN_ERR_ARG, "k must be a positive multiple of 4");
    if (live_in < 0) return say(err, err_len, SPDNN_ERR_ARG, "live_in must be >= 0");
    if (live_in > SPDNN_STATIC_MAX_IMAGES) {
        char msg[160];
        snprintf(msg, sizeof msg, "live_in %d exceeds the static scratch limit of %d images per call: split the batch",
                 live_in, SPDNN_STATIC_MAX_IMAGES);
        return say(err, err_len, SPDNN_ERR_LIMIT, msg);
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return say(err, err_len, SPDNN_ERR_CUDA, "no current CUDA device");
    PerDevice pd;
    {
        // first call on this device: resolve the device address of the scratch array and the
        // launch shape.  (Do this once before any stream capture.)
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_dev[dev].scratch) {
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p) return say(err, err_len, SPDNN_ERR_CUDA, cudaGetErrorString(e));
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return say(err, err_len, SPDNN_ERR_CUDA, cudaGetErrorString(e));
            PerDevice n;
            n.sm_count = sms;
            if (occupancy<32, true>(&n.blocks_per_sm[0]) != cudaSuccess || occupancy<32, false>(&n.blocks_per_sm[1]) != cudaSuccess ||
                occupancy<0, true>(&n.blocks_per_sm[2]) != cudaSuccess || occupancy<0, false>(&n.blocks_per_sm[3]) != cudaSuccess)
                return say(err, err_len, SPDNN_ERR_CUDA, "occupancy query failed");
            n.scratch = static_cast<StaticScratch *>(p);
            g_dev[dev] = n;
        }
        pd = g_dev[dev];
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    const int ntiles = (live_in + 31) / 32;
    // the scratch keeps the last call's contents: clear what must start at zero
    e = cudaMemsetAsync(pd.scratch, 0, offsetof(StaticScratch, mask) + sizeof(uint32_t) * (size_t)(ntiles > 0 ? ntiles : 1), stream);
    if (e != cudaSuccess) return say(err, err_len, SPDNN_ERR_CUDA, cudaGetErrorString(e));
    StaticArgs a;
    a.yin = yin; a.yout = yout; a.tile_stride = ((long long)neurons + 1) * 32;
    a.in_positions = in_positions; a.off = off; a.vals = vals;
    a.survivors = survivors; a.survivor_count = survivor_count; a.scratch = pd.scratch;
    a.neurons = neurons; a.k = k; a.live_in = live_in;
    a.classes_per_item = neurons < 256 ? neurons : 256;
    a.w = w; a.bias = bias; a.clip = clip;
    const bool uniform = (vals == nullptr);
    const int variant = (k == 32 ? 0 : 2) + (uniform ? 0 : 1);
    const int grid = pd.sm_count * (pd.blocks_per_sm[variant] > 0 ? pd.blocks_per_sm[variant] : 1);
    if (k == 32) {
        if (uniform) layer_static_kernel<32, true><<<grid, kThreads, 0, stream>>>(a);
        else layer_static_kernel<32, false><<<grid, kThreads, 0, stream>>>(a);
    } else {
        if (uniform) layer_static_kernel<0, true><<<grid, kThreads, 0, stream>>>(a);
        else layer_static_kernel<0, false><<<grid, kThreads, 0, stream>>>(a);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return say(err, err_len, SPDNN_ERR_CUDA, cudaGetErrorString(e));
    return SPDNN_OK;
}
