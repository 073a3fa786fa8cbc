// sm_100a kernels of the sparse-DNN inference path.
//
// Activation layout ("tiles"): images are grouped 32 to a tile; a tile stores row r
// (neuron r) of its 32 images contiguously: Y[tile][r][lane], lane = image within the tile,
// r = 0..N, where row N is a permanent all-zero row that padded column entries point at.
// One warp lane owns one image, so every gather of a weight row is one coalesced 128-byte
// request and the per-image "any non-zero" test is a warp ballot.
//
// One launch per layer does what the reference spreads over a kernel, a D2H copy, a host
// scan and an H2D copy (src/microbenchmark/all_network.cu:344-510): SpMM + bias + ReLU +
// clip (its kernels :15-153 with __ReLU :8-10), the active[] flags (:57-59) as ballots, and
// the rebuild of the work list (:455-463) by the last block to finish (prefix sum over
// the per-tile ballots).  Dead images are dropped on read by the next layer: lane j of tile
// t reads the image in slot[32 t + j] and writes position 32 t + j, so outputs are always
// dense and no separate compaction pass over the activations exists.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace spdnn_impl {

constexpr int kThreads = 256;          // 8 warps per block
constexpr int kWarps = kThreads / 32;
// Blocks per SM the register allocator plans for: 3 leaves room (<= 85 registers) to issue
// all 32 gathers of a class before the first add, which is what hides the memory latency.
#ifndef SPDNN_MIN_BLOCKS
#define SPDNN_MIN_BLOCKS 3
#endif

// Per-layer weights as the kernel reads them (passed by value).
struct LayerDesc {
    const int32_t *off;       // [U][K] element offset (row*32) of each class's inputs, ascending input order
    const float *vals;        // [U][K] weights, or nullptr: every weight is w
    const int32_t *mem_ptr;   // [U+1] member ranges, or nullptr: class u is column u
    const int32_t *mem;       // member column offsets (column*32)
    int classes;              // U
    int k;                    // entries per class, multiple of 4
    float w;                  // the uniform weight (power of two)
    int classes_per_item;     // classes one block handles for one tile
};

// Loop state kept on the device, one record per layer boundary (record l = state entering
// layer l; record L = final result).
struct LoopCtl {
    int32_t live;        // images alive
    int32_t identity;    // 1: image j sits in slot j of the input buffer (no indirection)
    int32_t ids_buf;     // which of the two id arrays holds the ids in current order
    int32_t reserved;
};

struct LayerArgs {
    const float *yin;
    float *yout;
    long long tile_stride;     // elements per tile = (N+1)*32
    const LoopCtl *ctl_in;
    LoopCtl *ctl_out;
    int32_t *slot;             // work list: slot[j] = position in yin of live image j
    uint32_t *mask;            // per output tile: ballot of alive lanes (zero on entry, zero on exit)
    int32_t *ids0, *ids1;      // global image numbers, double buffered
    unsigned int *counter;     // blocks finished (zero on entry, zero on exit)
    unsigned int *work;        // next work item to hand out (zero on entry, zero on exit)
    int32_t *status;           // set non-zero when the kernel finds an inconsistency
    int32_t *died_at;          // where the per-layer kernel records how many images died in its layer (or nullptr)
    int first_member_only;     // 1: the next launch reads one row per class (its first member): store only that row
    float bias, clip;
    // BITS variant (first layer of a pass on a binary input): the input is one word per (tile, neuron),
    // nw words per tile, bit i = image i of the tile is 1.0 (spdnn_front.cuh)
    const uint32_t *xw;
    int nw;
    // the launch runs only when *gate == gate_want (nullptr: always): the first layer exists in a variant
    // for binary inputs and one for any input, and the flag raised while the input was converted picks one
    const int32_t *gate;
    int gate_want;
};

// L2 residency hints of the per-layer kernel (SPDNN_L2_HINT: 0 none, 1 input rows are read
// with an evict-first policy, 2 output rows are also written with evict-last).  The input of
// a layer is dead once read and its output is the next layer's input, so when both together
// exceed the L2 but the output alone fits, keeping the output and letting go of the input
// turns the next layer's DRAM reads into L2 hits.
#ifndef SPDNN_L2_HINT
#define SPDNN_L2_HINT 0
#endif
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ unsigned long long l2_policy_evict_last() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ float load_row(const float *p, unsigned long long pol) {
#if SPDNN_L2_HINT >= 1
    float v;
    asm volatile("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
    return v;
#else
    (void)pol;
    return __ldg(p);
#endif
}
__device__ __forceinline__ void store_row(float *p, float v, unsigned long long pol) {
#if SPDNN_L2_HINT >= 2
    asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(p), "f"(v), "l"(pol) : "memory");
#else
    (void)pol;
    *p = v;
#endif
}

__device__ __forceinline__ float relu_clip(float x, float clip) {
    // x<0 ? 0 : x>clip ? clip : x   (all_network.cu:8-10)
    return x < 0.0f ? 0.0f : (x > clip ? clip : x);
}

// Sum of one class for this lane's image: the K inputs in ascending input order, one fp32
// add after the other, starting from 0 -- the order of src/utils/cpu_spmm.h:14-43.
// One gathered input of this lane's image: element `o` (row * 32) of the tile at yin -- or, BITS, bit
// `lane` of word `o >> 5` of the tile's words (yin then points at those words).
template <bool BITS>
__device__ __forceinline__ float in_value(const float *__restrict__ yin, int o, unsigned long long pol, int lane) {
    if (BITS) return ((__ldg(reinterpret_cast<const uint32_t *>(yin) + (o >> 5)) >> lane) & 1u) ? 1.0f : 0.0f;
    return load_row(yin + o, pol);
}

template <int KT, bool UNIFORM, bool BITS = false>
__device__ __forceinline__ float class_sum(const LayerDesc &d, int u, const float *__restrict__ yin, unsigned long long pol = 0, int lane = 0) {
    float acc = 0.0f;
    if (KT > 0) {
        constexpr int KA = KT > 0 ? KT : 4;      // array extent (the branch is dead for KT == 0)
        const int4 *o4 = reinterpret_cast<const int4 *>(d.off + (size_t)u * KT);
        int o[KA];
#pragma unroll
        for (int i = 0; i < KT / 4; ++i) {
            const int4 t = __ldg(o4 + i);
            o[4 * i + 0] = t.x; o[4 * i + 1] = t.y; o[4 * i + 2] = t.z; o[4 * i + 3] = t.w;
        }
        float v[KA];
#pragma unroll
        for (int i = 0; i < KT; ++i) v[i] = in_value<BITS>(yin, o[i], pol, lane);
        if (UNIFORM) {
#pragma unroll
            for (int i = 0; i < KT; ++i) acc = __fadd_rn(acc, v[i]);
        } else {
            const float4 *w4 = reinterpret_cast<const float4 *>(d.vals + (size_t)u * KT);
#pragma unroll
            for (int i = 0; i < KT / 4; ++i) {
                const float4 t = __ldg(w4 + i);
                acc = __fadd_rn(acc, __fmul_rn(v[4 * i + 0], t.x));
                acc = __fadd_rn(acc, __fmul_rn(v[4 * i + 1], t.y));
                acc = __fadd_rn(acc, __fmul_rn(v[4 * i + 2], t.z));
                acc = __fadd_rn(acc, __fmul_rn(v[4 * i + 3], t.w));
            }
        }
    } else {
        const int k = d.k;
        const int4 *o4 = reinterpret_cast<const int4 *>(d.off + (size_t)u * k);
        const float4 *w4 = UNIFORM ? nullptr : reinterpret_cast<const float4 *>(d.vals + (size_t)u * k);
        for (int i = 0; i < k / 4; ++i) {
            const int4 t = __ldg(o4 + i);
            const float a = in_value<BITS>(yin, t.x, pol, lane), b = in_value<BITS>(yin, t.y, pol, lane), c = in_value<BITS>(yin, t.z, pol, lane),
                        e = in_value<BITS>(yin, t.w, pol, lane);
            if (UNIFORM) {
                acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, a), b), c), e);
            } else {
                const float4 q = __ldg(w4 + i);
                acc = __fadd_rn(acc, __fmul_rn(a, q.x));
                acc = __fadd_rn(acc, __fmul_rn(b, q.y));
                acc = __fadd_rn(acc, __fmul_rn(c, q.z));
                acc = __fadd_rn(acc, __fmul_rn(e, q.w));
            }
        }
    }
    // uniform power-of-two weight: w * sum(y) == sum(w * y) bit for bit
    return UNIFORM ? __fmul_rn(acc, d.w) : acc;
}

// The last block to finish turns the per-tile ballots into the next launch's work list: every
// warp takes a contiguous run of tiles, counts its survivors (lanes split the run, warp scan),
// a block scan over the warps gives each run its first position, and the warp then walks its
// tiles 32 at a time with lane b handling bit b, so that the writes of the work list are
// coalesced.  The global image numbers follow later and in parallel: when the order changed
// (ids_buf flips) the blocks of the NEXT launch copy ids[ids_buf ^ 1][slot[j]] to ids[ids_buf][j]
// for the images they own (move_id), and finalize_ids_kernel does it after the last launch.
__device__ __forceinline__ void rebuild_worklist(const LayerArgs &a, int live_in, int ids_buf) {
    __shared__ int s_warp[32];          // works for any block size up to 1024 threads
    __shared__ int s_total;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ntiles = (live_in + 31) >> 5;
    const int nwarps = blockDim.x >> 5;
    const int per_warp = (ntiles + nwarps - 1) / nwarps;
    const int w0 = min(warp * per_warp, ntiles), w1 = min(w0 + per_warp, ntiles);
    int cnt = 0;
    for (int t = w0 + lane; t < w1; t += 32) cnt += __popc(__ldcg(a.mask + t));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);      // survivors of the warp's run
    if (lane == 0) s_warp[warp] = cnt;
    __syncthreads();
    if (warp == 0) {
        int w = lane < nwarps ? s_warp[lane] : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, w, d);
            if (lane >= d) w += o;
        }
        if (lane < nwarps) s_warp[lane] = w;          // inclusive over warps
        if (lane == nwarps - 1) s_total = w;
    }
    __syncthreads();
    const int total = s_total;
    if (total > live_in && tid == 0) atomicExch(a.status, 2);
    const bool same = (total == live_in);      // nobody died: positions are already dense
    if (!same) {
        int run = warp ? s_warp[warp - 1] : 0;         // first position of this warp's run
        const uint32_t below = (1u << lane) - 1u;
        int32_t *__restrict__ slot = a.slot;
        for (int tb = w0; tb < w1; tb += 32) {
            const uint32_t mine = (tb + lane < w1) ? __ldcg(a.mask + tb + lane) : 0u;    // 32 ballots per load
            const int n = min(32, w1 - tb);
            for (int i = 0; i < n; ++i) {
                const uint32_t m = __shfl_sync(0xffffffffu, mine, i);
                if ((m >> lane) & 1u) slot[run + __popc(m & below)] = (tb + i) * 32 + lane;
                run += __popc(m);
            }
        }
    }
    for (int t = w0 + lane; t < w1; t += 32) a.mask[t] = 0u;
    if (tid == 0) {
        LoopCtl c;
        c.live = total;
        c.identity = same ? 1 : 0;
        c.ids_buf = same ? ids_buf : (ids_buf ^ 1);
        c.reserved = 0;
        *a.ctl_out = c;
        *a.counter = 0u;
        *a.work = 0u;
        if (a.died_at) *a.died_at = live_in - total;
    }
}

// The consumer's half of the id bookkeeping: image j of the new order came from position src.
__device__ __forceinline__ void move_id(const LoopCtl &ctl, int32_t *ids0, int32_t *ids1, int j, int src) {
    int32_t *to = ctl.ids_buf ? ids1 : ids0;
    const int32_t *from = ctl.ids_buf ? ids0 : ids1;
    to[j] = __ldg(from + src);
}

// One layer.  Grid: persistent blocks that draw work items (tile, block of classes) from an
// atomic counter, tile-major, so that blocks running at the same time work on neighbouring
// tiles and an uneven last wave costs one item, not one block's whole share.  Inside an item
// every warp takes a contiguous run of classes: the host orders classes so that neighbours
// share input rows, and the second read of a row then hits in L1.
template <int KT, bool UNIFORM, bool BITS = false>
__global__ void __launch_bounds__(kThreads, SPDNN_MIN_BLOCKS) layer_kernel(const LayerDesc d, const LayerArgs a) {
    __shared__ unsigned int s_mask;
    __shared__ unsigned int s_item;
    __shared__ int s_last;
    if (a.gate != nullptr && *a.gate != a.gate_want) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const LoopCtl ctl = *a.ctl_in;
    const int live_in = ctl.live;
    const int ntiles = (live_in + 31) >> 5;
    const int cpi = d.classes_per_item;
    const int ncb = (d.classes + cpi - 1) / cpi;
    const unsigned int items = (unsigned int)ntiles * (unsigned int)ncb;
    const int per_warp = (cpi + kWarps - 1) / kWarps;
    const unsigned long long pol_in = SPDNN_L2_HINT >= 1 ? l2_policy_evict_first() : 0ull;
    const unsigned long long pol_out = SPDNN_L2_HINT >= 2 ? l2_policy_evict_last() : 0ull;

    for (;;) {
        if (tid == 0) {
            s_item = atomicAdd(a.work, 1u);
            s_mask = 0u;
        }
        __syncthreads();
        const unsigned int item = s_item;
        if (item >= items) break;
        const int tile = (int)(item / (unsigned int)ncb);
        const int cb = (int)(item - (unsigned int)tile * (unsigned int)ncb);
        const int j = tile * 32 + lane;
        const bool valid = j < live_in;
        const int jj = valid ? j : tile * 32;               // padding lanes shadow lane 0 and are masked out
        const int src = ctl.identity ? jj : __ldg(a.slot + jj);
        if (!ctl.identity && cb == 0 && warp == 0 && valid) move_id(ctl, a.ids0, a.ids1, j, src);
        const float *__restrict__ yin = BITS ? reinterpret_cast<const float *>(a.xw + (size_t)(src >> 5) * a.nw)
                                             : a.yin + (size_t)(src >> 5) * a.tile_stride + (src & 31);
        float *__restrict__ yout = a.yout + (size_t)tile * a.tile_stride + lane;
        bool any = false;
        const int u_end = min(d.classes, (cb + 1) * cpi);
        const int u0 = cb * cpi + warp * per_warp;
        const int u1 = min(u0 + per_warp, u_end);
        for (int u = u0; u < u1; ++u) {
            // member list of the class, fetched before the gathers so that it is there when
            // the sum is: lane m holds member m
            int mb = u, me = u + 1, mreg = u * 32;
            if (d.mem_ptr != nullptr) {
                mb = __ldg(d.mem_ptr + u);
                me = __ldg(d.mem_ptr + u + 1);
                mreg = (mb + lane < me) ? __ldg(d.mem + mb + lane) : 0;
            }
            const float s = class_sum<KT, UNIFORM, BITS>(d, u, yin, pol_in, src & 31);
            const float y = relu_clip(__fadd_rn(s, a.bias), a.clip);
            any |= (y != 0.0f);
            const int cnt = a.first_member_only ? 1 : me - mb;
            if (cnt <= 32) {
                for (int m = 0; m < cnt; ++m) store_row(yout + __shfl_sync(0xffffffffu, mreg, m), y, pol_out);
            } else {
                for (int m = mb; m < me; ++m) store_row(yout + __ldg(d.mem + m), y, pol_out);
            }
        }
        const unsigned int m = __ballot_sync(0xffffffffu, any && valid);
        if (lane == 0 && m) atomicOr(&s_mask, m);
        __syncthreads();
        if (tid == 0 && s_mask) atomicOr(a.mask + tile, s_mask);
    }

    // last block done: rebuild the work list (wait-free: nobody spins)
    if (tid == 0) {
        __threadfence();
        const unsigned int t = atomicAdd(a.counter, 1u);
        s_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    rebuild_worklist(a, live_in, ctl.ids_buf);
}

// ---- layout conversion and bookkeeping kernels -------------------------------------------

// Row-major [batch][N] -> tiles.  Block (32, 8); a work item is 32 images x kLayoutCols neurons, 512 contiguous
// bytes of every image's row, so that the reads stay within few DRAM pages; all of a thread's 16 loads are in
// flight before the first store.  Blocks walk the items (tile-major) with a grid stride, so a launch that its
// gate switches off costs a few thousand blocks' worth of nothing, not one block per item.
// With a gate the kernel runs only once *gate is non-zero (the input is known not to be binary, see
// spdnn_front.cuh) and marks the tiles it wrote in has_floats.
constexpr int kLayoutCols = 128;
static __global__ void dense_to_tiles_kernel(const float *__restrict__ in, float *__restrict__ out, int n, int batch,
                                      long long tile_stride, int first_tile, const int32_t *gate, unsigned char *has_floats) {
    __shared__ float t[32][kLayoutCols + 1];
    if (gate != nullptr && *gate == 0) return;
    const int ncb = (n + kLayoutCols - 1) / kLayoutCols;
    const long long items = (long long)((batch + 31) / 32) * ncb;
    for (long long item = blockIdx.x; item < items; item += gridDim.x) {
        const int tile = (int)(item / ncb), c0 = (int)(item - (long long)tile * ncb) * kLayoutCols;
        if (gate != nullptr && c0 == 0 && threadIdx.x == 0 && threadIdx.y == 0) has_floats[first_tile + tile] = 1;
        const int img0 = tile * 32;
        float v[4][kLayoutCols / 32];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int img = img0 + threadIdx.y + 8 * q;
#pragma unroll
            for (int k = 0; k < kLayoutCols / 32; ++k) {
                const int c = c0 + 32 * k + threadIdx.x;
                v[q][k] = (img < batch && c < n) ? __ldg(in + (size_t)img * n + c) : 0.0f;
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int k = 0; k < kLayoutCols / 32; ++k) t[threadIdx.y + 8 * q][32 * k + threadIdx.x] = v[q][k];
        __syncthreads();
        float *o = out + (size_t)(first_tile + tile) * tile_stride;
#pragma unroll
        for (int r = threadIdx.y; r < kLayoutCols; r += 8) {
            const int c = c0 + r;
            if (c < n) o[(size_t)c * 32 + threadIdx.x] = t[threadIdx.x][r];
        }
        __syncthreads();
    }
}

// COO triplets -> tiles (the tiles must have been zeroed).  Out-of-range triplets raise status.
static __global__ void coo_to_tiles_kernel(const int32_t *__restrict__ img, const int32_t *__restrict__ neuron,
                                    const float *__restrict__ val, long long nnz, int index_base, int n, int batch,
                                    float *__restrict__ out, long long tile_stride, int32_t *status) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nnz; i += (long long)gridDim.x * blockDim.x) {
        const int b = img[i] - index_base, c = neuron[i] - index_base;
        if (b < 0 || b >= batch || c < 0 || c >= n) { atomicExch(status, 3); continue; }
        out[(size_t)(b >> 5) * tile_stride + (size_t)c * 32 + (b & 31)] = val ? val[i] : 1.0f;
    }
}

// Tiles -> row-major [rows][N] for the live images j_base, j_base+1, ... in work-list order
// (row 0 of `out` is image j_base).  Block (32, 8), grid (ceil(rows/32), ceil(N/32)).
static __global__ void tiles_to_dense_kernel(const float *__restrict__ y, long long tile_stride, const LoopCtl *ctl,
                                      const int32_t *__restrict__ slot, int n, float *__restrict__ out, int j_base) {
    __shared__ float t[32][33];
    const LoopCtl c = *ctl;
    const int j0 = j_base + blockIdx.x * 32;
    if (j0 >= c.live) return;
    const int c0 = blockIdx.y * 32;
    const int j = j0 + threadIdx.x;
    const int jj = j < c.live ? j : j0;
    const int src = c.identity ? jj : slot[jj];
    const float *base = y + (size_t)(src >> 5) * tile_stride + (src & 31);
#pragma unroll
    for (int r = threadIdx.y; r < 32; r += 8) {
        const int col = c0 + r;
        t[r][threadIdx.x] = col < n ? base[(size_t)col * 32] : 0.0f;    // t[col][image]
    }
    __syncthreads();
#pragma unroll
    for (int r = threadIdx.y; r < 32; r += 8) {
        const int img = j0 + r, col = c0 + threadIdx.x;
        if (img < c.live && col < n) out[(size_t)(img - j_base) * n + col] = t[threadIdx.x][r];
    }
}

// After the last launch: the ids of the final order, if that launch changed the order.
// After a pass whose last launch stored one row per class (its first member): copy that row to the
// other member rows of every tile the launch wrote, so that the tiles hold all N activations.
// One warp per (tile, class), lane = image; mem[] holds member column * 32.
static __global__ void expand_members_kernel(float *__restrict__ y, long long tile_stride, int tiles, const int32_t *__restrict__ mem_ptr,
                                             const int32_t *__restrict__ mem, int classes) {
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < (long long)tiles * classes; w += warps) {
        const int tile = (int)(w / classes), u = (int)(w - (long long)tile * classes);
        float *t = y + (size_t)tile * tile_stride + lane;
        const int mb = __ldg(mem_ptr + u), me = __ldg(mem_ptr + u + 1);
        const float v = t[__ldg(mem + mb)];
        for (int m = mb + 1; m < me; ++m) t[__ldg(mem + m)] = v;
    }
}

static __global__ void finalize_ids_kernel(const LoopCtl *ctl, const int32_t *__restrict__ slot, int32_t *ids0, int32_t *ids1) {
    const LoopCtl c = *ctl;
    if (c.identity) return;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < c.live; j += gridDim.x * blockDim.x)
        move_id(c, ids0, ids1, j, __ldg(slot + j));
}

// dense_cell: where the first launch of a pass finds the caller's row-major input when that launch
// reads it in place (dense_src, may be null: the input was converted to tiles).
static __global__ void init_loop_kernel(LoopCtl *ctl, int32_t *ids0, int batch, int first_global_id, int32_t *died_at,
                                        int layers, const float **dense_cell, const float *dense_src) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < batch; i += gridDim.x * blockDim.x)
        ids0[i] = first_global_id + i;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < layers; i += gridDim.x * blockDim.x) died_at[i] = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        LoopCtl c;
        c.live = batch; c.identity = 1; c.ids_buf = 0; c.reserved = 0;
        *ctl = c;
        *dense_cell = dense_src;
    }
}

}  // namespace spdnn_impl
