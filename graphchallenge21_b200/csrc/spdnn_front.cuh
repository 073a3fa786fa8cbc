// Binary inputs as a bit matrix.
//
// The challenge's input images are binary: every entry of the reference's input file carries the
// value 1 (src/network.cpp:49-51 logs any other value as an anomaly).  Such an input is kept on the
// device as one 32-bit word per (tile of 32 images, neuron): bit i of xw[tile][r] = image 32 tile + i
// has neuron r set.  That is N/8 bytes per image instead of 4 N, and layer 0 reads it directly:
//   * the per-layer kernel takes a gathered input as ((word >> lane) & 1) ? 1.0f : 0.0f, one
//     broadcast 4-byte load per gather instead of a 128-byte row;
//   * with a uniform weight w and 32 entries per class, front_count_kernel computes layer 0 for 32 images
//     at once: the K-term sum of zeros and ones in ascending order is the COUNT of ones, every partial
//     sum an integer and therefore exact in fp32, so the output is count * w + bias, clamped, computed
//     with the float path's own instructions from a bit-sliced count.
// Inputs that turn out not to be binary (a value other than 0 and 1) raise a flag on the device while
// they are converted; the launches of the first layer exist in both variants and each checks the
// flag at entry (`gate`), so no host round-trip decides.  For those inputs the float tiles are built
// as before.
#pragma once

#include "spdnn_kernels.cuh"

namespace spdnn_impl {

// words per tile: the neurons, then at least four words that stay zero (padded table entries point there)
__host__ __device__ __forceinline__ int front_words_per_tile(int n) { return (n + 4 + 31) / 32 * 32; }

// 32 x 32 bit transpose across a warp: on return bit i of lane r's word = bit r of lane i's word on entry.
__device__ __forceinline__ unsigned int warp_bit_transpose(unsigned int x, int lane) {
#pragma unroll
    for (int j = 16; j >= 1; j >>= 1) {
        // bits whose index has bit j clear
        const unsigned int m = j == 16 ? 0x0000ffffu : j == 8 ? 0x00ff00ffu : j == 4 ? 0x0f0f0f0fu : j == 2 ? 0x33333333u : 0x55555555u;
        const unsigned int t = __shfl_xor_sync(0xffffffffu, x, j);
        x = (lane & j) ? ((x & ~m) | ((t >> j) & m)) : ((x & m) | ((t & m) << j));
    }
    return x;
}

// Packed rows (image i = row_words words, bit (n & 31) of word n >> 5 = neuron n) -> words per (tile, neuron).
// One warp per (tile, 32 neurons).
static __global__ void rows_to_words_kernel(const uint32_t *__restrict__ in, long long row_words, int n, int batch,
                                            uint32_t *__restrict__ xw, int nw, int first_tile) {
    const int lane = threadIdx.x & 31;
    const int chunks = (n + 31) / 32;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    const long long total = (long long)((batch + 31) / 32) * chunks;
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total; w += warps) {
        const int tile = (int)(w / chunks), c = (int)(w - (long long)tile * chunks);
        const int img = tile * 32 + lane;
        unsigned int x = img < batch ? __ldg(in + (size_t)img * row_words + c) : 0u;
        if (c == chunks - 1 && (n & 31)) x &= (1u << (n & 31)) - 1u;        // bits past the last neuron do not count
        x = warp_bit_transpose(x, lane);
        if (c * 32 + lane < n) xw[(size_t)(first_tile + tile) * nw + c * 32 + lane] = x;
    }
}

// Row-major floats [batch][n] -> words, raising *nonbinary when a value is neither 0 nor 1.
// Block (32, 8): a warp takes 32 images x 128 neurons (512 contiguous bytes of every image's row), a lane
// four neighbouring neurons of all 32 images; grid (tiles, ceil(n / 1024)).
static __global__ void dense_to_words_kernel(const float *__restrict__ in, int n, int batch, uint32_t *__restrict__ xw, int nw,
                                             int first_tile, int32_t *nonbinary) {
    const int lane = threadIdx.x, tile = blockIdx.x;
    const int c0 = (blockIdx.y * 8 + threadIdx.y) * 128 + lane * 4;
    if (c0 >= n) return;
    const bool vec = (n & 3) == 0 && (reinterpret_cast<size_t>(in) & 15) == 0;
    unsigned int w0 = 0, w1 = 0, w2 = 0, w3 = 0;
    bool odd = false;
    for (int i0 = 0; i0 < 32; i0 += 8) {
        float4 v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int img = tile * 32 + i0 + q;
            v[q] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (img < batch) {
                const float *p = in + (size_t)img * n + c0;
                if (vec) v[q] = __ldg(reinterpret_cast<const float4 *>(p));
                else {
                    v[q].x = __ldg(p);
                    if (c0 + 1 < n) v[q].y = __ldg(p + 1);
                    if (c0 + 2 < n) v[q].z = __ldg(p + 2);
                    if (c0 + 3 < n) v[q].w = __ldg(p + 3);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int i = i0 + q;
            w0 |= (v[q].x != 0.0f ? 1u : 0u) << i; w1 |= (v[q].y != 0.0f ? 1u : 0u) << i;
            w2 |= (v[q].z != 0.0f ? 1u : 0u) << i; w3 |= (v[q].w != 0.0f ? 1u : 0u) << i;
            odd |= (v[q].x != 0.0f && v[q].x != 1.0f) || (v[q].y != 0.0f && v[q].y != 1.0f) || (v[q].z != 0.0f && v[q].z != 1.0f) ||
                   (v[q].w != 0.0f && v[q].w != 1.0f);
        }
    }
    uint32_t *o = xw + (size_t)(first_tile + tile) * nw + c0;
    if (c0 + 3 < n) *reinterpret_cast<uint4 *>(o) = make_uint4(w0, w1, w2, w3);       // nw and c0 are multiples of 4
    else {
        o[0] = w0;
        if (c0 + 1 < n) o[1] = w1;
        if (c0 + 2 < n) o[2] = w2;
    }
    if (odd) atomicExch(nonbinary, 1);
}

// Triplets -> words (the words must have been zeroed).  A value other than 1 raises *nonbinary, an
// out-of-range triplet raises status 3.
static __global__ void coo_to_words_kernel(const int32_t *__restrict__ img, const int32_t *__restrict__ neuron,
                                           const float *__restrict__ val, long long nnz, int index_base, int n, int batch,
                                           uint32_t *__restrict__ xw, int nw, int32_t *nonbinary, int32_t *status) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nnz; i += (long long)gridDim.x * blockDim.x) {
        const int b = img[i] - index_base, c = neuron[i] - index_base;
        if (b < 0 || b >= batch || c < 0 || c >= n) { atomicExch(status, 3); continue; }
        const float v = val ? val[i] : 1.0f;
        if (v != 1.0f) atomicExch(nonbinary, 1);
        if (v != 0.0f) atomicOr(xw + (size_t)(b >> 5) * nw + c, 1u << (b & 31));
    }
}

// Words -> float tiles (1.0 / 0.0) for every tile whose floats were not written (has_floats[tile] == 0).
// Runs when *gate == gate_want.  One warp per (tile, neuron); lane = image.
static __global__ void words_to_tiles_kernel(const uint32_t *__restrict__ xw, int nw, int n, int tiles, float *__restrict__ y,
                                             long long tile_stride, const unsigned char *has_floats, const int32_t *gate, int gate_want) {
    if (*gate != gate_want) return;
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < (long long)tiles * n; w += warps) {
        const int tile = (int)(w / n), r = (int)(w - (long long)tile * n);
        if (has_floats && has_floats[tile]) continue;
        const unsigned int x = __ldg(xw + (size_t)tile * nw + r);
        y[(size_t)tile * tile_stride + (size_t)r * 32 + lane] = ((x >> lane) & 1u) ? 1.0f : 0.0f;
    }
}

// Marks the tiles [first_tile, first_tile + tiles) as holding floats; runs when *gate == gate_want.
static __global__ void mark_tiles_kernel(unsigned char *has_floats, int first_tile, int tiles, const int32_t *gate, int gate_want) {
    if (*gate != gate_want) return;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < tiles; t += gridDim.x * blockDim.x) has_floats[first_tile + t] = 1;
}

// ---- layer 0 of a binary input, 32 images at a time -----------------------------------------------------
//
// For a layer with a uniform weight and 32 entries per class the sum of a class over a binary input is
// count * w with count = the number of its inputs that are set, every partial sum an integer and so exact in
// fp32 whatever the order.  A lane owns a CLASS: it gathers the class's 32 row words of the tile (bit i =
// image i) and adds them with a tree of 31 carry-save adders into a six-plane bit-sliced count of all 32
// images at once -- about a third of the instructions of the per-image gather-and-add.  The planes are then
// handed round the warp, class by class, and lane i turns image i's count into the float output with the
// per-layer kernel's own instructions (multiply by w, add the bias, clamp) and stores a coalesced row.
// Same launch protocol as layer_kernel: work items from an atomic counter, ballots, last-block rebuild.
__device__ __forceinline__ void front_csa(unsigned int &h, unsigned int &l, unsigned int a, unsigned int b, unsigned int c) {
    const unsigned int u = a ^ b;
    h = (a & b) | (u & c);
    l = u ^ c;
}

constexpr int kFrontClassesPerItem = 256;

static __global__ void __launch_bounds__(kThreads, 4) front_count_kernel(const LayerDesc d, const LayerArgs a) {
    __shared__ unsigned int s_mask;
    __shared__ unsigned int s_item;
    __shared__ int s_last;
    if (a.gate != nullptr && *a.gate != a.gate_want) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const LoopCtl ctl = *a.ctl_in;                 // first launch of a pass: image j sits at position j
    const int live_in = ctl.live;
    const int ntiles = (live_in + 31) >> 5;
    const int ncb = (d.classes + kFrontClassesPerItem - 1) / kFrontClassesPerItem;
    const unsigned int items = (unsigned int)ntiles * (unsigned int)ncb;
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
        const uint32_t *__restrict__ xw = a.xw + (size_t)tile * a.nw;
        float *__restrict__ yout = a.yout + (size_t)tile * a.tile_stride + lane;
        const bool valid = tile * 32 + lane < live_in;
        bool any = false;
        const int u_end = min(d.classes, (cb + 1) * kFrontClassesPerItem);
        for (int u0 = cb * kFrontClassesPerItem + warp * 32; u0 < u_end; u0 += kWarps * 32) {
            const int u = u0 + lane;
            const bool in = u < u_end;
            const int4 *o4 = reinterpret_cast<const int4 *>(d.off + (size_t)(in ? u : u0) * 32);
            unsigned int pl[6] = {0u, 0u, 0u, 0u, 0u, 0u};       // ones, twos, fours, eights, sixteens, thirty-twos
            unsigned int s16[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                unsigned int e8[2];
#pragma unroll
                for (int quarter = 0; quarter < 2; ++quarter) {
                    const int4 r0 = __ldg(o4 + half * 4 + quarter * 2), r1 = __ldg(o4 + half * 4 + quarter * 2 + 1);
                    const unsigned int w0 = __ldg(xw + (r0.x >> 5)), w1 = __ldg(xw + (r0.y >> 5)), w2 = __ldg(xw + (r0.z >> 5)),
                                       w3 = __ldg(xw + (r0.w >> 5)), w4 = __ldg(xw + (r1.x >> 5)), w5 = __ldg(xw + (r1.y >> 5)),
                                       w6 = __ldg(xw + (r1.z >> 5)), w7 = __ldg(xw + (r1.w >> 5));
                    unsigned int t2a, t2b, f4a, f4b;
                    front_csa(t2a, pl[0], pl[0], w0, w1);
                    front_csa(t2b, pl[0], pl[0], w2, w3);
                    front_csa(f4a, pl[1], pl[1], t2a, t2b);
                    front_csa(t2a, pl[0], pl[0], w4, w5);
                    front_csa(t2b, pl[0], pl[0], w6, w7);
                    front_csa(f4b, pl[1], pl[1], t2a, t2b);
                    front_csa(e8[quarter], pl[2], pl[2], f4a, f4b);
                }
                front_csa(s16[half], pl[3], pl[3], e8[0], e8[1]);
            }
            front_csa(pl[5], pl[4], pl[4], s16[0], s16[1]);
            // where the class's output goes: its first member's row, or all of them
            int mb = u, me = u + 1, mrow = u * 32;
            if (d.mem_ptr != nullptr && in) {
                mb = __ldg(d.mem_ptr + u);
                me = __ldg(d.mem_ptr + u + 1);
                mrow = __ldg(d.mem + mb);
            }
            const int n_here = min(32, u_end - u0);
            for (int cidx = 0; cidx < n_here; ++cidx) {
                unsigned int cnt = (__shfl_sync(0xffffffffu, pl[0], cidx) >> lane) & 1u;
                cnt |= ((__shfl_sync(0xffffffffu, pl[1], cidx) >> lane) & 1u) << 1;
                cnt |= ((__shfl_sync(0xffffffffu, pl[2], cidx) >> lane) & 1u) << 2;
                cnt |= ((__shfl_sync(0xffffffffu, pl[3], cidx) >> lane) & 1u) << 3;
                cnt |= ((__shfl_sync(0xffffffffu, pl[4], cidx) >> lane) & 1u) << 4;
                cnt |= ((__shfl_sync(0xffffffffu, pl[5], cidx) >> lane) & 1u) << 5;
                const float y = relu_clip(__fadd_rn(__fmul_rn((float)cnt, d.w), a.bias), a.clip);
                any |= (y != 0.0f);
                const int row = __shfl_sync(0xffffffffu, mrow, cidx);
                yout[row] = y;
                if (!a.first_member_only && d.mem_ptr != nullptr) {
                    const int b0 = __shfl_sync(0xffffffffu, mb, cidx), b1 = __shfl_sync(0xffffffffu, me, cidx);
                    for (int m = b0 + 1; m < b1; ++m) yout[__ldg(d.mem + m)] = y;
                }
            }
        }
        const unsigned int m = __ballot_sync(0xffffffffu, any && valid);
        if (lane == 0 && m) atomicOr(&s_mask, m);
        __syncthreads();
        if (tid == 0 && s_mask) atomicOr(a.mask + tile, s_mask);
    }
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

}  // namespace spdnn_impl
