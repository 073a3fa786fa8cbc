// Resident kernel: a chunk of consecutive layers in ONE launch, with the activations of a
// group of images held in shared memory from the first to the last layer of the chunk.
//
// Images are independent through the network, so a block that owns TI images can apply layer
// after layer without touching global memory for Y.  This is the idea of the reference's
// two-layer fusion (src/fuse/fuse.h:9-53, src/microbenchmark/fuse.cu:16-110: layer-0 output kept
// in shared memory for layer 1) taken to whole chunks of layers, which B200's 227 KB of shared
// memory per block allow.
//
// Inside a chunk the activations are stored by VALUE ID, not by neuron: all columns of a
// class (identical inputs and weights) hold the same value, so a layer writes one row per
// class and the next layer's tables name those rows directly (layer_inspect.h).  Two buffers
// of rows x TI floats ping-pong; for the challenge networks that is N/16 rows instead of N.
// At the start of a chunk one representative row per value id is read from the N-row tiles in
// global memory, at its end every class is expanded back to all its member rows, so between
// launches the layout is the one of the per-layer kernel.
//
// Thread mapping: a thread owns one class for FOUR images and keeps a float4 of accumulators;
// a gather is one 16-byte shared-memory load, two adds are one packed add.rn.f32x2 (sm_100
// packed fp32).  Each element is added in ascending-input order, so results are bit-identical
// to the per-layer kernel and to the CPU loop of src/utils/cpu_spmm.h:14-43.  Two table forms:
//   GENERIC  K row numbers per class, gathered one by one: resident_kernel, in this file;
//   ALT2     the K terms alternate between two rows a,b,a,b,... (what a 16-wide butterfly block
//            looks like in value ids): two loads, then K adds in that order: alt2_kernel
//            (spdnn_alt2.cuh), which shares the helpers defined here.
// The per-layer tables come into shared memory by bulk asynchronous copy (TMA, cp.async.bulk
// completing on an mbarrier), the table of layer l+1 while layer l is computed.
//
// Rows of the shared-memory buffers are permuted (row r sits at r ^ parity(r >> 1)) so that
// classes whose rows share one parity do not pile onto the same half of the banks; the
// permutation is folded into the tables on the host.
//
// Survivors: an image dies in the layer after which all its activations are zero
// (all_network.cu:57-59, 455-463) and stays dead; inside a chunk its activations are forced to
// zero from then on, the layer of death is counted in died_at[], and at the end of the chunk the
// per-tile ballots and the last-block work-list rebuild are those of the per-layer kernel.
#pragma once

#include "spdnn_kernels.cuh"

namespace spdnn_impl {

constexpr int kResGeneric = 0, kResAlt2 = 1;

// Per-layer tables of the resident kernel (one entry per layer, in device memory).
struct ResLayer {
    const int32_t *blob;      // header {classes, k, bits of w, 0}, then
                              // GENERIC: int32 t[U][k+4] (k input rows, then the output row) [+ float vals[U][k+4]]
                              // ALT2:    int32 t[U][4] = {row a, row b, output row, 0}
    const int32_t *rep;       // [v_in] neuron*32 carrying value id v, or nullptr (value id == neuron)
    const int32_t *mem_ptr;   // [U+1] member ranges, or nullptr (class u == column u)
    const int32_t *mem;       // member column*32
    int blob_bytes;           // multiple of 16
    int o_vals;               // word offset of the weights inside the blob (0: uniform weight)
    int classes, k;
    int v_in;                 // rows of the input buffer
    float w;
};

struct ResArgs {
    const float *yin;
    float *yout;
    long long tile_stride;
    const LoopCtl *ctl_in;
    LoopCtl *ctl_out;
    int32_t *slot;
    uint32_t *mask;
    int32_t *ids0, *ids1;
    unsigned int *counter, *work;
    int32_t *status;
    const ResLayer *layers;   // first layer of this chunk
    int32_t *died_at;         // first layer of this chunk
    int nlayers;
    int buf_rows;             // rows of one activation buffer (largest layer of the chunk, even, + 2)
    int table_bytes;          // shared memory reserved per staged table (0 = read the tables from global memory)
    int n;                    // neurons
    int reps_only;            // 1: the next launch is a resident chunk, which reads one row per class (the first
                              // member): write only that row at the end of this chunk
    int exact_ok;             // the inputs of every layer of the chunk are activations in [0, clip], clip <= 1024
    float bias, clip;
    // ALT2 chunks (alt2_kernel) read their tables from one packed stream per chunk instead of the per-layer blobs
    const unsigned char *stream;   // stream_stride bytes per layer of the chunk (alt2_pack_kernel)
    int stream_stride;
    int tgroup_shift;         // staged: one bulk copy brings 1 << tgroup_shift layers of the stream
    int tring;                // staged: buffers of one such group (2 or 4); 0 = read the stream from global memory
    int wring;                // bit form: buffers of one word per row (>= 2)
    int rows_w;               // bit form: words per buffer (>= buf_rows and >= 32; a row past it belongs to no class)
    int bit_ok;               // bit form allowed (clip > 0, not switched off)
    int bit_multi;            // bit form: some layer of the chunk has more than 64 classes
    // First launch of a pass that reads the caller's row-major input (batch x n floats) in place: the cell
    // that holds its address (init_loop_kernel), else nullptr (the input is in yin, in tiles).  Loading the
    // block's rows into shared memory does the change of layout that dense_to_tiles_kernel would do.
    const float *const *dense_in;
    int sm_count;             // SMs of the device (alt2_kernel spreads the working warps of its blocks by it)
    // ALT2 chunks with a bits_kernel pre-pass (spdnn_bits.cuh): one byte per tile of 32 images of the work list,
    // 1 = the pre-pass finished the tile and alt2_kernel's blocks of that tile skip their work; nullptr = no pre-pass
    unsigned char *tile_done;
    int wwords;               // bits_kernel: words per word buffer (a multiple of 64)
    // bits_kernel, cached records: the distinct records of the chunk's stream (cache_records of stream_stride bytes,
    // held in shared memory for the whole launch) and which of them each layer uses; nullptr = stream per layer
    const unsigned char *cache;
    const unsigned short *rec_of;
    int cache_records;
    // the launch runs only when *gate == gate_want (nullptr: always), see LayerArgs
    const int32_t *gate;
    int gate_want;
};

__host__ __device__ __forceinline__ int resident_phys_row(int r) {
    // flip the low bit by the parity of the upper bits: a bijection on [0, 2m)
#ifdef __CUDA_ARCH__
    return r ^ (__popc((unsigned int)(r >> 1)) & 1);
#else
    int x = r >> 1;
    x ^= x >> 16; x ^= x >> 8; x ^= x >> 4; x ^= x >> 2; x ^= x >> 1;
    return r ^ (x & 1);
#endif
}

// Two fp32 values in one 64-bit register pair, added by ONE instruction (add.rn.f32x2, sm_100):
// each half is an ordinary IEEE round-to-nearest add, so results equal two scalar adds.
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
#ifndef SPDNN_NO_F32X2
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
#else
    float al, ah, bl, bh;
    unpack2(a, al, ah);
    unpack2(b, bl, bh);
    return pack2(__fadd_rn(al, bl), __fadd_rn(ah, bh));
#endif
}

// Four accumulators (one per image of the thread) as two packed pairs.
struct Acc4 {
    f32x2 lo, hi;
};

__device__ __forceinline__ Acc4 acc_zero() { return Acc4{pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)}; }
__device__ __forceinline__ Acc4 acc_from(const float4 v) { return Acc4{pack2(v.x, v.y), pack2(v.z, v.w)}; }
__device__ __forceinline__ void acc_add(Acc4 &acc, const Acc4 &v) {
    acc.lo = add2(acc.lo, v.lo);
    acc.hi = add2(acc.hi, v.hi);
}
__device__ __forceinline__ float4 acc_get(const Acc4 &acc) {
    float4 r;
    unpack2(acc.lo, r.x, r.y);
    unpack2(acc.hi, r.z, r.w);
    return r;
}

__device__ __forceinline__ float4 mul4(const float4 v, float w) {
    return make_float4(__fmul_rn(v.x, w), __fmul_rn(v.y, w), __fmul_rn(v.z, w), __fmul_rn(v.w, w));
}

// ---- bulk asynchronous copy (TMA) of a layer's table blob into shared memory -------------------
__device__ __forceinline__ unsigned int smem_u32(const void *p) { return (unsigned int)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void bulk_load_table(void *dst, const void *src, unsigned int bytes, unsigned long long *bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

#ifndef SPDNN_MBAR_POLL
#define SPDNN_MBAR_POLL "try_wait"      // "test_wait": poll without the hardware's suspend
#endif
// Bounded wait: returns false when the copy has not landed after kMbarSpinLimit polls.
constexpr int kMbarSpinLimit = 1 << 22;
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned int parity) {
    for (int i = 0; i < kMbarSpinLimit; ++i) {
        unsigned int done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier." SPDNN_MBAR_POLL ".parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Sum of one class for this thread's four images, GENERIC tables.  `in` points at the thread's
// 16-byte column of the current buffer, `rows`/`vals` at the class's K entries (in shared
// memory when STAGED, else in global memory); a row number times RS is its byte offset.
template <int KT, bool UNIFORM, bool STAGED, int RS>
__device__ __forceinline__ float4 class_sum_generic(const int32_t *rows, const float *vals, int k, float w,
                                                    const unsigned char *in) {
    Acc4 acc = acc_zero();
    const int4 *o4 = reinterpret_cast<const int4 *>(rows);
    const float4 *w4 = reinterpret_cast<const float4 *>(vals);
    if (KT > 0) {
        constexpr int KA = KT > 0 ? KT : 4;
        int o[KA];
#pragma unroll
        for (int i = 0; i < KT / 4; ++i) {
            const int4 t = STAGED ? o4[i] : __ldg(o4 + i);
            o[4 * i + 0] = t.x * RS; o[4 * i + 1] = t.y * RS; o[4 * i + 2] = t.z * RS; o[4 * i + 3] = t.w * RS;
        }
        if (UNIFORM) {
#pragma unroll
            for (int i = 0; i < KT; ++i) acc_add(acc, acc_from(*reinterpret_cast<const float4 *>(in + o[i])));
        } else {
#pragma unroll
            for (int i = 0; i < KT / 4; ++i) {
                const float4 t = STAGED ? w4[i] : __ldg(w4 + i);
                acc_add(acc, acc_from(mul4(*reinterpret_cast<const float4 *>(in + o[4 * i + 0]), t.x)));
                acc_add(acc, acc_from(mul4(*reinterpret_cast<const float4 *>(in + o[4 * i + 1]), t.y)));
                acc_add(acc, acc_from(mul4(*reinterpret_cast<const float4 *>(in + o[4 * i + 2]), t.z)));
                acc_add(acc, acc_from(mul4(*reinterpret_cast<const float4 *>(in + o[4 * i + 3]), t.w)));
            }
        }
    } else {
        for (int i = 0; i < k / 4; ++i) {
            const int4 t = STAGED ? o4[i] : __ldg(o4 + i);
            float4 a = *reinterpret_cast<const float4 *>(in + t.x * RS), b = *reinterpret_cast<const float4 *>(in + t.y * RS);
            float4 c = *reinterpret_cast<const float4 *>(in + t.z * RS), e = *reinterpret_cast<const float4 *>(in + t.w * RS);
            if (!UNIFORM) {
                const float4 q = STAGED ? w4[i] : __ldg(w4 + i);
                a = mul4(a, q.x); b = mul4(b, q.y); c = mul4(c, q.z); e = mul4(e, q.w);
            }
            acc_add(acc, acc_from(a)); acc_add(acc, acc_from(b)); acc_add(acc, acc_from(c)); acc_add(acc, acc_from(e));
        }
    }
    const float4 r = acc_get(acc);
    return UNIFORM ? mul4(r, w) : r;
}

// ALT2: the K terms are a, b, a, b, ...
//
// Shortcut (exact_ok: K == 32, inputs are activations of an earlier layer, clip <= 1024): when
// all of a and b are multiples of 1/16 -- which (x + M) - M == x tests for M = 1.5 * 2^19,
// whose ulp is 2^-4 -- every partial sum of a+b+a+b+... is a multiple of 1/16 below 2^15 and so
// exactly representable in fp32: each of the 32 adds is exact and the sequential sum EQUALS
// 16 (a + b), which is computed directly; the result bits are the same.  Off unless SPDNN_EXACT_SHORTCUT=1:
// saturated tiles (activations 0 or 32, the steady state of the challenge networks) run in the bit form,
// and on the layers before that state the test of eight inputs costs more than the few classes that pass
// it save (measured on all four challenge sizes).
template <int KT>
__device__ __forceinline__ float4 class_sum_alt2(const float4 a, const float4 b, int k, float w, bool exact_ok, bool *took = nullptr) {
    const Acc4 pa = acc_from(a), pb = acc_from(b);
    if (KT == 32 && exact_ok) {
        const f32x2 M = pack2(786432.0f, 786432.0f), NM = pack2(-786432.0f, -786432.0f);
        const f32x2 d = (add2(add2(pa.lo, M), NM) ^ pa.lo) | (add2(add2(pa.hi, M), NM) ^ pa.hi) |
                        (add2(add2(pb.lo, M), NM) ^ pb.lo) | (add2(add2(pb.hi, M), NM) ^ pb.hi);
        if (d == 0ull) {
            Acc4 s = pa;
            acc_add(s, pb);
            if (took) *took = true;
            return mul4(acc_get(s), 16.0f * w);
        }
    }
    Acc4 acc = acc_zero();
    if (KT > 0) {
#pragma unroll
        for (int i = 0; i < KT / 2; ++i) { acc_add(acc, pa); acc_add(acc, pb); }
    } else {
        for (int i = 0; i < k / 2; ++i) { acc_add(acc, pa); acc_add(acc, pb); }
    }
    return mul4(acc_get(acc), w);
}

// x<0 ? 0 : x>clip ? clip : x of the biased sum (all_network.cu:8-10); for the finite x that occur
// this is min(max(x, 0), clip), two instructions instead of two compares and two selects.
__device__ __forceinline__ float finish_output(float sum, float bias, float clip) {
    return fminf(fmaxf(__fadd_rn(sum, bias), 0.0f), clip);
}

// Load phase of a first launch that reads the caller's row-major input in place, for layers whose
// value ids are the neurons themselves: image j0 + i, rows [0, rows) -> cur[phys_row(r)][i].
// A warp covers 32 / TI groups of four consecutive rows for each of the TI images with one 16-byte
// load per lane (4 * 32 / TI lanes read 16 * 32 / TI contiguous bytes of an image), all loads of a
// thread in flight before its stores; the scattered 4-byte stores are the change of layout.
// Requires n % 4 == 0 and a 16-byte aligned base.  Returns (WANT_NS) whether any loaded value is
// neither 0 nor clip.
template <int TI, int NT, bool WANT_NS, bool PERMUTE>
__device__ __forceinline__ bool load_dense_rows(const float *dense, int n, int j0, int live_in, int rows, unsigned char *cur,
                                                float clip) {
    constexpr int RS = TI * 4;
    constexpr int GPW = 32 / TI;                 // groups of four rows per warp and step
    constexpr int STEP = (NT / 32) * GPW * 4;    // rows the block covers per step
    constexpr int UNR = 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i = lane % TI, g = lane / TI;
    const bool valid = j0 + i < live_in;
    const float *src = dense + (size_t)(valid ? j0 + i : j0) * n;
    bool ns = false;
    for (int r0 = (warp * GPW + g) * 4; r0 < rows; r0 += STEP * UNR) {
        float4 x[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int r = r0 + u * STEP;
            x[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (valid && r < rows) x[u] = __ldg(reinterpret_cast<const float4 *>(src + r));
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int r = r0 + u * STEP;
            if (r < rows) {
                // resident_phys_row flips the low bit of a row by the parity of the bits above it; r is a
                // multiple of 4, so rows r, r+1 share the parity of r >> 1 and rows r+2, r+3 have the other one
                const int par = PERMUTE ? (__popc((unsigned int)(r >> 1)) & 1) : 0;
                unsigned char *dst = cur + r * RS + i * 4;
                *reinterpret_cast<float *>(dst + (0 ^ par) * RS) = x[u].x;
                *reinterpret_cast<float *>(dst + (1 ^ par) * RS) = x[u].y;
                *reinterpret_cast<float *>(dst + (3 ^ par) * RS) = x[u].z;
                *reinterpret_cast<float *>(dst + (2 ^ par) * RS) = x[u].w;
                if (WANT_NS)
                    ns |= (x[u].x != 0.0f && x[u].x != clip) || (x[u].y != 0.0f && x[u].y != clip) || (x[u].z != 0.0f && x[u].z != clip) ||
                          (x[u].w != 0.0f && x[u].w != clip);
            }
        }
    }
    return ns;
}

// Grid: one block per TI live images (launched for the worst case; surplus blocks only take
// part in the last-block ticket).  Dynamic shared memory: two activation buffers of
// buf_rows * TI * 4 bytes, then (STAGED) two table buffers of table_bytes each.
// Threads per block: the GENERIC form is bound by shared-memory latency with one or two blocks
// per SM (its buffers fill the shared memory), so it runs 16 warps.
#ifndef SPDNN_GENERIC_THREADS
#define SPDNN_GENERIC_THREADS 512
#endif
#ifndef SPDNN_GENERIC_MIN_BLOCKS
#define SPDNN_GENERIC_MIN_BLOCKS 2      // <= 64 registers: two blocks of 16 warps per SM where the shared memory allows
#endif
// IPT = images per thread (4 here; the ALT2 kernel also runs 8).
template <int TI, int IPT, int KT, bool UNIFORM, bool STAGED>
__global__ void __launch_bounds__(SPDNN_GENERIC_THREADS, SPDNN_GENERIC_MIN_BLOCKS)
resident_kernel(const ResArgs a) {
    constexpr int NT = SPDNN_GENERIC_THREADS;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ unsigned int s_alive[3];
    __shared__ int s_last, s_fail;
    __shared__ __align__(8) unsigned long long s_bar[2];
    if (a.gate != nullptr && *a.gate != a.gate_want) return;
    constexpr int NQ = IPT / 4;                  // float4 halves per thread
    constexpr int LPC = TI / IPT;                // threads per class
    constexpr int CPI = NT / LPC;                // classes per pass of the block
    constexpr int RS = TI * 4;                   // bytes per row
    constexpr int TB = IPT * 4;                  // bytes of a row one thread owns
    const int tid = threadIdx.x, lane = tid & 31;
    const int sub = tid % LPC, grp = tid / LPC;
    const LoopCtl ctl = *a.ctl_in;
    const int live_in = ctl.live;
    const int nblk = (live_in + TI - 1) / TI;
    const int buf_bytes = a.buf_rows * RS;

    // a tile that the count_kernel pre-pass finished is skipped (TI divides 32: a block lies inside one tile)
    const bool tile_finished = a.tile_done != nullptr && (int)blockIdx.x < nblk && a.tile_done[(blockIdx.x * TI) >> 5] != 0;
    if ((int)blockIdx.x < nblk && !tile_finished) {
        unsigned char *cur = smem, *nxt = smem + buf_bytes;
        unsigned char *const tbl0 = smem + 2 * buf_bytes;      // table buffer q sits at tbl0 + q * table_bytes
        const int j0 = blockIdx.x * TI;
        if (tid == 0) {
            s_alive[0] = 0u;
            s_fail = 0;
            if (STAGED) {
                mbar_init(&s_bar[0], 1);
                mbar_init(&s_bar[1], 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                bulk_load_table(tbl0, a.layers[0].blob, (unsigned int)a.layers[0].blob_bytes, &s_bar[0]);
            }
        }
        // ---- load one row per value id of the block's images (dead images were dropped: read
        //      through the work list)
        unsigned int my_valid;
        {
            // Thread -> (image, row): the lanes of a warp that share a row read the TI images of the block, which lie
            // side by side in a tile unless images died in between; a thread has one source image and up to UNR
            // scalar loads in flight (a block that has an SM to itself cannot hide the latency of a load behind
            // another block's arithmetic).
            constexpr int RPP = NT / TI;             // rows per pass of the block
            constexpr int UNR = 16;
            const int img = tid % TI, rgrp = tid / TI;
            const float *const dense = a.dense_in ? *a.dense_in : nullptr;
            const int j = j0 + img;
            const bool valid = j < live_in;
            my_valid = valid ? 1u << img : 0u;
            const int src = ctl.identity ? (valid ? j : j0) : __ldg(a.slot + (valid ? j : j0));
            const ResLayer L0 = a.layers[0];
            if (!ctl.identity && rgrp == 0 && valid) move_id(ctl, a.ids0, a.ids1, j, src);
            const float *const pimg = dense ? dense + (size_t)src * a.n : a.yin + (size_t)(src >> 5) * a.tile_stride + (src & 31);
            const bool fast_dense = dense && !L0.rep && L0.v_in == a.n && (a.n & 3) == 0 && (reinterpret_cast<size_t>(dense) & 15) == 0;
            if (fast_dense) load_dense_rows<TI, NT, false, true>(dense, a.n, j0, live_in, L0.v_in, cur, a.clip);
            for (int v0 = rgrp; v0 < L0.v_in && !fast_dense; v0 += RPP * UNR) {
                float x[UNR];
                int e[UNR];
#pragma unroll
                for (int t = 0; t < UNR; ++t) {
                    const int v = min(v0 + t * RPP, L0.v_in - 1);
                    // element of row r: r * 32 floats into a tile's column, r floats into a row-major image
                    e[t] = L0.rep ? __ldg(L0.rep + v) : v * 32;
                    if (dense) e[t] >>= 5;
                }
#pragma unroll
                for (int t = 0; t < UNR; ++t) x[t] = valid ? __ldg(pimg + e[t]) : 0.0f;
#pragma unroll
                for (int t = 0; t < UNR; ++t) {
                    const int v = v0 + t * RPP;
                    if (v >= L0.v_in) break;
                    *reinterpret_cast<float *>(cur + resident_phys_row(v) * RS + img * 4) = x[t];
                }
            }
            // rows v_in .. even(v_in) + 1 are the zero rows padded table entries point at
            const int ve = (L0.v_in + 1) & ~1;
            for (int r = L0.v_in + grp; r < ve + 2; r += CPI)
#pragma unroll
                for (int h = 0; h < NQ; ++h)
                    *reinterpret_cast<float4 *>(cur + (r < ve ? resident_phys_row(r) : r) * RS + sub * TB + 16 * h) = make_float4(0, 0, 0, 0);
        }
        // TI divides 32, so every warp holds all images: the OR over a warp is the block's mask of valid images
        // (bit i = image j0 + i), identical in every thread
        unsigned int alive_prev = __reduce_or_sync(0xffffffffu, my_valid);
        __syncthreads();

        // ---- the layers of this chunk
        // thread 0 keeps the address of the table after next in registers, so that the copy
        // it issues at the top of a layer does not wait for a load from global memory
        const int32_t *nb_ptr = nullptr;
        unsigned int nb_bytes = 0;
        if (STAGED && tid == 0 && a.nlayers > 1) {
            nb_ptr = a.layers[1].blob;
            nb_bytes = (unsigned int)a.layers[1].blob_bytes;
        }
        int li = 0;
        int last_classes = 0;
        const bool force_dead = a.bias > 0.0f;
        for (; li < a.nlayers; ++li) {
            const int32_t *T;
            bool ready = true;
            if (STAGED) {
                if (tid == 0) {
                    s_alive[(li + 1) % 3] = 0u;
                    // the other table buffer was last read in layer li - 1, which every thread has left
                    if (li + 1 < a.nlayers) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        bulk_load_table(tbl0 + ((li + 1) & 1) * a.table_bytes, nb_ptr, nb_bytes, &s_bar[(li + 1) & 1]);
                        if (li + 2 < a.nlayers) {
                            nb_ptr = a.layers[li + 2].blob;
                            nb_bytes = (unsigned int)a.layers[li + 2].blob_bytes;
                        }
                    }
                }
                ready = mbar_wait(&s_bar[li & 1], (unsigned int)((li >> 1) & 1));
                if (!ready) s_fail = 1;
                T = reinterpret_cast<const int32_t *>(tbl0 + (li & 1) * a.table_bytes);
            } else {
                if (tid == 0) s_alive[(li + 1) % 3] = 0u;
                T = a.layers[li].blob;
            }
            // per-layer scalars travel in the table's header
            const int4 hdr = (STAGED && ready) ? *reinterpret_cast<const int4 *>(T)
                                               : (STAGED ? make_int4(0, 4, 0, 0) : __ldg(reinterpret_cast<const int4 *>(T)));
            const int classes = hdr.x, lk = hdr.y;
            const float lw = __int_as_float(hdr.z);
            last_classes = classes;
            unsigned int bits = 0;
            const unsigned char *in = cur + sub * TB;
            for (int u = grp; u < classes; u += CPI) {
                float4 s[NQ];
                int out_row;
                const int kp = lk + 4;
                const int32_t *rows = T + 4 + (size_t)u * kp;
#pragma unroll
                for (int h = 0; h < NQ; ++h)
                    s[h] = class_sum_generic<KT, UNIFORM, STAGED, RS>(rows, reinterpret_cast<const float *>(rows) + (size_t)classes * kp,
                                                                      lk, lw, in + 16 * h);
                out_row = STAGED ? rows[lk] : __ldg(rows + lk);
#pragma unroll
                for (int h = 0; h < NQ; ++h) {
                    float4 y;
                    y.x = finish_output(s[h].x, a.bias, a.clip);
                    y.y = finish_output(s[h].y, a.bias, a.clip);
                    y.z = finish_output(s[h].z, a.bias, a.clip);
                    y.w = finish_output(s[h].w, a.bias, a.clip);
                    // dead images stay dead: with bias <= 0 an all-zero image stays all-zero by itself
                    if (force_dead) {
                        const unsigned int al = alive_prev >> (sub * IPT + 4 * h);
                        if (!(al & 1u)) y.x = 0.0f;
                        if (!(al & 2u)) y.y = 0.0f;
                        if (!(al & 4u)) y.z = 0.0f;
                        if (!(al & 8u)) y.w = 0.0f;
                    }
                    bits |= ((y.x != 0.0f ? 1u : 0u) | (y.y != 0.0f ? 2u : 0u) | (y.z != 0.0f ? 4u : 0u) | (y.w != 0.0f ? 8u : 0u)) << (4 * h);
                    *reinterpret_cast<float4 *>(nxt + out_row * RS + sub * TB + 16 * h) = y;
                }
            }
            {
                // zero rows of the buffer just written (the next layer's padded entries point there)
                const int ue = (classes + 1) & ~1;
                for (int r = classes + grp; r < ue + 2; r += CPI)
#pragma unroll
                    for (int h = 0; h < NQ; ++h)
                        *reinterpret_cast<float4 *>(nxt + (r < ue ? resident_phys_row(r) : r) * RS + sub * TB + 16 * h) = make_float4(0, 0, 0, 0);
            }
            const unsigned int wm = __reduce_or_sync(0xffffffffu, bits << (sub * IPT));
            if (lane == 0 && wm) atomicOr(&s_alive[li % 3], wm);
            __syncthreads();
            const unsigned int alive_now = s_alive[li % 3] & alive_prev;
            if (tid == 0) {
                const int died = __popc(alive_prev & ~alive_now);
                if (died) atomicAdd(a.died_at + li, died);
            }
            alive_prev = alive_now;
            unsigned char *t = cur; cur = nxt; nxt = t;
            if (s_fail) {                    // a table never arrived: report it and drop the block's images
                if (tid == 0) atomicExch(a.status, 4);
                alive_prev = 0u;
            }
            if (alive_prev == 0u) { ++li; break; }
        }
        if (STAGED && li < a.nlayers) {
            // the loop was left early with the table of layer li still on its way: wait for it
            // (bounded) so that the block does not exit, and its shared memory get reused, under
            // a copy in flight
            if (tid == 0 && !mbar_wait(&s_bar[li & 1], (unsigned int)((li >> 1) & 1))) atomicExch(a.status, 4);
            __syncthreads();
        }

        // ---- expand the survivors' classes to all member rows (dead blocks write nothing)
        if (alive_prev != 0u) {
            const ResLayer LL = a.layers[li - 1];
            const int tile = j0 >> 5, lane0 = j0 & 31;
            float *out = a.yout + (size_t)tile * a.tile_stride + lane0 + sub * IPT;
            if (LL.mem_ptr != nullptr && a.reps_only) {
                // one row per class: the offsets of SU classes are looked up together (two dependent loads each)
                constexpr int SU = 8;
                for (int u0 = grp; u0 < last_classes; u0 += CPI * SU) {
                    int o[SU];
#pragma unroll
                    for (int t = 0; t < SU; ++t) o[t] = __ldg(LL.mem_ptr + min(u0 + t * CPI, last_classes - 1));
#pragma unroll
                    for (int t = 0; t < SU; ++t) o[t] = __ldg(LL.mem + o[t]);
#pragma unroll
                    for (int t = 0; t < SU; ++t) {
                        const int u = u0 + t * CPI;
                        if (u >= last_classes) break;
                        const unsigned char *src = cur + resident_phys_row(u) * RS + sub * TB;
#pragma unroll
                        for (int h = 0; h < NQ; ++h)
                            *reinterpret_cast<float4 *>(out + o[t] + 4 * h) = *reinterpret_cast<const float4 *>(src + 16 * h);
                    }
                }
            } else {
                for (int u = grp; u < last_classes; u += CPI) {
                    const unsigned char *src = cur + resident_phys_row(u) * RS + sub * TB;
#pragma unroll
                    for (int h = 0; h < NQ; ++h) {
                        const float4 y = *reinterpret_cast<const float4 *>(src + 16 * h);
                        if (LL.mem_ptr == nullptr) {
                            *reinterpret_cast<float4 *>(out + (size_t)u * 32 + 4 * h) = y;
                        } else {
                            const int mb = __ldg(LL.mem_ptr + u), me = __ldg(LL.mem_ptr + u + 1);
                            for (int m = mb; m < me; ++m) *reinterpret_cast<float4 *>(out + __ldg(LL.mem + m) + 4 * h) = y;
                        }
                    }
                }
            }
            if (tid == 0) atomicOr(a.mask + tile, alive_prev << lane0);
        }
    }

    // ---- last block done: rebuild the work list
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_last = (atomicAdd(a.counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    LayerArgs la;
    la.yin = a.yin; la.yout = a.yout; la.tile_stride = a.tile_stride;
    la.ctl_in = a.ctl_in; la.ctl_out = a.ctl_out; la.slot = a.slot; la.mask = a.mask;
    la.ids0 = a.ids0; la.ids1 = a.ids1; la.counter = a.counter; la.work = a.work; la.status = a.status;
    la.died_at = nullptr;
    la.first_member_only = 0;
    la.bias = a.bias; la.clip = a.clip;
    la.xw = nullptr; la.nw = 0; la.gate = nullptr; la.gate_want = 0;
    rebuild_worklist(la, live_in, ctl.ids_buf);
}

}  // namespace spdnn_impl
