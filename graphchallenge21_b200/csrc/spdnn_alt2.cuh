// alt2_kernel: the resident kernel for chunks of layers in the ALT2 table form (every class adds
// the two rows a, b alternately: a+b+a+b+..., K terms -- a 16-wide butterfly block in value ids).
//
// It differs from resident_kernel (spdnn_resident.cuh), whose structure it shares -- one block
// owns TI images for all layers of the chunk, two activation buffers of one row per value id
// ping-pong in shared memory, dead images are dropped between launches -- in two ways.
//
// 1. Packed table stream.  The tables of a chunk are one contiguous array in global memory,
//    `stride` bytes per layer: a 16-byte header {classes, K, bits of w, truth table}, then per pass
//    of 64 classes 32 slots of 8 bytes; slot `lane` holds the entries of classes 64p + lane and
//    64p + 32 + lane, 4 bytes each: 4 * row a | (4 * row b) << 16 in plain row numbers (value ids;
//    the float buffers keep row r at alt2_row_pos(r)).  The output row of class u is u and is
//    not stored.  One bulk asynchronous copy (TMA) brings a GROUP of up
//    to 8 layers into shared memory, several groups ahead of the layer being computed.
//
// 2. Bit form of saturated activations.  Once every activation of a block's images is exactly 0
//    or exactly clip (the steady state of the challenge networks), a row of the block is one
//    32-bit word (bit i = image i holds clip) and a class is a boolean function of two words.  All
//    classes of an ALT2 layer share K, the weight, the bias and the clip, so the output for the
//    four combinations (a, b) in {0, clip}^2 is a property of the LAYER.  alt2_pack_kernel evaluates
//    those four outputs with the same fp32 code as the float form (class_sum_alt2 + finish_output)
//    and stores them as the truth table, one byte per combination q = [a == clip] + 2 [b == clip]:
//      bit 7 of byte q   output == clip
//      bit 6 of byte q   output is neither 0 nor clip
//    (the top bit of a byte, because prmt.b32 can spread it over a word in one instruction).
//    The kernel then applies a layer to all images of a block with a few logic instructions per
//    class.  It does so a group of layers at a time, writing every layer's words to the next
//    buffer of a small ring and checking only at the end of the group that no image met a
//    combination whose output is not saturated and that no image died; if one did, the group is
//    repeated from its first buffer (still intact) one layer at a time, so that the layer of a
//    death is counted exactly and the layer with the unsaturated output is computed in the float
//    form.  The results are therefore those of the float form, bit for bit, whatever the inputs.
#pragma once

#include "spdnn_resident.cuh"

namespace spdnn_impl {

// Bytes per layer of a packed stream whose largest layer has max_classes classes.
__host__ __device__ __forceinline__ int alt2_stream_stride(int max_classes) { return 16 + ((max_classes + 63) / 64) * 256; }

// Byte offset of class u's entry inside a layer's record.
__host__ __device__ __forceinline__ int alt2_entry_offset(int u) {
    return 16 + (u >> 6) * 256 + (u & 31) * 8 + ((u >> 5) & 1) * 4;
}

// Builds the packed stream of a chunk from the per-layer blobs (ALT2: int32 t[U][4] = {row a,
// row b, output row, 0} behind a 4-word header).  One block per layer.
static __global__ void alt2_pack_kernel(const ResLayer *layers, int stride, unsigned char *out, float bias, float clip) {
    const int32_t *blob = layers[blockIdx.x].blob;
    const int classes = blob[0], k = blob[1];
    const float w = __int_as_float(blob[2]);
    unsigned char *rec = out + (size_t)blockIdx.x * stride;
    if (threadIdx.x == 0) {
        const float4 s = class_sum_alt2<0>(make_float4(0.0f, clip, 0.0f, clip), make_float4(0.0f, 0.0f, clip, clip), k, w, false);
        const float y[4] = {finish_output(s.x, bias, clip), finish_output(s.y, bias, clip), finish_output(s.z, bias, clip),
                            finish_output(s.w, bias, clip)};
        unsigned int tt = 0u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (y[q] == clip) tt |= 0x80u << (8 * q);
            else if (y[q] != 0.0f) tt |= 0x40u << (8 * q);
        }
        *reinterpret_cast<int4 *>(rec) = make_int4(classes, k, blob[2], (int)tt);
    }
    const int slots = (stride - 16) / 4;
    for (int u = threadIdx.x; u < slots; u += blockDim.x) {
        unsigned int e = 0u;                 // a class past the end reads row 0 twice; its output row is never read
        if (u < classes) {
            // the blob names rows of the float buffers, which are permuted (resident_phys_row, an involution):
            // the stream holds the plain row numbers (value ids)
            const int pa = blob[4 + 4 * u], pb = blob[4 + 4 * u + 1];
            e = (unsigned int)(resident_phys_row(pa) * 4) | ((unsigned int)(resident_phys_row(pb) * 4) << 16);
        }
        *reinterpret_cast<unsigned int *>(rec + alt2_entry_offset(u)) = e;
    }
}

// The truth table of a layer as eight 32-bit masks: prmt.b32 with selector nibble 8 | q copies
// the top bit of byte q over every byte of the result, so one instruction per combination makes
// its mask (hi[q]: output == clip; ns[q], from the table shifted left by one: output unsaturated).
// All of this runs on the integer ALU; bit-field extract and population count go through the
// slow special-function pipe and are avoided.
__device__ __forceinline__ unsigned int spread_top_bit(unsigned int tt, unsigned int selector) {
    unsigned int r;
    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(tt), "r"(selector));
    return r;
}
struct TruthMasks {
    unsigned int hi[4], ns[4];
};
__device__ __forceinline__ TruthMasks truth_masks(unsigned int tt) {
    TruthMasks m;
    m.hi[0] = spread_top_bit(tt, 0x8888u); m.hi[1] = spread_top_bit(tt, 0x9999u);
    m.hi[2] = spread_top_bit(tt, 0xAAAAu); m.hi[3] = spread_top_bit(tt, 0xBBBBu);
    m.ns[0] = spread_top_bit(tt << 1, 0x8888u); m.ns[1] = spread_top_bit(tt << 1, 0x9999u);
    m.ns[2] = spread_top_bit(tt << 1, 0xAAAAu); m.ns[3] = spread_top_bit(tt << 1, 0xBBBBu);
    return m;
}
// 32 images at once: the mask of combination [a] + 2 [b], selected bit by bit.
__device__ __forceinline__ unsigned int select4(unsigned int wa, unsigned int wb, const unsigned int (&m)[4]) {
    const unsigned int t0 = (wa & m[1]) | (~wa & m[0]);
    const unsigned int t1 = (wa & m[3]) | (~wa & m[2]);
    return (wb & t1) | (~wb & t0);
}

// Where the float buffers keep row r.  With fewer than 32 images a row is shorter than the 128 bytes
// the banks span, and rows are permuted (resident_phys_row) so that classes whose rows share one
// parity do not pile onto the same banks; a row of 32 images covers all banks and stays where it is.
template <int TI>
__device__ __forceinline__ int alt2_row_pos(int r) { return TI == 32 ? r : resident_phys_row(r); }

#ifndef SPDNN_ALT2_MIN_BLOCKS
#define SPDNN_ALT2_MIN_BLOCKS 4      // blocks per SM asked of the compiler: <= 64 registers, no spills
#endif
constexpr int kAlt2MaxTableRing = 4;

// Grid: one block per TI live images (launched for the worst case; surplus blocks only take
// part in the last-block ticket).  Dynamic shared memory: two activation buffers of
// buf_rows * TI * 4 bytes, then (STAGED) tring buffers of (stream_stride << tgroup_shift) bytes for
// groups of layer records.  The bit form keeps its ring of wring word buffers (rows_w words each) in
// the activation buffer that is free at that moment: while a block is in the bit form it needs
// neither float buffer (it converts `cur` on the way in and rebuilds `cur` on the way out).
// IPT = images per thread (4 or 8): with 8 a thread carries two float4 halves through every step.
// NT = threads per block: 256; 128 for chunks whose layers have at most 64 classes -- there one warp
// does the bit form, and smaller blocks let twice as many of those warps share an SM; 512 for chunks whose
// buffers leave room for one block per SM only -- the float form is a chain of dependent adds per output,
// and sixteen warps fill the issue slots that eight leave empty.
template <int TI, int IPT, int KT, bool STAGED, int NT>
__global__ void __launch_bounds__(NT, NT == 128 ? 2 * SPDNN_ALT2_MIN_BLOCKS : NT == 512 ? 1 : SPDNN_ALT2_MIN_BLOCKS)
alt2_kernel(const ResArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ unsigned int s_alive[3];          // float form: images alive after layer li % 3
    __shared__ int s_ns[3];                      // float form: layer li % 3 produced an output that is neither 0 nor clip
    __shared__ unsigned int s_grp[2][2];         // bit form, many warps: {unsaturated, last layer's outputs} of a group
    __shared__ int s_x[4];                       // state handed from the bit form to the block
    __shared__ int s_last, s_fail;
    __shared__ int s_next_group;                 // the next group of tables to request (used by one thread at a time)
    __shared__ __align__(8) unsigned long long s_bar[kAlt2MaxTableRing];
    if (a.gate != nullptr && *a.gate != a.gate_want) return;
    constexpr int NQ = IPT / 4;                  // float4 halves per thread
    constexpr int LPC = TI / IPT;                // threads per class
    constexpr int CPI = NT / LPC;                // classes per pass of the block
    constexpr int RS = TI * 4;                   // bytes per row
    constexpr int TB = IPT * 4;                  // bytes of a row one thread owns
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = tid % LPC, grp = tid / LPC;
    const LoopCtl ctl = *a.ctl_in;
    const int live_in = ctl.live;
    const int nblk = (live_in + TI - 1) / TI;
    const int buf_bytes = a.buf_rows * RS;
    const int stride = a.stream_stride;

    // a tile that the bits_kernel pre-pass finished is skipped (TI divides 32: a block lies inside one tile)
    const bool tile_finished = a.tile_done != nullptr && (int)blockIdx.x < nblk && a.tile_done[(blockIdx.x * TI) >> 5] != 0;
    if ((int)blockIdx.x < nblk && !tile_finished) {
        unsigned char *cur = smem, *nxt = smem + buf_bytes;
        unsigned char *const tbl0 = smem + 2 * buf_bytes;
        // Staged tables: group g = layers [g << gshift, (g + 1) << gshift) lives in buffer g & (tring - 1)
        // and completes phase g / tring of that buffer's mbarrier.
        const int gshift = a.tgroup_shift, gmask = (1 << gshift) - 1;
        const int tring = STAGED ? a.tring : 0, tshift = tring == 4 ? 2 : 1;
        const int group_bytes = stride << gshift;
        const int ngroups = STAGED ? (a.nlayers + gmask) >> gshift : 0;
        unsigned int *wring0 = nullptr;      // bit form: its word buffers, in the float buffer that is not `cur`
        const bool use_bits = a.bit_ok != 0;
        const int j0 = blockIdx.x * TI;
        // One thread requests the groups in order (thread 0 in the float form, the leader of the working
        // warp in the bit form; barriers separate the two).  At the top of layer li every thread has left layer
        // li - 1, so the buffers of all groups before li's are free: groups up to (li's group) + tring - 1
        // may be on their way.
        auto issue_groups = [&](int li) {
            const int lim = min((li >> gshift) + tring, ngroups);
            int next_group = s_next_group;
            while (next_group < lim) {
                const int l0 = next_group << gshift, cnt = min(1 << gshift, a.nlayers - l0);
                // orders the block's earlier reads of this buffer before the copy that overwrites it
                // (measured: no cost at one copy per 32 layers)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                bulk_load_table(tbl0 + (size_t)(next_group & (tring - 1)) * group_bytes, a.stream + (size_t)l0 * stride,
                                (unsigned int)(cnt * stride), &s_bar[next_group & (tring - 1)]);
                ++next_group;
            }
            s_next_group = next_group;
        };
        auto wait_table = [&](int l) -> bool {        // bounded
            const int g = l >> gshift;
            return mbar_wait(&s_bar[g & (tring - 1)], (unsigned int)((g >> tshift) & 1));
        };
        auto table_of = [&](int l) -> const unsigned char * {
            return STAGED ? tbl0 + (size_t)((l >> gshift) & (tring - 1)) * group_bytes + (size_t)(l & gmask) * stride
                          : a.stream + (size_t)l * stride;
        };
        if (tid == 0) {
            s_next_group = 0;
            s_alive[0] = 0u;
            s_ns[0] = 0;
            s_grp[0][0] = s_grp[0][1] = s_grp[1][0] = s_grp[1][1] = 0u;
            s_fail = 0;
            if (STAGED) {
                for (int q = 0; q < tring; ++q) mbar_init(&s_bar[q], 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                issue_groups(0);         // travels while the block's activations are read
            }
        }
        // ---- load one row per value id of the block's images (dead images were dropped: read
        //      through the work list)
        bool load_ns = false;                    // a loaded value is neither 0 nor clip
        unsigned int my_valid;
        {
            // Thread -> (image, row): the lanes of a warp that share a row read the TI images of the block, which lie
            // side by side in a tile unless images died in between (at most 2 * 32 / TI lines per load instruction);
            // a thread has one source image and up to UNR scalar loads in flight, the whole block all of its rows or
            // half of them: one block per SM cannot hide the latency of a load behind another block's arithmetic.
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
            if (fast_dense) load_ns |= load_dense_rows<TI, NT, true, TI != 32>(dense, a.n, j0, live_in, L0.v_in, cur, a.clip);
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
                    *reinterpret_cast<float *>(cur + alt2_row_pos<TI>(v) * RS + img * 4) = x[t];
                    load_ns |= x[t] != 0.0f && x[t] != a.clip;
                }
            }
        }
        // TI divides 32, so every warp holds all images: the OR over a warp is the block's mask of valid images
        // (bit i = image j0 + i), identical in every thread
        unsigned int alive_prev = __reduce_or_sync(0xffffffffu, my_valid);
        const bool start_in_bits = !__syncthreads_or(load_ns ? 1 : 0) && use_bits;

        // float rows -> one word per row (bit i = image i is non-zero; called when every value is 0 or clip)
        auto rows_to_bits = [&](const unsigned char *buf, unsigned int *w) {
            for (int r0 = 0; r0 < a.buf_rows; r0 += CPI) {
                const int r = r0 + grp;
                unsigned int m = 0;
                if (r < a.buf_rows) {
#pragma unroll
                    for (int h = 0; h < NQ; ++h) {
                        const float4 v = *reinterpret_cast<const float4 *>(buf + r * RS + sub * TB + 16 * h);
                        m |= ((v.x != 0.0f ? 1u : 0u) | (v.y != 0.0f ? 2u : 0u) | (v.z != 0.0f ? 4u : 0u) | (v.w != 0.0f ? 8u : 0u)) << (4 * h);
                    }
                }
                m <<= sub * IPT;
#pragma unroll
                for (int s = 1; s < LPC; s <<= 1) m |= __shfl_xor_sync(0xffffffffu, m, s);
                if (sub == 0 && r < a.buf_rows) w[alt2_row_pos<TI>(r)] = m;       // words are kept by plain row number
            }
        };
        // ---- the layers of this chunk
        int li = 0;                  // layers of the chunk applied so far
        int last_classes = 0;
        const bool force_dead = a.bias > 0.0f;
        const bool multi = a.bit_multi != 0;     // layers of more than one pass of 64 classes: all warps work in the bit form
        // Otherwise ONE warp of the block does the bit form.  Warp w of every block sits on the same scheduler
        // of an SM, so blocks that are likely to share an SM (numbers a multiple of the SM count apart) use
        // different warps; a wrong guess only costs speed.
        const int work_warp = (int)((blockIdx.x / (unsigned int)max(a.sm_count, 1)) % (NT / 32));
        int ws = 0;                  // bit form: the word buffer that holds the current activations
        bool bitmode = false;
        bool took_exact = true;      // float form: the exact-sum shortcut applied to a class of this thread in the last layer
        if (start_in_bits) {
            wring0 = reinterpret_cast<unsigned int *>(nxt);
            rows_to_bits(cur, wring0);
            __syncthreads();
            bitmode = true;
        }
        while (li < a.nlayers) {
            if (bitmode) {
                // ---- bit form.  Worker warps (one warp when a layer is one pass of 64 classes, else
                //      all warps) apply groups of layers until the chunk ends, every image is dead, or a
                //      layer yields an output that is neither 0 nor clip (redone in the float form).
                if (multi || warp == work_warp) {
                    const bool leader = multi ? tid == 0 : lane == 0;
                    unsigned int alive = alive_prev;
                    int done_classes = last_classes;
                    int careful = 0;             // layers still to be applied one at a time
                    int par = 0;
                    int waited_group = -1;                   // the group of tables these threads have seen arrive
                    unsigned int tt_cur = 0xffffffffu;       // no truth table has this value
                    TruthMasks tm = truth_masks(0u);
                    while (li < a.nlayers) {
                        if (STAGED && (li >> gshift) != waited_group) {
                            if (leader) issue_groups(li);
                            const bool arrived = wait_table(li);
                            // one verdict for all workers, so that they leave the loop together
                            if (!(multi ? __syncthreads_and(arrived ? 1 : 0) != 0 : __all_sync(0xffffffffu, arrived))) {
                                s_fail = 1;
                                break;
                            }
                            waited_group = li >> gshift;
                        }
                        int cnt = min(a.wring - 1, a.nlayers - li);
                        if (STAGED) cnt = min(cnt, (1 << gshift) - (li & gmask));
                        if (careful > 0) cnt = 1;
                        const unsigned char *T = table_of(li);
                        // The layers of a group are applied with one truth table: lane g looks at layer g's, and
                        // a group whose layers differ (another K or weight) is cut down to its first layer.
                        {
                            const unsigned char *hp = T + (size_t)(lane < cnt ? lane : 0) * stride + 12;
                            const unsigned int tl = STAGED ? *reinterpret_cast<const unsigned int *>(hp) : __ldg(reinterpret_cast<const unsigned int *>(hp));
                            const unsigned int t0 = __shfl_sync(0xffffffffu, tl, 0);
                            const bool same = multi ? __syncthreads_and(tl == t0 ? 1 : 0) != 0 : __all_sync(0xffffffffu, tl == t0);
                            if (!same) cnt = 1;
                            if (t0 != tt_cur) {
                                tt_cur = t0;
                                tm = truth_masks(t0);
                            }
                        }
                        const unsigned int keep = force_dead ? alive : 0xffffffffu;
                        unsigned int ns = 0u, acc = 0u;
                        int s = ws;
                        const int wbytes = a.rows_w * 4;
                        unsigned char *const wbase = reinterpret_cast<unsigned char *>(wring0);
                        unsigned char *const wend = wbase + (size_t)a.wring * wbytes;
                        const unsigned char *wc = wbase + (size_t)s * wbytes;
                        unsigned int o1 = 0u, o2 = 0u;
                        if (!multi) {
                            // one pass of 64 classes: lane owns classes lane and lane + 32, whose words sit at
                            // lane * 4 and lane * 4 + 128 of a buffer (plain row numbers, see rows_to_bits).
                            // A slot past the layer's classes reads row 0 twice and writes a row nobody reads;
                            // its bits can only add to `ns` (a needless return to the float form, never a
                            // wrong one) -- an image with all-zero rows gets 0 there like everywhere else.
                            const uint2 *slot = reinterpret_cast<const uint2 *>(T + 16) + lane;
                            uint2 e = STAGED ? *slot : __ldg(slot);
                            for (int g = 0; g < cnt; ++g) {
                                slot = reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned char *>(slot) + stride);
                                uint2 en = e;
                                if (g + 1 < cnt) en = STAGED ? *slot : __ldg(slot);      // next layer's entries, early
                                const unsigned int a1 = *reinterpret_cast<const unsigned int *>(wc + (e.x & 0xffffu));
                                const unsigned int b1 = *reinterpret_cast<const unsigned int *>(wc + (e.x >> 16));
                                const unsigned int a2 = *reinterpret_cast<const unsigned int *>(wc + (e.y & 0xffffu));
                                const unsigned int b2 = *reinterpret_cast<const unsigned int *>(wc + (e.y >> 16));
                                unsigned char *wn = const_cast<unsigned char *>(wc) + wbytes;
                                if (wn == wend) wn = wbase;
                                o1 = select4(a1, b1, tm.hi) & keep;
                                o2 = select4(a2, b2, tm.hi) & keep;
                                ns |= (select4(a1, b1, tm.ns) | select4(a2, b2, tm.ns)) & keep;
                                reinterpret_cast<unsigned int *>(wn)[lane] = o1;         // rows_w >= 32
                                if (lane + 32 < a.rows_w) reinterpret_cast<unsigned int *>(wn)[lane + 32] = o2;
                                wc = wn;
                                e = en;
                                __syncwarp();
                            }
                            s += cnt;
                            if (s >= a.wring) s -= a.wring;
                        } else {
                            const unsigned char *Tg = T;
                            for (int g = 0; g < cnt; ++g) {
                                const int classes = STAGED ? *reinterpret_cast<const int *>(Tg) : __ldg(reinterpret_cast<const int *>(Tg));
                                const int passes = (classes + 63) >> 6;
                                unsigned char *wn = const_cast<unsigned char *>(wc) + wbytes;
                                if (wn == wend) wn = wbase;
                                o1 = 0u; o2 = 0u;
                                for (int p = warp; p < passes; p += NT / 32) {
                                    const uint2 *slot = reinterpret_cast<const uint2 *>(Tg + 16 + p * 256) + lane;
                                    const uint2 e = STAGED ? *slot : __ldg(slot);
                                    const unsigned int a1 = *reinterpret_cast<const unsigned int *>(wc + (e.x & 0xffffu));
                                    const unsigned int b1 = *reinterpret_cast<const unsigned int *>(wc + (e.x >> 16));
                                    const unsigned int a2 = *reinterpret_cast<const unsigned int *>(wc + (e.y & 0xffffu));
                                    const unsigned int b2 = *reinterpret_cast<const unsigned int *>(wc + (e.y >> 16));
                                    const unsigned int x1 = select4(a1, b1, tm.hi) & keep, x2 = select4(a2, b2, tm.hi) & keep;
                                    ns |= (select4(a1, b1, tm.ns) | select4(a2, b2, tm.ns)) & keep;
                                    if (p * 64 + lane < a.rows_w) reinterpret_cast<unsigned int *>(wn)[p * 64 + lane] = x1;
                                    if (p * 64 + 32 + lane < a.rows_w) reinterpret_cast<unsigned int *>(wn)[p * 64 + 32 + lane] = x2;
                                    o1 |= p * 64 + lane < classes ? x1 : 0u;         // a slot past the classes does not count
                                    o2 |= p * 64 + 32 + lane < classes ? x2 : 0u;
                                }
                                wc = wn;
                                Tg += stride;
                                __syncthreads();
                            }
                            s += cnt;
                            if (s >= a.wring) s -= a.wring;
                        }
                        const unsigned char *hl = T + (size_t)(cnt - 1) * stride;      // classes of the group's last layer
                        const int classes = STAGED ? *reinterpret_cast<const int *>(hl) : __ldg(reinterpret_cast<const int *>(hl));
                        // outputs of the group's last layer; here a slot past the classes must not count, or an
                        // image whose real outputs are all zero could pass for alive one layer longer
                        if (!multi) acc = (lane < classes ? o1 : 0u) | (lane + 32 < classes ? o2 : 0u);
                        else acc = o1 | o2;
                        // what the group did: an unsaturated output anywhere, and who is alive after it
                        unsigned int ns_any = __reduce_or_sync(0xffffffffu, ns), now = __reduce_or_sync(0xffffffffu, acc);
                        if (multi) {
                            if (lane == 0) {
                                if (ns_any) atomicOr(&s_grp[par][0], ns_any);
                                if (now) atomicOr(&s_grp[par][1], now);
                            }
                            __syncthreads();
                            ns_any = s_grp[par][0];
                            now = s_grp[par][1];
                            if (tid == 0) s_grp[par ^ 1][0] = s_grp[par ^ 1][1] = 0u;
                            par ^= 1;
                        }
                        now &= alive;
                        if (ns_any != 0u || (now != alive && cnt > 1)) {
                            if (cnt == 1) break;         // layer li has an unsaturated output: the float form applies it
                            careful = cnt;               // repeat the group from its first buffer, layer by layer
                            continue;
                        }
                        if (now != alive && leader) atomicAdd(a.died_at + li, __popc(alive & ~now));     // cnt == 1
                        alive = now;
                        ws = s;
                        li += cnt;
                        done_classes = classes;
                        if (careful > 0) --careful;
                        if (alive == 0u) break;
                    }
                    if (leader) {
                        s_x[0] = li; s_x[1] = (int)alive; s_x[2] = done_classes; s_x[3] = ws;
                        s_alive[li % 3] = 0u;        // the float form may take over at layer li
                        s_ns[li % 3] = 0;
                    }
                }
                __syncthreads();
                li = s_x[0];
                alive_prev = (unsigned int)s_x[1];
                last_classes = s_x[2];
                ws = s_x[3];
                // back to floats: the rows the next float layer (or the expansion below) reads
                const unsigned int *wcur = wring0 + (size_t)ws * a.rows_w;
                for (int r = grp; r < a.buf_rows; r += CPI) {
                    const unsigned int wv = wcur[alt2_row_pos<TI>(r)] >> (sub * IPT);
#pragma unroll
                    for (int h = 0; h < NQ; ++h) {
                        const unsigned int q = wv >> (4 * h);
                        *reinterpret_cast<float4 *>(cur + r * RS + sub * TB + 16 * h) =
                            make_float4((q & 1u) ? a.clip : 0.0f, (q & 2u) ? a.clip : 0.0f, (q & 4u) ? a.clip : 0.0f, (q & 8u) ? a.clip : 0.0f);
                    }
                }
                bitmode = false;
                __syncthreads();
                if (s_fail) {
                    if (tid == 0) atomicExch(a.status, 4);
                    alive_prev = 0u;
                }
                if (alive_prev == 0u) break;
                continue;
            }

            // ---- float form of layer li
            bool ready = true;
            if (tid == 0) {
                s_alive[(li + 1) % 3] = 0u;
                s_ns[(li + 1) % 3] = 0;
            }
            if (STAGED) {
                if (tid == 0) issue_groups(li);
                ready = wait_table(li);
                if (!ready) s_fail = 1;
            }
            const unsigned char *T = table_of(li);
            // per-layer scalars travel in the record's header
            const int4 hdr = (STAGED && ready) ? *reinterpret_cast<const int4 *>(T)
                                               : (STAGED ? make_int4(0, 4, 0, 0) : __ldg(reinterpret_cast<const int4 *>(T)));
            const int classes = hdr.x, lk = hdr.y;
            const float lw = __int_as_float(hdr.z);
            last_classes = classes;
            unsigned int bits = 0;
            bool ns = false;
            const unsigned char *in = cur + sub * TB;
            // The exact-sum shortcut needs a test of all eight inputs of a class; a thread whose classes all failed it
            // in the last layer skips the test (same bits either way) and tries again every eighth layer.
            const bool try_exact = a.exact_ok != 0 && (took_exact || (li & 7) == 0);
            took_exact = false;
            for (int u = grp; u < classes; u += CPI) {
                const unsigned int *ep = reinterpret_cast<const unsigned int *>(T + alt2_entry_offset(u));
                const unsigned int e = STAGED ? *ep : __ldg(ep);
                const int ao = alt2_row_pos<TI>((int)(e & 0xffffu) >> 2) * RS, bo = alt2_row_pos<TI>((int)(e >> 18)) * RS;
                unsigned char *out = nxt + alt2_row_pos<TI>(u) * RS + sub * TB;
#pragma unroll
                for (int h = 0; h < NQ; ++h) {
                    const float4 va = *reinterpret_cast<const float4 *>(in + ao + 16 * h);
                    const float4 vb = *reinterpret_cast<const float4 *>(in + bo + 16 * h);
                    const float4 s = class_sum_alt2<KT>(va, vb, lk, lw, try_exact, &took_exact);
                    float4 y;
                    y.x = finish_output(s.x, a.bias, a.clip);
                    y.y = finish_output(s.y, a.bias, a.clip);
                    y.z = finish_output(s.z, a.bias, a.clip);
                    y.w = finish_output(s.w, a.bias, a.clip);
                    // dead images stay dead: with bias <= 0 an all-zero image stays all-zero by itself
                    if (force_dead) {
                        const unsigned int al = alive_prev >> (sub * IPT + 4 * h);
                        if (!(al & 1u)) y.x = 0.0f;
                        if (!(al & 2u)) y.y = 0.0f;
                        if (!(al & 4u)) y.z = 0.0f;
                        if (!(al & 8u)) y.w = 0.0f;
                    }
                    bits |= ((y.x != 0.0f ? 1u : 0u) | (y.y != 0.0f ? 2u : 0u) | (y.z != 0.0f ? 4u : 0u) | (y.w != 0.0f ? 8u : 0u)) << (4 * h);
                    ns |= (y.x != 0.0f && y.x != a.clip) || (y.y != 0.0f && y.y != a.clip) || (y.z != 0.0f && y.z != a.clip) ||
                          (y.w != 0.0f && y.w != a.clip);
                    *reinterpret_cast<float4 *>(out + 16 * h) = y;
                }
            }
            const unsigned int wm = __reduce_or_sync(0xffffffffu, bits << (sub * IPT));
            if (lane == 0 && wm) atomicOr(&s_alive[li % 3], wm);
            if (use_bits && __any_sync(0xffffffffu, ns) && lane == 0) s_ns[li % 3] = 1;
            __syncthreads();
            const unsigned int alive_now = s_alive[li % 3] & alive_prev;
            const bool saturated = use_bits && s_ns[li % 3] == 0;
            if (tid == 0) {
                const int died = __popc(alive_prev & ~alive_now);
                if (died) atomicAdd(a.died_at + li, died);
            }
            alive_prev = alive_now;
            unsigned char *t = cur; cur = nxt; nxt = t;
            ++li;
            if (s_fail) {                    // a table never arrived: report it and drop the block's images
                if (tid == 0) atomicExch(a.status, 4);
                alive_prev = 0u;
            }
            if (alive_prev == 0u) break;
            if (saturated && li < a.nlayers) {
                // every output of the layer is 0 or clip: continue in the bit form
                wring0 = reinterpret_cast<unsigned int *>(nxt);
                rows_to_bits(cur, wring0);
                ws = 0;
                __syncthreads();
                bitmode = true;
            }
        }
        if (STAGED) {
            // tables may still be on their way: wait for them (bounded) so that the block does not
            // exit, and its shared memory get reused, under a copy in flight
            if (tid == 0)
                for (int g = min(li, a.nlayers - 1) >> gshift; g < s_next_group; ++g)
                    if (!mbar_wait(&s_bar[g & (tring - 1)], (unsigned int)((g >> tshift) & 1))) atomicExch(a.status, 4);
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
                        const unsigned char *src = cur + alt2_row_pos<TI>(u) * RS + sub * TB;
#pragma unroll
                        for (int h = 0; h < NQ; ++h)
                            *reinterpret_cast<float4 *>(out + o[t] + 4 * h) = *reinterpret_cast<const float4 *>(src + 16 * h);
                    }
                }
            } else {
                for (int u = grp; u < last_classes; u += CPI) {
                    const unsigned char *src = cur + alt2_row_pos<TI>(u) * RS + sub * TB;
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
