// bits_kernel: a chunk of ALT2 layers for tiles of 32 images whose activations are all exactly 0
// or clip, with one 32-bit word per row (bit i = image i holds clip) and nothing else in shared
// memory -- so a block owns 32 images whatever the number of neurons is.
//
// alt2_kernel (spdnn_alt2.cuh) has the same bit form, but keeps it inside the float buffers of a
// block; at 16384 and 65536 neurons those buffers fill the shared memory with 16 or 8 images, a
// quarter to a half of every word goes unused, one block per SM is resident and the tables no
// longer fit beside them.  This kernel is the steady state of the large challenge networks (the
// role of the reference's n16384_l11_kernel, src/microbenchmark/all_network.cu:115-153, which also
// runs one thread per image over gathered rows): two word buffers of one word per value id, the
// per-layer tables streamed through a small ring by bulk asynchronous copies, all warps of the
// block sharing the classes of a layer, one block barrier per layer.
//
// It runs as a PRE-PASS of the chunk's alt2_kernel launch and decides per tile:
//   * every value the tile reads is 0 or clip, and no layer of the chunk produced an output that is
//     neither: the tile is finished here (outputs written, survivor ballot set, deaths counted) and
//     tile_done[tile] = 1 tells alt2_kernel's blocks of that tile to skip their work;
//   * otherwise nothing is written, tile_done[tile] = 0, and alt2_kernel computes the tile from the
//     chunk's input as if this kernel had not run (its float form handles any value).
// Either way the results are those of the float form, bit for bit: the truth table of a layer is
// computed by the float code itself (alt2_pack_kernel).  The work-list rebuild stays with the last
// block of the alt2_kernel launch that follows.
#pragma once

#include "spdnn_alt2.cuh"

namespace spdnn_impl {

constexpr int kBitsMaxThreads = 1024;
constexpr int kBitsCheckEvery = 32;      // layers between two checks for an unsaturated output

// Where the layer records come from.  kBitsCached: the chunk's layers repeat a few distinct records (a periodic
// network in its steady state): all of them are brought into shared memory once, a.rec_of[layer] names the
// record of every layer, and the layer loop touches no global memory at all.  kBitsRing: records stream through
// a ring of a.tring buffers, groups of 1 << tgroup_shift layers per bulk copy.  kBitsGlobal: read in place.
constexpr int kBitsGlobal = 0, kBitsRing = 1, kBitsCached = 2;

// Dynamic shared memory: two word buffers of a.wwords words (a multiple of 64, at least the largest
// v_in / classes of the chunk), then kBitsRing: a.tring buffers of (stream_stride << tgroup_shift) bytes;
// kBitsCached: a.cache_records records of stream_stride bytes, then one uint16 per layer of the chunk (rounded up to
// 16 bytes), then a.wwords words that hold a copy of a segment's input.
template <int MODE>
__global__ void __launch_bounds__(kBitsMaxThreads, 1) bits_kernel(const ResArgs a) {
    constexpr bool STAGED = (MODE == kBitsRing);
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ unsigned int s_or[3];             // OR of the outputs of layer li % 3: who is alive after it
    __shared__ int s_next_group;
    __shared__ int s_nev, s_ev_layer[32], s_ev_cnt[32];      // deaths seen so far (at most one per image)
    __shared__ __align__(8) unsigned long long s_bar[kAlt2MaxTableRing];
    if (a.gate != nullptr && *a.gate != a.gate_want) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const LoopCtl ctl = *a.ctl_in;
    const int live_in = ctl.live;
    const int tile = blockIdx.x;
    if (tile >= ((live_in + 31) >> 5)) return;
    unsigned int *wc = reinterpret_cast<unsigned int *>(smem), *wn = wc + a.wwords;
    unsigned char *const tbl0 = smem + (size_t)a.wwords * 8;
    const int stride = a.stream_stride;
    const int gshift = a.tgroup_shift, gmask = (1 << gshift) - 1;
    const int tring = STAGED ? a.tring : 0, tshift = tring == 4 ? 2 : 1;
    const int group_bytes = stride << gshift;
    const int ngroups = STAGED ? (a.nlayers + gmask) >> gshift : 0;

    // ---- the tile's input: one word per value id, read through the work list
    const int j = tile * 32 + lane;
    const bool valid = j < live_in;
    const int jj = valid ? j : tile * 32;
    const int src = ctl.identity ? jj : __ldg(a.slot + jj);
    if (!ctl.identity && warp == 0 && valid) move_id(ctl, a.ids0, a.ids1, j, src);
    const float *__restrict__ p = a.yin + (size_t)(src >> 5) * a.tile_stride + (src & 31);
    const ResLayer L0 = a.layers[0];
    bool ns_in = false;
    for (int v0 = warp * 8; v0 < L0.v_in; v0 += nwarps * 8) {
        int e[8];
        float x[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int v = min(v0 + q, L0.v_in - 1);
            e[q] = L0.rep ? __ldg(L0.rep + v) : v * 32;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) x[q] = valid ? __ldg(p + e[q]) : 0.0f;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const unsigned int w = __ballot_sync(0xffffffffu, x[q] != 0.0f);
            ns_in |= (x[q] != 0.0f && x[q] != a.clip);
            if (lane == 0 && v0 + q < L0.v_in) wc[v0 + q] = w;
        }
    }
    if (tid == 0) {
        s_or[0] = 0u;
        s_next_group = 0;
        s_nev = 0;
        if (STAGED) {
            for (int q = 0; q < tring; ++q) mbar_init(&s_bar[q], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    if (__syncthreads_or(ns_in ? 1 : 0)) {          // a value that is neither 0 nor clip: the float form's tile
        if (tid == 0) a.tile_done[tile] = 0;
        return;
    }
    unsigned short *const s_rec = reinterpret_cast<unsigned short *>(tbl0 + (size_t)a.cache_records * stride);
    if (MODE == kBitsCached) {
        // every distinct record of the chunk in one bulk copy, the layer -> record map by plain loads
        if (tid == 0) {
            mbar_init(&s_bar[0], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            bulk_load_table(tbl0, a.cache, (unsigned int)(a.cache_records * stride), &s_bar[0]);
        }
        for (int q = tid; q < a.nlayers; q += blockDim.x) s_rec[q] = __ldg(a.rec_of + q);
        __syncthreads();                                // the barrier's initialisation is visible to every waiter
        const bool arrived = mbar_wait(&s_bar[0], 0u);
        if (!__syncthreads_and(arrived ? 1 : 0)) {      // bounded wait ran out: report it, drop the tile's images
            if (tid == 0) { atomicExch(a.status, 4); a.tile_done[tile] = 1; }
            return;
        }
    }

    auto issue_groups = [&](int li) {               // thread 0; every thread has left layer li - 1
        const int lim = min((li >> gshift) + tring, ngroups);
        int next_group = s_next_group;
        while (next_group < lim) {
            const int l0 = next_group << gshift, cnt = min(1 << gshift, a.nlayers - l0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            bulk_load_table(tbl0 + (size_t)(next_group & (tring - 1)) * group_bytes, a.stream + (size_t)l0 * stride,
                            (unsigned int)(cnt * stride), &s_bar[next_group & (tring - 1)]);
            ++next_group;
        }
        s_next_group = next_group;
    };
    auto drain = [&](int li) {                      // thread 0: copies still on their way must land before the block exits
        bool ok = true;
        for (int g = min(li, a.nlayers - 1) >> gshift; g < s_next_group; ++g)
            ok &= mbar_wait(&s_bar[g & (tring - 1)], (unsigned int)((g >> tshift) & 1));
        if (!ok) atomicExch(a.status, 4);
    };

    unsigned int alive = __ballot_sync(0xffffffffu, valid);
    const bool force_dead = a.bias > 0.0f;
    unsigned int tt_cur = 0xffffffffu;               // no truth table has this value
    TruthMasks tm = truth_masks(0u);
    unsigned int ns = 0u;
    int li = 0, last_classes = 0;
    int waited_group = -1;
    bool failed = false, unsat = false;
    auto run_tracked = [&](int lend) {
    while (li < lend) {
        if (STAGED && (li >> gshift) != waited_group) {
            if (tid == 0) issue_groups(li);
            const int g = li >> gshift;
            const bool arrived = mbar_wait(&s_bar[g & (tring - 1)], (unsigned int)((g >> tshift) & 1));
            if (!__syncthreads_and(arrived ? 1 : 0)) { failed = true; break; }
            waited_group = g;
        }
        constexpr bool IN_SMEM = (MODE != kBitsGlobal);
        const unsigned char *T = MODE == kBitsCached ? tbl0 + (size_t)s_rec[li] * stride
                                 : STAGED ? tbl0 + (size_t)((li >> gshift) & (tring - 1)) * group_bytes + (size_t)(li & gmask) * stride
                                          : a.stream + (size_t)li * stride;
        const int4 hdr = IN_SMEM ? *reinterpret_cast<const int4 *>(T) : __ldg(reinterpret_cast<const int4 *>(T));
        const int classes = hdr.x;
        if ((unsigned int)hdr.w != tt_cur) {
            tt_cur = (unsigned int)hdr.w;
            tm = truth_masks(tt_cur);
        }
        const unsigned int keep = force_dead ? alive : 0xffffffffu;
        const int passes = (classes + 63) >> 6;
        unsigned int o = 0u;
        const unsigned char *wcb = reinterpret_cast<const unsigned char *>(wc);
        // The usual table -- (0, 0) -> 0, (clip, clip) -> clip, one clip-valued input -> an unsaturated output -- is
        // a & b with a ^ b marking the unsaturated ones: two instructions instead of four table selections.
        const bool usual = (tt_cur == 0x80404000u);
        for (int ps = warp; ps < passes; ps += nwarps) {
            const uint2 *slot = reinterpret_cast<const uint2 *>(T + 16 + ps * 256) + lane;
            const uint2 e = IN_SMEM ? *slot : __ldg(slot);
            const unsigned int a1 = *reinterpret_cast<const unsigned int *>(wcb + (e.x & 0xffffu));
            const unsigned int b1 = *reinterpret_cast<const unsigned int *>(wcb + (e.x >> 16));
            const unsigned int a2 = *reinterpret_cast<const unsigned int *>(wcb + (e.y & 0xffffu));
            const unsigned int b2 = *reinterpret_cast<const unsigned int *>(wcb + (e.y >> 16));
            unsigned int x1, x2, n1, n2;
            if (usual) {
                x1 = a1 & b1; x2 = a2 & b2;
                n1 = a1 ^ b1; n2 = a2 ^ b2;
            } else {
                x1 = select4(a1, b1, tm.hi); x2 = select4(a2, b2, tm.hi);
                n1 = select4(a1, b1, tm.ns); n2 = select4(a2, b2, tm.ns);
            }
            if (force_dead) { x1 &= keep; x2 &= keep; n1 &= keep; n2 &= keep; }
            wn[ps * 64 + lane] = x1;
            wn[ps * 64 + 32 + lane] = x2;
            if ((ps + 1) * 64 <= classes) {
                ns |= n1 | n2;
                o |= x1 | x2;
            } else {
                // the layer's last pass: a slot past the classes (it read row 0 twice) does not count
                const bool in1 = ps * 64 + lane < classes, in2 = ps * 64 + 32 + lane < classes;
                ns |= (in1 ? n1 : 0u) | (in2 ? n2 : 0u);
                o |= (in1 ? x1 : 0u) | (in2 ? x2 : 0u);
            }
        }
        o = __reduce_or_sync(0xffffffffu, o);
        if (lane == 0 && o) atomicOr(&s_or[li % 3], o);
        if (tid == 0) s_or[(li + 1) % 3] = 0u;      // layer li + 1's slot: last read after layer li - 2, which every thread has left
        __syncthreads();
        const unsigned int now = s_or[li % 3] & alive;
        if (now != alive && tid == 0) {
            s_ev_layer[s_nev] = li;
            s_ev_cnt[s_nev] = __popc(alive & ~now);
            ++s_nev;
        }
        alive = now;
        unsigned int *t = wc; wc = wn; wn = t;
        last_classes = classes;
        ++li;
        if ((li % kBitsCheckEvery) == 0 || li == lend || alive == 0u) {
            if (__syncthreads_or(ns != 0u ? 1 : 0)) { unsat = true; break; }
        }
        if (alive == 0u) break;
    }
    };
    if (MODE == kBitsCached && a.wwords <= nwarps * 128 && !force_dead) {
        // Every record is in shared memory and a warp has at most two passes per layer.  The records are checked
        // once: if all carry the usual truth table ((0, 0) -> 0, (clip, clip) -> clip, one clip-valued input -> an
        // unsaturated output), a layer is x = a & b with a ^ b marking the unsaturated outputs, and the loop below
        // runs SEGMENTS of up to kBitsCheckEvery layers with nothing per layer but that: the next layer's entries
        // are fetched while this one computes, and who is alive is not tracked -- a dead image's words are all zero
        // and stay so, therefore the OR of the words after the segment tells who is alive then.  Only if that
        // differs from before (an image died inside the segment: rare) are the segment's layers run again from a
        // copy of its input, with the per-layer bookkeeping that finds the layer of death.
        bool all_usual = true;
        for (int q = 0; q < a.cache_records; ++q)
            all_usual &= (*reinterpret_cast<const unsigned int *>(tbl0 + (size_t)q * stride + 12) == 0x80404000u);
        if (all_usual) {
            unsigned int *const ckpt = reinterpret_cast<unsigned int *>(reinterpret_cast<unsigned char *>(s_rec) +
                                                                        (((size_t)a.nlayers * 2 + 15) & ~(size_t)15));
            const int spasses = (stride - 16) >> 8;                 // passes a record has room for
            const int p0 = warp, p1 = warp + nwarps;
            auto entries = [&](const unsigned char *rec, int ps) -> uint2 {
                return ps < spasses ? (reinterpret_cast<const uint2 *>(rec + 16 + ps * 256))[lane] : make_uint2(0u, 0u);
            };
            while (li < a.nlayers && !unsat && !failed) {
                const int l0 = li, l1 = min(li + kBitsCheckEvery, a.nlayers);
                for (int q = tid; q < a.wwords; q += blockDim.x) ckpt[q] = wc[q];      // read before layer l0's barrier, which precedes any write to wc
                const unsigned char *T = tbl0 + (size_t)s_rec[li] * stride;
                int classes = *reinterpret_cast<const int *>(T);
                uint2 e0 = entries(T, p0), e1 = entries(T, p1);
                unsigned int nsx = 0u;
                for (; li < l1; ++li) {
                    const unsigned char *wcb = reinterpret_cast<const unsigned char *>(wc);
                    const int passes = (classes + 63) >> 6;
                    // a pass the layer does not have is skipped; a slot past the classes in its last pass reads row 0
                    // twice (a ^ a = 0) and writes a row that nobody reads
                    const unsigned int a1 = *reinterpret_cast<const unsigned int *>(wcb + (e0.x & 0xffffu));
                    const unsigned int b1 = *reinterpret_cast<const unsigned int *>(wcb + (e0.x >> 16));
                    const unsigned int a2 = *reinterpret_cast<const unsigned int *>(wcb + (e0.y & 0xffffu));
                    const unsigned int b2 = *reinterpret_cast<const unsigned int *>(wcb + (e0.y >> 16));
                    const unsigned int a3 = *reinterpret_cast<const unsigned int *>(wcb + (e1.x & 0xffffu));
                    const unsigned int b3 = *reinterpret_cast<const unsigned int *>(wcb + (e1.x >> 16));
                    const unsigned int a4 = *reinterpret_cast<const unsigned int *>(wcb + (e1.y & 0xffffu));
                    const unsigned int b4 = *reinterpret_cast<const unsigned int *>(wcb + (e1.y >> 16));
                    const bool has0 = p0 < passes, has1 = p1 < passes;
                    last_classes = classes;
                    if (li + 1 < a.nlayers) {                       // the next layer's record, while the words arrive
                        const unsigned char *Tn = tbl0 + (size_t)s_rec[li + 1] * stride;
                        classes = *reinterpret_cast<const int *>(Tn);
                        e0 = entries(Tn, p0);
                        e1 = entries(Tn, p1);
                    }
                    if (has0) {
                        wn[p0 * 64 + lane] = a1 & b1;
                        wn[p0 * 64 + 32 + lane] = a2 & b2;
                        nsx |= (a1 ^ b1) | (a2 ^ b2);
                    }
                    if (has1) {
                        wn[p1 * 64 + lane] = a3 & b3;
                        wn[p1 * 64 + 32 + lane] = a4 & b4;
                        nsx |= (a3 ^ b3) | (a4 ^ b4);
                    }
                    __syncthreads();
                    unsigned int *t = wc; wc = wn; wn = t;
                }
                // who is alive after the segment: the OR of the last layer's rows
                unsigned int o = 0u;
                for (int q = tid; q < last_classes; q += blockDim.x) o |= wc[q];
                o = __reduce_or_sync(0xffffffffu, o);
                if (lane == 0 && o) atomicOr(&s_or[0], o);
                const bool any_ns = __syncthreads_or(nsx != 0u ? 1 : 0) != 0;      // (the barrier also publishes the atomics)
                const unsigned int now = s_or[0] & alive;
                __syncthreads();                               // everyone has read s_or[0]
                if (tid == 0) s_or[0] = s_or[1] = s_or[2] = 0u;
                if (any_ns) { unsat = true; break; }
                if (now != alive) {
                    // somebody died inside the segment: again from its input, layer by layer (the tracked loop wants
                    // its three slots zero and leaves them in any state)
                    for (int q = tid; q < a.wwords; q += blockDim.x) wc[q] = ckpt[q];
                    li = l0;
                    __syncthreads();
                    run_tracked(l1);
                    __syncthreads();
                    if (tid == 0) s_or[0] = s_or[1] = s_or[2] = 0u;
                }
                if (alive == 0u) break;
            }
        } else {
            run_tracked(a.nlayers);
        }
    } else {
        run_tracked(a.nlayers);
    }
    if (STAGED) {
        if (tid == 0) drain(li);
        __syncthreads();
    }
    if (failed) {                      // a table never arrived: report it and drop the tile's images
        if (tid == 0) { atomicExch(a.status, 4); a.tile_done[tile] = 1; }
        return;
    }
    if (unsat) {                       // an output that is neither 0 nor clip: the float form redoes the tile from the chunk's input
        if (tid == 0) a.tile_done[tile] = 0;
        return;
    }
    if (tid == 0) {
        a.tile_done[tile] = 1;
        for (int q = 0; q < s_nev; ++q) atomicAdd(a.died_at + s_ev_layer[q], s_ev_cnt[q]);
        if (alive) atomicOr(a.mask + tile, alive);
    }
    if (alive == 0u) return;
    // ---- the survivors' rows back to floats: all member rows, or the one row per class the next chunk reads
    const ResLayer LL = a.layers[li - 1];
    float *out = a.yout + (size_t)tile * a.tile_stride + lane;
    if (LL.mem_ptr != nullptr && a.reps_only) {
        // one row per class: the offsets of SU rows are looked up together (two dependent loads each) before their stores
        constexpr int SU = 8;
        for (int u0 = warp; u0 < last_classes; u0 += nwarps * SU) {
            int o[SU];
#pragma unroll
            for (int t = 0; t < SU; ++t) o[t] = __ldg(LL.mem_ptr + min(u0 + t * nwarps, last_classes - 1));
#pragma unroll
            for (int t = 0; t < SU; ++t) o[t] = __ldg(LL.mem + o[t]);
#pragma unroll
            for (int t = 0; t < SU; ++t) {
                const int u = u0 + t * nwarps;
                if (u >= last_classes) break;
                out[o[t]] = ((wc[u] >> lane) & 1u) ? a.clip : 0.0f;
            }
        }
        return;
    }
    for (int u = warp; u < last_classes; u += nwarps) {
        const float y = ((wc[u] >> lane) & 1u) ? a.clip : 0.0f;
        if (LL.mem_ptr == nullptr) {
            out[(size_t)u * 32] = y;
        } else {
            const int mb = __ldg(LL.mem_ptr + u), me = __ldg(LL.mem_ptr + u + 1);
            for (int m = mb; m < me; ++m) out[__ldg(LL.mem + m)] = y;
        }
    }
}

// ---- count_kernel: the same pre-pass for chunks of GENERIC layers (K gathered rows per class) ------------
//
// With a uniform weight and inputs that are all 0 or clip, the K-term sum of a class, added in any
// order, is the sequential sum of c copies of clip, c = the number of its inputs that hold clip (adding
// 0.0 never changes a sum).  So the output is a function of the COUNT alone, tabulated per layer with
// the float form's own instructions (sequential adds, one multiply, bias, clamp), and because the
// weight is positive that function does not decrease: outputs are 0 up to some count, clip from some
// count on, unsaturated in between.  For 32 images at once the count is a bit-sliced number: a lane owns
// a class, gathers its K = 32 row words and adds them with a tree of 31 carry-save adders (two 3-input
// logic instructions each) into six planes, then compares the planes with the two thresholds.  A
// count in the unsaturated range sends the tile back to the float form, as in bits_kernel.
//
// Word buffers are indexed by the PHYSICAL row numbers the GENERIC tables hold (resident_phys_row), the
// tables are read from global memory (a class's 32 row numbers are 128 contiguous bytes of one lane).
__device__ __forceinline__ void csa(unsigned int &h, unsigned int &l, unsigned int a, unsigned int b, unsigned int c) {
    const unsigned int u = a ^ b;
    h = (a & b) | (u & c);
    l = u ^ c;
}

// bit i of the result = (the six-plane number of image i) >= t
__device__ __forceinline__ unsigned int planes_ge(const unsigned int (&p)[6], int t) {
    unsigned int gt = 0u, eq = 0xffffffffu;
#pragma unroll
    for (int q = 5; q >= 0; --q) {
        if ((t >> q) & 1) eq &= p[q];
        else { gt |= eq & p[q]; eq &= ~p[q]; }
    }
    return t > 63 ? 0u : (gt | eq);
}

__global__ void __launch_bounds__(kBitsMaxThreads, 1) count_kernel(const ResArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ unsigned int s_or[3];
    __shared__ int s_nev, s_ev_layer[32], s_ev_cnt[32];
    __shared__ float s_tab[64];                  // output of the current layer for every count 0 .. K
    if (a.gate != nullptr && *a.gate != a.gate_want) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const LoopCtl ctl = *a.ctl_in;
    const int live_in = ctl.live;
    const int tile = blockIdx.x;
    if (tile >= ((live_in + 31) >> 5)) return;
    unsigned int *wc = reinterpret_cast<unsigned int *>(smem), *wn = wc + a.wwords;

    // ---- the tile's input: one word per value id, read through the work list
    const int j = tile * 32 + lane;
    const bool valid = j < live_in;
    const int jj = valid ? j : tile * 32;
    const int src = ctl.identity ? jj : __ldg(a.slot + jj);
    if (!ctl.identity && warp == 0 && valid) move_id(ctl, a.ids0, a.ids1, j, src);
    const float *__restrict__ p = a.yin + (size_t)(src >> 5) * a.tile_stride + (src & 31);
    const ResLayer L0 = a.layers[0];
    bool ns_in = false;
    for (int v0 = warp * 8; v0 < L0.v_in; v0 += nwarps * 8) {
        int e[8];
        float x[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int v = min(v0 + q, L0.v_in - 1);
            e[q] = L0.rep ? __ldg(L0.rep + v) : v * 32;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) x[q] = valid ? __ldg(p + e[q]) : 0.0f;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const unsigned int w = __ballot_sync(0xffffffffu, x[q] != 0.0f);
            ns_in |= (x[q] != 0.0f && x[q] != a.clip);
            if (lane == 0 && v0 + q < L0.v_in) wc[resident_phys_row(v0 + q)] = w;
        }
    }
    // every word past the value ids is zero in both buffers: padded table entries point at the first even row behind them
    for (int r = L0.v_in + tid; r < a.wwords; r += blockDim.x) wc[(r < ((L0.v_in + 1) & ~1)) ? resident_phys_row(r) : r] = 0u;
    for (int r = tid; r < a.wwords; r += blockDim.x) wn[r] = 0u;
    if (tid == 0) {
        s_or[0] = 0u;
        s_nev = 0;
    }
    if (__syncthreads_or(ns_in ? 1 : 0)) {
        if (tid == 0) a.tile_done[tile] = 0;
        return;
    }

    unsigned int alive = __ballot_sync(0xffffffffu, valid);
    const bool force_dead = a.bias > 0.0f;
    unsigned int ns = 0u;
    int li = 0, last_classes = 0;
    bool unsat = false;
    int tab_k = -1, sat_lo = 0, zero_hi = 0;
    float tab_w = 0.0f;
    while (li < a.nlayers) {
        const ResLayer RL = a.layers[li];
        const int classes = RL.classes, k = RL.k;
        if (k != tab_k || RL.w != tab_w) {
            // the layer's output for every count of clip-valued inputs, by the float form's instructions
            __syncthreads();
            if (tid <= k && tid < 64) {
                float sum = 0.0f;
                for (int q = 0; q < tid; ++q) sum = __fadd_rn(sum, a.clip);
                s_tab[tid] = finish_output(__fmul_rn(sum, RL.w), a.bias, a.clip);
            }
            __syncthreads();
            int zeros = 0, sats = 0;
            bool shaped = true;
            for (int q = 0; q <= k; ++q) {
                const float f = s_tab[q];
                if (f == 0.0f) { ++zeros; shaped &= (q == zeros - 1); }          // zeros first
                if (f == a.clip) ++sats;
                else shaped &= (sats == 0);                                       // clip last
            }
            zero_hi = zeros - 1;
            sat_lo = k + 1 - sats;
            tab_k = k; tab_w = RL.w;
            if (!shaped) { unsat = true; break; }         // not a step function of the count: leave it to the float form
        }
        const unsigned int keep = force_dead ? alive : 0xffffffffu;
        const int passes = (classes + 31) >> 5;
        const int kp = k + 4;
        const int32_t *__restrict__ tb = RL.blob + 4;
        unsigned int o = 0u;
        for (int ps = warp; ps < passes; ps += nwarps) {
            const int u = ps * 32 + lane;
            const bool in = u < classes;
            const int4 *rows = reinterpret_cast<const int4 *>(tb + (size_t)(in ? u : 0) * kp);
            unsigned int pl[6] = {0u, 0u, 0u, 0u, 0u, 0u};       // ones, twos, fours, eights, sixteens, thirty-twos
            unsigned int s16[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                unsigned int e8[2];
#pragma unroll
                for (int quarter = 0; quarter < 2; ++quarter) {
                    const int4 r0 = __ldg(rows + half * 4 + quarter * 2), r1 = __ldg(rows + half * 4 + quarter * 2 + 1);
                    const unsigned int w0 = wc[r0.x], w1 = wc[r0.y], w2 = wc[r0.z], w3 = wc[r0.w];
                    const unsigned int w4 = wc[r1.x], w5 = wc[r1.y], w6 = wc[r1.z], w7 = wc[r1.w];
                    unsigned int t2a, t2b, f4a, f4b;
                    csa(t2a, pl[0], pl[0], w0, w1);
                    csa(t2b, pl[0], pl[0], w2, w3);
                    csa(f4a, pl[1], pl[1], t2a, t2b);
                    csa(t2a, pl[0], pl[0], w4, w5);
                    csa(t2b, pl[0], pl[0], w6, w7);
                    csa(f4b, pl[1], pl[1], t2a, t2b);
                    csa(e8[quarter], pl[2], pl[2], f4a, f4b);
                }
                csa(s16[half], pl[3], pl[3], e8[0], e8[1]);
            }
            csa(pl[5], pl[4], pl[4], s16[0], s16[1]);
            const unsigned int x = planes_ge(pl, sat_lo) & keep;
            const unsigned int nz = planes_ge(pl, zero_hi + 1) & keep;
            if (in) {
                ns |= nz & ~x;
                wn[resident_phys_row(u)] = x;
                o |= x;
            }
        }
        {
            // zero rows of the buffer just written (the next layer's padded entries point there; the buffer may
            // hold outputs of a wider layer from two layers ago)
            const int ue = (classes + 1) & ~1;
            for (int r = classes + tid; r < ue + 2; r += blockDim.x) wn[r < ue ? resident_phys_row(r) : r] = 0u;
        }
        o = __reduce_or_sync(0xffffffffu, o);
        if (lane == 0 && o) atomicOr(&s_or[li % 3], o);
        if (tid == 0) s_or[(li + 1) % 3] = 0u;
        __syncthreads();
        const unsigned int now = s_or[li % 3] & alive;
        if (now != alive && tid == 0) {
            s_ev_layer[s_nev] = li;
            s_ev_cnt[s_nev] = __popc(alive & ~now);
            ++s_nev;
        }
        alive = now;
        unsigned int *t = wc; wc = wn; wn = t;
        last_classes = classes;
        ++li;
        if ((li % kBitsCheckEvery) == 0 || li == a.nlayers || alive == 0u) {
            if (__syncthreads_or(ns != 0u ? 1 : 0)) { unsat = true; break; }
        }
        if (alive == 0u) break;
    }
    if (unsat) {
        if (tid == 0) a.tile_done[tile] = 0;
        return;
    }
    if (tid == 0) {
        a.tile_done[tile] = 1;
        for (int q = 0; q < s_nev; ++q) atomicAdd(a.died_at + s_ev_layer[q], s_ev_cnt[q]);
        if (alive) atomicOr(a.mask + tile, alive);
    }
    if (alive == 0u) return;
    const ResLayer LL = a.layers[li - 1];
    float *out = a.yout + (size_t)tile * a.tile_stride + lane;
    for (int u = warp; u < last_classes; u += nwarps) {
        const float y = ((wc[resident_phys_row(u)] >> lane) & 1u) ? a.clip : 0.0f;
        if (LL.mem_ptr == nullptr) {
            out[(size_t)u * 32] = y;
        } else {
            const int mb = __ldg(LL.mem_ptr + u), me = a.reps_only ? mb + 1 : __ldg(LL.mem_ptr + u + 1);
            for (int m = mb; m < me; ++m) out[__ldg(LL.mem + m)] = y;
        }
    }
}

}  // namespace spdnn_impl
