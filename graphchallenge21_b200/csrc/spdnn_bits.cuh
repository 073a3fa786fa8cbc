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

// Dynamic shared memory: two word buffers of a.wwords words (a multiple of 64, at least the largest
// v_in / classes of the chunk), then (STAGED) a.tring buffers of (stream_stride << tgroup_shift) bytes.
template <bool STAGED>
__global__ void __launch_bounds__(kBitsMaxThreads, 1) bits_kernel(const ResArgs a) {
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
    while (li < a.nlayers) {
        if (STAGED && (li >> gshift) != waited_group) {
            if (tid == 0) issue_groups(li);
            const int g = li >> gshift;
            const bool arrived = mbar_wait(&s_bar[g & (tring - 1)], (unsigned int)((g >> tshift) & 1));
            if (!__syncthreads_and(arrived ? 1 : 0)) { failed = true; break; }
            waited_group = g;
        }
        const unsigned char *T = STAGED ? tbl0 + (size_t)((li >> gshift) & (tring - 1)) * group_bytes + (size_t)(li & gmask) * stride
                                        : a.stream + (size_t)li * stride;
        const int4 hdr = STAGED ? *reinterpret_cast<const int4 *>(T) : __ldg(reinterpret_cast<const int4 *>(T));
        const int classes = hdr.x;
        if ((unsigned int)hdr.w != tt_cur) {
            tt_cur = (unsigned int)hdr.w;
            tm = truth_masks(tt_cur);
        }
        const unsigned int keep = force_dead ? alive : 0xffffffffu;
        const int passes = (classes + 63) >> 6;
        unsigned int o = 0u;
        const unsigned char *wcb = reinterpret_cast<const unsigned char *>(wc);
        for (int ps = warp; ps < passes; ps += nwarps) {
            const uint2 *slot = reinterpret_cast<const uint2 *>(T + 16 + ps * 256) + lane;
            const uint2 e = STAGED ? *slot : __ldg(slot);
            const unsigned int a1 = *reinterpret_cast<const unsigned int *>(wcb + (e.x & 0xffffu));
            const unsigned int b1 = *reinterpret_cast<const unsigned int *>(wcb + (e.x >> 16));
            const unsigned int a2 = *reinterpret_cast<const unsigned int *>(wcb + (e.y & 0xffffu));
            const unsigned int b2 = *reinterpret_cast<const unsigned int *>(wcb + (e.y >> 16));
            const bool in1 = ps * 64 + lane < classes, in2 = ps * 64 + 32 + lane < classes;   // a slot past the classes does not count
            const unsigned int x1 = select4(a1, b1, tm.hi) & keep, x2 = select4(a2, b2, tm.hi) & keep;
            ns |= ((in1 ? select4(a1, b1, tm.ns) : 0u) | (in2 ? select4(a2, b2, tm.ns) : 0u)) & keep;
            wn[ps * 64 + lane] = x1;
            wn[ps * 64 + 32 + lane] = x2;
            o |= (in1 ? x1 : 0u) | (in2 ? x2 : 0u);
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
        if ((li % kBitsCheckEvery) == 0 || li == a.nlayers || alive == 0u) {
            if (__syncthreads_or(ns != 0u ? 1 : 0)) { unsat = true; break; }
        }
        if (alive == 0u) break;
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
    for (int u = warp; u < last_classes; u += nwarps) {
        const float y = ((wc[u] >> lane) & 1u) ? a.clip : 0.0f;
        if (LL.mem_ptr == nullptr) {
            out[(size_t)u * 32] = y;
        } else {
            const int mb = __ldg(LL.mem_ptr + u), me = a.reps_only ? mb + 1 : __ldg(LL.mem_ptr + u + 1);
            for (int m = mb; m < me; ++m) out[__ldg(LL.mem + m)] = y;
        }
    }
}

}  // namespace spdnn_impl
