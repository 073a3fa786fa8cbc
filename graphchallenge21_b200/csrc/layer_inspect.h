// Host-side preparation of the weight layers for the sm_100a kernels.
//
// Takes the role of the reference's per-layer inspector pass (src/network.cpp:97-121:
// COOMatrix -> reorder -> CSRCSCMatrix -> BlockContainer -> MaxInReuseBSchedule::get_data,
// src/inspector/gpu_block_scheduler.h:160-171) but makes no assumption on the pattern: any CSC
// goes in.  What it derives:
//   * per column the input rows in ascending order (the summation order of the reference's CPU
//     loop, src/utils/cpu_spmm.h:12-43), padded to a common K that is a multiple of 4;
//   * column classes: columns with identical (rows, weights) produce identical outputs, so each
//     class is computed once.  The challenge networks have 16 such columns per class (the
//     16-wide blocks the reference's n16384_l11_kernel shares its gathered rows over,
//     all_network.cu:134-149);
//   * value ids across layers: the members of one class of layer l-1 hold the same value for
//     every image, so layer l can read ONE stored value per class of layer l-1 instead of one
//     row per neuron.  Expressed in value ids, even more columns of layer l may coincide, and
//     the activations between two layers shrink from N rows to one row per class;
//   * whether all weights are one power-of-two constant w: then sum(y*w) == w*sum(y) bit for bit
//     in fp32 (scaling by 2^e commutes with rounding), and the kernels add first.
// None of this changes a result bit: every output is still the sum of its K terms in ascending
// input-neuron order.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

namespace spdnn_impl {

inline uint64_t mix64(uint64_t x) {
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

inline bool is_pow2_float(float w) {
    if (!(w > 0.0f) || !std::isfinite(w)) return false;
    int e;
    return std::frexp(w, &e) == 0.5f;
}

// Row permutation of the resident kernel's shared-memory buffers: the low bit is flipped by the
// parity of the upper bits (a bijection on [0, 2m)), which spreads rows of equal parity over
// both halves of the shared-memory banks.
inline int phys_row(int r) {
    int x = r >> 1;
    x ^= x >> 16; x ^= x >> 8; x ^= x >> 4; x ^= x >> 2; x ^= x >> 1;
    return r ^ (x & 1);
}

// One layer in canonical form, kept on the host.
struct HostLayer {
    int n = 0;                     // neurons
    int k = 0;                     // entries per column, padded to a multiple of 4
    bool uniform = false;          // all weights == w, w a power of two
    float w = 0.0f;
    int64_t nnz = 0;
    std::vector<int32_t> rows;     // [n][k] ascending input neuron per output neuron; padding = n
    std::vector<float> vals;       // [n][k]; padding 0
    uint64_t hash1 = 0, hash2 = 0; // content hashes (128 bits together)
};

// Returns an empty string on success, else the reason the layer is rejected.
inline std::string canonicalize_layer(int n, const int32_t *col_ptr, const int32_t *row_idx, const float *val, HostLayer &out) {
    if (n <= 0 || n > (1 << 26)) return "neurons must be in [1, 2^26]";
    if (!col_ptr || !row_idx) return "col_ptr/row_idx is null";
    if (col_ptr[0] != 0) return "col_ptr[0] must be 0";
    int kmax = 0;
    for (int c = 0; c < n; ++c) {
        const int64_t cnt = (int64_t)col_ptr[c + 1] - col_ptr[c];
        if (cnt < 0) return "col_ptr must be non-decreasing";
        if (cnt > 4096) return "more than 4096 non-zeros in one column is not supported";
        kmax = std::max<int>(kmax, (int)cnt);
    }
    const int64_t nnz = col_ptr[n];
    const int k = std::max(4, (kmax + 3) / 4 * 4);
    const float w0 = val ? (nnz ? val[0] : 0.0625f) : 0.0625f;
    bool uniform = is_pow2_float(w0);
    out = HostLayer();
    out.n = n; out.k = k; out.nnz = nnz; out.w = w0;
    // ascending row, stable for equal rows (repeated entries stay separate terms, as a COO with
    // repeated triplets would be summed)
    out.rows.assign((size_t)n * k, n);
    out.vals.assign((size_t)n * k, 0.0f);
    std::vector<std::pair<int32_t, float>> tmp;
    uint64_t h1 = mix64(0x5EEDull ^ (uint64_t)n ^ ((uint64_t)k << 32));
    uint64_t h2 = mix64(0xC0FFEEull + (uint64_t)n * 31 + (uint64_t)k);
    for (int c = 0; c < n; ++c) {
        const int s = col_ptr[c], e = col_ptr[c + 1];
        tmp.clear();
        for (int i = s; i < e; ++i) {
            const int32_t r = row_idx[i];
            if (r < 0 || r >= n) return "row index out of range in column " + std::to_string(c);
            const float v = val ? val[i] : 0.0625f;
            if (v != w0) uniform = false;
            tmp.emplace_back(r, v);
        }
        std::stable_sort(tmp.begin(), tmp.end(),
                         [](const std::pair<int32_t, float> &a, const std::pair<int32_t, float> &b) { return a.first < b.first; });
        uint64_t h = 0x9E3779B97F4A7C15ull;
        for (size_t i = 0; i < tmp.size(); ++i) {
            out.rows[(size_t)c * k + i] = tmp[i].first;
            out.vals[(size_t)c * k + i] = tmp[i].second;
            uint32_t vb;
            std::memcpy(&vb, &tmp[i].second, 4);
            h = mix64(h ^ (((uint64_t)(uint32_t)tmp[i].first << 32) | vb));
        }
        h1 = mix64(h1 ^ h);
        h2 = mix64(h2 + h * 0x9E3779B97F4A7C15ull + (uint64_t)c);
    }
    out.uniform = uniform;
    out.hash1 = h1; out.hash2 = h2;
    return std::string();
}

// Groups the columns of a layer whose (id sequence, weights) coincide.  ids == nullptr: the
// sequences are the raw rows.  Classes are numbered in order of their first column.
inline int group_columns(const HostLayer &h, const int32_t *ids, std::vector<int> &class_of, std::vector<int> &first_col) {
    const int n = h.n, k = h.k;
    std::unordered_map<uint64_t, std::vector<int>> by_hash;
    by_hash.reserve((size_t)n * 2);
    class_of.assign(n, 0);
    first_col.clear();
    std::vector<int32_t> seq((size_t)n * k);
    for (size_t i = 0; i < seq.size(); ++i) {
        const int32_t r = h.rows[i];
        seq[i] = (r < n && ids) ? ids[r] : r;       // padding stays n (ids are below n)
    }
    const bool has_vals = !h.vals.empty();      // a uniform layer may have dropped its weights
    for (int c = 0; c < n; ++c) {
        const int32_t *s = &seq[(size_t)c * k];
        const float *v = has_vals ? &h.vals[(size_t)c * k] : nullptr;
        uint64_t hh = 0x9E3779B97F4A7C15ull;
        for (int i = 0; i < k; ++i) {
            uint32_t vb = 0;
            if (v) std::memcpy(&vb, &v[i], 4);
            hh = mix64(hh ^ (((uint64_t)(uint32_t)s[i] << 32) | vb));
        }
        auto &cands = by_hash[hh];
        int found = -1;
        for (int cls : cands) {
            const int fc = first_col[cls];
            if (!std::memcmp(s, &seq[(size_t)fc * k], sizeof(int32_t) * k) &&
                (!v || !std::memcmp(v, &h.vals[(size_t)fc * k], sizeof(float) * k))) { found = cls; break; }
        }
        if (found < 0) {
            found = (int)first_col.size();
            first_col.push_back(c);
            cands.push_back(found);
        }
        class_of[c] = found;
    }
    return (int)first_col.size();
}

// ---- tables of the per-layer kernel (activations stored as N rows per image) -------------------
struct PerLayerTables {
    int classes = 0;
    bool identity_members = false;      // class u == column u (no two columns alike)
    std::vector<int32_t> off;           // [U][k] input row * 32 (element offset inside a tile); padding -> row n (always zero)
    std::vector<float> vals;            // [U][k] (empty when uniform)
    std::vector<int32_t> mem_ptr;       // [U+1]
    std::vector<int32_t> mem;           // member column * 32, ascending inside a class
};

inline void build_per_layer_tables(const HostLayer &h, PerLayerTables &out) {
    const int n = h.n, k = h.k;
    std::vector<int> class_of, first_col;
    const int u = group_columns(h, nullptr, class_of, first_col);

    // Order of the classes in device memory.  Where columns repeat (u well below n) classes are
    // chained greedily so that each is followed by the unvisited class sharing most input rows
    // with it: a warp that walks a run of such classes re-reads the shared rows while they are
    // still in L1.  Without repeats every row is shared by ~k unrelated classes and the order of
    // first appearance is kept.
    std::vector<int> order;
    order.reserve(u);
    if (u <= n / 2) {
        std::vector<int> rp((size_t)n + 2, 0);
        for (int cls = 0; cls < u; ++cls)
            for (int i = 0; i < k; ++i) {
                const int r = h.rows[(size_t)first_col[cls] * k + i];
                if (r < n) rp[r + 2]++;
            }
        for (int r = 0; r < n; ++r) rp[r + 2] += rp[r + 1];
        std::vector<int> rc((size_t)rp[n + 1]);
        for (int cls = 0; cls < u; ++cls)
            for (int i = 0; i < k; ++i) {
                const int r = h.rows[(size_t)first_col[cls] * k + i];
                if (r < n) rc[rp[r + 1]++] = cls;
            }
        // rp[r] .. rp[r+1] now delimits the classes that read row r
        std::vector<char> visited(u, 0);
        std::vector<int> cnt(u, 0), touched;
        for (int start = 0; start < u; ++start) {
            if (visited[start]) continue;
            int cur = start;
            for (;;) {
                visited[cur] = 1;
                order.push_back(cur);
                touched.clear();
                for (int i = 0; i < k; ++i) {
                    const int r = h.rows[(size_t)first_col[cur] * k + i];
                    if (r >= n) continue;
                    for (int q = rp[r]; q < rp[r + 1]; ++q) {
                        const int other = rc[q];
                        if (!visited[other] && cnt[other]++ == 0) touched.push_back(other);
                    }
                }
                int best = -1, best_cnt = 0;
                for (int t : touched) {
                    if (cnt[t] > best_cnt || (cnt[t] == best_cnt && t < best)) { best = t; best_cnt = cnt[t]; }
                    cnt[t] = 0;
                }
                if (best < 0 || best_cnt * 4 < k) break;
                cur = best;
            }
        }
    } else {
        for (int cls = 0; cls < u; ++cls) order.push_back(cls);
    }
    std::vector<int> new_id(u);
    for (int pos = 0; pos < u; ++pos) new_id[order[pos]] = pos;

    out = PerLayerTables();
    out.classes = u;
    out.identity_members = (u == n);
    out.off.resize((size_t)u * k);
    if (!h.uniform) out.vals.resize((size_t)u * k);
    for (int pos = 0; pos < u; ++pos) {
        const int fc = first_col[order[pos]];
        for (int i = 0; i < k; ++i) {
            out.off[(size_t)pos * k + i] = h.rows[(size_t)fc * k + i] * 32;
            if (!h.uniform) out.vals[(size_t)pos * k + i] = h.vals[(size_t)fc * k + i];
        }
    }
    out.mem_ptr.assign(u + 1, 0);
    for (int c = 0; c < n; ++c) out.mem_ptr[new_id[class_of[c]] + 1]++;
    for (int cls = 0; cls < u; ++cls) out.mem_ptr[cls + 1] += out.mem_ptr[cls];
    out.mem.resize(n);
    std::vector<int32_t> fill(out.mem_ptr.begin(), out.mem_ptr.end() - 1);
    for (int c = 0; c < n; ++c) out.mem[fill[new_id[class_of[c]]]++] = c * 32;
}

// ---- tables of the resident kernel (activations stored as one row per value id) ------------------
enum ResidentMode { RES_GENERIC = 0, RES_ALT2 = 1 };

struct ResidentTables {
    int classes = 0;                // U: rows of the output buffer (class u writes row u)
    int v_in = 0;                   // value ids of the input: rows of the input buffer
    int mode = RES_GENERIC;
    int o_vals = 0;                 // word offset of the weights inside the blob (0: uniform)
    // blob: a 4-word header {classes, k, bits of w, 0}, then, all entries being (permuted) row
    // numbers of the shared-memory buffers:
    //   RES_GENERIC: int32 t[U][k + 4]: the k input rows in summation order, then {output row, 0, 0, 0};
    //                followed, when the weights are not uniform, by float vals[U][k + 4]
    //   RES_ALT2:    int32 t[U][4] = {row a, row b, output row, 0 (filled on the device: truth table)}: the sum is a+b+a+b+... (k terms)
    std::vector<int32_t> blob;
    std::vector<int32_t> rep;       // [v_in] neuron * 32 holding value id v (empty: value id == neuron)
    std::vector<int32_t> mem_ptr;   // [U+1] member ranges (empty: class u == column u)
    std::vector<int32_t> mem;       // member column * 32
    std::vector<int32_t> class_of;  // [n] class of every column = value ids of the next layer's input
    uint64_t partition_hash = 0;    // of class_of
};

// vid_in: value id of every input neuron (nullptr: identity, v_in == n).
inline void build_resident_tables(const HostLayer &h, const int32_t *vid_in, int v_in, ResidentTables &out) {
    const int n = h.n, k = h.k;
    std::vector<int> class_of, first_col;
    const int u = group_columns(h, vid_in, class_of, first_col);
    out = ResidentTables();
    out.classes = u;
    out.v_in = vid_in ? v_in : n;
    const int zero_in = (out.v_in + 1) & ~1;        // first row past the permuted range of the input buffer
    auto in_row = [&](int r) { return r < n ? phys_row(vid_in ? vid_in[r] : r) : zero_in; };

    // alternating pair: k even, terms a,b,a,b,... with at most two distinct ids, uniform weight
    bool alt2 = h.uniform && (k % 2 == 0);
    for (int cls = 0; cls < u && alt2; ++cls) {
        const int32_t *r = &h.rows[(size_t)first_col[cls] * k];
        if (r[k - 1] >= n) { alt2 = false; break; }            // padded column
        const int a = in_row(r[0]), b = in_row(r[1]);
        for (int i = 0; i < k; ++i)
            if (in_row(r[i]) != ((i & 1) ? b : a)) { alt2 = false; break; }
    }
    out.mode = alt2 ? RES_ALT2 : RES_GENERIC;
    constexpr size_t H = 4;      // header words
    if (alt2) {
        out.blob.assign(H + (size_t)u * 4, 0);
        for (int cls = 0; cls < u; ++cls) {
            const int32_t *r = &h.rows[(size_t)first_col[cls] * k];
            out.blob[H + (size_t)cls * 4 + 0] = in_row(r[0]);
            out.blob[H + (size_t)cls * 4 + 1] = in_row(r[1]);
            out.blob[H + (size_t)cls * 4 + 2] = phys_row(cls);
        }
    } else {
        const int kp = k + 4;
        const size_t words = (size_t)u * kp;
        out.o_vals = h.uniform ? 0 : (int)(H + words);
        out.blob.assign(H + words * (h.uniform ? 1 : 2), 0);
        for (int cls = 0; cls < u; ++cls) {
            const int fc = first_col[cls];
            for (int i = 0; i < k; ++i) {
                out.blob[H + (size_t)cls * kp + i] = in_row(h.rows[(size_t)fc * k + i]);
                if (!h.uniform) std::memcpy(&out.blob[H + words + (size_t)cls * kp + i], &h.vals[(size_t)fc * k + i], 4);
            }
            out.blob[H + (size_t)cls * kp + k] = phys_row(cls);
        }
    }
    out.blob[0] = u;
    out.blob[1] = k;
    std::memcpy(&out.blob[2], &h.w, 4);
    if (vid_in) {
        out.rep.assign(out.v_in, -1);
        for (int r = 0; r < n; ++r)
            if (out.rep[vid_in[r]] < 0) out.rep[vid_in[r]] = r * 32;
        for (auto &x : out.rep)
            if (x < 0) x = 0;      // an id no neuron carries is never read
    }
    if (u < n) {
        out.mem_ptr.assign(u + 1, 0);
        for (int c = 0; c < n; ++c) out.mem_ptr[class_of[c] + 1]++;
        for (int cls = 0; cls < u; ++cls) out.mem_ptr[cls + 1] += out.mem_ptr[cls];
        out.mem.resize(n);
        std::vector<int32_t> fill(out.mem_ptr.begin(), out.mem_ptr.end() - 1);
        for (int c = 0; c < n; ++c) out.mem[fill[class_of[c]]++] = c * 32;
    }
    out.class_of.assign(class_of.begin(), class_of.end());
    uint64_t ph = mix64(0xABCDEFull + (uint64_t)u);
    for (int c = 0; c < n; ++c) ph = mix64(ph ^ ((uint64_t)(uint32_t)class_of[c] + ((uint64_t)c << 32)));
    out.partition_hash = ph;
}

}  // namespace spdnn_impl
