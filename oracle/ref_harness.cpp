// Harness around the REFERENCE's own CPU checkers, compiled against the reference's
// headers where they lie (see build.py: -I<reference>/src).  TEST INFRASTRUCTURE ONLY.
//
// It feeds a case file written by oracle/make_case.py to
//   ftxj::CpuSpmm::run_and_cmp      (src/utils/cpu_spmm.h:11-55)   one layer, raw product
//   ftxj::CpuSpmmFuse::run_and_cmp  (src/utils/cpu_spmm_fuse.h:11-95) chained layers + clip
// which recompute the layer(s) with the reference's loop nest and abort (assert_msg,
// src/utils/debug.h:5-22) when a value differs from the supplied one by more than 1e-3.
// A clean exit therefore means "the oracle's numbers agree with the reference's CPU
// implementation to the reference's own tolerance".  Mode `time` runs the same loop nest
// on image slices in host threads and reports the wall time, which is the reference's CPU
// path as timed by the benchmark.
//
// Case file (little endian): char magic[8]="SPDNNC01"; int32 N,B,L; float bias;
// float input[B*N]; then per layer: int32 nnz; int32 a[nnz] (input neuron, 1-based);
// int32 b[nnz] (output neuron, 1-based); float v[nnz]; float raw[B*N]; float act[B*N].
#include "utils/header.h"

#include <chrono>
#include <cstdio>
#include <cstring>
#include <sstream>
#include <thread>

using namespace ftxj;

struct Layer {
    std::vector<int> a, b;
    std::vector<float> v, raw, act;
};
struct Case {
    int n = 0, batch = 0, layers = 0;
    float bias = 0;
    std::vector<float> input;
    std::vector<Layer> layer;
};

// Discards everything and keeps no state, so concurrent writers cannot race on it.
struct NullBuf : std::streambuf {
    int overflow(int ch) override { return ch; }
    std::streamsize xsputn(const char *, std::streamsize n) override { return n; }
};

static bool read_exact(FILE *f, void *p, size_t bytes) { return fread(p, 1, bytes, f) == bytes; }

static bool load_case(const char *path, Case &c) {
    FILE *f = fopen(path, "rb");
    if (!f) return false;
    char magic[8];
    bool ok = read_exact(f, magic, 8) && !memcmp(magic, "SPDNNC01", 8) && read_exact(f, &c.n, 4) &&
              read_exact(f, &c.batch, 4) && read_exact(f, &c.layers, 4) && read_exact(f, &c.bias, 4);
    if (ok) {
        size_t bn = (size_t)c.batch * c.n;
        c.input.resize(bn);
        ok = read_exact(f, c.input.data(), bn * 4);
        c.layer.resize(c.layers);
        for (int l = 0; ok && l < c.layers; ++l) {
            Layer &L = c.layer[l];
            int nnz = 0;
            ok = read_exact(f, &nnz, 4);
            if (!ok) break;
            L.a.resize(nnz); L.b.resize(nnz); L.v.resize(nnz); L.raw.resize(bn); L.act.resize(bn);
            ok = read_exact(f, L.a.data(), (size_t)nnz * 4) && read_exact(f, L.b.data(), (size_t)nnz * 4) &&
                 read_exact(f, L.v.data(), (size_t)nnz * 4) && read_exact(f, L.raw.data(), bn * 4) &&
                 read_exact(f, L.act.data(), bn * 4);
        }
    }
    fclose(f);
    return ok;
}

// The reference's loader stores file line `a b v` as Elm{row = b-1, col = a-1}
// (src/utils/matrix.h:273-277, T == false); add_edge builds the same element list.
static COOMatrix make_coo(const Layer &L) {
    COOMatrix coo;
    for (size_t i = 0; i < L.a.size(); ++i) coo.add_edge(L.b[i] - 1, L.a[i] - 1, L.v[i]);
    return coo;
}

int main(int argc, char **argv) {
    if (argc < 3) {
        fprintf(stderr, "usage: %s verify|fuse|time <case file> [tsv dir | threads [repetitions]]\n", argv[0]);
        return 2;
    }
    std::string mode = argv[1];
    Case c;
    if (!load_case(argv[2], c)) {
        fprintf(stderr, "cannot read case file %s\n", argv[2]);
        return 2;
    }
    if (mode == "verify") {
        // optional argv[3]: directory holding n{N}-l{k}.tsv, read by the reference's own loader
        for (int l = 0; l < c.layers; ++l) {
            const float *in = l == 0 ? c.input.data() : c.layer[l - 1].act.data();
            if (argc > 3) {
                std::ostringstream p;
                p << argv[3] << "/n" << c.n << "-l" << (l + 1) << ".tsv";
                COOMatrix coo(p.str(), 1, false);
                CpuSpmm::run_and_cmp(coo, const_cast<float *>(in), c.n, c.batch, c.layer[l].raw.data(), false, true, true);
            } else {
                COOMatrix coo = make_coo(c.layer[l]);
                CpuSpmm::run_and_cmp(coo, const_cast<float *>(in), c.n, c.batch, c.layer[l].raw.data(), false, true, true);
            }
        }
        printf("REF_VERIFY_OK layers=%d batch=%d neurons=%d\n", c.layers, c.batch, c.n);
        return 0;
    }
    if (mode == "fuse") {
        // CpuSpmmFuse takes an INT bias (src/utils/cpu_spmm_fuse.h:11): the case must have
        // been produced with bias == (int)bias.
        std::vector<COOMatrix> w;
        for (int l = 0; l < c.layers; ++l) w.push_back(make_coo(c.layer[l]));
        CpuSpmmFuse::run_and_cmp(w, c.input.data(), c.n, c.batch, (int)c.bias, c.layer[c.layers - 1].act.data(),
                                 c.layers, false, true, true);
        printf("REF_FUSE_OK layers=%d batch=%d neurons=%d bias=%d\n", c.layers, c.batch, c.n, (int)c.bias);
        return 0;
    }
    if (mode == "time") {
        int threads = argc > 3 ? atoi(argv[3]) : (int)std::thread::hardware_concurrency();
        if (threads < 1) threads = 1;
        if (threads > c.batch) threads = c.batch;
        int reps = argc > 4 ? atoi(argv[4]) : 1;
        if (reps < 1) reps = 1;
        std::vector<COOMatrix> w;
        for (int l = 0; l < c.layers; ++l) {
            w.push_back(make_coo(c.layer[l]));
            w.back().to_row_first_ordered();   // sorted once: later calls only read it
        }
        NullBuf sink;                                          // the checker prints per call
        std::streambuf *old = std::cout.rdbuf(&sink);
        auto t0 = std::chrono::steady_clock::now();
        for (int rep = 0; rep < reps; ++rep)
        for (int l = 0; l < c.layers; ++l) {
            const float *in = l == 0 ? c.input.data() : c.layer[l - 1].act.data();
            std::vector<std::thread> pool;
            for (int t = 0; t < threads; ++t) {
                int lo = (int)((long)c.batch * t / threads), hi = (int)((long)c.batch * (t + 1) / threads);
                pool.emplace_back([&, lo, hi, in, l] {
                    CpuSpmm::run_and_cmp(w[l], const_cast<float *>(in) + (size_t)lo * c.n, c.n, hi - lo,
                                         c.layer[l].raw.data() + (size_t)lo * c.n, false, true, true);
                });
            }
            for (auto &th : pool) th.join();
        }
        double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        std::cout.rdbuf(old);
        double edges = (double)c.batch * c.n * 32.0 * c.layers * reps;
        printf("{\"seconds\": %.6f, \"threads\": %d, \"batch\": %d, \"neurons\": %d, \"layers\": %d, \"repetitions\": %d, \"edges_per_s\": %.6e}\n",
               s, threads, c.batch, c.n, c.layers, reps, edges / s);
        return 0;
    }
    fprintf(stderr, "unknown mode %s\n", mode.c_str());
    return 2;
}
