// Harness around the REFERENCE's own structure-agnostic GPU inference loop, compiled against the
// reference's sources where they lie (see build.py: nvcc -I<reference>/src).  TEST INFRASTRUCTURE ONLY.
//
// It feeds a network and a batch of images to
//   ftxj::test_benchmark_SNIG   (src/microbenchmark/snig.cu:124-257: the layer loop around the
//                                kernel snig_inference, :19-120)
// through the reference's own matrix type ftxj::SNIGMatrix (src/utils/matrix.h:856-974), exactly as
// the reference's driver does (src/SNIG.cpp:73-110), and lets that function print what it prints: one
// line "layer = l, batch = k, time = t" per layer (k = images that still hold a non-zero activation)
// and the total "Kernel Exec Time [SNIG] = T ms".  The Python side parses those lines: the counts
// pin the oracle's survivors against the reference's own CUDA implementation, the time is the
// reference's GPU code timed on the same device as this repository's kernels.
//
// Why this loop and not all_network.cu: read for bounds, snig_inference and its host loop index only
// inside their arrays for any network whose every INPUT neuron has exactly 32 outgoing edges and
// whose neuron count is a multiple of the section size (col_w has num_secs * N + 1 entries and is read
// up to [num_secs * N], snig.cu:89-90; the shared array has sec_size floats and is indexed by
// row - section start, :98; Y_0/Y_1 by image * N + neuron < batch * N, :85, :109).  This harness
// checks both conditions and refuses anything else.  The per-pattern kernels of all_network.cu read
// their work list past its end (all_network.cu:83-87 against :293, :510) and are not run.
//
// SNIGMatrix only reads layer files, so every DISTINCT layer is written once as a file in the
// reference's format (line "a b v": input neuron, output neuron, weight; 1-based) into a scratch directory.
//
// Case file (little endian): char magic[8]="SPDNNS01"; int32 N, B, L, K, P; float bias;
// int32 pattern_of_layer[L]; int32 rows[P][N][K] (input neurons of every output neuron, 0-based);
// uint8 bits[B][ceil(N/8)] (bit n & 7 of byte n >> 3 = image has neuron n set).  All weights 0.0625.
#include "microbenchmark/snig.cu"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

using namespace ftxj;

static bool read_exact(FILE *f, void *p, size_t bytes) { return fread(p, 1, bytes, f) == bytes; }

int main(int argc, char **argv) {
    if (argc < 3) {
        fprintf(stderr, "usage: %s <case file> <scratch dir>\n", argv[0]);
        return 2;
    }
    FILE *f = fopen(argv[1], "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", argv[1]); return 2; }
    char magic[8];
    int n = 0, batch = 0, layers = 0, k = 0, patterns = 0;
    float bias = 0;
    bool ok = read_exact(f, magic, 8) && !memcmp(magic, "SPDNNS01", 8) && read_exact(f, &n, 4) && read_exact(f, &batch, 4) &&
              read_exact(f, &layers, 4) && read_exact(f, &k, 4) && read_exact(f, &patterns, 4) && read_exact(f, &bias, 4);
    if (!ok || n <= 0 || batch <= 0 || layers <= 0 || patterns <= 0 || k != 32) { fprintf(stderr, "bad case header\n"); return 2; }
    std::vector<int> pattern_of(layers);
    std::vector<int> rows((size_t)patterns * n * k);
    std::vector<unsigned char> bits((size_t)batch * ((n + 7) / 8));
    ok = read_exact(f, pattern_of.data(), (size_t)layers * 4) && read_exact(f, rows.data(), rows.size() * 4) &&
         read_exact(f, bits.data(), bits.size());
    fclose(f);
    if (!ok) { fprintf(stderr, "short case file\n"); return 2; }

    // section size as src/SNIG.cpp:17-41 picks it: the largest N / d that fits the default shared memory
    cudaDeviceProp props;
    if (cudaGetDeviceProperties(&props, 0) != cudaSuccess) { fprintf(stderr, "no CUDA device\n"); return 3; }
    const size_t max_per_block = props.sharedMemPerBlock / sizeof(float);
    int sec_size = n;
    if ((size_t)n > max_per_block) {
        int d = 2;
        while (n % d != 0 || max_per_block < (size_t)(n / d)) ++d;
        sec_size = n / d;
    }
    if (n % sec_size != 0) { fprintf(stderr, "refused: %d neurons are not a multiple of the section size %d\n", n, sec_size); return 4; }

    // the conditions under which every index of the reference's loop stays inside its array
    for (int p = 0; p < patterns; ++p) {
        std::vector<int> out_degree(n, 0);
        for (size_t i = 0; i < (size_t)n * k; ++i) {
            const int r = rows[(size_t)p * n * k + i];
            if (r < 0 || r >= n) { fprintf(stderr, "refused: row index out of range\n"); return 4; }
            out_degree[r]++;
        }
        for (int r = 0; r < n; ++r)
            if (out_degree[r] != 32) {
                fprintf(stderr, "refused: input neuron %d of pattern %d has %d outgoing edges, the reference's format needs 32\n", r, p,
                        out_degree[r]);
                return 4;
            }
    }

    std::vector<SNIGMatrix> distinct;
    for (int p = 0; p < patterns; ++p) {
        const std::string path = std::string(argv[2]) + "/snig-p" + std::to_string(p) + ".tsv";
        FILE *t = fopen(path.c_str(), "w");
        if (!t) { fprintf(stderr, "cannot write %s\n", path.c_str()); return 2; }
        for (int c = 0; c < n; ++c)
            for (int i = 0; i < k; ++i) fprintf(t, "%d\t%d\t0.0625\n", rows[((size_t)p * n + c) * k + i] + 1, c + 1);
        fclose(t);
        distinct.push_back(SNIGMatrix(path, 32 * n, sec_size, n));
    }
    std::vector<SNIGMatrix> weights;
    for (int l = 0; l < layers; ++l) {
        if (pattern_of[l] < 0 || pattern_of[l] >= patterns) { fprintf(stderr, "bad pattern index\n"); return 2; }
        weights.push_back(distinct[pattern_of[l]]);
    }
    std::vector<std::vector<float>> input(batch, std::vector<float>(n, 0.0f));
    const size_t rb = (n + 7) / 8;
    for (int b = 0; b < batch; ++b)
        for (int c = 0; c < n; ++c)
            if ((bits[(size_t)b * rb + (c >> 3)] >> (c & 7)) & 1) input[b][c] = 1.0f;

    printf("[snig harness] neurons = %d, batch = %d, layers = %d, sec_size = %d\n", n, batch, layers, sec_size);
    fflush(stdout);
    GpuEnv env(0);
    test_benchmark_SNIG(input, weights, batch, n, sec_size, 32 * n, bias, env);
    fflush(stdout);
    return 0;
}
