// Single-layer testbed with the reference's command line (src/main.cpp:12-133):
//     main <layer> [neuron = 1024] [batch = 1024]
// reads ONE layer file, fills the input with random values in [0, 32) as the reference's kernel tests do
// (e.g. src/microbenchmark/n16384-l2-l10.cu:83-89), runs that layer once on the GPU as a plain product (bias 0,
// no clip) and checks every output against a CPU loop in the order of CpuSpmm::run_and_cmp
// (src/utils/cpu_spmm.h:14-52, abs tolerance 1e-3), printing the reference's success line.
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdio>
#include <iostream>
#include <numeric>
#include <vector>

#include "spdnn_b200.h"
#include "tsv_loader.h"

int main(int argc, char *argv[]) {
    if (argc < 2) {
        std::cout << "Usage: exe layer [neuron] [batch]" << std::endl;
        return 0;
    }
    const int layer = atoi(argv[1]);
    const int neuron = argc > 2 ? atoi(argv[2]) : 1024, batch = argc > 3 ? atoi(argv[3]) : 1024;
    drivers::Triplets w;
    const std::string path = drivers::weight_file_name(neuron, layer);
    if (!drivers::read_triplets(path, w)) {
        std::cout << "File:" << path << " does not exists.\n";
        return 1;
    }
    std::cout << "[" << path << "] to COO success!" << std::endl;
    std::vector<float> in((size_t)batch * neuron), out((size_t)batch * neuron, 0.0f);
    srand(12345);
    for (auto &x : in) x = (float)(rand() % 32);
    spdnn_t *ctx = nullptr;
    spdnn_stats_t st;
    if (spdnn_create(&ctx, 0, neuron, 1, 0.0f, FLT_MAX) ||
        spdnn_set_layer_coo(ctx, 0, (int64_t)w.a.size(), w.a.data(), w.b.data(), w.v.data(), 1) ||
        spdnn_set_input_dense(ctx, in.data(), batch, 0) || spdnn_infer(ctx, &st)) {
        std::cerr << spdnn_last_error(ctx) << std::endl;
        spdnn_destroy(ctx);
        return 1;
    }
    std::vector<int32_t> cats(batch);
    int count = 0;
    spdnn_get_categories(ctx, cats.data(), batch, &count);
    std::vector<float> act((size_t)std::max(count, 1) * neuron);
    spdnn_get_activations(ctx, act.data(), count);
    for (int i = 0; i < count; ++i)
        std::copy(act.begin() + (size_t)i * neuron, act.begin() + (size_t)(i + 1) * neuron, out.begin() + (size_t)cats[i] * neuron);
    std::cout << "Kernel Exec Time = " << st.infer_ms << "ms" << std::endl;
    // CPU check: per output, terms in ascending input order (the COO sorted by (output, input))
    std::vector<size_t> order(w.a.size());
    std::iota(order.begin(), order.end(), 0);
    std::sort(order.begin(), order.end(), [&](size_t x, size_t y) { return w.b[x] != w.b[y] ? w.b[x] < w.b[y] : w.a[x] < w.a[y]; });
    for (int b = 0; b < batch; ++b) {
        std::vector<float> res(neuron, 0.0f);
        for (size_t i : order) res[w.b[i] - 1] += in[(size_t)b * neuron + w.a[i] - 1] * w.v[i];
        for (int j = 0; j < neuron; ++j)
            if (std::abs(res[j] - out[(size_t)b * neuron + j]) > 1e-3) {
                std::cout << b << ", " << j << " cpu=" << res[j] << ", gpu=" << out[(size_t)b * neuron + j] << std::endl;
                spdnn_destroy(ctx);
                return 1;
            }
    }
    std::cout << "Compare with cpu result [Success]" << std::endl;
    spdnn_destroy(ctx);
    return 0;
}
