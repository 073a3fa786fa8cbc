// Single-GPU driver with the reference's command line and output (src/network.cpp:56-125):
//     network <neuron> <batch> <layer>
// reads ../data/sparse-images-{N}.tsv and ../data/neuron{N}/n{N}-l{1..L}.tsv (SPDNN_DATA_DIR overrides the
// directory), runs the layer loop on GPU 0 through the C ABI and prints the reference's progress lines
// ("layer l, batch = k", "Kernel Exec Time [...]", all_network.cu:508, 522-523).  In addition it writes the
// category list the reference never emitted: neuron{N}-l{L}-categories.tsv, one 1-based image number per line.
#include <algorithm>
#include <cstdio>
#include <iostream>
#include <vector>

#include "spdnn_b200.h"
#include "tsv_loader.h"

static int die(spdnn_t *ctx, const char *what) {
    std::cerr << what << ": " << spdnn_last_error(ctx) << std::endl;
    spdnn_destroy(ctx);
    return 1;
}

int main(int argc, char *argv[]) {
    if (argc != 4) {
        std::cout << "Usage: exe neuron batch layer" << std::endl;
        return 0;
    }
    const int neuron = atoi(argv[1]), batch = atoi(argv[2]), layer = atoi(argv[3]);
    std::cout << "[BEGIN]..." << std::endl;
    drivers::Triplets in;
    if (!drivers::read_triplets(drivers::input_file_name(neuron), in, batch)) {
        std::cout << "FILE:" << drivers::input_file_name(neuron) << " does not exists.\n";
        return 1;
    }
    for (size_t i = 0; i < in.v.size(); ++i)
        if (in.v[i] != 1.0f) printf("read input %d, %f\n", in.a[i], in.v[i]);
    std::cout << "Read Input success! read_numeber = " << in.a.size() << std::endl;
    std::cout << "Read Input success!" << std::endl;

    spdnn_t *ctx = nullptr;
    if (spdnn_create(&ctx, 0, neuron, layer, drivers::bias_for(neuron), 32.0f)) return die(ctx, "create");
    for (int l = 0; l < layer; ++l) {
        drivers::Triplets w;
        const std::string path = drivers::weight_file_name(neuron, l);
        if (!drivers::read_triplets(path, w)) {
            std::cout << "File:" << path << " does not exists.\n";
            spdnn_destroy(ctx);
            return 1;
        }
        std::cout << "[" << path << "] to COO success!" << std::endl;
        if (spdnn_set_layer_coo(ctx, l, (int64_t)w.a.size(), w.a.data(), w.b.data(), w.v.data(), 1)) return die(ctx, "set_layer");
    }
    if (spdnn_set_input_coo(ctx, (int64_t)in.a.size(), in.a.data(), in.b.data(), in.v.data(), batch, 0, 1))
        return die(ctx, "set_input");
    spdnn_stats_t st;
    if (spdnn_infer(ctx, &st)) return die(ctx, "infer");
    std::vector<int32_t> live(layer), cats(batch > 0 ? batch : 1);
    if (spdnn_get_layer_live(ctx, live.data(), layer)) return die(ctx, "layer_live");
    for (int l = 0; l < layer; ++l) std::cout << "layer " << l << ", batch = " << live[l] << std::endl;
    std::cout << "Kernel Exec Time [20-uiuc-row-succ] = " << st.infer_ms << "ms" << std::endl;
    // the reference's lower bound: live rows * N * 8 bytes at 700 GB/s (all_network.cu:335-340)
    std::cout << "Kernel Exec Upper Time = " << st.algorithmic_bytes / 1e9 / 700.0 * 1000.0 << "ms" << std::endl;
    int count = 0;
    if (spdnn_get_categories(ctx, cats.data(), (int)cats.size(), &count)) return die(ctx, "categories");
    const std::string out = "neuron" + std::to_string(neuron) + "-l" + std::to_string(layer) + "-categories.tsv";
    if (FILE *f = fopen(out.c_str(), "w")) {
        for (int i = 0; i < count; ++i) fprintf(f, "%d\n", cats[i] + 1);
        fclose(f);
    }
    std::cout << "categories = " << count << " -> " << out << std::endl;
    {
        // the challenge's truth categories, when they were downloaded next to the data
        // (tools/get_dataset.sh:15): 1-based image numbers, one per line
        const std::string truth = drivers::data_dir() + "/neuron" + std::to_string(neuron) + "-l" + std::to_string(layer) + "-categories.tsv";
        if (FILE *f = fopen(truth.c_str(), "r")) {
            std::vector<int32_t> want;
            double x;
            while (fscanf(f, "%lf", &x) == 1)
                if ((int)x <= batch) want.push_back((int32_t)x - 1);
            fclose(f);
            const bool same = (int)want.size() == count && std::equal(want.begin(), want.end(), cats.begin());
            std::cout << "Challenge " << (same ? "PASSED" : "FAILED") << ": " << count << " categories, truth " << want.size() << std::endl;
        }
    }
    spdnn_destroy(ctx);
    std::cout << "[END]..." << std::endl;
    return 0;
}
