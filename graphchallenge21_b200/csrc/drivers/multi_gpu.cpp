// Multi-GPU driver with the reference's command line (src/multi_gpu.cpp:57-155):
//     multi_gpu <neuron> <batch> <layer>
// The reference starts one MPI rank per GPU; every rank reads all data, runs a contiguous slice of the images
// on its GPU and prints its own survivor count, with no exchange at all (multi_gpu.cpp:146-154,
// multi_gpu.cu:251-258).  Here one process drives all visible GPUs (SPDNN_GPUS limits the number) with one host
// thread and one context per GPU, weights replicated, nothing exchanged inside the layer loop, and the
// per-GPU category lists are concatenated at the end (slices are contiguous, so the result is ascending).
#include <algorithm>
#include <cstdio>
#include <iostream>
#include <mutex>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "spdnn_b200.h"
#include "tsv_loader.h"

int main(int argc, char *argv[]) {
    if (argc != 4) {
        std::cout << "Usage: exe neuron batch layer" << std::endl;
        return 0;
    }
    const int neuron = atoi(argv[1]), batch = atoi(argv[2]), layer = atoi(argv[3]);
    int gpus = 0;
    if (cudaGetDeviceCount(&gpus) != cudaSuccess || gpus < 1) {
        std::cerr << "no CUDA device" << std::endl;
        return 1;
    }
    if (const char *e = getenv("SPDNN_GPUS")) gpus = std::max(1, std::min(gpus, atoi(e)));
    printf("task_count = %d\n", gpus);
    drivers::Triplets in;
    if (!drivers::read_triplets(drivers::input_file_name(neuron), in, batch)) {
        std::cout << "FILE:" << drivers::input_file_name(neuron) << " does not exists.\n";
        return 1;
    }
    std::vector<drivers::Triplets> w(layer);
    for (int l = 0; l < layer; ++l)
        if (!drivers::read_triplets(drivers::weight_file_name(neuron, l), w[l])) {
            std::cout << "File:" << drivers::weight_file_name(neuron, l) << " does not exists.\n";
            return 1;
        }
    const int per = (batch + gpus - 1) / gpus;      // the reference hard-wires (batch + 1) / 2 for two ranks
    std::vector<std::vector<int32_t>> cats(gpus);
    std::vector<float> ms(gpus, 0.0f);
    std::vector<int> rc(gpus, 0);
    std::mutex io;
    auto worker = [&](int g) {
        const int lo = std::min(g * per, batch), hi = std::min(lo + per, batch);
        auto say = [&](const std::string &s) { std::lock_guard<std::mutex> k(io); std::cout << "GPU[" << g << "] " << s << std::endl; };
        say("[BEGIN]...");
        spdnn_t *ctx = nullptr;
        auto fail = [&](const char *what) { say(std::string(what) + ": " + spdnn_last_error(ctx)); spdnn_destroy(ctx); rc[g] = 1; };
        if (spdnn_create(&ctx, g, neuron, layer, drivers::bias_for(neuron), 32.0f)) return fail("create");
        for (int l = 0; l < layer; ++l)
            if (spdnn_set_layer_coo(ctx, l, (int64_t)w[l].a.size(), w[l].a.data(), w[l].b.data(), w[l].v.data(), 1)) return fail("set_layer");
        drivers::Triplets mine;
        for (size_t i = 0; i < in.a.size(); ++i)
            if (in.a[i] > lo && in.a[i] <= hi) { mine.a.push_back(in.a[i] - lo); mine.b.push_back(in.b[i]); mine.v.push_back(in.v[i]); }
        if (spdnn_set_input_coo(ctx, (int64_t)mine.a.size(), mine.a.data(), mine.b.data(), mine.v.data(), hi - lo, lo, 1)) return fail("set_input");
        spdnn_stats_t st;
        if (spdnn_infer(ctx, &st)) return fail("infer");
        std::vector<int32_t> live(layer);
        spdnn_get_layer_live(ctx, live.data(), layer);
        for (int l = 0; l < layer; l += 100)      // multi_gpu.cu:517-518
            say("[GPU " + std::to_string(g) + "], Layer " + std::to_string(l) + ", Batch = " + std::to_string(live[l]));
        cats[g].resize(std::max(hi - lo, 1));
        int count = 0;
        if (spdnn_get_categories(ctx, cats[g].data(), (int)cats[g].size(), &count)) return fail("categories");
        cats[g].resize(count);
        ms[g] = st.infer_ms;
        say("Kernel Exec Time = " + std::to_string(st.infer_ms) + "ms, survivors = " + std::to_string(count));
        spdnn_destroy(ctx);
        say("[END]...");
    };
    std::vector<std::thread> pool;
    for (int g = 0; g < gpus; ++g) pool.emplace_back(worker, g);
    for (auto &t : pool) t.join();
    for (int g = 0; g < gpus; ++g)
        if (rc[g]) return 1;
    const std::string out = "neuron" + std::to_string(neuron) + "-l" + std::to_string(layer) + "-categories.tsv";
    size_t total = 0;
    if (FILE *f = fopen(out.c_str(), "w")) {
        for (int g = 0; g < gpus; ++g)
            for (int32_t id : cats[g]) { fprintf(f, "%d\n", id + 1); ++total; }
        fclose(f);
    }
    std::cout << "categories = " << total << " -> " << out << ", max kernel time = " << *std::max_element(ms.begin(), ms.end())
              << "ms" << std::endl;
    return 0;
}
