// Loaders for the reference's text formats, shared by the drivers.
//   weight layer  "../data/neuron{N}/n{N}-l{k}.tsv": lines `a b v`, 1-based, W[a][b] = v with a the input
//                 and b the output neuron (src/utils/matrix.h:255-282, T == false; path src/network.cpp:14-19)
//   inputs        "../data/sparse-images-{N}.tsv": lines `img neuron val`, 1-based, only img <= batch kept
//                 (src/network.cpp:33-54)
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

namespace drivers {

struct Triplets {
    std::vector<int32_t> a, b;
    std::vector<float> v;
};

inline std::string data_dir() {
    const char *e = getenv("SPDNN_DATA_DIR");
    return e ? std::string(e) : std::string("../data");
}

inline std::string weight_file_name(int neuron, int layer) {
    const std::string n = std::to_string(neuron);
    return data_dir() + "/neuron" + n + "/n" + n + "-l" + std::to_string(layer + 1) + ".tsv";
}

inline std::string input_file_name(int neuron) { return data_dir() + "/sparse-images-" + std::to_string(neuron) + ".tsv"; }

// Whole-file read and a hand-rolled scan: the files hold millions of short lines.
inline bool read_triplets(const std::string &path, Triplets &t, int keep_a_upto = 0) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END);
    const long size = ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<char> buf((size_t)size + 1);
    const size_t got = fread(buf.data(), 1, (size_t)size, f);
    fclose(f);
    buf[got] = 0;
    char *p = buf.data(), *end = buf.data() + got;
    while (p < end) {
        char *q;
        const long a = strtol(p, &q, 10);
        if (q == p) break;
        p = q;
        const long b = strtol(p, &q, 10);
        if (q == p) break;
        p = q;
        const float v = strtof(p, &q);
        if (q == p) break;
        p = q;
        if (keep_a_upto > 0 && a > keep_a_upto) continue;
        t.a.push_back((int32_t)a);
        t.b.push_back((int32_t)b);
        t.v.push_back(v);
    }
    return true;
}

inline float bias_for(int neuron) {          // src/network.cpp:73-78
    switch (neuron) {
        case 65536: return -0.45f;
        case 16384: return -0.4f;
        case 4096: return -0.35f;
        default: return -0.3f;
    }
}

}  // namespace drivers
