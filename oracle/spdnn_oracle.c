/*
 * CPU oracle (plain C + OpenMP) for the sparse-DNN inference loop
 *     Y <- min(clip, ReLU(Y W + bias)),  W: N x N, K non-zeros per column.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; the tests, the smoke check and the benchmark's CPU-baseline
 * leg use it as the checker / as the timed CPU port.
 *
 * What it restates (paths are the reference's, relative to its project root):
 *  - raw product of one layer: CpuSpmm::run_and_cmp, src/utils/cpu_spmm.h:11-43.
 *    For every image it walks the COO sorted by (output, input)
 *    (src/utils/matrix.h:245-253) doing `res[out] += in * val`, so every output
 *    accumulates its terms in ASCENDING INPUT-NEURON order from 0.0f in fp32,
 *    each product rounded before it is added.
 *  - epilogue: __ReLU(acc + bias) = x<0 ? 0 : x>32 ? 32 : x,
 *    src/microbenchmark/all_network.cu:8-10 applied at :57, :108, :147; the same
 *    chain on the CPU is src/utils/cpu_spmm_fuse.h:46,74.
 *  - survivors: an image is alive after a layer when any activation is non-zero
 *    (all_network.cu:57-59 sets active[img], :455-463 rebuilds the work list).
 *  - categories: ascending original image numbers alive after the last layer
 *    (the reference prints only the count, all_network.cu:508).
 *
 * Parity status: checked against the reference's CpuSpmm / CpuSpmmFuse compiled
 * from its own sources (oracle/build.py builds it as _ref/ref_harness); the reference holds no golden
 * vectors for this path and the challenge's truth files are unavailable, so
 * parity against the official data set is unpinned.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC (no -ffast-math).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float relu_clip(float x, float clip) {
    return x < 0.0f ? 0.0f : (x > clip ? clip : x);
}

/* One layer for one image.  rows: [N*K] (entry < 0 = padding), vals: [N*K] or NULL. */
static int layer_one_image(const float *in, float *out, int n, int k, const int32_t *rows, const float *vals,
                           float value, float bias, float clip) {
    int any = 0;
    for (int c = 0; c < n; ++c) {
        const int32_t *r = rows + (size_t)c * k;
        float acc = 0.0f;
        if (vals) {
            const float *v = vals + (size_t)c * k;
            for (int j = 0; j < k; ++j)
                if (r[j] >= 0) { float p = in[r[j]] * v[j]; acc = acc + p; }
        } else {
            for (int j = 0; j < k; ++j)
                if (r[j] >= 0) { float p = in[r[j]] * value; acc = acc + p; }
        }
        float y = relu_clip(acc + bias, clip);
        out[c] = y;
        any |= (y != 0.0f);
    }
    return any;
}

/*
 * Full inference.  rows[l] / vals[l] describe layer l (vals == NULL or vals[l] == NULL
 * means the constant `value`).  y0 is batch x N row-major.  When prune != 0 dead images
 * are skipped in later layers (same results: a zero row maps to relu(bias) = 0 for
 * bias <= 0); prune == 0 recomputes every image in every layer as the reference's CPU
 * loop does.  Outputs: categories (capacity batch), activations (count x N, may be
 * NULL), live[l] = survivors after layer l (may be NULL).  Returns the survivor count,
 * or -1 on allocation failure.
 */
int64_t spdnn_oracle_infer(int n, int layers, int k, const int32_t *const *rows, const float *const *vals,
                           float value, float bias, float clip, int64_t batch, const float *y0,
                           int32_t first_image, int32_t *categories, float *activations, int64_t *live,
                           int threads, int prune) {
    float *a = (float *)malloc(sizeof(float) * (size_t)n * (size_t)(batch ? batch : 1));
    float *b = (float *)malloc(sizeof(float) * (size_t)n * (size_t)(batch ? batch : 1));
    unsigned char *alive = (unsigned char *)malloc((size_t)(batch ? batch : 1));
    if (!a || !b || !alive) { free(a); free(b); free(alive); return -1; }
    memcpy(a, y0, sizeof(float) * (size_t)n * (size_t)batch);
    memset(alive, 1, (size_t)batch);
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
    for (int l = 0; l < layers; ++l) {
        const int32_t *r = rows[l];
        const float *v = (vals && vals[l]) ? vals[l] : NULL;
        int64_t cnt = 0;
#pragma omp parallel for schedule(dynamic, 8) reduction(+ : cnt)
        for (int64_t i = 0; i < batch; ++i) {
            float *out = b + (size_t)i * n;
            if (prune && !alive[i]) continue;      /* its row in `a` is already all zero */
            int any = layer_one_image(a + (size_t)i * n, out, n, k, r, v, value, bias, clip);
            if (!any && prune) memset(out, 0, sizeof(float) * (size_t)n);
            alive[i] = (unsigned char)any;
            cnt += any;
        }
        if (prune) {
            /* rows of dead images must read as zero in both buffers from now on */
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < batch; ++i)
                if (!alive[i]) memset(a + (size_t)i * n, 0, sizeof(float) * (size_t)n);
        }
        if (live) live[l] = cnt;
        float *t = a; a = b; b = t;
    }
    int64_t count = 0;
    for (int64_t i = 0; i < batch; ++i) {
        if (!alive[i]) continue;
        if (categories) categories[count] = first_image + (int32_t)i;
        if (activations) memcpy(activations + (size_t)count * n, a + (size_t)i * n, sizeof(float) * (size_t)n);
        ++count;
    }
    free(a); free(b); free(alive);
    return count;
}

/* Raw product of one layer (no bias, no clip) for `batch` images: the quantity
 * CpuSpmm::run_and_cmp recomputes and compares (src/utils/cpu_spmm.h:14-52). */
void spdnn_oracle_layer_raw(int n, int k, const int32_t *rows, const float *vals, float value, int64_t batch,
                            const float *in, float *out, int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(dynamic, 8)
    for (int64_t i = 0; i < batch; ++i) {
        const float *x = in + (size_t)i * n;
        float *o = out + (size_t)i * n;
        for (int c = 0; c < n; ++c) {
            const int32_t *r = rows + (size_t)c * k;
            float acc = 0.0f;
            for (int j = 0; j < k; ++j) {
                if (r[j] < 0) continue;
                float p = x[r[j]] * (vals ? vals[(size_t)c * k + j] : value);
                acc = acc + p;
            }
            o[c] = acc;
        }
    }
}

int spdnn_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
