// add_chain_ceiling: what one SM sustains on the arithmetic of the float form, measured in isolation.
//
// The float form of a layer (alt2_kernel, spdnn_alt2.cuh) computes every output as 32 fp32 additions in
// the order of the reference's loop, a + b + a + b + ..., so an output is a chain of 32 dependent adds and
// its cost is set by the FP32 pipe, not by memory.  This program runs that inner loop alone -- one block
// per SM, the rows of 16 images resident in shared memory, a synthetic table of row pairs, the same
// per-class work (two 16-byte loads, the sum, scale, bias, clamp, survivor and saturation bits, a 16-byte
// store, one barrier per layer) -- with the additions packed (add.rn.f32x2, two images per instruction,
// as the library does) or scalar, and prints the cycles one SM sub-partition spends per warp and class
// (128 outputs = 4096 additions).  The hardware limit is 128 cycles (32 lanes, one add per lane and cycle);
// what this loop reaches is the practical ceiling the library's float form is compared with.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o add_chain_ceiling add_chain_ceiling.cu && ./add_chain_ceiling
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>

typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { f32x2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
// rows are stored with the low bit flipped by the parity of the bits above it (spdnn_resident.cuh, resident_phys_row)
__device__ __forceinline__ int phys(int r) { return r ^ (__popc((unsigned)(r >> 1)) & 1); }

template <int NT, bool PACKED>
__global__ void __launch_bounds__(NT, 1) loop_kernel(const unsigned int *tab, int classes, int layers, float bias, float clip, float w,
                                                      unsigned int *out, long long *cycles) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ unsigned int s_alive[3];
    __shared__ int s_ns[3];
    constexpr int RS = 64, TB = 16, LPC = 4, CPI = NT / LPC;        // 16 images per block, 4 per thread
    const int tid = threadIdx.x, lane = tid & 31, sub = tid % LPC, grp = tid / LPC;
    unsigned char *cur = smem, *nxt = smem + classes * RS;
    unsigned int *T = reinterpret_cast<unsigned int *>(smem + 2 * classes * RS);
    for (int i = tid; i < classes * 16; i += NT) reinterpret_cast<float *>(cur)[i] = (float)((i * 7 + blockIdx.x) % 33) * 0.37f;
    for (int i = tid; i < classes; i += NT) T[i] = tab[i];
    if (tid < 3) { s_alive[tid] = 0; s_ns[tid] = 0; }
    __syncthreads();
    const long long t0 = clock64();
    unsigned int alive_prev = 0xffffu;
    for (int li = 0; li < layers; ++li) {
        if (tid == 0) { s_alive[(li + 1) % 3] = 0u; s_ns[(li + 1) % 3] = 0; }
        unsigned int bits = 0;
        bool ns = false;
        const unsigned char *in = cur + sub * TB;
        for (int u = grp; u < classes; u += CPI) {
            const unsigned int e = T[u];
            const int ao = phys((int)(e & 0xffffu) >> 2) * RS, bo = phys((int)(e >> 18)) * RS, oo = phys(u) * RS;
            const float4 va = *reinterpret_cast<const float4 *>(in + ao);
            const float4 vb = *reinterpret_cast<const float4 *>(in + bo);
            float4 s;
            if (PACKED) {
                const f32x2 al = pack2(va.x, va.y), ah = pack2(va.z, va.w), bl = pack2(vb.x, vb.y), bh = pack2(vb.z, vb.w);
                f32x2 lo = pack2(0.f, 0.f), hi = lo;
#pragma unroll
                for (int i = 0; i < 16; ++i) { lo = add2(lo, al); hi = add2(hi, ah); lo = add2(lo, bl); hi = add2(hi, bh); }
                unpack2(lo, s.x, s.y);
                unpack2(hi, s.z, s.w);
            } else {
                s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    s.x = __fadd_rn(s.x, va.x); s.y = __fadd_rn(s.y, va.y); s.z = __fadd_rn(s.z, va.z); s.w = __fadd_rn(s.w, va.w);
                    s.x = __fadd_rn(s.x, vb.x); s.y = __fadd_rn(s.y, vb.y); s.z = __fadd_rn(s.z, vb.z); s.w = __fadd_rn(s.w, vb.w);
                }
            }
            float4 y;
            y.x = fminf(fmaxf(__fadd_rn(__fmul_rn(s.x, w), bias), 0.f), clip);
            y.y = fminf(fmaxf(__fadd_rn(__fmul_rn(s.y, w), bias), 0.f), clip);
            y.z = fminf(fmaxf(__fadd_rn(__fmul_rn(s.z, w), bias), 0.f), clip);
            y.w = fminf(fmaxf(__fadd_rn(__fmul_rn(s.w, w), bias), 0.f), clip);
            bits |= (y.x != 0.0f ? 1u : 0u) | (y.y != 0.0f ? 2u : 0u) | (y.z != 0.0f ? 4u : 0u) | (y.w != 0.0f ? 8u : 0u);
            ns |= (y.x != 0.0f && y.x != clip) || (y.y != 0.0f && y.y != clip) || (y.z != 0.0f && y.z != clip) || (y.w != 0.0f && y.w != clip);
            *reinterpret_cast<float4 *>(nxt + oo + sub * TB) = y;
        }
        const unsigned int wm = __reduce_or_sync(0xffffffffu, bits << (sub * 4));
        if (lane == 0 && wm) atomicOr(&s_alive[li % 3], wm);
        if (__any_sync(0xffffffffu, ns) && lane == 0) s_ns[li % 3] = 1;
        __syncthreads();
        alive_prev &= s_alive[li % 3];
        unsigned char *t = cur; cur = nxt; nxt = t;
        if (alive_prev == 0u) break;
    }
    const long long t1 = clock64();
    if (tid == 0) { cycles[blockIdx.x] = t1 - t0; out[blockIdx.x] = alive_prev + reinterpret_cast<unsigned int *>(cur)[5]; }
}

template <int NT, bool PACKED>
void run(const char *name, const unsigned int *d_tab, int classes, int layers, unsigned int *d_out, long long *d_cyc, int sms, int khz) {
    const size_t smem = (size_t)classes * 64 * 2 + (size_t)classes * 4;
    cudaFuncSetAttribute(loop_kernel<NT, PACKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float best = 1e9f;
    for (int it = 0; it < 3; ++it) {
        cudaEventRecord(e0);
        loop_kernel<NT, PACKED><<<sms, NT, smem>>>(d_tab, classes, layers, -0.4f, 32.0f, 0.0625f, d_out, d_cyc);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms < best) best = ms;
    }
    const cudaError_t err = cudaGetLastError();
    std::vector<long long> cyc(sms);
    cudaMemcpy(cyc.data(), d_cyc, sms * 8, cudaMemcpyDeviceToHost);
    long long mx = 0;
    for (long long c : cyc) mx = c > mx ? c : mx;
    const double per_smsp = (double)layers * classes * 4 / 32 / 4;           // warp-classes one sub-partition executes
    const double adds = (double)layers * classes * 16 * 32 * sms;
    printf("%-8s %4d threads  %7.3f ms  %6.1f cycles per warp and class on a sub-partition (limit 128)  %6.2f T adds/s of %6.2f\n", name, NT,
           best, (double)mx / per_smsp, adds / (best * 1e-3) * 1e-12, (double)sms * 128 * khz * 1e3 * 1e-12);
    if (err != cudaSuccess) printf("  CUDA error: %s\n", cudaGetErrorString(err));
}

int main() {
    int sms = 148, khz = 1965000;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
    const int classes = 1024, layers = 64;                       // one layer of the 16384-neuron network has 1024 classes
    std::vector<unsigned int> tab(classes);
    for (int u = 0; u < classes; ++u) {
        const int a = (u * 16) % 1024 + (u / 64), b = (a + 8 * 16 + 3) % 1024;      // scattered row pairs
        tab[u] = (unsigned)(a * 4) | ((unsigned)(b * 4) << 16);
    }
    unsigned int *d_tab, *d_out;
    long long *d_cyc;
    cudaMalloc(&d_tab, classes * 4);
    cudaMalloc(&d_out, sms * 4);
    cudaMalloc(&d_cyc, sms * 8);
    cudaMemcpy(d_tab, tab.data(), classes * 4, cudaMemcpyHostToDevice);
    run<512, true>("packed", d_tab, classes, layers, d_out, d_cyc, sms, khz);
    run<512, false>("scalar", d_tab, classes, layers, d_out, d_cyc, sms, khz);
    run<1024, true>("packed", d_tab, classes, layers, d_out, d_cyc, sms, khz);
    run<256, true>("packed", d_tab, classes, layers, d_out, d_cyc, sms, khz);
    return 0;
}
