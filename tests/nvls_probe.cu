// What does the NVSwitch compute for multimem.ld_reduce?  N GPUs in one process, 2^20 fp16
// (and fp32) values per GPU, N(0,1) and a wide-exponent mix.  Prints one JSON line per form
// of the instruction: how many results differ between two runs, how many differ from the
// rank-ordered fp32 sum rounded once to fp16, and the histogram of the difference to that
// sum in fp16 ulps.  Built and run by tests/test_multigpu.py; uses the library's fabric layer
// (saga_b200/csrc/fabric.cpp) for the multicast set-up.
//
//   nvcc -std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a -I include \
//        tests/nvls_probe.cu saga_b200/csrc/fabric.cpp -o nvls_probe && ./nvls_probe N
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <string>
#include <vector>
#include <unistd.h>
#include "../saga_b200/csrc/fabric.h"  // relative to this file
using namespace b200;

template <int MODE>
__global__ void probe(const uint16_t *mc, uint16_t *out, size_t n8)
{
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if(i >= n8) return;
    uint4 v;
    const void *p = mc + i * 8;
    if(MODE == 0)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else  // (.acc::f16 is not accepted by ptxas for f16x2)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    reinterpret_cast<uint4 *>(out)[i] = v;
}

__global__ void probe_f32(const float *mc, float *out, size_t n4)
{
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if(i >= n4) return;
    uint4 v;
    const void *p = mc + i * 4;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    reinterpret_cast<uint4 *>(out)[i] = v;
}

static float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
static uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

#define CKC(x) do { cudaError_t e = (x); if(e != cudaSuccess) { printf("CUDA %s: %s\n", #x, cudaGetErrorString(e)); return 1; } } while(0)
#define CKF(x) do { int rc_ = (x); if(rc_) { printf("fabric %s: %d %s\n", #x, rc_, err.c_str()); return 1; } } while(0)

int main(int argc, char **argv)
{
    int N = argc > 1 ? atoi(argv[1]) : 2;
    size_t n = 1 << 20;  // fp16 elements
    std::string err;
    bool yes = false;
    CKC(cudaSetDevice(0));
    CKF(fabric_multicast_supported(0, &yes, &err));
    if(!yes) { printf("{\"multicast\": false}\n"); return 0; }
    size_t gran = 0;
    CKF(fabric_granularity(0, N, true, &gran, &err));
    size_t bytes = (n * 4 + gran - 1) / gran * gran;  // room for f32 too
    std::vector<FabricMapping> arena(N);
    std::vector<FabricMulticast> mc(N);
    for(int r = 0; r < N; r++) {
        CKC(cudaSetDevice(r));
        CKF(fabric_alloc(&arena[r], r, bytes, &err));
        CKC(cudaMemset((void *)arena[r].va, 0, bytes));
    }
    CKC(cudaSetDevice(0));
    CKF(fabric_mc_create(&mc[0], N, bytes, &err));
    int fd = -1;
    CKF(fabric_export_fd(mc[0].mc, &fd, &err));
    for(int r = 1; r < N; r++) { CKC(cudaSetDevice(r)); CKF(fabric_mc_import(&mc[r], fd, bytes, &err)); }
    close(fd);
    for(int r = 0; r < N; r++) { CKC(cudaSetDevice(r)); CKF(fabric_mc_add_device(&mc[r], r, &err)); }
    for(int r = 0; r < N; r++) { CKC(cudaSetDevice(r)); CKF(fabric_mc_bind(&mc[r], arena[r], r, &err)); }

    // data: config-like gradients N(0,1) plus some wide-exponent pairs
    std::vector<std::vector<uint16_t>> G(N, std::vector<uint16_t>(n));
    srand(1234);
    auto gauss = [] { double u = (rand() + 1.0) / (RAND_MAX + 2.0), v = (rand() + 1.0) / (RAND_MAX + 2.0); return sqrt(-2 * log(u)) * cos(6.283185307179586 * v); };
    for(int r = 0; r < N; r++)
        for(size_t i = 0; i < n; i++) {
            double x = gauss();
            if(i >= n / 2) x *= pow(2.0, (rand() % 16) - 8);
            G[r][i] = f2h((float)x);
        }
    for(int r = 0; r < N; r++) { CKC(cudaSetDevice(r)); CKC(cudaMemcpy((void *)arena[r].va, G[r].data(), n * 2, cudaMemcpyHostToDevice)); CKC(cudaDeviceSynchronize()); }

    CKC(cudaSetDevice(0));
    uint16_t *out;
    CKC(cudaMalloc(&out, n * 2));
    std::vector<uint16_t> res(n), res2(n);
    for(int mode = 0; mode < 2; mode++) {
        for(int rep = 0; rep < 2; rep++) {
            const uint16_t *mcp = (const uint16_t *)mc[0].va;
            if(mode == 0) probe<0><<<(n / 8 + 255) / 256, 256>>>(mcp, out, n / 8);
            if(mode == 1) probe<1><<<(n / 8 + 255) / 256, 256>>>(mcp, out, n / 8);
            CKC(cudaDeviceSynchronize());
            CKC(cudaMemcpy(rep ? res2.data() : res.data(), out, n * 2, cudaMemcpyDeviceToHost));
        }
        long hist[9] = {0}, nondet = 0, other = 0, vs_f32order = 0, vs_f16chain = 0;
        for(size_t i = 0; i < n; i++) {
            if(res[i] != res2[i]) nondet++;
            double ex = 0; float a32 = 0; uint16_t c16 = 0;
            for(int r = 0; r < N; r++) { ex += h2f(G[r][i]); a32 += h2f(G[r][i]); c16 = r ? f2h(h2f(c16) + h2f(G[r][i])) : G[r][i]; }
            uint16_t rn = f2h((float)ex);  // exact sum of <= 8 halves fits double; float rounding first is fine for N=2
            if(res[i] != f2h(a32)) vs_f32order++;
            if(res[i] != c16) vs_f16chain++;
            int d = (int)(res[i] & 0x7fff) - (int)(rn & 0x7fff);
            if((res[i] ^ rn) & 0x8000) { other++; continue; }
            if(d < -4 || d > 4) other++; else hist[d + 4]++;
        }
        printf("{\"form\": \"%s\", \"ranks\": %d, \"values\": %zu, \"differ_between_runs\": %ld, "
               "\"differ_from_rank_ordered_sum\": %ld, \"differ_from_fp16_chain_sum\": %ld, "
               "\"ulps_minus4_to_plus4\": [",
               mode == 0 ? "f16x2" : "f16x2 acc::f32", N, n, nondet, vs_f32order, vs_f16chain);
        for(int k = 0; k < 9; k++) printf("%s%ld", k ? ", " : "", hist[k]);
        printf("], \"beyond\": %ld}\n", other);
    }
    // f32
    {
        std::vector<std::vector<float>> F(N, std::vector<float>(n));
        for(int r = 0; r < N; r++) for(size_t i = 0; i < n; i++) F[r][i] = (float)(gauss() * pow(2.0, (rand() % 16) - 8));
        for(int r = 0; r < N; r++) { CKC(cudaSetDevice(r)); CKC(cudaMemcpy((void *)arena[r].va, F[r].data(), n * 4, cudaMemcpyHostToDevice)); CKC(cudaDeviceSynchronize()); }
        CKC(cudaSetDevice(0));
        float *outf; CKC(cudaMalloc(&outf, n * 4));
        probe_f32<<<(n / 4 + 255) / 256, 256>>>((const float *)mc[0].va, outf, n / 4);
        CKC(cudaDeviceSynchronize());
        std::vector<float> rf(n);
        CKC(cudaMemcpy(rf.data(), outf, n * 4, cudaMemcpyDeviceToHost));
        long diff_order = 0, diff_exact = 0;
        for(size_t i = 0; i < n; i++) {
            float a = 0; double ex = 0;
            for(int r = 0; r < N; r++) { a += F[r][i]; ex += F[r][i]; }
            if(memcmp(&a, &rf[i], 4)) diff_order++;
            float e = (float)ex;
            if(memcmp(&e, &rf[i], 4)) diff_exact++;
        }
        printf("{\"form\": \"f32\", \"ranks\": %d, \"values\": %zu, \"differ_from_rank_ordered_sum\": %ld, "
               "\"differ_from_correctly_rounded_sum\": %ld}\n", N, n, diff_order, diff_exact);
    }
    for(int r = 0; r < N; r++) { cudaSetDevice(r); cudaDeviceSynchronize(); }
    for(int r = 0; r < N; r++) { cudaSetDevice(r); fabric_mc_release(&mc[r]); }
    for(int r = 0; r < N; r++) { cudaSetDevice(r); fabric_unmap(&arena[r]); }
    return 0;
}
