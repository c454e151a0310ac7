// Multi-threaded driver in Saga's own execution model: ONE process, one
// std::thread per GPU, every thread bound to its device and calling the step
// on its own stream with no host barrier between ranks inside the loop
// (test/test_classifier.cpp:689-691 and test/test_mp.cpp:131-167 of the Saga
// tree do the same around Program::run).  It goes through the C ABI only.
//
//   mt_driver <nranks> <n_half> <steps> [timeout_ms] [skip_rank]
//
// Prints one JSON line: per-step device time (max over ranks), the flag sums
// and loss scale after every step of rank 0, a checksum of every rank's weight
// buffer (all must agree).  skip_rank >= 0 makes that rank never call step, to
// show that the others give up after the wait limit instead of hanging.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "b200_adam_op.hpp"

namespace {

struct Lcg {
    uint64_t s;
    explicit Lcg(uint64_t seed) : s(seed * 2862933555777941757ull + 3037000493ull) {}
    float uniform()  // (-1, 1)
    {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        return ((s >> 40) / 8388608.0f) - 1.0f;
    }
};

struct RankResult {
    int status = 0;
    std::string error;
    float ms_per_step = 0;
    uint64_t checksum = 0;
    std::vector<uint32_t> flags;
    std::vector<float> scales;
};

uint64_t fnv(const std::vector<uint16_t> &v)
{
    uint64_t h = 1469598103934665603ull;
    for(uint16_t x : v) {
        h ^= x;
        h *= 1099511628211ull;
    }
    return h;
}

}  // namespace

int main(int argc, char **argv)
{
    if(argc < 4) {
        fprintf(stderr, "usage: %s nranks n_half steps [timeout_ms] [skip_rank]\n", argv[0]);
        return 2;
    }
    const int nranks = atoi(argv[1]);
    const size_t n = strtoull(argv[2], nullptr, 10);
    const int steps = atoi(argv[3]);
    const long timeout_ms = argc > 4 ? atol(argv[4]) : 10000;
    const int skip_rank = argc > 5 ? atoi(argv[5]) : -1;

    int ndev = 0;
    cudaGetDeviceCount(&ndev);
    if(ndev < nranks) {
        printf("{\"skipped\": \"needs %d GPUs, found %d\"}\n", nranks, ndev);
        return 0;
    }

    saga::B200Rendezvous rendezvous(nranks);
    std::vector<RankResult> results(nranks);
    std::vector<b200opt_t *> handles(nranks, nullptr);
    std::vector<std::thread> threads;

    for(int rank = 0; rank < nranks; rank++) {
        threads.emplace_back([&, rank] {
            RankResult &res = results[rank];
            cudaSetDevice(rank);
            cudaStream_t stream;
            cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
            b200opt_t *h = nullptr;
            int rc = b200opt_create(&h, rank, nranks, rank, n, 0);
            if(rc) {
                // the other threads would wait for this rank at the rendezvous
                fprintf(stderr, "rank %d: b200opt_create failed: %s\n", rank,
                        b200opt_strerror(rc));
                exit(1);
            }
            b200opt_set_option(h, B200OPT_OPT_TIMEOUT_MS, timeout_ms);
            b200opt_set_option(h, B200OPT_OPT_PATH, B200OPT_PATH_PEER);
            try {
                rendezvous.join(rank, h);
            } catch(const std::exception &e) {
                res.status = B200OPT_ESTATE;
                res.error = e.what();
                return;
            }
            void *w = nullptr, *g = nullptr;
            b200opt_buffers(h, B200OPT_HALF, &w, &g, nullptr);
            std::vector<__half> hw(n), hg(n);
            Lcg wl(1), gl(1000 + rank);  // same weights everywhere, own gradients
            for(size_t i = 0; i < n; i++) {
                hw[i] = __float2half(0.05f * wl.uniform());
                hg[i] = __float2half(2.0f * gl.uniform());
            }
            cudaMemcpyAsync(w, hw.data(), n * 2, cudaMemcpyHostToDevice, stream);
            cudaMemcpyAsync(g, hg.data(), n * 2, cudaMemcpyHostToDevice, stream);
            b200opt_init_master(h, stream);
            cudaStreamSynchronize(stream);

            float scale = 1024.0f;
            cudaEvent_t e0, e1;
            cudaEventCreate(&e0);
            cudaEventCreate(&e1);
            float total_ms = 0;
            for(int step = 0; step < steps && !res.status; step++) {
                if(rank == skip_rank)
                    break;  // this rank "dies" between steps, nothing in flight
                cudaEventRecord(e0, stream);
                rc = b200opt_step(h, 1e-3f, 0.01f, scale, stream);
                cudaEventRecord(e1, stream);
                uint32_t fl[3] = {0, 0, 0};
                if(!rc)
                    rc = b200opt_flags(h, stream, fl);
                if(rc) {
                    res.status = rc;
                    res.error = b200opt_last_error(h);
                    break;
                }
                float ms = 0;
                cudaEventElapsedTime(&ms, e0, e1);
                total_ms += ms;
                b200opt_policy_update(&scale, fl, B200OPT_POLICY_REFERENCE, nullptr, 0);
                res.flags.insert(res.flags.end(), fl, fl + 3);
                res.scales.push_back(scale);
            }
            res.ms_per_step = steps ? total_ms / steps : 0;
            cudaStreamSynchronize(stream);
            std::vector<uint16_t> back(n);
            cudaMemcpy(back.data(), w, n * 2, cudaMemcpyDeviceToHost);
            res.checksum = fnv(back);
            handles[rank] = h;  // destroyed by main once every rank is done
        });
    }
    for(auto &t : threads)
        t.join();
    for(auto h : handles)
        if(h)
            b200opt_destroy(h);

    float worst = 0;
    bool same = true, ok = true;
    for(int r = 0; r < nranks; r++) {
        worst = results[r].ms_per_step > worst ? results[r].ms_per_step : worst;
        if(r != skip_rank) {
            same &= results[r].checksum == results[skip_rank == 0 ? 1 : 0].checksum;
            ok &= results[r].status == 0;
        }
    }
    printf("{\"nranks\": %d, \"n_half\": %zu, \"steps\": %d, \"ok\": %s, "
           "\"weights_identical\": %s, \"ms_per_step_max\": %.6f, \"status\": [",
           nranks, n, steps, ok ? "true" : "false", same ? "true" : "false", worst);
    for(int r = 0; r < nranks; r++)
        printf("%s%d", r ? ", " : "", results[r].status);
    printf("], \"errors\": [");
    for(int r = 0; r < nranks; r++)
        printf("%s\"%s\"", r ? ", " : "", results[r].error.c_str());
    const RankResult &r0 = results[skip_rank == 0 ? 1 % nranks : 0];
    printf("], \"flags\": [");
    for(size_t i = 0; i < r0.flags.size(); i++)
        printf("%s%u", i ? ", " : "", r0.flags[i]);
    printf("], \"scales\": [");
    for(size_t i = 0; i < r0.scales.size(); i++)
        printf("%s%.9g", i ? ", " : "", r0.scales[i]);
    printf("], \"checksum\": \"%016llx\"}\n", (unsigned long long)r0.checksum);
    return 0;
}
