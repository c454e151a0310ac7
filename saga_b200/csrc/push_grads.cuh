// Push half of the "push" collective path (several ranks): every rank WRITES
// the parts of its own gradient buffers that other ranks own into staging
// slots in those ranks' memory, then announces "my contributions have landed".
// The step kernel that follows on the same stream then sums its own shard with
// the staged contributions in rank order -- all loads local -- and pushes the
// updated weights as before.
//
// Why: over NVLink a load is a request packet one way and the data the other
// way, a store is data one way only.  With every rank pulling from every other
// rank the request packets take a measurable share of each direction; with
// stores only they are gone.  The price is one more launch and one more pass
// of the staged bytes through local HBM, which has headroom when the links
// are the bottleneck.  Needs no wait on entry: the slots written here were
// last read before the previous step's completion protocol ended.
#pragma once

#include "fused_step.cuh"

namespace b200 {

struct PushParams {
    const uint16_t *Gh;          // this rank's fp16 gradient buffer
    const float *Gf;             // this rank's fp32 gradient buffer
    // staging slot reserved for THIS rank on rank q, as a virtual base: the
    // element with flat index i goes to Sh[q][i]
    uint16_t *Sh[kMaxRanks];
    float *Sf[kMaxRanks];
    size_t sh, sf;               // shard lengths (n / nranks)
    int rank, nranks;
    uint32_t epoch;
    Ctrl *ctrl[kMaxRanks];
};

constexpr int kPushThreads = 256;
constexpr int kPushUnroll = 4;  // 16-byte vectors per thread per work item

// One work item = kPushThreads * kPushUnroll 16-byte vectors of one peer's
// shard; consecutive items go to different peers so that at any time every
// link carries traffic.
__global__ void __launch_bounds__(kPushThreads)
    push_grads_kernel(const __grid_constant__ PushParams p)
{
    __shared__ int s_last;
    const int tid = threadIdx.x;
    const int npeers = p.nranks - 1;
    constexpr size_t kItemVecs = (size_t)kPushThreads * kPushUnroll;

    // fp16 group: 8 elements per vector; the copied range is the peer's shard
    // widened to whole vectors (the few extra elements land in slot padding
    // and are never read)
    {
        const size_t vec_per_shard_max = (p.sh + 2 * kVec) / kVec + 1;
        const size_t items_per_peer = (vec_per_shard_max + kItemVecs - 1) / kItemVecs;
        const size_t items = p.sh ? items_per_peer * npeers : 0;
        for(size_t t = blockIdx.x; t < items; t += gridDim.x) {
            const int j = (int)(t % npeers);
            const size_t c = t / npeers;
            const int q = (p.rank + 1 + j) % p.nranks;
            const size_t lo = (p.sh * q) & ~(size_t)(kVec - 1);
            const size_t hi = (p.sh * q + p.sh + kVec - 1) & ~(size_t)(kVec - 1);
            const size_t nvec = (hi - lo) / kVec;
            uint4 v[kPushUnroll];
#pragma unroll
            for(int u = 0; u < kPushUnroll; u++) {
                const size_t k = c * kItemVecs + (size_t)u * kPushThreads + tid;
                if(k < nvec)
                    v[u] = ld_stream(p.Gh + lo + k * kVec);
            }
#pragma unroll
            for(int u = 0; u < kPushUnroll; u++) {
                const size_t k = c * kItemVecs + (size_t)u * kPushThreads + tid;
                if(k < nvec)
                    *reinterpret_cast<uint4 *>(p.Sh[q] + lo + k * kVec) = v[u];
            }
        }
    }
    // fp32 group: 4 elements per vector
    {
        const size_t vec_per_shard_max = (p.sf + 8) / 4 + 1;
        const size_t items_per_peer = (vec_per_shard_max + kItemVecs - 1) / kItemVecs;
        const size_t items = p.sf ? items_per_peer * npeers : 0;
        for(size_t t = blockIdx.x; t < items; t += gridDim.x) {
            const int j = (int)(t % npeers);
            const size_t c = t / npeers;
            const int q = (p.rank + 1 + j) % p.nranks;
            const size_t lo = (p.sf * q) & ~(size_t)3;
            const size_t hi = (p.sf * q + p.sf + 3) & ~(size_t)3;
            const size_t nvec = (hi - lo) / 4;
#pragma unroll
            for(int u = 0; u < kPushUnroll; u++) {
                const size_t k = c * kItemVecs + (size_t)u * kPushThreads + tid;
                if(k < nvec)
                    *reinterpret_cast<uint4 *>(p.Sf[q] + lo + k * 4) =
                        ld_stream(p.Gf + lo + k * 4);
            }
        }
    }

    // the last CTA to finish tells every rank (itself included) that this
    // rank's contributions of step `epoch` are in place
    Ctrl *const my = p.ctrl[p.rank];
    __threadfence_system();
    __syncthreads();
    if(tid == 0)
        s_last = atomicAdd(&my->push_done, 1u) == gridDim.x - 1;
    __syncthreads();
    if(!s_last)
        return;
    __threadfence();
    if(tid < p.nranks) {
        __threadfence_system();
        st_release_sys(&p.ctrl[tid]->ready[p.rank], p.epoch);
    }
    if(tid == 0)
        my->push_done = 0;
}

}  // namespace b200
