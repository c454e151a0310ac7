// Step kernel over an NVSwitch multicast mapping (sm_100a, N > 1 GPUs): the
// gradients of the rank's shard are fetched with ONE switch-reduced load per
// 16 bytes (multimem.ld_reduce: the switch reads the same address in every
// rank's gradient buffer, adds the values and returns the fp16 sum) and
// the updated fp16 weights leave the GPU ONCE (multimem.st: the switch writes
// them into every rank's weight buffer).  Per rank and NVLink direction that
// is about 2n + 2n/N bytes for n fp16 parameters instead of the 4n(N-1)/N of
// the peer-pointer kernel, which loads every peer's copy and stores to every
// peer separately.
//
// The sum is the switch's: measured on B200 / NVSwitch, multimem.ld_reduce on
// f16x2 is deterministic but lands one fp16 ulp beside the correctly rounded
// sum for about a fifth of the elements (with or without .acc::f32; the f32
// form of the instruction is exact).  That is the arithmetic NCCL's own NVLS
// reduce-scatter has on this machine, i.e. what Saga gets from
// ncclReduceScatter (src/cuda/cuda_optimizer.cpp:160-166 of the Saga tree);
// the peer-pointer kernel, which adds in fp32 in rank order and rounds once,
// stays the path that is bit for bit equal to the rank-ordered oracle.
// Everything after the sum (classification, unscale, Adam, rounding) is the
// same code on both paths and bit-exact given the sum.
//
// The fp32 group (a few tens of thousands of BatchNorm parameters) and the
// ragged 8-element groups at the shard's ends go through the peer pointers.
#pragma once

#include "fused_step.cuh"

namespace b200 {

// 8 fp16 values summed over all ranks by the switch.
__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void *mc)
{
    uint4 v;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 "
        "{%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(mc)
        : "memory");
    return v;
}

// 16 bytes stored into the same address of every rank's buffer.
__device__ __forceinline__ void multimem_st_16(void *mc, const uint4 &v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::
                     "l"(mc),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Direct loads, one 8-element group per thread per trip; the loads of the first
// trip's shard state are issued before the wait for the peers.
template <int NR, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
    nvls_step_kernel(const __grid_constant__ StepParams p)
{
    __shared__ int s_flag;
    const int tid = threadIdx.x;
    uint32_t fl = 0;
    const size_t stride = (size_t)gridDim.x * kThreads;
    const size_t ng = p.h.ngroups;
    const size_t lo = p.h.o, hi = p.h.o + p.h.s;
    size_t base = (size_t)blockIdx.x * kThreads;
    HalfLoads<1> L;
    bool full = false;
    size_t idx0 = 0;

    auto classify = [&](size_t b) {
        const size_t gid = b + tid;
        idx0 = p.h.B + gid * kVec;
        full = gid < ng && idx0 >= lo && idx0 + kVec <= hi;
    };

    step_announce<NR>(p);
    bool state_loaded = false;
    if(base < ng) {
        classify(base);
        if(full)
            half_load_state(p, idx0, L);
        state_loaded = true;
    }
    if(!step_wait<NR>(p)) {
        const float alpha = step_alpha(p);
        for(; base < ng; base += stride) {
            if(!state_loaded) {
                classify(base);
                if(full)
                    half_load_state(p, idx0, L);
            }
            state_loaded = false;
            if(full) {
                L.g[0] = multimem_ld_reduce_f16x8(p.mcG + idx0);
                uint4 out[7];
                // the sum is already formed: the one-rank arithmetic
                half_compute<1>(p, alpha, idx0, L, fl, out);
                const size_t li = idx0 - p.h.A;
                st_stream(p.h.m + li, out[0]);
                st_stream(p.h.m + li + 4, out[1]);
                st_stream(p.h.v + li, out[2]);
                st_stream(p.h.v + li + 4, out[3]);
                st_stream(p.h.c + li, out[4]);
                st_stream(p.h.c + li + 4, out[5]);
                multimem_st_16(p.mcW + idx0, out[6]);
                if(p.keep_reduced)
                    *reinterpret_cast<uint4 *>(
                        const_cast<uint16_t *>(p.h.G[p.rank]) + idx0) = L.g[0];
            } else if(base + tid < ng && idx0 + kVec > lo) {
                fl |= half_scalar<NR>(p, alpha, idx0);
            }
        }
        float_group_pass<NR>(p, fl);
    }
    step_finish<NR>(p, fl, &s_flag);
}

}  // namespace b200
