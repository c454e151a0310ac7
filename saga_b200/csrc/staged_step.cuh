// Step kernel with shared-memory staging of the shard (sm_100a): bulk
// asynchronous copies (cp.async.bulk, completion on an mbarrier) stream
// 2048-element tiles of the gradient buffers of all ranks and of the local
// m / v / master shard into a ring of shared-memory stages; the CTA updates a
// tile in place in shared memory and bulk-stores m, v, master and the fp16
// weights (to every rank's weight buffer) straight from the stage.  Loads of
// later tiles are in flight while a tile is computed, independent of how many
// registers a thread holds.  No cluster multicast is used anywhere.
#pragma once

#include "fused_step.cuh"

namespace b200 {

// bytes of one stage: the gradient tiles of NR ranks, then m, v, master tiles
__host__ __device__ constexpr size_t stage_bytes(int nr, int tile)
{
    return (size_t)nr * tile * 2 + 3 * (size_t)tile * 4;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(count)
                 : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait for a stage to fill: gives up after limit_ns.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity,
                                          unsigned long long limit_ns)
{
    if(mbar_try_wait(bar, parity))
        return true;
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    for(;;) {
        if(mbar_try_wait(bar, parity))
            return true;
        if((++spins & 255u) == 0 && globaltimer_ns() - t0 > limit_ns)
            return false;
    }
}
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc,
                                          uint32_t bytes, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void bulk_store(void *gdst, const void *smem_src,
                                           uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::
                     "l"(gdst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until at most N of this thread's store groups still READ shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until all of this thread's bulk stores are complete.
__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all()
{
    asm volatile("fence.proxy.async;" ::: "memory");
}

// VEC consecutive elements of a tile per thread, to and from shared memory.
template <int VEC>
__device__ __forceinline__ void lds_halves(const unsigned char *base, int tid,
                                           uint32_t (&u)[VEC])
{
    if(VEC == 8) {
        const uint4 g = reinterpret_cast<const uint4 *>(base)[tid];
        u[0] = g.x & 0xffffu;
        u[1] = g.x >> 16;
        u[2] = g.y & 0xffffu;
        u[3] = g.y >> 16;
        u[VEC - 4] = g.z & 0xffffu;
        u[VEC - 3] = g.z >> 16;
        u[VEC - 2] = g.w & 0xffffu;
        u[VEC - 1] = g.w >> 16;
    } else {
        const uint2 g = reinterpret_cast<const uint2 *>(base)[tid];
        u[0] = g.x & 0xffffu;
        u[1] = g.x >> 16;
        u[2] = g.y & 0xffffu;
        u[3] = g.y >> 16;
    }
}
template <int VEC>
__device__ __forceinline__ void sts_halves(unsigned char *base, int tid,
                                           const uint32_t (&u)[VEC])
{
    if(VEC == 8) {
        reinterpret_cast<uint4 *>(base)[tid] = make_uint4(
            u[0] | (u[1] << 16), u[2] | (u[3] << 16),
            u[VEC - 4] | (u[VEC - 3] << 16), u[VEC - 2] | (u[VEC - 1] << 16));
    } else {
        reinterpret_cast<uint2 *>(base)[tid] =
            make_uint2(u[0] | (u[1] << 16), u[2] | (u[3] << 16));
    }
}
template <int VEC>
__device__ __forceinline__ void lds_floats(const unsigned char *base, int tid,
                                           float (&x)[VEC])
{
    const float4 *s4 = reinterpret_cast<const float4 *>(base) + tid * (VEC / 4);
#pragma unroll
    for(int k = 0; k < VEC / 4; k++) {
        const float4 t = s4[k];
        x[4 * k + 0] = t.x;
        x[4 * k + 1] = t.y;
        x[4 * k + 2] = t.z;
        x[4 * k + 3] = t.w;
    }
}
template <int VEC>
__device__ __forceinline__ void sts_floats(unsigned char *base, int tid,
                                           const float (&x)[VEC])
{
    float4 *s4 = reinterpret_cast<float4 *>(base) + tid * (VEC / 4);
#pragma unroll
    for(int k = 0; k < VEC / 4; k++)
        s4[k] = make_float4(x[4 * k], x[4 * k + 1], x[4 * k + 2], x[4 * k + 3]);
}

// Updates, in place in one filled stage, the VEC elements this thread owns.
template <int NR, int VEC, int TILE>
__device__ __forceinline__ void staged_update(const StepParams &p, float alpha,
                                              unsigned char *st, int tid,
                                              size_t gidx, uint32_t &fl)
{
    constexpr uint32_t kOffM = NR * TILE * 2;
    constexpr uint32_t kOffV = kOffM + TILE * 4;
    constexpr uint32_t kOffC = kOffV + TILE * 4;
    uint32_t u[VEC];
    lds_halves<VEC>(st, tid, u);
    if(NR > 1) {
        // fp32 accumulation in rank order, one rounding to fp16
        float acc[VEC];
#pragma unroll
        for(int e = 0; e < VEC; e++)
            acc[e] = half_bits_to_float(u[e]);
#pragma unroll
        for(int q = 1; q < NR; q++) {
            uint32_t t[VEC];
            lds_halves<VEC>(st + q * TILE * 2, tid, t);
#pragma unroll
            for(int e = 0; e < VEC; e++)
                acc[e] += half_bits_to_float(t[e]);
        }
#pragma unroll
        for(int e = 0; e < VEC; e++)
            u[e] = float_to_half_bits(acc[e]);
    }
    float m[VEC], v[VEC], c[VEC];
    lds_floats<VEC>(st + kOffM, tid, m);
    lds_floats<VEC>(st + kOffV, tid, v);
    lds_floats<VEC>(st + kOffC, tid, c);
    uint32_t wbits[VEC];
    half_update<VEC>(p, alpha, u, m, v, c, wbits, p.h.W[p.rank] + gidx, fl);
    sts_floats<VEC>(st + kOffM, tid, m);
    sts_floats<VEC>(st + kOffV, tid, v);
    sts_floats<VEC>(st + kOffC, tid, c);
    sts_halves<VEC>(st, tid, wbits);  // the new weights take the place of g[0]
}

constexpr int kMaxStages = 16;

// THREADS threads update tiles of THREADS*VEC elements through a ring of
// p.stages shared-memory stages (dynamic shared memory sized by the launcher).
template <int NR, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS)
    staged_step_kernel(const __grid_constant__ StepParams p)
{
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ int s_flag;
    const int STAGES = p.stages;

    constexpr int TILE = THREADS * VEC;
    constexpr uint32_t kStage = (uint32_t)stage_bytes(NR, TILE);
    constexpr uint32_t kOffM = NR * TILE * 2;
    constexpr uint32_t kOffV = kOffM + TILE * 4;
    constexpr uint32_t kOffC = kOffV + TILE * 4;

    const int tid = threadIdx.x;
    if(tid == 0) {
        for(int s = 0; s < STAGES; s++)
            mbar_init(&full_bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    uint32_t fl = 0;
    if(!step_begin<NR>(p)) {
        const float alpha = step_alpha(p);
        // full 8-element groups of the shard: [F0, F1); the (at most two)
        // ragged groups at the shard's ends go through the element-wise path
        const size_t lo = p.h.o, hi = p.h.o + p.h.s;
        const size_t F0 = (lo + kVec - 1) & ~(size_t)(kVec - 1);
        const size_t F1 = hi & ~(size_t)(kVec - 1);
        const bool any_full = p.h.s && F1 > F0;
        // Tiles are cut on multiples of TILE of the flat buffer's index, so that
        // all but the first and last tile of a shard start on a 2 KB boundary of
        // the fp16 arrays (4 KB of the fp32 arrays) whatever the shard's offset.
        const size_t t_first = F0 / TILE;
        const size_t ntiles = any_full ? (F1 - 1) / TILE - t_first + 1 : 0;
        const size_t nmine =
            ntiles > blockIdx.x
                ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x
                : 0;

        auto tile_start = [&](size_t k) -> size_t {
            const size_t t = t_first + blockIdx.x + k * gridDim.x;
            const size_t b = t * TILE;
            return b > F0 ? b : F0;
        };
        auto tile_elems = [&](size_t k) -> uint32_t {
            const size_t t = t_first + blockIdx.x + k * gridDim.x;
            const size_t e = (t + 1) * TILE;
            return (uint32_t)((e < F1 ? e : F1) - tile_start(k));
        };
        auto issue_loads = [&](size_t k) {
            const int s = (int)(k % STAGES);
            const size_t e0 = tile_start(k);    // global element index
            const size_t l0 = e0 - p.h.A;       // index into the shard state
            const uint32_t te = tile_elems(k);
            unsigned char *st = stage_mem + (size_t)s * kStage;
            mbar_expect_tx(&full_bar[s], te * (2u * NR + 12u));
#pragma unroll
            for(int q = 0; q < NR; q++)
                bulk_load(st + q * TILE * 2, p.h.G[q] + e0, te * 2u,
                          &full_bar[s]);
            bulk_load(st + kOffM, p.h.m + l0, te * 4u, &full_bar[s]);
            bulk_load(st + kOffV, p.h.v + l0, te * 4u, &full_bar[s]);
            bulk_load(st + kOffC, p.h.c + l0, te * 4u, &full_bar[s]);
        };

        if(tid == 0 && !p.force_scalar) {
            // loads of peer gradients are ordered after the peers' announcements
            fence_proxy_async_all();
            for(size_t k = 0; k < nmine && k < (size_t)STAGES; k++)
                issue_loads(k);
        }

        bool failed = false;
        for(size_t k = 0; k < nmine && !p.force_scalar; k++) {
            const int s = (int)(k % STAGES);
            const uint32_t parity = (uint32_t)((k / STAGES) & 1);
            unsigned char *st = stage_mem + (size_t)s * kStage;
            if(!mbar_wait(&full_bar[s], parity, p.timeout_ns))
                failed = true;
            // a stage that did not fill is not touched by anyone
            if(__syncthreads_or(failed)) {
                failed = true;
                break;
            }
            const uint32_t te = tile_elems(k);
            const size_t e0 = tile_start(k);
            if((uint32_t)tid * VEC < te) {
                staged_update<NR, VEC, TILE>(p, alpha, st, tid,
                                             e0 + (size_t)tid * VEC, fl);
                fence_proxy_async_smem();
            }
            __syncthreads();
            if(tid == 0) {
                const size_t l0 = e0 - p.h.A;
                bulk_store(p.h.m + l0, st + kOffM, te * 4u);
                bulk_store(p.h.v + l0, st + kOffV, te * 4u);
                bulk_store(p.h.c + l0, st + kOffC, te * 4u);
#pragma unroll
                for(int q = 0; q < NR; q++)
                    bulk_store(p.h.W[q] + e0, st, te * 2u);
                bulk_commit();
                // refill the stage whose stores were issued one trip ago
                if(STAGES > 1 && k >= 1 && k - 1 + STAGES < nmine) {
                    bulk_wait_read<1>();
                    issue_loads(k - 1 + STAGES);
                }
            }
        }
        if(tid == 0) {
            bulk_wait_all();          // stores complete, not merely read
            fence_proxy_async_all();  // ... and ordered before the signals below
        }
        if(failed) {
            // Loads may still be landing in this CTA's shared memory: give each
            // outstanding stage a bounded chance to fill before returning.
            for(int s = 0; s < STAGES; s++) {
                mbar_wait(&full_bar[s], 0, 1000000ull);
                mbar_wait(&full_bar[s], 1, 1000000ull);
            }
            if(tid == 0) {
                Ctrl *const my = p.ctrl[p.rank];
                if(my)
                    atomicCAS(&my->status, 0u, (uint32_t)(-B200OPT_ETIMEOUT));
                if(p.host)
                    p.host->where = 3;
            }
        }

        // ragged groups at the shard's ends (and everything, for unaligned
        // caller memory in kernel-seam mode)
        if(p.force_scalar) {
            const size_t ng = p.h.ngroups;
            for(size_t gid = (size_t)blockIdx.x * THREADS + tid; gid < ng;
                gid += (size_t)gridDim.x * THREADS)
                fl |= half_scalar<NR>(p, alpha, p.h.B + gid * kVec);
        } else if(blockIdx.x == 0 && p.h.s) {
            if(tid == 0 && lo != F0)
                fl |= half_scalar<NR>(p, alpha, lo & ~(size_t)(kVec - 1));
            if(tid == 1 && F1 < hi && F1 >= F0)
                fl |= half_scalar<NR>(p, alpha, F1);
        }
        float_group_pass<NR>(p, fl);
    }
    step_finish<NR>(p, fl, &s_flag);
}

}  // namespace b200
