// Step kernel with a shared-memory ring PER WARP: the same bulk-copy staging
// as staged_step_kernel, but every warp owns its own stages, its own mbarriers
// and issues its own bulk loads and stores, so no CTA-wide barrier sits between
// a tile's loads, its update and its stores.  Warps of a CTA only meet in the
// step prologue and epilogue.  No cluster multicast anywhere.
#pragma once

#include "staged_step.cuh"

namespace b200 {

constexpr int kMaxWarpStages = 8;

// WARPS warps per CTA; a warp-tile is 32*VEC elements; p.stages stages per warp.
template <int NR, int VEC, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
    warp_ring_step_kernel(const __grid_constant__ StepParams p)
{
    extern __shared__ __align__(128) unsigned char stage_mem[];
    __shared__ __align__(8) uint64_t full_bar[WARPS * kMaxWarpStages];
    __shared__ int s_flag;
    __shared__ int s_failed;

    constexpr int TILE = 32 * VEC;
    constexpr uint32_t kStage = (uint32_t)stage_bytes(NR, TILE);
    constexpr uint32_t kOffM = NR * TILE * 2;
    constexpr uint32_t kOffV = kOffM + TILE * 4;
    constexpr uint32_t kOffC = kOffV + TILE * 4;

    const int STAGES = p.stages;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    uint64_t *bars = full_bar + warp * kMaxWarpStages;
    unsigned char *ring = stage_mem + (size_t)warp * STAGES * kStage;

    if(lane == 0)
        for(int s = 0; s < STAGES; s++)
            mbar_init(&bars[s], 1);
    if(tid == 0) {
        s_failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    uint32_t fl = 0;
    if(!step_begin<NR>(p)) {
        const float alpha = step_alpha(p);
        const size_t lo = p.h.o, hi = p.h.o + p.h.s;
        const size_t F0 = (lo + kVec - 1) & ~(size_t)(kVec - 1);
        const size_t F1 = hi & ~(size_t)(kVec - 1);
        const bool any_full = p.h.s && F1 > F0;
        // warp-tiles are cut on multiples of TILE of the flat buffer's index
        const size_t t_first = F0 / TILE;
        const size_t ntiles = any_full ? (F1 - 1) / TILE - t_first + 1 : 0;
        const size_t gw = (size_t)blockIdx.x * WARPS + warp;   // this warp, grid-wide
        const size_t nw = (size_t)gridDim.x * WARPS;
        const size_t nmine = ntiles > gw ? (ntiles - gw + nw - 1) / nw : 0;

        auto tile_start = [&](size_t k) -> size_t {
            const size_t b = (t_first + gw + k * nw) * TILE;
            return b > F0 ? b : F0;
        };
        auto tile_elems = [&](size_t k) -> uint32_t {
            const size_t e = (t_first + gw + k * nw + 1) * TILE;
            return (uint32_t)((e < F1 ? e : F1) - tile_start(k));
        };
        auto issue_loads = [&](size_t k) {  // lane 0 only
            const int s = (int)(k % STAGES);
            const size_t e0 = tile_start(k);
            const size_t l0 = e0 - p.h.A;
            const uint32_t te = tile_elems(k);
            unsigned char *st = ring + (size_t)s * kStage;
            mbar_expect_tx(&bars[s], te * (2u * NR + 12u));
#pragma unroll
            for(int q = 0; q < NR; q++)
                bulk_load(st + q * TILE * 2, p.h.G[q] + e0, te * 2u, &bars[s]);
            bulk_load(st + kOffM, p.h.m + l0, te * 4u, &bars[s]);
            bulk_load(st + kOffV, p.h.v + l0, te * 4u, &bars[s]);
            bulk_load(st + kOffC, p.h.c + l0, te * 4u, &bars[s]);
        };

        if(lane == 0 && !p.force_scalar) {
            fence_proxy_async_all();  // after the peers' announcements
            for(size_t k = 0; k < nmine && k < (size_t)STAGES; k++)
                issue_loads(k);
        }
        __syncwarp();

        bool failed = false;
        for(size_t k = 0; k < nmine && !p.force_scalar; k++) {
            const int s = (int)(k % STAGES);
            const uint32_t parity = (uint32_t)((k / STAGES) & 1);
            unsigned char *st = ring + (size_t)s * kStage;
            const bool ok = mbar_wait(&bars[s], parity, p.timeout_ns);
            if(__any_sync(0xffffffffu, !ok)) {
                failed = true;  // a stage that did not fill is not touched
                break;
            }
            const uint32_t te = tile_elems(k);
            const size_t e0 = tile_start(k);
            if((uint32_t)lane * VEC < te) {
                staged_update<NR, VEC, TILE>(p, alpha, st, lane,
                                             e0 + (size_t)lane * VEC, fl);
                fence_proxy_async_smem();
            }
            __syncwarp();
            if(lane == 0) {
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
            __syncwarp();
        }
        if(lane == 0) {
            bulk_wait_all();          // stores complete, not merely read
            fence_proxy_async_all();  // ... and ordered before the signals below
        }
        if(failed) {
            // loads may still be landing in this warp's stages: bounded wait
            for(int s = 0; s < STAGES; s++) {
                mbar_wait(&bars[s], 0, 1000000ull);
                mbar_wait(&bars[s], 1, 1000000ull);
            }
            if(lane == 0)
                s_failed = 1;
        }

        if(p.force_scalar) {
            const size_t ng = p.h.ngroups;
            for(size_t gid = (size_t)blockIdx.x * (WARPS * 32) + tid; gid < ng;
                gid += (size_t)gridDim.x * (WARPS * 32))
                fl |= half_scalar<NR>(p, alpha, p.h.B + gid * kVec);
        } else if(blockIdx.x == 0 && p.h.s) {
            if(tid == 0 && lo != F0)
                fl |= half_scalar<NR>(p, alpha, lo & ~(size_t)(kVec - 1));
            if(tid == 1 && F1 < hi && F1 >= F0)
                fl |= half_scalar<NR>(p, alpha, F1);
        }
        float_group_pass<NR>(p, fl);
    }
    __syncthreads();
    if(tid == 0 && s_failed) {
        Ctrl *const my = p.ctrl[p.rank];
        if(my)
            atomicCAS(&my->status, 0u, (uint32_t)(-B200OPT_ETIMEOUT));
        if(p.host)
            p.host->where = 3;
    }
    step_finish<NR>(p, fl, &s_flag);
}

}  // namespace b200
