// Host side of the b200opt C ABI (include/b200opt.h): handle management, peer
// wiring, launch of the fused step kernel.  Host-only arithmetic (loss-scale
// policy, bias corrections, flat layout) lives in host_logic.cpp.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include <unistd.h>

#include "fabric.h"
#include "fused_step.cuh"
#include "staged_step.cuh"
#include "nvls_step.cuh"
#include "nccl_path.h"

using namespace b200;

namespace {

constexpr size_t kCtrlBytes = 4096;
// Shard state is padded so that element i of the flat buffer sits at [i - A]
// with A = the shard start rounded down to this many elements: every array
// (gradients, weights, m, v, master) then has the same phase relative to the
// tiles of the step kernels, and interior tiles start on 2 KB / 4 KB boundaries
// whatever the reference's shard boundary r*(n/N) happens to be.
constexpr size_t kStateAlign = 4096;
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block must fit its page");

inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

struct b200opt {
    int rank = 0, nranks = 1, device = 0;
    size_t n_half = 0, n_float = 0;
    // shard geometry
    size_t sh = 0, oh = 0, Ah = 0, sf = 0, of = 0, Af = 0;
    // peer-mapped arena: [Ctrl page | W half | G half | W float | G float]
    char *arena = nullptr;
    size_t arena_bytes = 0;
    size_t off_wh = 0, off_gh = 0, off_wf = 0, off_gf = 0;
    char *peer_arena[kMaxRanks] = {};
    bool peer_is_ipc[kMaxRanks] = {};
    bool peer_seen[kMaxRanks] = {};
    int peers_attached = 0;
    // a peer whose memory this GPU cannot reach counts as attached but keeps a
    // null arena pointer: only the NCCL path can step such a group
    bool peers_reachable = true;
    // arena from the virtual-memory API (shareable by fd, bindable to a
    // multicast object) instead of cudaMalloc
    bool fabric = false;
    FabricMapping fab;
    FabricMapping peer_map[kMaxRanks];
    FabricMulticast mc;
    // local state
    float *mh = nullptr, *vh = nullptr, *ch = nullptr, *mf = nullptr,
          *vf = nullptr;
    char *state = nullptr;  // one allocation holding the five arrays above
    size_t state_bytes = 0;
    size_t state_h_elems = 0, state_f_elems = 0;
    HostResult *host = nullptr;      // pinned + mapped
    HostResult *host_dev = nullptr;  // device alias of `host`
    int iter = 0;
    uint32_t epoch = 0;
    bool serial = false;  // peers share a device: no in-kernel waits
    bool failed = false;
    int num_sms = 0;
    long timeout_ms = 10000;
    long path = B200OPT_PATH_AUTO;
    long ctas_per_sm = 0;  // 0 = built-in default
    long variant = 0;
    long stages = 0;
    long grid = 0;
    long timing = 0;
    long keep_reduced = 0;
    long assume_no_peer_access = 0;  // test aid: wire as if the GPUs had no peer access
    long nccl_crossover = 0;
    uint64_t launches = 0;
    NcclPath *nccl = nullptr;
    bool device_scale = false;   // loss scale lives in the control page
    float device_scale_initial = 0;
    bool step_open = false;      // between b200opt_step_begin and the last bucket
    uint32_t *scale_log = nullptr;
    uint32_t scale_log_cap = 0;
    // b200opt_step_host on one rank: the gradient copy runs on a stream of its own,
    // chunk by chunk, while the step consumes the chunks that have arrived
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t copy_fork = nullptr;
    cudaEvent_t copy_done[16] = {};
    std::string err;
};

namespace {

int fail(b200opt *h, int code, const char *what, cudaError_t ce = cudaSuccess)
{
    if(h) {
        char buf[512];
        if(ce != cudaSuccess)
            snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(ce));
        else
            snprintf(buf, sizeof(buf), "%s", what);
        h->err = buf;
    }
    return code;
}

#define CK(h, call)                                     \
    do {                                                \
        cudaError_t ce_ = (call);                       \
        if(ce_ != cudaSuccess)                          \
            return fail((h), B200OPT_ECUDA, #call, ce_); \
    } while(0)

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev)
    {
        if(cudaGetDevice(&prev) != cudaSuccess)
            prev = -1;
        ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard()
    {
        if(prev >= 0)
            cudaSetDevice(prev);
    }
};

template <typename T>
T *arena_ptr(char *base, size_t off)
{
    return base ? reinterpret_cast<T *>(base + off) : nullptr;
}

// Part of the flat buffers one launch works on: the whole shard, or the shard
// clipped to [first, first + count) of each dtype group (a bucket of a step).
struct StepRange {
    bool whole = true;
    size_t h_first = 0, h_count = 0, f_first = 0, f_count = 0;
};

void clip(size_t o, size_t s, bool whole, size_t first, size_t count, size_t *lo,
          size_t *len)
{
    size_t a = o, b = o + s;
    if(!whole) {
        a = std::max(a, first);
        b = std::min(b, first + count);
    }
    *lo = a;
    *len = b > a ? b - a : 0;
}

void fill_groups(const b200opt *h, StepParams &p, const StepRange &r = StepRange())
{
    for(int q = 0; q < h->nranks; q++) {
        char *base = h->peer_arena[q];
        p.ctrl[q] = arena_ptr<Ctrl>(base, 0);
        p.h.W[q] = arena_ptr<uint16_t>(base, h->off_wh);
        p.h.G[q] = arena_ptr<uint16_t>(base, h->off_gh);
        p.f.W[q] = arena_ptr<float>(base, h->off_wf);
        p.f.G[q] = arena_ptr<float>(base, h->off_gf);
    }
    p.h.m = h->mh;
    p.h.v = h->vh;
    p.h.c = h->ch;
    clip(h->oh, h->sh, r.whole, r.h_first, r.h_count, &p.h.o, &p.h.s);
    p.h.A = h->Ah;
    p.h.B = p.h.o & ~(size_t)(kStateAlign - 1);
    p.h.ngroups = p.h.s ? (p.h.o + p.h.s - p.h.B + kVec - 1) / kVec : 0;
    p.f.m = h->mf;
    p.f.v = h->vf;
    clip(h->of, h->sf, r.whole, r.f_first, r.f_count, &p.f.o, &p.f.s);
    p.f.A = h->Af;
    p.f.B = p.f.o & ~(size_t)(kStateAlign - 1);
    p.f.ngroups = p.f.s ? (p.f.o + p.f.s - p.f.B + kVec - 1) / kVec : 0;
}

template <int NR, int UNR, int MINB>
cudaError_t launch_direct(const StepParams &p, int grid, cudaStream_t st)
{
    fused_step_kernel<NR, UNR, MINB><<<grid, kThreads, 0, st>>>(p);
    return cudaGetLastError();
}

template <int NR>
cudaError_t launch_nvls(const StepParams &p, int grid, cudaStream_t st)
{
    nvls_step_kernel<NR, 3><<<grid, kThreads, 0, st>>>(p);
    return cudaGetLastError();
}

// Tuning knobs of a launch (0 = the variant's default).
struct LaunchTuning {
    long ctas_per_sm = 0;
    long variant = 0;
    long stages = 0;
    long grid = 0;
    bool nvls = false;
};

constexpr int kStagedVec = 4, kStagedThreads = 256;
constexpr int kStagedTile = kStagedVec * kStagedThreads;
constexpr size_t kSmemBudget = 227 * 1024 - 1024;

// Ring depth of the staged kernel for `cps` CTAs per SM: the rings of all CTAs
// resident on an SM must fit its shared memory.  0 if not even one stage fits.
int staged_stages(int nranks, long want, long cps)
{
    const size_t per_stage = stage_bytes(nranks, kStagedTile);
    int stages = (int)want;
    while(stages > 1 && (size_t)stages * per_stage * (size_t)cps > kSmemBudget)
        stages--;
    if(stages > kMaxStages)
        stages = kMaxStages;
    return (size_t)stages * per_stage <= kSmemBudget ? stages : 0;
}

template <int NR>
cudaError_t launch_staged(StepParams p, int num_sms, const LaunchTuning &t,
                          cudaStream_t st)
{
    constexpr int def_stages = 4, def_ctas = 2;
    const long cps = t.ctas_per_sm > 0 ? t.ctas_per_sm : def_ctas;
    const int stages = staged_stages(NR, t.stages > 0 ? t.stages : def_stages, cps);
    if(stages < 1)
        return cudaErrorInvalidValue;
    const size_t smem = (size_t)stages * stage_bytes(NR, kStagedTile);
    auto kern = staged_step_kernel<NR, kStagedVec, kStagedThreads>;
    // opting in to large dynamic shared memory is per device and sticky
    static std::atomic<uint64_t> opted{0};
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if(ce != cudaSuccess)
        return ce;
    if(dev >= 64 || !(opted.load() & (1ull << dev))) {
        ce = cudaFuncSetAttribute(
            kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
        if(ce != cudaSuccess)
            return ce;
        if(dev < 64)
            opted.fetch_or(1ull << dev);
    }
    const size_t tiles_h = (p.h.ngroups * kVec + kStagedTile - 1) / kStagedTile;
    const size_t tiles_f = (p.f.ngroups + kStagedThreads - 1) / kStagedThreads;
    size_t want = std::max<size_t>(std::max(tiles_h, tiles_f), 1);
    const size_t cap = t.grid > 0 ? (size_t)t.grid : (size_t)num_sms * cps;
    const int grid = (int)std::min<size_t>(want, cap);
    p.stages = stages;
    kern<<<grid, kStagedThreads, smem, st>>>(p);
    return cudaGetLastError();
}

// Launch shape: a persistent grid of ctas_per_sm CTAs on every SM, shrunk for
// small inputs so that no CTA starts without work.
//   variant 0: the default of the rank count (staged for one rank, direct else)
//   variant 1: direct 16-byte loads, one 8-element group per thread per trip
//   variant 2: bulk-copy staging through a ring of shared-memory stages
//              (256 threads x 4 elements per tile)
// Measured on B200s at 25.6 M fp16 parameters.  One rank: staged, two CTAs per
// SM, four stages; the direct-load shape is about 4 % slower.  Several ranks
// over NVLink: both shapes land within a few percent of one another (the
// links bind, not the SMs), so the simpler direct kernel is the default there.
// With t.nvls the fp16 group goes through the multicast mapping instead
// (nvls_step_kernel, direct loads only).
cudaError_t launch_step(const StepParams &p, int nranks, int num_sms,
                        const LaunchTuning &t, cudaStream_t st)
{
    const long variant = t.variant > 0 ? t.variant : (nranks == 1 ? 2 : 1);
    if(variant == 2 && !t.nvls) {
        switch(nranks) {
        case 1: return launch_staged<1>(p, num_sms, t, st);
        case 2: return launch_staged<2>(p, num_sms, t, st);
        case 3: return launch_staged<3>(p, num_sms, t, st);
        case 4: return launch_staged<4>(p, num_sms, t, st);
        case 5: return launch_staged<5>(p, num_sms, t, st);
        case 6: return launch_staged<6>(p, num_sms, t, st);
        case 7: return launch_staged<7>(p, num_sms, t, st);
        case 8: return launch_staged<8>(p, num_sms, t, st);
        }
        return cudaErrorInvalidValue;
    }
    const size_t groups = std::max(p.h.ngroups, p.f.ngroups);
    // measured at 25.6 M parameters: 2 CTAs per SM up to four ranks, 3 beyond;
    // the multicast kernel does best with 2
    const long def_ctas = t.nvls ? 2 : (nranks <= 4 ? 2 : 3);
    const long cps = t.ctas_per_sm > 0 ? t.ctas_per_sm : def_ctas;
    size_t want = (groups + (size_t)kThreads - 1) / (size_t)kThreads;
    if(want == 0)
        want = 1;
    const int grid = (int)std::min<size_t>(
        want, t.grid > 0 ? (size_t)t.grid : (size_t)num_sms * cps);
    if(t.nvls) {
        switch(nranks) {
        case 2: return launch_nvls<2>(p, grid, st);
        case 3: return launch_nvls<3>(p, grid, st);
        case 4: return launch_nvls<4>(p, grid, st);
        case 5: return launch_nvls<5>(p, grid, st);
        case 6: return launch_nvls<6>(p, grid, st);
        case 7: return launch_nvls<7>(p, grid, st);
        case 8: return launch_nvls<8>(p, grid, st);
        }
        return cudaErrorInvalidValue;
    }
    switch(nranks) {
    case 1: return launch_direct<1, 1, 3>(p, grid, st);
    case 2: return launch_direct<2, 1, 3>(p, grid, st);
    case 3: return launch_direct<3, 1, 2>(p, grid, st);
    case 4: return launch_direct<4, 1, 2>(p, grid, st);
    case 5: return launch_direct<5, 1, 2>(p, grid, st);
    case 6: return launch_direct<6, 1, 2>(p, grid, st);
    case 7: return launch_direct<7, 1, 2>(p, grid, st);
    case 8: return launch_direct<8, 1, 2>(p, grid, st);
    }
    return cudaErrorInvalidValue;
}

// Would launch_step refuse this combination?  Checked before a step moves any
// counter, so that a refused step leaves the rank in step with its peers.
bool launch_possible(int nranks, const LaunchTuning &t)
{
    if(nranks < 1 || nranks > kMaxRanks)
        return false;
    if(t.nvls)
        return nranks >= 2;
    const long variant = t.variant > 0 ? t.variant : (nranks == 1 ? 2 : 1);
    if(variant == 2) {
        const long cps = t.ctas_per_sm > 0 ? t.ctas_per_sm : 2;
        return staged_stages(nranks, t.stages > 0 ? t.stages : 4, cps) >= 1;
    }
    return variant == 1;
}

LaunchTuning tuning_of(const b200opt *h)
{
    LaunchTuning t;
    t.ctas_per_sm = h->ctas_per_sm;
    t.variant = h->variant;
    t.stages = h->stages;
    t.grid = h->grid;
    return t;
}

LaunchTuning seam_tuning()
{
    LaunchTuning t;
    return t;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace

extern "C" {

const char *b200opt_version(void) { return "b200opt 0.1 sm_100a"; }

const char *b200opt_strerror(int status)
{
    switch(status) {
    case B200OPT_OK: return "ok";
    case B200OPT_EINVAL: return "invalid argument";
    case B200OPT_ECUDA: return "CUDA runtime error";
    case B200OPT_ENOMEM: return "out of memory";
    case B200OPT_ETIMEOUT: return "a peer rank did not arrive in time";
    case B200OPT_ESTATE: return "call not valid in this state";
    case B200OPT_EUNSUPPORTED: return "not supported by this build";
    case B200OPT_ETOOBIG:
        return "size exceeds what this entry point's fixed scratch covers";
    }
    return "unknown status";
}

const char *b200opt_last_error(const b200opt_t *h)
{
    return h ? h->err.c_str() : "";
}

int b200opt_create_ex(b200opt_t **out, int rank, int nranks, int device,
                      size_t n_half, size_t n_float, unsigned flags)
{
    if(!out || nranks < 1 || nranks > kMaxRanks || rank < 0 || rank >= nranks ||
       device < 0 || (flags & ~(B200OPT_CREATE_FABRIC | B200OPT_CREATE_MULTICAST)))
        return B200OPT_EINVAL;
    *out = nullptr;
    int ndev = 0;
    if(cudaGetDeviceCount(&ndev) != cudaSuccess || device >= ndev)
        return B200OPT_ECUDA;

    b200opt *h = new(std::nothrow) b200opt;
    if(!h)
        return B200OPT_ENOMEM;
    h->rank = rank;
    h->nranks = nranks;
    h->device = device;
    h->n_half = n_half;
    h->n_float = n_float;
    h->fabric = flags != 0;
    // the reference's partition: plain integer division
    // (src/cuda/cuda_optimizer.cpp:85-86,157-158 of the Saga tree)
    h->sh = n_half / nranks;
    h->oh = h->sh * rank;
    h->Ah = h->oh & ~(size_t)(kStateAlign - 1);
    h->sf = n_float / nranks;
    h->of = h->sf * rank;
    h->Af = h->of & ~(size_t)(kStateAlign - 1);

    h->off_wh = kCtrlBytes;
    h->off_gh = h->off_wh + round_up(n_half * 2, 256);
    h->off_wf = h->off_gh + round_up(n_half * 2, 256);
    h->off_gf = h->off_wf + round_up(n_float * 4, 256);
    h->arena_bytes = h->off_gf + round_up(n_float * 4, 256);

    DeviceGuard guard(device);
    int rc = B200OPT_OK;
    cudaError_t ce = cudaSuccess;
    std::string ferr;
    do {
        if(!guard.ok) {
            rc = B200OPT_ECUDA;
            break;
        }
        cudaDeviceProp prop;
        if((ce = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) {
            rc = B200OPT_ECUDA;
            break;
        }
        h->num_sms = prop.multiProcessorCount;
        if(h->fabric) {
            // every rank of the group rounds to the same size, so that the
            // arenas can be bound to one multicast object at offset 0
            size_t gran = 0;
            if((rc = fabric_granularity(device, nranks, true, &gran, &ferr)) != 0 &&
               (rc = fabric_granularity(device, nranks, false, &gran, &ferr)) != 0)
                break;
            h->arena_bytes = round_up(h->arena_bytes, gran);
            if((rc = fabric_alloc(&h->fab, device, h->arena_bytes, &ferr)) != 0)
                break;
            h->arena = reinterpret_cast<char *>(h->fab.va);
        } else if((ce = cudaMalloc(&h->arena, h->arena_bytes)) != cudaSuccess) {
            rc = B200OPT_ENOMEM;
            break;
        }
        if((ce = cudaMemset(h->arena, 0, h->arena_bytes)) != cudaSuccess) {
            rc = B200OPT_ECUDA;
            break;
        }
        // shard state, padded so that element i of the flat buffer sits at [i - A]
        h->state_h_elems = h->sh ? round_up(h->oh + h->sh - h->Ah, kVec) : 0;
        h->state_f_elems = h->sf ? round_up(h->of + h->sf - h->Af, kVec) : 0;
        // one allocation for all shard state: [m | v | master | m32 | v32]
        {
            const size_t hb = round_up(h->state_h_elems * 4, 256);
            const size_t fb = round_up(h->state_f_elems * 4, 256);
            h->state_bytes = 3 * hb + 2 * fb;
            if(h->state_bytes) {
                if((ce = cudaMalloc(&h->state, h->state_bytes)) != cudaSuccess) {
                    rc = B200OPT_ENOMEM;
                    break;
                }
                if((ce = cudaMemset(h->state, 0, h->state_bytes)) != cudaSuccess) {
                    rc = B200OPT_ECUDA;
                    break;
                }
                if(hb) {
                    h->mh = (float *)(h->state);
                    h->vh = (float *)(h->state + hb);
                    h->ch = (float *)(h->state + 2 * hb);
                }
                if(fb) {
                    h->mf = (float *)(h->state + 3 * hb);
                    h->vf = (float *)(h->state + 3 * hb + fb);
                }
            }
        }
        if((ce = cudaHostAlloc(&h->host, sizeof(HostResult),
                               cudaHostAllocMapped | cudaHostAllocPortable)) !=
           cudaSuccess) {
            rc = B200OPT_ENOMEM;
            break;
        }
        memset(h->host, 0, sizeof(HostResult));
        if((ce = cudaHostGetDevicePointer((void **)&h->host_dev, h->host, 0)) !=
           cudaSuccess) {
            rc = B200OPT_ECUDA;
            break;
        }
        if((ce = cudaDeviceSynchronize()) != cudaSuccess) {
            rc = B200OPT_ECUDA;
            break;
        }
    } while(0);
    if(rc) {
        (void)ce;
        cudaGetLastError();
        b200opt_destroy(h);
        return rc;
    }
    h->peer_arena[rank] = h->arena;
    h->peers_attached = 1;
    *out = h;
    return B200OPT_OK;
}

int b200opt_create(b200opt_t **out, int rank, int nranks, int device,
                   size_t n_half, size_t n_float)
{
    return b200opt_create_ex(out, rank, nranks, device, n_half, n_float, 0);
}

int b200opt_destroy(b200opt_t *h)
{
    if(!h)
        return B200OPT_EINVAL;
    DeviceGuard guard(h->device);
    cudaDeviceSynchronize();
    if(h->nccl)
        nccl_path_destroy(h->nccl);
    // the multicast view goes first: unmap, unbind this GPU's memory, drop the
    // handle; only then the memory that was bound to it
    fabric_mc_release(&h->mc);
    for(int q = 0; q < h->nranks; q++) {
        if(q == h->rank || !h->peer_arena[q])
            continue;
        if(h->peer_is_ipc[q])
            cudaIpcCloseMemHandle(h->peer_arena[q]);
        fabric_unmap(&h->peer_map[q]);
    }
    if(h->fabric)
        fabric_unmap(&h->fab);
    else
        cudaFree(h->arena);
    cudaFree(h->state);
    cudaFree(h->scale_log);
    if(h->copy_stream) {
        cudaStreamDestroy(h->copy_stream);
        cudaEventDestroy(h->copy_fork);
        for(cudaEvent_t e : h->copy_done)
            if(e)
                cudaEventDestroy(e);
    }
    if(h->host)
        cudaFreeHost(h->host);
    cudaGetLastError();
    delete h;
    return B200OPT_OK;
}

int b200opt_attach_local(b200opt_t *h, int peer_rank, b200opt_t *peer)
{
    if(!h || !peer || peer_rank < 0 || peer_rank >= h->nranks ||
       peer_rank == h->rank || peer->rank != peer_rank ||
       peer->nranks != h->nranks)
        return B200OPT_EINVAL;
    if(peer->n_half != h->n_half || peer->n_float != h->n_float)
        return fail(h, B200OPT_EINVAL, "peer was created with other sizes");
    if(peer->fabric != h->fabric)
        return fail(h, B200OPT_EINVAL, "peer was created with other creation flags");
    if(h->peer_seen[peer_rank])
        return fail(h, B200OPT_ESTATE, "peer already attached");
    bool reachable = true;
    if(peer->device == h->device) {
        h->serial = true;
    } else {
        DeviceGuard guard(h->device);
        int can = 0;
        CK(h, cudaDeviceCanAccessPeer(&can, h->device, peer->device));
        if(h->assume_no_peer_access)
            can = 0;
        if(!can) {
            // counted as attached without memory: the NCCL path can still step
            reachable = false;
        } else if(h->fabric) {
            std::string err;
            int rc = fabric_grant(peer->fab, h->device, &err);
            if(rc)
                return fail(h, rc, err.c_str());
        } else {
            cudaError_t ce = cudaDeviceEnablePeerAccess(peer->device, 0);
            if(ce == cudaErrorPeerAccessAlreadyEnabled)
                cudaGetLastError();
            else if(ce != cudaSuccess)
                return fail(h, B200OPT_ECUDA, "cudaDeviceEnablePeerAccess", ce);
        }
    }
    if(reachable)
        h->peer_arena[peer_rank] = peer->arena;
    else
        h->peers_reachable = false;
    h->peer_seen[peer_rank] = true;
    h->peers_attached++;
    return B200OPT_OK;
}

static int group_multicast(b200opt_t **hs, int nranks)
{
    // rank 0 creates the object; the others take their own reference to it
    // through a file descriptor, exactly as separate processes would
    b200opt *h0 = hs[0];
    std::string err;
    int rc = fabric_mc_create(&h0->mc, nranks, h0->arena_bytes, &err);
    if(rc)
        return fail(h0, rc, err.c_str());
    int fd = -1;
    rc = fabric_export_fd(h0->mc.mc, &fd, &err);
    if(rc)
        return fail(h0, rc, err.c_str());
    for(int r = 1; r < nranks && !rc; r++) {
        DeviceGuard guard(hs[r]->device);
        rc = fabric_mc_import(&hs[r]->mc, fd, hs[r]->arena_bytes, &err);
        if(rc)
            fail(hs[r], rc, err.c_str());
    }
    close(fd);
    for(int r = 0; r < nranks && !rc; r++) {
        DeviceGuard guard(hs[r]->device);
        rc = fabric_mc_add_device(&hs[r]->mc, hs[r]->device, &err);
        if(rc)
            fail(hs[r], rc, err.c_str());
    }
    for(int r = 0; r < nranks && !rc; r++) {
        DeviceGuard guard(hs[r]->device);
        rc = fabric_mc_bind(&hs[r]->mc, hs[r]->fab, hs[r]->device, &err);
        if(rc)
            fail(hs[r], rc, err.c_str());
    }
    return rc;
}

int b200opt_create_group_ex(b200opt_t **out, int nranks, const int *devices,
                            size_t n_half, size_t n_float, unsigned flags)
{
    if(!out || !devices || nranks < 1 || nranks > kMaxRanks)
        return B200OPT_EINVAL;
    for(int r = 0; r < nranks; r++)
        out[r] = nullptr;
    bool any_shared = false;
    for(int r = 0; r < nranks; r++)
        for(int q = 0; q < r; q++)
            any_shared |= devices[r] == devices[q];
    if((flags & B200OPT_CREATE_MULTICAST) && (any_shared || nranks < 2))
        return B200OPT_EUNSUPPORTED;
    int rc = B200OPT_OK;
    for(int r = 0; r < nranks && !rc; r++)
        rc = b200opt_create_ex(&out[r], r, nranks, devices[r], n_half, n_float,
                               flags);
    for(int r = 0; r < nranks && !rc; r++)
        for(int q = 0; q < nranks && !rc; q++)
            if(q != r)
                rc = b200opt_attach_local(out[r], q, out[q]);
    if(!rc && any_shared)
        for(int r = 0; r < nranks; r++)
            out[r]->serial = true;
    if(!rc && (flags & B200OPT_CREATE_MULTICAST))
        rc = group_multicast(out, nranks);
    if(rc) {
        for(int r = 0; r < nranks; r++) {
            if(out[r])
                b200opt_destroy(out[r]);
            out[r] = nullptr;
        }
    }
    return rc;
}

int b200opt_create_group(b200opt_t **out, int nranks, const int *devices,
                         size_t n_half, size_t n_float)
{
    return b200opt_create_group_ex(out, nranks, devices, n_half, n_float, 0);
}

int b200opt_ipc_export(b200opt_t *h, void *handle_out)
{
    if(!h || !handle_out)
        return B200OPT_EINVAL;
    if(h->fabric)
        return fail(h, B200OPT_EUNSUPPORTED,
                    "this arena is shared by file descriptor (b200opt_fd_export)");
    static_assert(sizeof(cudaIpcMemHandle_t) == B200OPT_IPC_HANDLE_BYTES,
                  "IPC handle size");
    DeviceGuard guard(h->device);
    cudaIpcMemHandle_t mh;
    CK(h, cudaIpcGetMemHandle(&mh, h->arena));
    memcpy(handle_out, &mh, sizeof(mh));
    return B200OPT_OK;
}

int b200opt_ipc_attach(b200opt_t *h, int peer_rank, const void *handle)
{
    if(!h || !handle || peer_rank < 0 || peer_rank >= h->nranks ||
       peer_rank == h->rank)
        return B200OPT_EINVAL;
    if(h->peer_seen[peer_rank])
        return fail(h, B200OPT_ESTATE, "peer already attached");
    DeviceGuard guard(h->device);
    cudaIpcMemHandle_t mh;
    memcpy(&mh, handle, sizeof(mh));
    void *p = nullptr;
    cudaError_t ce = h->assume_no_peer_access
                         ? cudaErrorPeerAccessUnsupported
                         : cudaIpcOpenMemHandle(&p, mh, cudaIpcMemLazyEnablePeerAccess);
    if(ce == cudaErrorPeerAccessUnsupported) {
        // counted as attached without memory: the NCCL path can still step
        cudaGetLastError();
        h->peers_reachable = false;
    } else if(ce != cudaSuccess) {
        return fail(h, B200OPT_ECUDA, "cudaIpcOpenMemHandle", ce);
    } else {
        h->peer_arena[peer_rank] = (char *)p;
        h->peer_is_ipc[peer_rank] = true;
    }
    h->peer_seen[peer_rank] = true;
    h->peers_attached++;
    return B200OPT_OK;
}

int b200opt_fd_export(b200opt_t *h, int *fd)
{
    if(!h || !fd)
        return B200OPT_EINVAL;
    if(!h->fabric)
        return fail(h, B200OPT_EUNSUPPORTED,
                    "this arena is shared by CUDA IPC handle (b200opt_ipc_export)");
    DeviceGuard guard(h->device);
    std::string err;
    int rc = fabric_export_fd(h->fab.mem, fd, &err);
    return rc ? fail(h, rc, err.c_str()) : B200OPT_OK;
}

int b200opt_fd_attach(b200opt_t *h, int peer_rank, int fd)
{
    if(!h || fd < 0 || peer_rank < 0 || peer_rank >= h->nranks ||
       peer_rank == h->rank)
        return B200OPT_EINVAL;
    if(!h->fabric)
        return fail(h, B200OPT_EUNSUPPORTED, "created without B200OPT_CREATE_FABRIC");
    if(h->peer_seen[peer_rank])
        return fail(h, B200OPT_ESTATE, "peer already attached");
    DeviceGuard guard(h->device);
    std::string err;
    int rc = fabric_import(&h->peer_map[peer_rank], fd, h->device, h->arena_bytes,
                           &err);
    if(rc)
        return fail(h, rc, err.c_str());
    h->peer_arena[peer_rank] = reinterpret_cast<char *>(h->peer_map[peer_rank].va);
    h->peer_seen[peer_rank] = true;
    h->peers_attached++;
    return B200OPT_OK;
}

int b200opt_multicast_supported(int device, int *yes)
{
    if(!yes || device < 0)
        return B200OPT_EINVAL;
    DeviceGuard guard(device);
    bool y = false;
    std::string err;
    int rc = fabric_multicast_supported(device, &y, &err);
    *yes = y ? 1 : 0;
    return rc;
}

int b200opt_mc_create(b200opt_t *h, int *fd)
{
    if(!h || !fd)
        return B200OPT_EINVAL;
    if(!h->fabric || h->nranks < 2 || h->serial)
        return fail(h, B200OPT_EUNSUPPORTED,
                    "a multicast object needs B200OPT_CREATE_FABRIC and one GPU per rank");
    if(h->mc.mc)
        return fail(h, B200OPT_ESTATE, "multicast object already present");
    DeviceGuard guard(h->device);
    std::string err;
    int rc = fabric_mc_create(&h->mc, h->nranks, h->arena_bytes, &err);
    if(!rc)
        rc = fabric_export_fd(h->mc.mc, fd, &err);
    if(!rc)
        rc = fabric_mc_add_device(&h->mc, h->device, &err);
    if(rc) {
        fabric_mc_release(&h->mc);
        return fail(h, rc, err.c_str());
    }
    return B200OPT_OK;
}

int b200opt_mc_join(b200opt_t *h, int fd)
{
    if(!h || fd < 0)
        return B200OPT_EINVAL;
    if(!h->fabric || h->nranks < 2 || h->serial)
        return fail(h, B200OPT_EUNSUPPORTED,
                    "a multicast object needs B200OPT_CREATE_FABRIC and one GPU per rank");
    if(h->mc.mc)
        return fail(h, B200OPT_ESTATE, "multicast object already present");
    DeviceGuard guard(h->device);
    std::string err;
    int rc = fabric_mc_import(&h->mc, fd, h->arena_bytes, &err);
    if(!rc)
        rc = fabric_mc_add_device(&h->mc, h->device, &err);
    if(rc) {
        fabric_mc_release(&h->mc);
        return fail(h, rc, err.c_str());
    }
    return B200OPT_OK;
}

int b200opt_mc_bind(b200opt_t *h)
{
    if(!h)
        return B200OPT_EINVAL;
    if(!h->mc.mc || h->mc.bound)
        return fail(h, B200OPT_ESTATE,
                    "b200opt_mc_create / b200opt_mc_join first, and bind once");
    DeviceGuard guard(h->device);
    std::string err;
    int rc = fabric_mc_bind(&h->mc, h->fab, h->device, &err);
    if(rc) {
        fabric_mc_release(&h->mc);
        return fail(h, rc, err.c_str());
    }
    return B200OPT_OK;
}

int b200opt_nccl_unique_id(void *unique_id_out)
{
    if(!unique_id_out)
        return B200OPT_EINVAL;
    return nccl_path_unique_id(unique_id_out);
}

int b200opt_nccl_init(b200opt_t *h, const void *unique_id)
{
    if(!h || !unique_id)
        return B200OPT_EINVAL;
    if(h->nccl)
        return fail(h, B200OPT_ESTATE, "NCCL communicator already created");
    DeviceGuard guard(h->device);
    std::string err;
    int rc = nccl_path_create(&h->nccl, h->rank, h->nranks, unique_id, &err);
    if(rc)
        return fail(h, rc, err.c_str());
    return B200OPT_OK;
}

int b200opt_buffers(b200opt_t *h, int dtype, void **weights, void **gradients,
                    size_t *n)
{
    if(!h || (dtype != B200OPT_HALF && dtype != B200OPT_FLOAT))
        return B200OPT_EINVAL;
    const bool half = dtype == B200OPT_HALF;
    if(weights)
        *weights = h->arena + (half ? h->off_wh : h->off_wf);
    if(gradients)
        *gradients = h->arena + (half ? h->off_gh : h->off_gf);
    if(n)
        *n = half ? h->n_half : h->n_float;
    return B200OPT_OK;
}

int b200opt_init_master(b200opt_t *h, void *stream)
{
    if(!h)
        return B200OPT_EINVAL;
    DeviceGuard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    if(h->state_h_elems) {
        CK(h, cudaMemsetAsync(h->mh, 0, h->state_h_elems * 4, st));
        CK(h, cudaMemsetAsync(h->vh, 0, h->state_h_elems * 4, st));
        CK(h, cudaMemsetAsync(h->ch, 0, h->state_h_elems * 4, st));
        const int grid = (int)std::min<size_t>((h->sh + 255) / 256,
                                               (size_t)h->num_sms * 8);
        init_master_kernel<<<grid, 256, 0, st>>>(
            arena_ptr<uint16_t>(h->arena, h->off_wh), h->ch, h->oh, h->sh,
            h->Ah);
        CK(h, cudaGetLastError());
        h->launches++;
    }
    if(h->state_f_elems) {
        CK(h, cudaMemsetAsync(h->mf, 0, h->state_f_elems * 4, st));
        CK(h, cudaMemsetAsync(h->vf, 0, h->state_f_elems * 4, st));
    }
    h->iter = 0;
    return B200OPT_OK;
}

static int step_impl(b200opt_t *h, float lr, float l2_lambda, float scale,
                     bool device_scale, void *stream,
                     const StepRange &range = StepRange(), bool begins = true,
                     bool last = true)
{
    if(!h)
        return B200OPT_EINVAL;
    if(device_scale && !h->device_scale)
        return fail(h, B200OPT_ESTATE,
                    "b200opt_device_scale_enable has not been called");
    if(h->failed)
        return fail(h, B200OPT_ESTATE,
                    "an earlier step timed out; the handle is unusable");
    if(h->peers_attached != h->nranks)
        return fail(h, B200OPT_ESTATE, "not every peer rank is attached");
    // Everything that can refuse the call is checked before any counter moves:
    // a rank whose step was refused must not run one epoch and one Adam
    // iteration ahead of its peers.
    int path = B200OPT_PATH_PEER;
    int rc = b200opt_choose_path((int)h->path, h->nranks, h->serial ? 1 : 0,
                                 h->peers_reachable ? 1 : 0, h->nccl ? 1 : 0,
                                 h->mc.va ? 1 : 0, h->n_half,
                                 (size_t)h->nccl_crossover, &path);
    if(rc == B200OPT_ESTATE)
        return fail(h, rc,
                    (int)h->path == B200OPT_PATH_NVLS
                        ? "multicast path selected but no multicast object is bound"
                        : "NCCL path selected but b200opt_nccl_init was not called");
    if(rc)
        return fail(h, rc,
                    "no collective path is usable: this GPU cannot reach a peer's "
                    "memory and there is no NCCL communicator (or the requested "
                    "path needs one GPU per rank)");
    const bool use_nccl = path == B200OPT_PATH_NCCL;
    LaunchTuning tune = tuning_of(h);
    tune.nvls = path == B200OPT_PATH_NVLS;
    if(use_nccl) {
        if(!range.whole)
            return fail(h, B200OPT_EUNSUPPORTED,
                        "bucketed steps need a peer-memory path");
        if(device_scale)
            return fail(h, B200OPT_EUNSUPPORTED,
                        "the device-resident loss scale needs a peer-memory path");
    }
    if(!launch_possible(use_nccl ? 1 : h->nranks, tune))
        return fail(h, B200OPT_EINVAL,
                    "kernel variant / stage options do not fit this rank count");
    DeviceGuard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;

    // src/cuda/cuda_optimizer.cpp:150-152,169 of the Saga tree
    if(begins)
        ++h->iter;
    const int iter = h->iter;
    StepParams p;
    memset(&p, 0, sizeof(p));
    b200opt_bias_corrections(iter, &p.b1t, &p.b2t);
    p.alpha = 1.0f / scale;
    p.device_scale = device_scale ? 1 : 0;
    p.scale_log = h->scale_log;
    p.scale_log_cap = h->scale_log_cap;
    p.lr = lr;
    p.l2 = l2_lambda;
    p.rank = h->rank;
    p.epoch = ++h->epoch;
    p.timeout_ns = (unsigned long long)h->timeout_ms * 1000000ull;
    p.host = h->host_dev;
    p.timing = h->timing ? 1 : 0;

    if(use_nccl) {
        // reduce-scatter in place, Adam on the local shard, all-gather, flag sum
        std::string err;
        uint16_t *wh = arena_ptr<uint16_t>(h->arena, h->off_wh);
        uint16_t *gh = arena_ptr<uint16_t>(h->arena, h->off_gh);
        float *wf = arena_ptr<float>(h->arena, h->off_wf);
        float *gf = arena_ptr<float>(h->arena, h->off_gf);
        Ctrl *ctrl = arena_ptr<Ctrl>(h->arena, 0);
        rc = nccl_path_reduce_scatter(h->nccl, gh, h->sh, gf, h->sf, st, &err);
        if(rc)
            return fail(h, rc, err.c_str());
        // one-rank view of this rank's own memory: the shard now holds the sum
        fill_groups(h, p);
        for(int q = 0; q < kMaxRanks; q++) {
            p.ctrl[q] = nullptr;
            p.h.W[q] = nullptr;
            p.h.G[q] = nullptr;
            p.f.W[q] = nullptr;
            p.f.G[q] = nullptr;
        }
        p.rank = 0;
        p.ctrl[0] = ctrl;
        p.h.W[0] = wh;
        p.h.G[0] = gh;
        p.f.W[0] = wf;
        p.f.G[0] = gf;
        p.host = nullptr;
        p.timing = 0;
        p.flags_dev = ctrl->coll_flags;
        p.barrier = 0;
        CK(h, launch_step(p, 1, h->num_sms, tune, st));
        rc = nccl_path_all_gather_and_flags(h->nccl, wh, h->sh, wf, h->sf,
                                            ctrl->coll_flags, st, &err);
        if(rc)
            return fail(h, rc, err.c_str());
        CK(h, cudaMemcpyAsync(&h->host->range, ctrl->coll_flags, 12,
                              cudaMemcpyDeviceToHost, st));
        h->launches += 6;
        return B200OPT_OK;
    }

    fill_groups(h, p, range);
    p.partial = last ? 0 : 1;
    p.barrier = (h->nranks > 1 && !h->serial) ? 1 : 0;
    if(tune.nvls) {
        p.keep_reduced = h->keep_reduced ? 1 : 0;
        p.mcG = reinterpret_cast<const uint16_t *>(h->mc.va + h->off_gh);
        p.mcW = reinterpret_cast<uint16_t *>(h->mc.va + h->off_wh);
    }
    const cudaError_t ce = launch_step(p, h->nranks, h->num_sms, tune, st);
    if(ce != cudaSuccess) {
        // nothing was enqueued: stay in step with the peers
        --h->epoch;
        if(begins)
            --h->iter;
        return fail(h, B200OPT_ECUDA, "launch of the step kernel", ce);
    }
    h->launches++;
    return B200OPT_OK;
}

int b200opt_step(b200opt_t *h, float lr, float l2_lambda, float scale,
                 void *stream)
{
    if(h && h->step_open)
        return fail(h, B200OPT_ESTATE, "a bucketed step is open");
    return step_impl(h, lr, l2_lambda, scale, false, stream);
}

int b200opt_step_begin(b200opt_t *h)
{
    if(!h)
        return B200OPT_EINVAL;
    if(h->step_open)
        return fail(h, B200OPT_ESTATE, "the previous bucketed step has no last bucket yet");
    ++h->iter;
    h->step_open = true;
    return B200OPT_OK;
}

int b200opt_step_bucket(b200opt_t *h, size_t half_first, size_t half_count,
                        size_t float_first, size_t float_count, float lr,
                        float l2_lambda, float scale, void *stream, int last)
{
    if(!h)
        return B200OPT_EINVAL;
    if(!h->step_open)
        return fail(h, B200OPT_ESTATE, "b200opt_step_begin has not been called");
    if(half_first + half_count > h->n_half || float_first + float_count > h->n_float)
        return fail(h, B200OPT_EINVAL, "bucket reaches beyond the flat buffer");
    StepRange r;
    r.whole = false;
    r.h_first = half_first;
    r.h_count = half_count;
    r.f_first = float_first;
    r.f_count = float_count;
    const int rc = step_impl(h, lr, l2_lambda, scale, false, stream, r, false, last != 0);
    if(rc == B200OPT_OK && last)
        h->step_open = false;
    return rc;
}

int b200opt_step_device_scale(b200opt_t *h, float lr, float l2_lambda,
                              void *stream)
{
    return step_impl(h, lr, l2_lambda, 1.0f, true, stream);
}

int b200opt_device_scale_enable(b200opt_t *h, float initial_scale, int policy,
                                int interval, size_t log_capacity)
{
    if(!h || !(initial_scale > 0) ||
       (policy != B200OPT_POLICY_REFERENCE && policy != B200OPT_POLICY_INTERVAL) ||
       (policy == B200OPT_POLICY_INTERVAL && interval < 1) ||
       log_capacity > (1u << 24))
        return B200OPT_EINVAL;
    if(h->serial)
        return fail(h, B200OPT_EUNSUPPORTED,
                    "serial mode forms the flag sums on the host");
    DeviceGuard guard(h->device);
    CK(h, cudaDeviceSynchronize());
    if(h->scale_log) {
        cudaFree(h->scale_log);
        h->scale_log = nullptr;
        h->scale_log_cap = 0;
    }
    if(log_capacity) {
        if(cudaMalloc(&h->scale_log, log_capacity * 16) != cudaSuccess)
            return fail(h, B200OPT_ENOMEM, "cudaMalloc of the scale log");
        CK(h, cudaMemset(h->scale_log, 0, log_capacity * 16));
        h->scale_log_cap = (uint32_t)log_capacity;
    }
    Ctrl *ctrl = arena_ptr<Ctrl>(h->arena, 0);
    struct {
        float scale;
        uint32_t policy;
        int32_t clean;
        int32_t interval;
        uint32_t log_pos;
    } init = {initial_scale, (uint32_t)policy, 0, interval, 0};
    static_assert(offsetof(Ctrl, log_pos) - offsetof(Ctrl, scale) == 16,
                  "device scale fields are contiguous");
    CK(h, cudaMemcpy(&ctrl->scale, &init, sizeof(init), cudaMemcpyHostToDevice));
    h->device_scale = true;
    h->device_scale_initial = initial_scale;
    h->host->scale_bits = 0;
    return B200OPT_OK;
}

int b200opt_device_scale_ptr(b200opt_t *h, const float **scale_dev)
{
    if(!h || !scale_dev)
        return B200OPT_EINVAL;
    if(!h->device_scale)
        return fail(h, B200OPT_ESTATE,
                    "b200opt_device_scale_enable has not been called");
    *scale_dev = &arena_ptr<Ctrl>(h->arena, 0)->scale;
    return B200OPT_OK;
}

int b200opt_device_scale_peek(b200opt_t *h, float *scale, uint32_t *step)
{
    if(!h)
        return B200OPT_EINVAL;
    if(!h->device_scale)
        return fail(h, B200OPT_ESTATE,
                    "b200opt_device_scale_enable has not been called");
    // no wait and no CUDA call: the pinned page as the last finished kernel left it
    const volatile HostResult *hr = h->host;
    if(hr->status) {
        h->failed = true;
        return fail(h, B200OPT_ETIMEOUT, "a step gave up waiting for a peer rank");
    }
    const uint32_t bits = hr->scale_bits;
    if(step)
        *step = hr->epoch;
    if(scale) {
        if(bits)
            memcpy(scale, &bits, 4);
        else
            *scale = h->device_scale_initial;  // no step has finished yet
    }
    return B200OPT_OK;
}

int b200opt_device_scale_read(b200opt_t *h, void *stream, float *scale,
                              uint32_t *log_out, size_t capacity, size_t *count)
{
    if(!h)
        return B200OPT_EINVAL;
    if(!h->device_scale)
        return fail(h, B200OPT_ESTATE,
                    "b200opt_device_scale_enable has not been called");
    DeviceGuard guard(h->device);
    CK(h, cudaStreamSynchronize((cudaStream_t)stream));
    if(h->host->status) {
        h->failed = true;
        return fail(h, B200OPT_ETIMEOUT, "a step gave up waiting for a peer rank");
    }
    Ctrl *ctrl = arena_ptr<Ctrl>(h->arena, 0);
    struct {
        float scale;
        uint32_t policy;
        int32_t clean;
        int32_t interval;
        uint32_t log_pos;
    } cur;
    CK(h, cudaMemcpy(&cur, &ctrl->scale, sizeof(cur), cudaMemcpyDeviceToHost));
    if(scale)
        *scale = cur.scale;
    // the ring holds the last scale_log_cap steps, oldest first
    size_t have = std::min<size_t>(cur.log_pos, h->scale_log_cap);
    if(count)
        *count = have;
    if(log_out && have) {
        if(capacity < have)
            return B200OPT_EINVAL;
        const size_t cap = h->scale_log_cap;
        const size_t first = (cur.log_pos - have) % cap;
        const size_t run = std::min(have, cap - first);
        CK(h, cudaMemcpy(log_out, h->scale_log + 4 * first, run * 16,
                         cudaMemcpyDeviceToHost));
        if(run < have)
            CK(h, cudaMemcpy(log_out + 4 * run, h->scale_log, (have - run) * 16,
                             cudaMemcpyDeviceToHost));
    }
    return B200OPT_OK;
}

int b200opt_flags(b200opt_t *h, void *stream, uint32_t flags_out[3])
{
    if(!h || !flags_out)
        return B200OPT_EINVAL;
    DeviceGuard guard(h->device);
    CK(h, cudaStreamSynchronize((cudaStream_t)stream));
    if(h->host->status) {
        h->failed = true;
        char buf[160];
        snprintf(buf, sizeof(buf),
                 "step %u: rank %d gave up waiting for rank %u (%s)",
                 h->epoch, h->rank, h->host->peer,
                 h->host->where == 1 ? "gradients not announced"
                                     : "completion not announced");
        return fail(h, B200OPT_ETIMEOUT, buf);
    }
    if(h->serial && h->nranks > 1) {
        // every rank's launch left its flag word in this rank's slot array
        uint32_t words[32];
        const Ctrl *c = arena_ptr<Ctrl>(h->arena, 0);
        CK(h, cudaMemcpy(words, c->flagword[h->epoch & 1], sizeof(words),
                         cudaMemcpyDeviceToHost));
        flags_out[0] = flags_out[1] = flags_out[2] = 0;
        for(int q = 0; q < h->nranks; q++) {
            if(!(words[q] & kFlagValid))
                return fail(h, B200OPT_ESTATE,
                            "serial mode: not every rank has stepped yet");
            flags_out[0] += (words[q] & kFlagRange) ? 1 : 0;
            flags_out[1] += (words[q] & kFlagInf) ? 1 : 0;
            flags_out[2] += (words[q] & kFlagNan) ? 1 : 0;
        }
        CK(h, cudaMemset((void *)c->flagword[h->epoch & 1], 0, sizeof(words)));
    } else {
        flags_out[0] = h->host->range;
        flags_out[1] = h->host->inf;
        flags_out[2] = h->host->nan;
    }
    h->host->range = h->host->inf = h->host->nan = 0;
    return B200OPT_OK;
}

int b200opt_step_host(b200opt_t *h, const void *grads_half,
                      const void *grads_float, float lr, float l2_lambda,
                      float scale, void *stream, uint32_t flags_out[3])
{
    if(!h || !flags_out)
        return B200OPT_EINVAL;
    if((h->n_half && !grads_half) || (h->n_float && !grads_float))
        return B200OPT_EINVAL;
    DeviceGuard guard(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    // One rank, a buffer worth splitting: the copy is cut into chunks on a copy
    // stream and the step is issued as one bucket per chunk behind it, so that the
    // update of a chunk overlaps the transfer of the next ones.  Buckets of one
    // step give bit for bit the result of one whole step.
    constexpr size_t kPipelineMin = (size_t)1 << 22;  // fp16 elements
    constexpr int kChunks = 8;
    if(h->nranks == 1 && !h->serial && h->n_half >= kPipelineMin && !h->step_open &&
       !h->failed) {
        if(!h->copy_stream) {
            CK(h, cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking));
            CK(h, cudaEventCreateWithFlags(&h->copy_fork, cudaEventDisableTiming));
            for(int c = 0; c < kChunks; c++)
                CK(h, cudaEventCreateWithFlags(&h->copy_done[c], cudaEventDisableTiming));
        }
        // the copy may not overtake what the caller's stream still does with the buffers
        CK(h, cudaEventRecord(h->copy_fork, st));
        CK(h, cudaStreamWaitEvent(h->copy_stream, h->copy_fork, 0));
        int rc = b200opt_step_begin(h);
        if(rc)
            return rc;
        const size_t per = (h->n_half / kChunks + 4095) & ~(size_t)4095;
        size_t first = 0;
        for(int c = 0; c < kChunks && rc == B200OPT_OK; c++) {
            const bool last = c == kChunks - 1;
            const size_t count = last ? h->n_half - first : std::min(per, h->n_half - first);
            if(c == 0 && h->n_float)
                CK(h, cudaMemcpyAsync(h->arena + h->off_gf, grads_float, h->n_float * 4,
                                      cudaMemcpyHostToDevice, h->copy_stream));
            if(count)
                CK(h, cudaMemcpyAsync(h->arena + h->off_gh + first * 2,
                                      (const char *)grads_half + first * 2, count * 2,
                                      cudaMemcpyHostToDevice, h->copy_stream));
            CK(h, cudaEventRecord(h->copy_done[c], h->copy_stream));
            CK(h, cudaStreamWaitEvent(st, h->copy_done[c], 0));
            // the fp32 group travels with the first chunk
            rc = b200opt_step_bucket(h, first, count, 0, c == 0 ? h->n_float : 0, lr, l2_lambda,
                                     scale, stream, last ? 1 : 0);
            first += count;
        }
        if(rc)
            return rc;
        return b200opt_flags(h, stream, flags_out);
    }
    if(h->n_half)
        CK(h, cudaMemcpyAsync(h->arena + h->off_gh, grads_half, h->n_half * 2,
                              cudaMemcpyHostToDevice, st));
    if(h->n_float)
        CK(h, cudaMemcpyAsync(h->arena + h->off_gf, grads_float,
                              h->n_float * 4, cudaMemcpyHostToDevice, st));
    int rc = b200opt_step(h, lr, l2_lambda, scale, stream);
    if(rc)
        return rc;
    return b200opt_flags(h, stream, flags_out);
}

int b200opt_adam_mixed(size_t n, float alpha, void *weights,
                       const void *gradients, float *mvec, float *vvec,
                       float *cvec, float b1t, float b2t, float learning_rate,
                       float l2_lambda, uint32_t *aux, void *stream)
{
    if(n && (!weights || !gradients || !mvec || !vvec || !cvec || !aux))
        return B200OPT_EINVAL;
    if(!n)
        return B200OPT_OK;
    int dev = 0, sms = 0;
    if(cudaGetDevice(&dev) != cudaSuccess ||
       cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) !=
           cudaSuccess)
        return B200OPT_ECUDA;
    StepParams p;
    memset(&p, 0, sizeof(p));
    p.h.W[0] = (uint16_t *)weights;
    p.h.G[0] = (const uint16_t *)gradients;
    p.h.m = mvec;
    p.h.v = vvec;
    p.h.c = cvec;
    p.h.s = n;
    p.h.ngroups = (n + kVec - 1) / kVec;
    p.alpha = alpha;
    p.b1t = b1t;
    p.b2t = b2t;
    p.lr = learning_rate;
    p.l2 = l2_lambda;
    p.aux = aux;
    p.timeout_ns = 10000000000ull;
    p.force_scalar = !(aligned16(weights) && aligned16(gradients) &&
                       aligned16(mvec) && aligned16(vvec) && aligned16(cvec));
    return launch_step(p, 1, sms, seam_tuning(), (cudaStream_t)stream) == cudaSuccess
               ? B200OPT_OK
               : B200OPT_ECUDA;
}

int b200opt_adam_float(size_t n, float *weights, const float *gradients,
                       float *mvec, float *vvec, float b1t, float b2t,
                       float learning_rate, float l2_lambda, uint32_t *aux,
                       void *stream)
{
    if(n && (!weights || !gradients || !mvec || !vvec || !aux))
        return B200OPT_EINVAL;
    if(!n)
        return B200OPT_OK;
    int dev = 0, sms = 0;
    if(cudaGetDevice(&dev) != cudaSuccess ||
       cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) !=
           cudaSuccess)
        return B200OPT_ECUDA;
    StepParams p;
    memset(&p, 0, sizeof(p));
    p.f.W[0] = weights;
    p.f.G[0] = gradients;
    p.f.m = mvec;
    p.f.v = vvec;
    p.f.s = n;
    p.f.ngroups = (n + kVec - 1) / kVec;
    p.b1t = b1t;
    p.b2t = b2t;
    p.lr = learning_rate;
    p.l2 = l2_lambda;
    p.aux = aux;
    p.timeout_ns = 10000000000ull;
    p.force_scalar = !(aligned16(weights) && aligned16(gradients) &&
                       aligned16(mvec) && aligned16(vvec));
    return launch_step(p, 1, sms, seam_tuning(), (cudaStream_t)stream) == cudaSuccess
               ? B200OPT_OK
               : B200OPT_ECUDA;
}

// ---------------------------------------------------------------------------
// Entry point for callers that must not allocate: its scratch is this array.
// In host code the array's name stands for the symbol, not for a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
static __device__ __align__(256) unsigned char
    g_static_scratch[B200OPT_STATIC_SCRATCH_BYTES];
static_assert(sizeof(Ctrl) <= B200OPT_STATIC_SCRATCH_BYTES,
              "the control block must fit the static scratch");

static int static_scratch_address(Ctrl **out)
{
    static std::mutex mu;
    static void *per_device[64] = {};
    int dev = 0;
    if(cudaGetDevice(&dev) != cudaSuccess)
        return B200OPT_ECUDA;
    if(dev < 0 || dev >= 64)
        return B200OPT_EUNSUPPORTED;
    std::lock_guard<std::mutex> lock(mu);
    if(!per_device[dev]) {
        void *ptr = nullptr;
        if(cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return B200OPT_ECUDA;
        }
        per_device[dev] = ptr;
    }
    *out = static_cast<Ctrl *>(per_device[dev]);
    return B200OPT_OK;
}

int b200opt_adam_mixed_static(size_t n, float alpha, void *weights,
                              const void *gradients, float *mvec, float *vvec,
                              float *cvec, float b1t, float b2t,
                              float learning_rate, float l2_lambda,
                              uint32_t *flags_out, void *stream)
{
    if(n > B200OPT_STATIC_MAX_ELEMS)
        return B200OPT_ETOOBIG;
    if(!flags_out ||
       (n && (!weights || !gradients || !mvec || !vvec || !cvec)))
        return B200OPT_EINVAL;
    if(!(aligned16(weights) && aligned16(gradients) && aligned16(mvec) &&
         aligned16(vvec) && aligned16(cvec)))
        return B200OPT_EINVAL;
    Ctrl *ctrl = nullptr;
    int rc = static_scratch_address(&ctrl);
    if(rc)
        return rc;
    int dev = 0, sms = 0;
    if(cudaGetDevice(&dev) != cudaSuccess ||
       cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) !=
           cudaSuccess)
        return B200OPT_ECUDA;
    cudaStream_t st = (cudaStream_t)stream;
    // the shared array keeps the last call's contents: start from zero
    if(cudaMemsetAsync(ctrl, 0, sizeof(Ctrl), st) != cudaSuccess)
        return B200OPT_ECUDA;
    StepParams p;
    memset(&p, 0, sizeof(p));
    p.h.W[0] = (uint16_t *)weights;
    p.h.G[0] = (const uint16_t *)gradients;
    p.h.m = mvec;
    p.h.v = vvec;
    p.h.c = cvec;
    p.h.s = n;
    p.h.ngroups = (n + kVec - 1) / kVec;
    p.alpha = alpha;
    p.b1t = b1t;
    p.b2t = b2t;
    p.lr = learning_rate;
    p.l2 = l2_lambda;
    p.timeout_ns = 10000000000ull;
    p.ctrl[0] = ctrl;        // the fixed array, not an allocation
    p.flags_dev = flags_out;  // written by the last CTA, also when n == 0
    p.flags_dev_status = 1;   // a wait that ran out shows as 0xFFFFFFFF there
    return launch_step(p, 1, sms, seam_tuning(), st) == cudaSuccess
               ? B200OPT_OK
               : B200OPT_ECUDA;
}

int b200opt_rank_info(const b200opt_t *h, int *rank, int *nranks)
{
    if(!h)
        return B200OPT_EINVAL;
    if(rank)
        *rank = h->rank;
    if(nranks)
        *nranks = h->nranks;
    return B200OPT_OK;
}

int b200opt_get_iter(const b200opt_t *h, int *iter)
{
    if(!h || !iter)
        return B200OPT_EINVAL;
    *iter = h->iter;
    return B200OPT_OK;
}

int b200opt_set_iter(b200opt_t *h, int iter)
{
    if(!h || iter < 0)
        return B200OPT_EINVAL;
    h->iter = iter;
    return B200OPT_OK;
}

static int state_array(b200opt_t *h, int dtype, int which, float **base,
                       size_t *skip, size_t *count)
{
    if(dtype == B200OPT_HALF) {
        float *a[3] = {h->mh, h->vh, h->ch};
        if(which < 0 || which > 2)
            return B200OPT_EINVAL;
        *base = a[which];
        *skip = h->oh - h->Ah;
        *count = h->sh;
    } else if(dtype == B200OPT_FLOAT) {
        float *a[2] = {h->mf, h->vf};
        if(which < 0 || which > 1)
            return B200OPT_EINVAL;
        *base = a[which];
        *skip = h->of - h->Af;
        *count = h->sf;
    } else {
        return B200OPT_EINVAL;
    }
    return B200OPT_OK;
}

int b200opt_export_state(b200opt_t *h, int dtype, int which, float *host_dst,
                         size_t capacity, size_t *count)
{
    if(!h)
        return B200OPT_EINVAL;
    float *base;
    size_t skip, cnt;
    int rc = state_array(h, dtype, which, &base, &skip, &cnt);
    if(rc)
        return rc;
    if(count)
        *count = cnt;
    if(!host_dst)
        return B200OPT_OK;
    if(capacity < cnt)
        return B200OPT_EINVAL;
    DeviceGuard guard(h->device);
    if(cnt)
        CK(h, cudaMemcpy(host_dst, base + skip, cnt * 4,
                         cudaMemcpyDeviceToHost));
    return B200OPT_OK;
}

int b200opt_import_state(b200opt_t *h, int dtype, int which,
                         const float *host_src, size_t count)
{
    if(!h || !host_src)
        return B200OPT_EINVAL;
    float *base;
    size_t skip, cnt;
    int rc = state_array(h, dtype, which, &base, &skip, &cnt);
    if(rc)
        return rc;
    if(count != cnt)
        return B200OPT_EINVAL;
    DeviceGuard guard(h->device);
    if(cnt)
        CK(h, cudaMemcpy(base + skip, host_src, cnt * 4,
                         cudaMemcpyHostToDevice));
    return B200OPT_OK;
}

int b200opt_set_option(b200opt_t *h, int option, long value)
{
    if(!h)
        return B200OPT_EINVAL;
    switch(option) {
    case B200OPT_OPT_TIMEOUT_MS:
        if(value < 1)
            return B200OPT_EINVAL;
        h->timeout_ms = value;
        return B200OPT_OK;
    case B200OPT_OPT_PATH:
        if(value < B200OPT_PATH_AUTO || value > B200OPT_PATH_NVLS)
            return B200OPT_EINVAL;
        h->path = value;
        return B200OPT_OK;
    case B200OPT_OPT_CTAS_PER_SM:
        if(value < 0 || value > 32)
            return B200OPT_EINVAL;
        h->ctas_per_sm = value;
        return B200OPT_OK;
    case B200OPT_OPT_KERNEL_VARIANT:
        if(value < 0 || value > 2)
            return B200OPT_EINVAL;
        h->variant = value;
        return B200OPT_OK;
    case B200OPT_OPT_NCCL_CROSSOVER:
        if(value < 0)
            return B200OPT_EINVAL;
        h->nccl_crossover = value;
        return B200OPT_OK;
    case B200OPT_OPT_STAGES:
        if(value < 0 || value > 16)
            return B200OPT_EINVAL;
        h->stages = value;
        return B200OPT_OK;
    case B200OPT_OPT_GRID:
        if(value < 0 || value > 65535)
            return B200OPT_EINVAL;
        h->grid = value;
        return B200OPT_OK;
    case B200OPT_OPT_PHASE_TIMERS:
        h->timing = value != 0;
        return B200OPT_OK;
    case B200OPT_OPT_KEEP_REDUCED:
        h->keep_reduced = value != 0;
        return B200OPT_OK;

    case B200OPT_OPT_ASSUME_NO_PEER_ACCESS:
        if(h->peers_attached > 1)
            return fail(h, B200OPT_ESTATE, "set before any peer is attached");
        h->assume_no_peer_access = value != 0;
        return B200OPT_OK;
    }
    return B200OPT_EINVAL;
}

int b200opt_get_option(const b200opt_t *h, int option, long *value)
{
    if(!h || !value)
        return B200OPT_EINVAL;
    switch(option) {
    case B200OPT_OPT_TIMEOUT_MS: *value = h->timeout_ms; return B200OPT_OK;
    case B200OPT_OPT_PATH: *value = h->path; return B200OPT_OK;
    case B200OPT_OPT_CTAS_PER_SM: *value = h->ctas_per_sm; return B200OPT_OK;
    case B200OPT_OPT_KERNEL_VARIANT: *value = h->variant; return B200OPT_OK;
    case B200OPT_OPT_NCCL_CROSSOVER: *value = h->nccl_crossover; return B200OPT_OK;
    case B200OPT_OPT_STAGES: *value = h->stages; return B200OPT_OK;
    case B200OPT_OPT_GRID: *value = h->grid; return B200OPT_OK;
    case B200OPT_OPT_PHASE_TIMERS: *value = h->timing; return B200OPT_OK;
    case B200OPT_OPT_KEEP_REDUCED: *value = h->keep_reduced; return B200OPT_OK;
    case B200OPT_OPT_ASSUME_NO_PEER_ACCESS:
        *value = h->assume_no_peer_access;
        return B200OPT_OK;
    }
    return B200OPT_EINVAL;
}

int b200opt_peer_copy(b200opt_t *h, int peer_rank, size_t bytes, void *stream)
{
    if(!h || peer_rank < 0 || peer_rank >= h->nranks || peer_rank == h->rank)
        return B200OPT_EINVAL;
    if(!h->peer_arena[peer_rank] || h->serial)
        return fail(h, B200OPT_ESTATE, "the peer's memory is not mapped from another GPU");
    if(bytes > h->n_half * 2)
        return fail(h, B200OPT_EINVAL, "more bytes than the fp16 weight buffer holds");
    DeviceGuard guard(h->device);
    CK(h, cudaMemcpyAsync(h->arena + h->off_wh, h->peer_arena[peer_rank] + h->off_wh,
                          bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return B200OPT_OK;
}

int b200opt_phase_times(const b200opt_t *h, uint64_t ns_out[4])
{
    if(!h || !ns_out)
        return B200OPT_EINVAL;
    if(!h->timing)
        return B200OPT_ESTATE;
    for(int k = 0; k < 4; k++)
        ns_out[k] = h->host->phase_ns[k];
    return B200OPT_OK;
}

int b200opt_launch_count(const b200opt_t *h, uint64_t *launches)
{
    if(!h || !launches)
        return B200OPT_EINVAL;
    *launches = h->launches;
    return B200OPT_OK;
}

}  // extern "C"
