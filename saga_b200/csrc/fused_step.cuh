// Fused reduce-scatter + mixed-precision Adam + all-gather step kernel for
// sm_100a, and the small helper kernels around it.
//
// What one launch does on rank r of N (one launch per rank per training step):
//   1. (N > 1) tells every peer "my gradients are final" and waits, bounded,
//      until every peer said the same;
//   2. for its shard of each dtype group: loads the gradient vectors of all N
//      ranks through peer-mapped pointers (16 bytes per thread per rank), sums
//      them in fp32 in rank order, rounds once to the buffer dtype, classifies
//      overflow on the rounded value, unscales, applies Adam to the local fp32
//      m / v / master shard, and stores the new fp16 (or fp32) weights into the
//      weight buffer of EVERY rank;
//   3. the last CTA to finish publishes this rank's flag word to all peers,
//      waits (bounded) for theirs, and writes the sums to pinned host memory.
//
// The arithmetic per element follows Saga's adam_kernel_mp / adam_kernel
// (src/cuda/cuda_kernels.cu:159-230 of the Saga tree) expression by expression
// so that nvcc contracts the same multiply-add pairs.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200opt.h"

namespace b200 {

constexpr int kThreads = 256;
constexpr int kMaxRanks = B200OPT_MAX_RANKS;
constexpr int kVec = 8;  // elements per thread per group (16 B of fp16)

// flag bits carried in registers / flag words
constexpr uint32_t kFlagRange = 1u;
constexpr uint32_t kFlagInf = 2u;
constexpr uint32_t kFlagNan = 4u;
constexpr uint32_t kFlagValid = 0x80000000u;

// Adam constants of the reference (src/cuda/cuda_kernels.hpp:54-55,
// src/cuda/cuda_kernels.cu:157): double literals narrowed to float.
#define B200OPT_ADAM_B1 0.9
#define B200OPT_ADAM_B2 0.999
#define B200OPT_ADAM_EPS 1e-8

// Per-rank control block at the start of the peer-mapped arena.  Peers write
// ready[], done[] and flagword[][]; the rest is touched by the owner only.
struct alignas(128) Ctrl {
    uint32_t ready[32];        // ready[q] = step number rank q has reached
    uint32_t done[32];         // done[q]  = step number rank q has finished
    uint32_t flagword[2][32];  // [step parity][q] flag bits of rank q | valid
    uint32_t cta_done;         // CTAs of the running launch that finished
    uint32_t local_flags;      // OR of this rank's flag bits
    uint32_t status;           // sticky B200OPT_E* (as positive number) or 0
    uint32_t reserved0;
    uint32_t coll_flags[4];    // NCCL path: {range, inf, nan} to be all-reduced
    // device-resident loss scale (optional): updated by the last CTA of a step
    float scale;               // current loss scale
    uint32_t policy;           // B200OPT_POLICY_*
    int32_t clean_steps;       // interval policy: clean steps since the last change
    int32_t interval;          // interval policy: growth interval
    uint32_t log_pos;          // steps logged so far
    uint32_t reserved1;
    // phase timers (optional): %globaltimer at kernel entry and the time CTA 0
    // spent waiting for the peers' announcements
    unsigned long long t_start;
    unsigned long long t_entry_wait;
    uint32_t pad[14];
};
static_assert(sizeof(Ctrl) == 640, "control block layout");

// Written by the last CTA of a launch, read by the host after a stream sync.
struct HostResult {
    uint32_t range, inf, nan;
    uint32_t status;  // 0 or -B200OPT_ETIMEOUT
    uint32_t epoch;
    uint32_t where;   // 1 = wait for gradients, 2 = wait for completion
    uint32_t peer;    // rank that did not arrive
    uint32_t scale_bits;  // device-resident loss scale after this step's policy
                          // update (bit pattern; 0 when the scale lives on the host)
    // phase timers of the last launch, nanoseconds of %globaltimer (only with
    // B200OPT_OPT_PHASE_TIMERS): wait for the peers' announcements in CTA 0,
    // kernel entry until the last CTA finished its share, the completion
    // protocol in the last CTA, and kernel entry until the end of it
    unsigned long long phase_ns[4];
};

struct HalfGroup {
    uint16_t *W[kMaxRanks];        // weight buffer of every rank
    const uint16_t *G[kMaxRanks];  // gradient buffer of every rank
    float *m, *v, *c;  // local shard state; element i (global index) at [i - A]
    size_t o, s;       // shard start and length, elements
    size_t A;          // flat index of the element stored at [0] of m, v, c
    size_t B;          // index the group grid starts at: o rounded down so that a
                       // warp's 512-byte access starts on a 512-byte boundary
    size_t ngroups;    // kVec-element groups covering [B, o+s)
};

struct FloatGroup {
    float *W[kMaxRanks];
    const float *G[kMaxRanks];
    float *m, *v;
    size_t o, s, A, B, ngroups;
};

struct StepParams {
    HalfGroup h;
    FloatGroup f;
    float alpha, b1t, b2t, lr, l2;
    int rank;
    int barrier;      // 1: wait for peers inside the kernel
    int force_scalar; // 1: pointers are not 16-byte aligned, element-wise path
    int stages;       // staged kernel: depth of the shared-memory ring
    int partial;      // 1: a bucket of a step that is not its last (no completion
                      // protocol across ranks, flags keep accumulating)
    uint32_t epoch;
    unsigned long long timeout_ns;
    Ctrl *ctrl[kMaxRanks];  // control block of every rank (ctrl[rank] local)
    HostResult *host;       // pinned, may be null
    uint32_t *aux;          // kernel-seam mode: store 1 into aux[0..2], no ctrl
    uint32_t *flags_dev;    // NCCL path: this rank's {range, inf, nan} as 0/1
    int flags_dev_status;   // 1: a wait that ran out is reported as 0xFFFFFFFF in
                            // all three words of flags_dev (no host page to carry it)
    int device_scale;       // 1: 1/scale comes from ctrl[rank]->scale, and the last
                            // CTA applies the loss-scale policy to it
    uint32_t *scale_log;    // ring of {range, inf, nan, bits of the new scale} per step
    uint32_t scale_log_cap; // entries in the ring (0: no log)
    int timing;             // 1: record the phase timers
    int keep_reduced;       // 1 (multicast path): leave the reduced gradients of the own
                            // shard in the own gradient buffer, where ncclReduceScatter
                            // leaves them in Saga (src/cuda/cuda_optimizer.cpp:160-166)
    // multicast views of the fp16 gradient and weight buffers of all ranks
    // (switch-reduced loads, switch-replicated stores); null off that path
    const uint16_t *mcG;
    uint16_t *mcW;
};

// 1/scale of this step: from the launch arguments, or from the scale that
// lives in device memory (the reference divides in float,
// src/cuda/cuda_optimizer.cpp:169 of the Saga tree).
__device__ __forceinline__ float step_alpha(const StepParams &p)
{
    if(!p.device_scale)
        return p.alpha;
    const float s = *reinterpret_cast<const volatile float *>(&p.ctrl[p.rank]->scale);
    return __fdiv_rn(1.0f, s);
}

// CudaProgram::step's policy (src/cuda/cuda_program.cpp:295-302 of the Saga
// tree) evaluated on the device: float state, double factors.
__device__ __forceinline__ void device_scale_update(const StepParams &p, Ctrl *my,
                                                    const uint32_t (&sums)[3])
{
    float s = my->scale;
    const bool overflow = sums[1] != 0 || sums[2] != 0;
    if(my->policy == B200OPT_POLICY_INTERVAL) {
        if(overflow) {
            s = (float)((double)s * 0.5);
            my->clean_steps = 0;
        } else if(++my->clean_steps >= my->interval) {
            s = (float)((double)s * 2.0);
            my->clean_steps = 0;
        }
    } else {
        const double factor = overflow ? 0.5 : (sums[0] > 1 ? 0.9 : 1.02);
        s = (float)((double)s * factor);
    }
    my->scale = s;
    if(p.scale_log_cap) {
        uint32_t *e = p.scale_log + 4 * (size_t)(my->log_pos % p.scale_log_cap);
        e[0] = sums[0];
        e[1] = sums[1];
        e[2] = sums[2];
        e[3] = __float_as_uint(s);
    }
    my->log_pos++;
}

// ---------------------------------------------------------------- memory ops

__device__ __forceinline__ uint4 ld_stream(const void *p)
{
    return __ldcs(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ void st_stream(void *p, uint4 v)
{
    __stcs(reinterpret_cast<uint4 *>(p), v);
}
// Load that always goes to the point of coherence of the owning GPU.
__device__ __forceinline__ uint4 ld_peer(const void *p)
{
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v)
                 : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];"
                 : "=r"(v)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Waits until *p has reached `epoch`.  Gives up after timeout_ns and returns
// false; never spins without a limit.
__device__ __forceinline__ bool wait_epoch(const uint32_t *p, uint32_t epoch,
                                           unsigned long long timeout_ns)
{
    if((int32_t)(ld_acquire_sys(p) - epoch) >= 0)
        return true;
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    for(;;) {
        if((int32_t)(ld_acquire_sys(p) - epoch) >= 0)
            return true;
        __nanosleep(64);
        if((++spins & 63u) == 0 && globaltimer_ns() - t0 > timeout_ns)
            return false;
    }
}

// ---------------------------------------------------------------- arithmetic

// One element of the update.  The reference writes it as plain expressions
// (src/cuda/cuda_kernels.cu:177-187,212-228 of the Saga tree) and lets nvcc
// contract multiply-add pairs; which pairs it fuses differs between the
// reference's two kernels (in adam_kernel_mp the gradient is itself a product,
// in adam_kernel a plain load).  The roundings are spelled out here with
// intrinsics, one variant per reference kernel, so that the results equal the
// compiled reference bit for bit whatever this file's surroundings make the
// compiler prefer.
template <bool MIXED>
__device__ __forceinline__ void adam_element(float dw, float &m, float &v,
                                             float &w, float b1t, float b2t,
                                             float lr, float lambda)
{
    const float b1 = B200OPT_ADAM_B1;
    const float b2 = B200OPT_ADAM_B2;
    const float e = B200OPT_ADAM_EPS;
    const float omb1 = 1.0f - b1;
    const float omb2 = 1.0f - b2;
    if(MIXED) {
        // m = b1*m + (1-b1)*dw ; v = b2*v + (1-b2)*dw*dw : left product fused
        m = __fmaf_rn(b1, m, __fmul_rn(omb1, dw));
        v = __fmaf_rn(b2, v, __fmul_rn(__fmul_rn(omb2, dw), dw));
    } else {
        // same source text, right product fused
        m = __fmaf_rn(omb1, dw, __fmul_rn(b1, m));
        v = __fmaf_rn(__fmul_rn(omb2, dw), dw, __fmul_rn(b2, v));
    }
    const float m_hat = __fmul_rn(m, b1t);
    // v_hat + e is a single fma: v_hat = v*b2t is never rounded on its own
    const float r = __frsqrt_rn(__fmaf_rn(v, b2t, e));
    // w - lr*m_hat*r - lr*lambda*w, each subtraction of a product one fma
    const float t = __fmaf_rn(-__fmul_rn(lr, m_hat), r, w);
    w = __fmaf_rn(-__fmul_rn(lr, lambda), w, t);
}

// Overflow classes of an fp16 bit pattern (src/cuda/cuda_kernels.cu:198-210).
// Returns true when the element must be skipped.
__device__ __forceinline__ bool classify_half(uint32_t u16, uint32_t &fl)
{
    if((u16 & 0x7800u) == 0x7800u) {
        fl |= kFlagRange;
        if((u16 & 0x7c00u) == 0x7c00u) {
            fl |= (u16 & 0x3ffu) ? kFlagNan : kFlagInf;
            return true;
        }
    }
    return false;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t u16)
{
    return __half2float(__ushort_as_half((unsigned short)u16));
}
__device__ __forceinline__ uint32_t float_to_half_bits(float f)
{
    return (uint32_t)__half_as_ushort(__float2half_rn(f));
}

// Classifies and updates VEC elements whose reduced gradient bit patterns are
// u[].  Nearly every group holds no value of magnitude >= 32768: that is
// tested once for the whole group, and the common case then runs the VEC
// independent update chains without a branch between them.  wold points at
// the owner's current fp16 weights of these elements (read only when an
// element is skipped and must keep its weight).
template <int VEC>
__device__ __forceinline__ void half_update(const StepParams &p, float alpha,
                                            const uint32_t (&u)[VEC],
                                            float (&m)[VEC], float (&v)[VEC],
                                            float (&c)[VEC],
                                            uint32_t (&wbits)[VEC],
                                            const uint16_t *wold, uint32_t &fl)
{
    bool any = false;
#pragma unroll
    for(int e = 0; e < VEC; e++)
        any |= (u[e] & 0x7800u) == 0x7800u;
    if(!any) {
#pragma unroll
        for(int e = 0; e < VEC; e++) {
            const float dw = __fmul_rn(half_bits_to_float(u[e]), alpha);
            adam_element<true>(dw, m[e], v[e], c[e], p.b1t, p.b2t, p.lr, p.l2);
            wbits[e] = float_to_half_bits(c[e]);
        }
        return;
    }
#pragma unroll
    for(int e = 0; e < VEC; e++) {
        if(classify_half(u[e], fl)) {
            wbits[e] = wold[e];  // skipped: m, v, master and weight stay
        } else {
            const float dw = __fmul_rn(half_bits_to_float(u[e]), alpha);
            adam_element<true>(dw, m[e], v[e], c[e], p.b1t, p.b2t, p.lr, p.l2);
            wbits[e] = float_to_half_bits(c[e]);
        }
    }
}

// ------------------------------------------------------ fp16 group, 8 elements

template <int NR>
struct HalfLoads {
    uint4 g[NR];
    uint4 m0, m1, v0, v1, c0, c1;
};

// The local half of a group's loads: m, v and the master copy of the shard.
template <int NR>
__device__ __forceinline__ void half_load_state(const StepParams &p, size_t idx0,
                                                HalfLoads<NR> &L)
{
    const size_t li = idx0 - p.h.A;
    L.m0 = ld_stream(p.h.m + li);
    L.m1 = ld_stream(p.h.m + li + 4);
    L.v0 = ld_stream(p.h.v + li);
    L.v1 = ld_stream(p.h.v + li + 4);
    L.c0 = ld_stream(p.h.c + li);
    L.c1 = ld_stream(p.h.c + li + 4);
}

// The other half: the gradients of every rank (peers' through NVLink).
template <int NR>
__device__ __forceinline__ void half_load_grads(const StepParams &p, size_t idx0,
                                                HalfLoads<NR> &L)
{
#pragma unroll
    for(int q = 0; q < NR; q++) {
        if(NR == 1)
            L.g[q] = ld_stream(p.h.G[q] + idx0);
        else
            L.g[q] = ld_peer(p.h.G[q] + idx0);
    }
}

__device__ __forceinline__ void unpack8(const uint4 &a, const uint4 &b,
                                        float (&x)[8])
{
    x[0] = __uint_as_float(a.x);
    x[1] = __uint_as_float(a.y);
    x[2] = __uint_as_float(a.z);
    x[3] = __uint_as_float(a.w);
    x[4] = __uint_as_float(b.x);
    x[5] = __uint_as_float(b.y);
    x[6] = __uint_as_float(b.z);
    x[7] = __uint_as_float(b.w);
}
__device__ __forceinline__ void pack8(const float (&x)[8], uint4 &a, uint4 &b)
{
    a = make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]),
                   __float_as_uint(x[2]), __float_as_uint(x[3]));
    b = make_uint4(__float_as_uint(x[4]), __float_as_uint(x[5]),
                   __float_as_uint(x[6]), __float_as_uint(x[7]));
}
__device__ __forceinline__ void halves8(const uint4 &g, uint32_t (&u)[8])
{
    u[0] = g.x & 0xffffu;
    u[1] = g.x >> 16;
    u[2] = g.y & 0xffffu;
    u[3] = g.y >> 16;
    u[4] = g.z & 0xffffu;
    u[5] = g.z >> 16;
    u[6] = g.w & 0xffffu;
    u[7] = g.w >> 16;
}

// Reduces, classifies and updates one 8-element group held in registers.
// out[0..1] = m, out[2..3] = v, out[4..5] = master, out[6] = fp16 weights.
template <int NR>
__device__ __forceinline__ void half_compute(const StepParams &p, float alpha,
                                             size_t idx0,
                                             const HalfLoads<NR> &L,
                                             uint32_t &fl, uint4 (&out)[7])
{
    uint32_t u[8];
    halves8(L.g[0], u);
    if(NR > 1) {
        // fp32 accumulation in rank order, one rounding to fp16
        float acc[8];
#pragma unroll
        for(int e = 0; e < 8; e++)
            acc[e] = half_bits_to_float(u[e]);
#pragma unroll
        for(int q = 1; q < NR; q++) {
            uint32_t t[8];
            halves8(L.g[q], t);
#pragma unroll
            for(int e = 0; e < 8; e++)
                acc[e] += half_bits_to_float(t[e]);
        }
#pragma unroll
        for(int e = 0; e < 8; e++)
            u[e] = float_to_half_bits(acc[e]);
    }

    float m[8], v[8], c[8];
    unpack8(L.m0, L.m1, m);
    unpack8(L.v0, L.v1, v);
    unpack8(L.c0, L.c1, c);

    uint32_t wbits[8];
    half_update<8>(p, alpha, u, m, v, c, wbits, p.h.W[p.rank] + idx0, fl);
    pack8(m, out[0], out[1]);
    pack8(v, out[2], out[3]);
    pack8(c, out[4], out[5]);
    out[6] = make_uint4(wbits[0] | (wbits[1] << 16), wbits[2] | (wbits[3] << 16),
                        wbits[4] | (wbits[5] << 16), wbits[6] | (wbits[7] << 16));
}

template <int NR>
__device__ __forceinline__ void half_compute_store(const StepParams &p,
                                                   float alpha, size_t idx0,
                                                   const HalfLoads<NR> &L,
                                                   uint32_t &fl)
{
    uint4 out[7];
    half_compute<NR>(p, alpha, idx0, L, fl, out);
    const size_t li = idx0 - p.h.A;
    st_stream(p.h.m + li, out[0]);
    st_stream(p.h.m + li + 4, out[1]);
    st_stream(p.h.v + li, out[2]);
    st_stream(p.h.v + li + 4, out[3]);
    st_stream(p.h.c + li, out[4]);
    st_stream(p.h.c + li + 4, out[5]);
#pragma unroll
    for(int q = 0; q < NR; q++)
        *reinterpret_cast<uint4 *>(p.h.W[q] + idx0) = out[6];
}

// Element-wise path for the (at most two) groups that straddle a shard edge,
// and for unaligned caller memory in kernel-seam mode.
template <int NR>
__device__ __noinline__ uint32_t half_scalar(const StepParams &p, float alpha,
                                             size_t idx0)
{
    uint32_t fl = 0;
    for(int e = 0; e < kVec; e++) {
        const size_t i = idx0 + e;
        if(i < p.h.o || i >= p.h.o + p.h.s)
            continue;
        uint32_t u = *reinterpret_cast<const volatile uint16_t *>(p.h.G[0] + i);
        if(NR > 1) {
            float acc = half_bits_to_float(u);
            for(int q = 1; q < NR; q++)
                acc += half_bits_to_float(
                    *reinterpret_cast<const volatile uint16_t *>(p.h.G[q] + i));
            u = float_to_half_bits(acc);
        }
        if(p.keep_reduced)
            const_cast<uint16_t *>(p.h.G[p.rank])[i] = (uint16_t)u;
        if(classify_half(u, fl))
            continue;
        const size_t li = i - p.h.A;
        float m = p.h.m[li], v = p.h.v[li], c = p.h.c[li];
        const float dw = __fmul_rn(half_bits_to_float(u), alpha);
        adam_element<true>(dw, m, v, c, p.b1t, p.b2t, p.lr, p.l2);
        p.h.m[li] = m;
        p.h.v[li] = v;
        p.h.c[li] = c;
        const uint16_t wb = (uint16_t)float_to_half_bits(c);
        for(int q = 0; q < NR; q++)
            p.h.W[q][i] = wb;
    }
    return fl;
}

// ------------------------------------------------------ fp32 group, 8 elements

template <int NR>
struct FloatLoads {
    uint4 g0[NR], g1[NR];
    uint4 w0, w1, m0, m1, v0, v1;
};

template <int NR>
__device__ __forceinline__ void float_load(const StepParams &p, size_t idx0,
                                           FloatLoads<NR> &L)
{
    const size_t li = idx0 - p.f.A;
#pragma unroll
    for(int q = 0; q < NR; q++) {
        if(NR == 1) {
            L.g0[q] = ld_stream(p.f.G[q] + idx0);
            L.g1[q] = ld_stream(p.f.G[q] + idx0 + 4);
        } else {
            L.g0[q] = ld_peer(p.f.G[q] + idx0);
            L.g1[q] = ld_peer(p.f.G[q] + idx0 + 4);
        }
    }
    L.w0 = ld_stream(p.f.W[p.rank] + idx0);
    L.w1 = ld_stream(p.f.W[p.rank] + idx0 + 4);
    L.m0 = ld_stream(p.f.m + li);
    L.m1 = ld_stream(p.f.m + li + 4);
    L.v0 = ld_stream(p.f.v + li);
    L.v1 = ld_stream(p.f.v + li + 4);
}

// Non-finite classes of an fp32 gradient (src/cuda/cuda_kernels.cu:166-175):
// no range flag in this group.
__device__ __forceinline__ bool classify_float(float dw, uint32_t &fl)
{
    if(!isfinite(dw)) {
        fl |= isnan(dw) ? kFlagNan : kFlagInf;
        return true;
    }
    return false;
}

template <int NR>
__device__ __forceinline__ void float_compute_store(const StepParams &p,
                                                    size_t idx0,
                                                    const FloatLoads<NR> &L,
                                                    uint32_t &fl)
{
    float g[8], w[8], m[8], v[8];
    unpack8(L.g0[0], L.g1[0], g);
#pragma unroll
    for(int q = 1; q < NR; q++) {
        float t[8];
        unpack8(L.g0[q], L.g1[q], t);
#pragma unroll
        for(int e = 0; e < 8; e++)
            g[e] += t[e];
    }
    unpack8(L.w0, L.w1, w);
    unpack8(L.m0, L.m1, m);
    unpack8(L.v0, L.v1, v);
#pragma unroll
    for(int e = 0; e < 8; e++) {
        if(!classify_float(g[e], fl))
            adam_element<false>(g[e], m[e], v[e], w[e], p.b1t, p.b2t, p.lr, p.l2);
    }
    const size_t li = idx0 - p.f.A;
    uint4 a, b;
    pack8(m, a, b);
    st_stream(p.f.m + li, a);
    st_stream(p.f.m + li + 4, b);
    pack8(v, a, b);
    st_stream(p.f.v + li, a);
    st_stream(p.f.v + li + 4, b);
    pack8(w, a, b);
#pragma unroll
    for(int q = 0; q < NR; q++) {
        *reinterpret_cast<uint4 *>(p.f.W[q] + idx0) = a;
        *reinterpret_cast<uint4 *>(p.f.W[q] + idx0 + 4) = b;
    }
}

template <int NR>
__device__ __noinline__ uint32_t float_scalar(const StepParams &p, size_t idx0)
{
    uint32_t fl = 0;
    for(int e = 0; e < kVec; e++) {
        const size_t i = idx0 + e;
        if(i < p.f.o || i >= p.f.o + p.f.s)
            continue;
        float g = *reinterpret_cast<const volatile float *>(p.f.G[0] + i);
        for(int q = 1; q < NR; q++)
            g += *reinterpret_cast<const volatile float *>(p.f.G[q] + i);
        if(classify_float(g, fl))
            continue;
        const size_t li = i - p.f.A;
        float m = p.f.m[li], v = p.f.v[li], w = p.f.W[p.rank][i];
        adam_element<false>(g, m, v, w, p.b1t, p.b2t, p.lr, p.l2);
        p.f.m[li] = m;
        p.f.v[li] = v;
        for(int q = 0; q < NR; q++)
            p.f.W[q][i] = w;
    }
    return fl;
}

// ------------------------------------------------- step prologue and epilogue

// (N > 1) Announces "my gradients are final" to every rank.  The step kernels
// call this first, start the loads of their own shard state, and only then
// wait for the peers (step_wait): the state is local and final, only the
// peers' gradients depend on the announcements.
template <int NR>
__device__ __forceinline__ void step_announce(const StepParams &p)
{
    Ctrl *const my = p.ctrl[p.rank];
    if(p.timing && blockIdx.x == 0 && threadIdx.x == 0 && my) {
        my->t_start = globaltimer_ns();
        my->t_entry_wait = 0;
    }
    if(NR == 1 || !p.barrier)
        return;
    if(blockIdx.x == 0 && threadIdx.x < NR)
        st_release_sys(&p.ctrl[threadIdx.x]->ready[p.rank], p.epoch);
}

// Waits, bounded, for every rank's announcement of this step.  Returns
// non-zero in every thread of the CTA when a wait ran out.
template <int NR>
__device__ __forceinline__ int step_wait(const StepParams &p)
{
    if(NR == 1 || !p.barrier)
        return 0;
    const int tid = threadIdx.x;
    Ctrl *const my = p.ctrl[p.rank];
    int bad = 0;
    if(tid < NR) {
        if(!wait_epoch(&my->ready[tid], p.epoch, p.timeout_ns)) {
            bad = 1;
            if(atomicCAS(&my->status, 0u, (uint32_t)(-B200OPT_ETIMEOUT)) == 0u &&
               p.host) {
                p.host->where = 1;
                p.host->peer = tid;
            }
        }
    }
    bad = __syncthreads_or(bad);
    if(p.timing && blockIdx.x == 0 && tid == 0)
        my->t_entry_wait = globaltimer_ns() -
                           *reinterpret_cast<volatile unsigned long long *>(&my->t_start);
    return bad;
}

template <int NR>
__device__ __forceinline__ int step_begin(const StepParams &p)
{
    step_announce<NR>(p);
    return step_wait<NR>(p);
}

// The fp32 group (BatchNorm scales and biases in an fp16 network: a few tens
// of thousands of elements) always takes the direct-load path.
template <int NR>
__device__ __forceinline__ void float_group_pass(const StepParams &p,
                                                 uint32_t &fl)
{
    const int tid = threadIdx.x;
    const size_t ng = p.f.ngroups;
    const size_t lo = p.f.o, hi = p.f.o + p.f.s;
    for(size_t base = (size_t)blockIdx.x * blockDim.x; base < ng;
        base += (size_t)gridDim.x * blockDim.x) {
        const size_t gid = base + tid;
        const size_t idx0 = p.f.B + gid * kVec;
        if(gid < ng) {
            if(idx0 >= lo && idx0 + kVec <= hi && !p.force_scalar) {
                FloatLoads<NR> L;
                float_load<NR>(p, idx0, L);
                float_compute_store<NR>(p, idx0, L, fl);
            } else if(idx0 + kVec > lo) {
                fl |= float_scalar<NR>(p, idx0);
            }
        }
    }
}

// Folds the per-thread flag bits into one word per rank and, in the last CTA
// of the launch to get here, finishes the step: publishes this rank's flag
// word to all ranks, waits (bounded) until every rank has finished reading
// gradients and writing weights, and leaves the flag sums in pinned host
// memory.  `s_flag` is one int of shared memory.
template <int NR>
__device__ __forceinline__ void step_finish(const StepParams &p, uint32_t fl,
                                            int *s_flag)
{
    const int tid = threadIdx.x;
    Ctrl *const my = p.ctrl[p.rank];

    // one flag word per warp, then at most one atomic per warp that saw any
    fl = __reduce_or_sync(0xffffffffu, fl);

    if(p.aux) {
        // kernel-seam mode: the reference's plain stores of 1 into CudaAux
        if((tid & 31) == 0 && fl) {
            if(fl & kFlagRange)
                p.aux[0] = 1;
            if(fl & kFlagInf)
                p.aux[1] = 1;
            if(fl & kFlagNan)
                p.aux[2] = 1;
        }
        return;
    }

    if((tid & 31) == 0 && fl)
        atomicOr(&my->local_flags, fl);

    // the last CTA of this launch finishes the step
    if(NR > 1)
        __threadfence_system();  // weight stores into peers before the signal
    else
        __threadfence();
    __syncthreads();
    if(tid == 0)
        *s_flag = atomicAdd(&my->cta_done, 1u) == gridDim.x - 1;
    __syncthreads();
    if(!*s_flag)
        return;
    __threadfence();

    if(p.partial) {
        // not the step's last bucket: later buckets of this stream follow in
        // order, and the last one runs the completion protocol for all of them
        if(tid == 0)
            my->cta_done = 0;
        return;
    }

    const unsigned long long t_body = p.timing ? globaltimer_ns() : 0;
    const uint32_t mine =
        *reinterpret_cast<volatile uint32_t *>(&my->local_flags);
    uint32_t status = *reinterpret_cast<volatile uint32_t *>(&my->status);
    uint32_t sums[3] = {(mine & kFlagRange) ? 1u : 0u,
                        (mine & kFlagInf) ? 1u : 0u,
                        (mine & kFlagNan) ? 1u : 0u};
    const int par = p.epoch & 1;

    if(NR > 1) {
        // publish this rank's flag word into every rank's slot array
        if(tid < NR)
            p.ctrl[tid]->flagword[par][p.rank] = mine | kFlagValid;
        if(p.barrier && !status) {
            int bad = 0;
            if(tid < NR) {
                __threadfence_system();
                st_release_sys(&p.ctrl[tid]->done[p.rank], p.epoch);
                if(!wait_epoch(&my->done[tid], p.epoch, p.timeout_ns)) {
                    bad = 1;
                    if(atomicCAS(&my->status, 0u,
                                 (uint32_t)(-B200OPT_ETIMEOUT)) == 0u &&
                       p.host) {
                        p.host->where = 2;
                        p.host->peer = tid;
                    }
                }
            }
            if(__syncthreads_or(bad))
                status = (uint32_t)(-B200OPT_ETIMEOUT);
            if(tid == 0 && !status) {
                sums[0] = sums[1] = sums[2] = 0;
                for(int q = 0; q < NR; q++) {
                    const uint32_t w = *reinterpret_cast<volatile uint32_t *>(
                        &my->flagword[par][q]);
                    sums[0] += (w & kFlagRange) ? 1u : 0u;
                    sums[1] += (w & kFlagInf) ? 1u : 0u;
                    sums[2] += (w & kFlagNan) ? 1u : 0u;
                }
            }
        }
    }
    if(tid == 0) {
        if(p.device_scale && !status)
            device_scale_update(p, my, sums);
        if(p.flags_dev) {
            const bool gave_up = p.flags_dev_status && status;
            p.flags_dev[0] = gave_up ? 0xFFFFFFFFu : sums[0];
            p.flags_dev[1] = gave_up ? 0xFFFFFFFFu : sums[1];
            p.flags_dev[2] = gave_up ? 0xFFFFFFFFu : sums[2];
        }
        if(p.host) {
            p.host->range = sums[0];
            p.host->inf = sums[1];
            p.host->nan = sums[2];
            p.host->status = status;
            p.host->scale_bits = p.device_scale ? __float_as_uint(my->scale) : 0u;
            p.host->epoch = p.epoch;
            if(p.timing) {
                const unsigned long long t_end = globaltimer_ns();
                const unsigned long long t_start =
                    *reinterpret_cast<volatile unsigned long long *>(&my->t_start);
                p.host->phase_ns[0] =
                    *reinterpret_cast<volatile unsigned long long *>(&my->t_entry_wait);
                p.host->phase_ns[1] = t_body - t_start;
                p.host->phase_ns[2] = t_end - t_body;
                p.host->phase_ns[3] = t_end - t_start;
            }
        }
        my->local_flags = 0;
        my->cta_done = 0;
        // no fence: the end of the kernel makes these stores visible to the host
        // and to the next launch on the stream
    }
}

// ------------------------------------------------ step kernel, direct loads

// Every thread loads its 8-element groups straight into registers (UNR groups
// before any is computed, to keep enough bytes in flight per SM).  The loads
// of the first trip's shard state are issued before the wait for the peers.
template <int NR, int UNR, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
    fused_step_kernel(const __grid_constant__ StepParams p)
{
    __shared__ int s_flag;
    const int tid = threadIdx.x;
    uint32_t fl = 0;
    const size_t stride = (size_t)gridDim.x * kThreads * UNR;
    const size_t ng = p.h.ngroups;
    const size_t lo = p.h.o, hi = p.h.o + p.h.s;
    size_t base = (size_t)blockIdx.x * kThreads * UNR;
    HalfLoads<NR> L[UNR];
    bool full[UNR];

    auto classify = [&](size_t b) {
#pragma unroll
        for(int k = 0; k < UNR; k++) {
            const size_t gid = b + (size_t)k * kThreads + tid;
            const size_t idx0 = p.h.B + gid * kVec;
            full[k] = gid < ng && idx0 >= lo && idx0 + kVec <= hi && !p.force_scalar;
        }
    };
    auto load_state = [&](size_t b) {
#pragma unroll
        for(int k = 0; k < UNR; k++)
            if(full[k])
                half_load_state<NR>(p, p.h.B + (b + (size_t)k * kThreads + tid) * kVec, L[k]);
    };

    step_announce<NR>(p);
    bool state_loaded = false;
    if(base < ng) {
        classify(base);
        load_state(base);
        state_loaded = true;
    }
    if(!step_wait<NR>(p)) {
        const float alpha = step_alpha(p);
        for(; base < ng; base += stride) {
            if(!state_loaded) {
                classify(base);
                load_state(base);
            }
            state_loaded = false;
#pragma unroll
            for(int k = 0; k < UNR; k++)
                if(full[k])
                    half_load_grads<NR>(p, p.h.B + (base + (size_t)k * kThreads + tid) * kVec,
                                        L[k]);
#pragma unroll
            for(int k = 0; k < UNR; k++) {
                const size_t gid = base + (size_t)k * kThreads + tid;
                const size_t idx0 = p.h.B + gid * kVec;
                if(full[k])
                    half_compute_store<NR>(p, alpha, idx0, L[k], fl);
                else if(gid < ng && idx0 + kVec > lo)
                    fl |= half_scalar<NR>(p, alpha, idx0);
            }
        }
        float_group_pass<NR>(p, fl);
    }
    step_finish<NR>(p, fl, &s_flag);
}

// master := float(fp16 weights) over the shard (AdamMixed constructor,
// src/cuda/cuda_optimizer.cpp:142-145); c is indexed like in the step kernel.
__global__ void init_master_kernel(const uint16_t *w, float *c, size_t o,
                                   size_t s, size_t A)
{
    for(size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < s;
        i += (size_t)gridDim.x * blockDim.x)
        c[o + i - A] = half_bits_to_float(w[o + i]);
}

}  // namespace b200
