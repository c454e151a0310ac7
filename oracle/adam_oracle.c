/*
 * CPU oracle for Saga's data-parallel parameter-update path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the parity tests,
 * the smoke test and the benchmark's cpu_baseline leg compare the CUDA path
 * against.  Nothing in the product (the saga_b200 package, the C-ABI library)
 * links, loads or calls it, and the product has no CPU fallback.
 *
 * It restates, in plain C, what the reference computes for one training
 * step's parameter update (paths are relative to the reference project):
 *
 *   src/cuda/cuda_kernels.cu:159-189   adam_kernel      (fp32 parameters)
 *   src/cuda/cuda_kernels.cu:191-230   adam_kernel_mp   (fp16 w/g, fp32 m,v,master)
 *   src/cuda/cuda_optimizer.cpp:76-113,148-186   iteration counter, bias
 *       corrections in double, alpha = 1.0f/scale, shard offsets, reduce-scatter,
 *       all-gather
 *   src/cuda/cuda_optimizer.cpp:122-146  master := float(fp16 weight shard)
 *   src/cuda/cuda_optimizer.cpp:196-260  flat [W|G] layout, 16-element padding
 *   src/cuda/cuda_program.cpp:282-307    flag sum over ranks, loss-scale policy
 *   src/fp16.h:17-19                     half<->float, round to nearest even
 *
 * Parity pin: the reference's own tests hold no golden vectors for this path
 * (test/test_mp.cpp prints, test/test_resnode.cpp checks activations only).
 * The pin is the reference's kernels themselves: src/cuda/cuda_kernels.cu is
 * compiled unmodified into oracle/_ref/ by oracle/Makefile, run on a B200 by
 * tests/golden/make_golden.py, and its outputs are committed as fixtures under
 * tests/golden/ which this oracle must reproduce.
 *
 * Cross-rank gradient sum.  The reference sums with NCCL in the buffer's own
 * dtype in an order NCCL chooses, which is not reproducible.  This oracle (and
 * the CUDA path it checks) defines the sum as fp32 accumulation in rank order
 * 0..N-1 followed by one round-to-nearest-even conversion to the buffer dtype.
 * For one rank there is no sum and the two definitions coincide.
 *
 * `model` argument of the Adam functions:
 *   0  every multiply and add rounded separately (no contraction)
 *   1  the multiply-add pairs fused the way nvcc's default -fmad=true contracts
 *      the reference's expressions (checked bit for bit against the compiled
 *      reference kernel on the GPU by the parity tests)
 * Build with -ffp-contract=off so that model 0 really is uncontracted.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <immintrin.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_MAX_RANKS 16

/* ------------------------------------------------------------------ fp16 */

/* src/fp16.h:17-19 converts with F16C (round to nearest even).  Restated on
 * the bit patterns so it does not depend on the host CPU. */
float
orc_h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if(exp == 0x1f) {
        bits = sign | 0x7f800000u | (man << 13);
    } else if(exp != 0) {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    } else if(man == 0) {
        bits = sign;
    } else {
        /* subnormal half: man * 2^-24, normalise */
        int e = -1;
        do {
            man <<= 1;
            e++;
        } while(!(man & 0x400u));
        bits = sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3ffu) << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* float -> half, round to nearest even.  NaN maps to 0x7fff as the CUDA
 * conversion used by the reference's `weights[i] = w` store does. */
uint16_t
orc_f2h(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7fffffffu;
    if(x > 0x7f800000u)
        return 0x7fff;
    if(x == 0x7f800000u)
        return sign | 0x7c00;
    const int e = (int)(x >> 23) - 127;
    const uint32_t man24 = (x & 0x7fffffu) | 0x800000u;
    if(e > 15)
        return sign | 0x7c00;
    if(e >= -14) {
        uint32_t h = ((uint32_t)(e + 15) << 10) | ((man24 >> 13) & 0x3ffu);
        const uint32_t rem = man24 & 0x1fffu;
        if(rem > 0x1000u || (rem == 0x1000u && (h & 1u)))
            h++; /* may carry into the exponent; 0x7c00 == inf is right */
        return sign | (uint16_t)h;
    }
    /* result is a half subnormal: q = round(man24 * 2^(e+1)) units of 2^-24 */
    const int shift = -(e + 1);
    if(shift > 24)
        return sign;
    uint32_t q = man24 >> shift;
    const uint32_t rem = man24 & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if(rem > half || (rem == half && (q & 1u)))
        q++;
    return sign | (uint16_t)q;
}

/* Counts disagreements between the bit-level conversions above and the CPU's
 * F16C instructions over `count` float patterns start, start+stride, ... and
 * all 65536 half patterns.  Used by the CPU tests; returns 0 when they agree.
 * NaN results are compared as "both NaN". */
__attribute__((target("f16c"))) uint64_t
orc_selfcheck_fp16(uint32_t start, uint32_t stride, uint64_t count)
{
    uint64_t bad = 0;
    uint32_t bits = start;
    for(uint64_t k = 0; k < count; k++, bits += stride) {
        float f;
        memcpy(&f, &bits, 4);
        uint16_t a = orc_f2h(f);
        uint16_t b = _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT);
        int a_nan = (a & 0x7c00) == 0x7c00 && (a & 0x3ff);
        int b_nan = (b & 0x7c00) == 0x7c00 && (b & 0x3ff);
        if(a_nan || b_nan) {
            bad += a_nan != b_nan;
        } else {
            bad += a != b;
        }
    }
    for(uint32_t h = 0; h < 65536; h++) {
        float a = orc_h2f((uint16_t)h);
        float b = _cvtsh_ss((uint16_t)h);
        uint32_t ab, bb;
        memcpy(&ab, &a, 4);
        memcpy(&bb, &b, 4);
        if(a != a || b != b) {
            bad += (a != a) != (b != b);
        } else {
            bad += ab != bb;
        }
    }
    return bad;
}

/* --------------------------------------------------------- step scalars */

/* src/cuda/cuda_optimizer.cpp:150-152 — pow and the divisions in double
 * (ADAM_B1/ADAM_B2 are double literals, src/cuda/cuda_kernels.hpp:54-55),
 * narrowed to float on assignment. */
void
orc_bias_corrections(int iter, float *b1t, float *b2t)
{
    *b1t = (float)(1.0 / (1.0 - pow(0.9, iter)));
    *b2t = (float)(1.0 / (1.0 - pow(0.999, iter)));
}

/* src/cuda/cuda_optimizer.cpp:169 — `1.0f / p.m_mp_scaling`, a float divide */
float
orc_alpha(float scale)
{
    return 1.0f / scale;
}

/* __frsqrt_rn (src/cuda/cuda_kernels.cu:186,223) is the correctly rounded
 * reciprocal square root.  A double evaluation is re-done in extended
 * precision in the rare case where it lies too close to a rounding boundary
 * of float to decide. */
static inline float
rsqrt_rn(float x)
{
    const double d = 1.0 / sqrt((double)x);
    const float lo = (float)(d * (1.0 - 0x1p-50));
    const float hi = (float)(d * (1.0 + 0x1p-50));
    if(lo == hi)
        return lo;
    return (float)(1.0L / sqrtl((long double)x));
}

float
orc_rsqrt_rn(float x)
{
    return rsqrt_rn(x);
}

/* ------------------------------------------------------- Adam, one element */

/* src/cuda/cuda_kernels.cu:177-187 and :212-228, same expression order.
 * w0 is the fp32 weight the update starts from (master copy or fp32 weight).
 * `mixed` selects which of the two reference kernels is being restated: nvcc
 * contracts `b*x + (1-b)*dw` differently in the two (in adam_kernel_mp dw is
 * itself a product, in adam_kernel it is a plain load), as the golden fixtures
 * show bit for bit. */
static inline void
adam_update(float dw, float *m_io, float *v_io, float *w_io, float b1t,
            float b2t, float lr, float lambda, int model, int mixed)
{
    const float b1 = (float)0.9;
    const float b2 = (float)0.999;
    const float e = (float)1e-8;
    const float omb1 = 1.0f - b1;
    const float omb2 = 1.0f - b2;
    float m, v, w = *w_io;

    if(model == 0) {
        m = b1 * *m_io + omb1 * dw;
        v = b2 * *v_io + omb2 * dw * dw;
        const float m_hat = m * b1t;
        const float v_hat = v * b2t;
        w = w - lr * m_hat * rsqrt_rn(v_hat + e) - lr * lambda * w;
    } else {
        if(mixed) {
            m = fmaf(b1, *m_io, omb1 * dw);
            v = fmaf(b2, *v_io, omb2 * dw * dw);
        } else {
            m = fmaf(omb1, dw, b1 * *m_io);
            v = fmaf(omb2 * dw, dw, b2 * *v_io);
        }
        /* v*b2t + e is one fma (v_hat never exists as a rounded value), and
         * each x - a*b is fma(-a, b, x) */
        const float m_hat = m * b1t;
        const float t = fmaf(-(lr * m_hat), rsqrt_rn(fmaf(v, b2t, e)), w);
        w = fmaf(-(lr * lambda), w, t);
    }
    *m_io = m;
    *v_io = v;
    *w_io = w;
}

/* flags[0]=range, [1]=inf, [2]=nan; set to 1 when seen, never cleared here
 * (the reference's kernels only ever store 1, src/cuda/cuda_kernels.cu:201-206). */

/* src/cuda/cuda_kernels.cu:191-230 over elements [0,n) of a shard */
void
orc_adam_mixed(size_t n, float alpha, uint16_t *w, const uint16_t *g, float *m,
               float *v, float *c, float b1t, float b2t, float lr,
               float lambda, uint32_t *flags, int model)
{
    for(size_t i = 0; i < n; i++) {
        const uint16_t u = g[i];
        if((u & 0x7800) == 0x7800) {
            flags[0] = 1;
            if((u & 0x7c00) == 0x7c00) {
                if(u & 0x3ff)
                    flags[2] = 1;
                else
                    flags[1] = 1;
                continue; /* only this element is skipped */
            }
        }
        const float dw = orc_h2f(u) * alpha;
        adam_update(dw, &m[i], &v[i], &c[i], b1t, b2t, lr, lambda, model, 1);
        w[i] = orc_f2h(c[i]);
    }
}

/* src/cuda/cuda_kernels.cu:159-189: no unscale, no range flag */
void
orc_adam_f32(size_t n, float *w, const float *g, float *m, float *v, float b1t,
             float b2t, float lr, float lambda, uint32_t *flags, int model)
{
    for(size_t i = 0; i < n; i++) {
        const float dw = g[i];
        if(!isfinite(dw)) {
            if(isnan(dw))
                flags[2] = 1;
            else
                flags[1] = 1;
            continue;
        }
        adam_update(dw, &m[i], &v[i], &w[i], b1t, b2t, lr, lambda, model, 0);
    }
}

/* src/cuda/cuda_optimizer.cpp:142-145 */
void
orc_master_init(size_t s, const uint16_t *w_shard, float *c)
{
    for(size_t i = 0; i < s; i++)
        c[i] = orc_h2f(w_shard[i]);
}

/* --------------------------------------------------- cross-rank reduction */

/* Stands for ncclReduceScatter(..., ncclFloat16, ncclSum) at
 * src/cuda/cuda_optimizer.cpp:160-166, with the summation order fixed as the
 * header says.  g[q] is rank q's whole gradient buffer; out receives elements
 * [off, off+count). */
void
orc_reduce_half(int nranks, const uint16_t *const *g, size_t off, size_t count,
                uint16_t *out)
{
    for(size_t i = 0; i < count; i++) {
        if(nranks == 1) {
            out[i] = g[0][off + i];
            continue;
        }
        float acc = orc_h2f(g[0][off + i]);
        for(int q = 1; q < nranks; q++)
            acc += orc_h2f(g[q][off + i]);
        out[i] = orc_f2h(acc);
    }
}

/* src/cuda/cuda_optimizer.cpp:88-94 (ncclFloat32, ncclSum) */
void
orc_reduce_f32(int nranks, const float *const *g, size_t off, size_t count,
               float *out)
{
    for(size_t i = 0; i < count; i++) {
        float acc = g[0][off + i];
        for(int q = 1; q < nranks; q++)
            acc += g[q][off + i];
        out[i] = acc;
    }
}

/* ------------------------------------------------------------ flat layout */

/* src/cuda/cuda_optimizer.cpp:199-219,235-258: every tensor starts at the sum
 * of the 16-element-rounded sizes before it.  Returns the padded total. */
size_t
orc_flat_layout(const size_t *sizes, size_t k, size_t *offsets)
{
    size_t total = 0;
    for(size_t j = 0; j < k; j++) {
        if(offsets)
            offsets[j] = total;
        total += (sizes[j] + 15) & ~(size_t)15;
    }
    return total;
}

/* --------------------------------------------------------- loss-scale policy */

/* src/cuda/cuda_program.cpp:295-307.  `scale` is a float and the literals are
 * double, so each update is float(double(scale) * k).  flags are the sums over
 * ranks of {range, inf, nan}. */
void
orc_policy_reference(float *scale, const uint32_t *flags)
{
    if(flags[1] || flags[2]) {
        *scale *= 0.5;
    } else if(flags[0] > 1) {
        *scale *= 0.9;
    } else {
        *scale *= 1.02;
    }
}

/* The policy the benchmark description words instead ("skip and halve; the
 * scale doubles after 2000 clean steps").  Not a reference behaviour; kept as
 * a separately selected mode with its own restatement. */
void
orc_policy_interval(float *scale, int *clean_steps, const uint32_t *flags,
                    int growth_interval)
{
    if(flags[1] || flags[2]) {
        *scale *= 0.5;
        *clean_steps = 0;
    } else if(++*clean_steps >= growth_interval) {
        *scale *= 2.0;
        *clean_steps = 0;
    }
}

/* --------------------------------------------------- one whole step, N ranks */

/* Appendix-style restatement of one optimizer step over all ranks:
 * AdamF32::exec then AdamMixed::exec on every rank
 * (src/cuda/cuda_optimizer.cpp:76-113,148-186) followed by the flag sum of
 * src/cuda/cuda_program.cpp:282-291.
 *
 *   W[q], G[q]     rank q's fp16 weight / gradient buffers, n_half elements
 *   m[q],v[q],c[q] rank q's shard state, n_half/nranks floats
 *   Wf,Gf,mf,vf    the same for the fp32 group (no master copy), n_f32 elements
 *   iter           value of the iteration counter AFTER its increment (>= 1)
 *   flag_sums      receives sums over ranks of {range, inf, nan}; a rank
 *                  contributes at most 1 per flag across both groups
 * Elements beyond nranks*(n/nranks) are never touched, as in the reference
 * (plain integer division at :85 and :157).
 */
void
orc_step_multi(int nranks, size_t n_half, uint16_t **W, uint16_t **G, float **m,
               float **v, float **c, size_t n_f32, float **Wf, float **Gf,
               float **mf, float **vf, int iter, float scale, float lr,
               float lambda, uint32_t *flag_sums, int model)
{
    float b1t, b2t;
    orc_bias_corrections(iter, &b1t, &b2t);
    const float alpha = orc_alpha(scale);
    uint32_t flags[ORC_MAX_RANKS][3];
    memset(flags, 0, sizeof(flags));

    const size_t sf = n_f32 / (size_t)nranks;
    const size_t sh = n_half / (size_t)nranks;

    /* reduce-scatter + local update; W of the owner holds the new shard */
    for(int r = 0; r < nranks; r++) {
        if(sf) {
            const size_t o = sf * (size_t)r;
            float *gs = Gf[r] + o; /* in place, like ncclReduceScatter */
            float tmp;
            for(size_t i = 0; i < sf; i++) {
                const float *srcs[ORC_MAX_RANKS];
                for(int q = 0; q < nranks; q++)
                    srcs[q] = Gf[q];
                orc_reduce_f32(nranks, srcs, o + i, 1, &tmp);
                gs[i] = tmp;
            }
            orc_adam_f32(sf, Wf[r] + o, gs, mf[r], vf[r], b1t, b2t, lr, lambda,
                         flags[r], model);
        }
    }
    for(int r = 0; r < nranks; r++) {
        if(sh) {
            const size_t o = sh * (size_t)r;
            uint16_t *gs = G[r] + o;
            const uint16_t *srcs[ORC_MAX_RANKS];
            for(int q = 0; q < nranks; q++)
                srcs[q] = G[q];
            /* Each rank reduces only its own shard, and shards are disjoint,
             * so reducing in place never feeds a sum back into another sum. */
            for(size_t i = 0; i < sh; i++) {
                uint16_t tmp;
                orc_reduce_half(nranks, srcs, o + i, 1, &tmp);
                gs[i] = tmp;
            }
            orc_adam_mixed(sh, alpha, W[r] + o, gs, m[r], v[r], c[r], b1t, b2t,
                           lr, lambda, flags[r], model);
        }
    }
    /* all-gather */
    for(int r = 0; r < nranks; r++) {
        for(int q = 0; q < nranks; q++) {
            if(q == r)
                continue;
            if(sf)
                memcpy(Wf[q] + sf * r, Wf[r] + sf * r, sf * sizeof(float));
            if(sh)
                memcpy(W[q] + sh * r, W[r] + sh * r, sh * sizeof(uint16_t));
        }
    }
    flag_sums[0] = flag_sums[1] = flag_sums[2] = 0;
    for(int r = 0; r < nranks; r++)
        for(int k = 0; k < 3; k++)
            flag_sums[k] += flags[r][k];
}

/* ------------------------------------------------ timed multi-thread variant */

int
orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Number of host threads the timed variants below use from now on. */
void
orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if(n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* orc_reduce_half over all host threads: the gradient sum of a whole buffer
 * (every shard) as the N-rank step needs it. */
__attribute__((target("f16c"))) void
orc_reduce_half_mt(int nranks, const uint16_t *const *g, size_t count,
                   uint16_t *out)
{
#pragma omp parallel for schedule(static)
    for(size_t i = 0; i < count; i++) {
        float acc = _cvtsh_ss(g[0][i]);
        for(int q = 1; q < nranks; q++)
            acc += _cvtsh_ss(g[q][i]);
        out[i] = nranks == 1 ? g[0][i] : _cvtss_sh(acc, _MM_FROUND_TO_NEAREST_INT);
    }
}

/* Same arithmetic as orc_adam_mixed (model 1), elements split across all host
 * threads, half conversions through the CPU's F16C instructions as the
 * reference's host code does (src/fp16.h).  This is the CPU figure the
 * benchmark reports beside the GPU numbers. */
__attribute__((target("f16c,fma"))) void
orc_adam_mixed_mt(size_t n, float alpha, uint16_t *w, const uint16_t *g,
                  float *m, float *v, float *c, float b1t, float b2t, float lr,
                  float lambda, uint32_t *flags)
{
    uint32_t f_range = 0, f_inf = 0, f_nan = 0;
    const float b1 = (float)0.9, b2 = (float)0.999, e = (float)1e-8;
    const float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
#pragma omp parallel for schedule(static) reduction(| : f_range, f_inf, f_nan)
    for(size_t i = 0; i < n; i++) {
        const uint16_t u = g[i];
        if((u & 0x7800) == 0x7800) {
            f_range = 1;
            if((u & 0x7c00) == 0x7c00) {
                if(u & 0x3ff)
                    f_nan = 1;
                else
                    f_inf = 1;
                continue;
            }
        }
        const float dw = _cvtsh_ss(u) * alpha;
        const float mi = fmaf(b1, m[i], omb1 * dw);
        const float vi = fmaf(b2, v[i], omb2 * dw * dw);
        const float m_hat = mi * b1t;
        float wi = c[i];
        const float r = rsqrt_rn(fmaf(vi, b2t, e));
        const float t = fmaf(-(lr * m_hat), r, wi);
        wi = fmaf(-(lr * lambda), wi, t);
        m[i] = mi;
        v[i] = vi;
        c[i] = wi;
        w[i] = _cvtss_sh(wi, _MM_FROUND_TO_NEAREST_INT);
    }
    if(f_range)
        flags[0] = 1;
    if(f_inf)
        flags[1] = 1;
    if(f_nan)
        flags[2] = 1;
}
