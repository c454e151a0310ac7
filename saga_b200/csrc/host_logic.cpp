// Host-only arithmetic of the b200opt C ABI: the loss-scale policy, the
// per-step bias corrections and the flat-buffer layout.  No CUDA in here.
#include <cmath>
#include <cstddef>
#include <cstdint>

#include "../../include/b200opt.h"

extern "C" {

// CudaProgram::step's policy block (src/cuda/cuda_program.cpp:295-302 of the
// Saga tree).  m_mp_scaling is a float and the factors are double literals, so
// every update is float(double(scale) * factor); a float factor would drift
// from the reference within two steps.
int b200opt_policy_update(float *scale, const uint32_t flags[3], int policy,
                          int *state, int interval)
{
    if(!scale || !flags)
        return B200OPT_EINVAL;
    const bool overflow = flags[1] != 0 || flags[2] != 0;
    if(policy == B200OPT_POLICY_REFERENCE) {
        double factor = 1.02;
        if(overflow)
            factor = 0.5;
        else if(flags[0] > 1)
            factor = 0.9;
        *scale = (float)((double)*scale * factor);
        return B200OPT_OK;
    }
    if(policy == B200OPT_POLICY_INTERVAL) {
        if(!state || interval < 1)
            return B200OPT_EINVAL;
        if(overflow) {
            *scale = (float)((double)*scale * 0.5);
            *state = 0;
        } else if(++*state >= interval) {
            *scale = (float)((double)*scale * 2.0);
            *state = 0;
        }
        return B200OPT_OK;
    }
    return B200OPT_EINVAL;
}

// AdamMixed::exec / AdamF32::exec (src/cuda/cuda_optimizer.cpp:78-80,150-152):
// double arithmetic on the double literals 0.9 and 0.999, narrowed to float.
int b200opt_bias_corrections(int iter, float *b1t, float *b2t)
{
    if(iter < 1 || !b1t || !b2t)
        return B200OPT_EINVAL;
    *b1t = (float)(1.0 / (1.0 - std::pow(0.9, iter)));
    *b2t = (float)(1.0 / (1.0 - std::pow(0.999, iter)));
    return B200OPT_OK;
}

// CudaProgram::create_optimizer (src/cuda/cuda_optimizer.cpp:199-219,235-258):
// tensors are laid end to end, each padded to a multiple of 16 elements.
int b200opt_layout(const size_t *sizes, size_t k, size_t *offsets,
                   size_t *total)
{
    if((k && !sizes) || !total)
        return B200OPT_EINVAL;
    const size_t align = 16;
    size_t at = 0;
    for(size_t j = 0; j < k; j++) {
        if(offsets)
            offsets[j] = at;
        at += (sizes[j] + align - 1) & ~(align - 1);
    }
    *total = at;
    return B200OPT_OK;
}

// Which collective path a step takes.  Kept free of CUDA so that the rule can
// be checked on a machine without a GPU.
int b200opt_choose_path(int requested, int nranks, int serial,
                        int peers_reachable, int have_nccl, int have_multicast,
                        size_t n_half, size_t nccl_crossover, int *chosen)
{
    if(!chosen || nranks < 1 || requested < B200OPT_PATH_AUTO ||
       requested > B200OPT_PATH_NVLS)
        return B200OPT_EINVAL;
    // one rank, or several ranks stepped one after the other on one GPU: the
    // peer-pointer kernel is the only arithmetic there is
    if(nranks == 1 || serial) {
        if(requested == B200OPT_PATH_NVLS && nranks > 1)
            return B200OPT_EUNSUPPORTED;
        *chosen = B200OPT_PATH_PEER;
        return B200OPT_OK;
    }
    switch(requested) {
    case B200OPT_PATH_NCCL:
        if(!have_nccl)
            return B200OPT_ESTATE;
        *chosen = B200OPT_PATH_NCCL;
        return B200OPT_OK;
    case B200OPT_PATH_NVLS:
        if(!have_multicast)
            return B200OPT_ESTATE;
        *chosen = B200OPT_PATH_NVLS;
        return B200OPT_OK;
    case B200OPT_PATH_PEER:
        if(!peers_reachable)
            return B200OPT_EUNSUPPORTED;
        *chosen = B200OPT_PATH_PEER;
        return B200OPT_OK;
    }
    // AUTO: the peer-pointer kernel (bit for bit the rank-ordered sum) unless
    // the GPUs cannot reach one another's memory or the buffer is below the
    // size at which NCCL was measured to win; never the multicast path, whose
    // sum order is the switch's
    if(!peers_reachable) {
        if(!have_nccl)
            return B200OPT_EUNSUPPORTED;
        *chosen = B200OPT_PATH_NCCL;
        return B200OPT_OK;
    }
    *chosen = (have_nccl && n_half < nccl_crossover) ? B200OPT_PATH_NCCL
                                                     : B200OPT_PATH_PEER;
    return B200OPT_OK;
}

}  // extern "C"
