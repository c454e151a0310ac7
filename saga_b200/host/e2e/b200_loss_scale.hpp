// -*-c++-*-
// Call-site side of the device-resident loss scale inside the Saga tree:
// included into src/cuda/cuda_dnn.cpp (after cuda_kernels.hpp) by
// build_saga_e2e.py, which re-routes the four loss-gradient calls that pass
// `scale * p.m_mp_scaling` by value (src/cuda/cuda_dnn.cpp:1310-1315,1424-1443)
// through the functions below.  When the program keeps its loss scale on the
// device (CudaProgram::m_b200_dscale, set by the b200opt optimizer op) the
// kernels read it there; otherwise the call is the original one.
#pragma once

namespace saga {

void catclassifier_bwd_half_i32_dscale(int n, const __half *x, __half *dx, const int32_t *y,
                                       const int32_t *dy, float *loss, unsigned int c,
                                       float scale, const float *dscale, cudaStream_t stream);
void loss_bwd_half_float_dscale(int n, const __half *x, __half *dx, const float *dy,
                                float *loss, unsigned int c, float scale, const float *dscale,
                                cudaStream_t stream);
void loss_bwd_half_half_dscale(int n, const __half *x, __half *dx, const __half *dy,
                               float *loss, unsigned int c, float scale, const float *dscale,
                               cudaStream_t stream);
void loss_bwd_float_float_dscale(int n, const float *x, float *dx, const float *dy,
                                 float *loss, unsigned int c, float scale, const float *dscale,
                                 cudaStream_t stream);

#define B200_LOSS_SCALE_ROUTE(NAME, XT, DYT)                                                  \
    static inline void b200_##NAME(int n, const XT *x, XT *dx, const DYT *dy, float *loss,    \
                                   unsigned int c, float scale, float host_scale,             \
                                   const float *dscale, cudaStream_t stream)                  \
    {                                                                                         \
        if(dscale)                                                                            \
            NAME##_dscale(n, x, dx, dy, loss, c, scale, dscale, stream);                      \
        else                                                                                  \
            NAME(n, x, dx, dy, loss, c, scale * host_scale, stream);                          \
    }

B200_LOSS_SCALE_ROUTE(loss_bwd_half_float, __half, float)
B200_LOSS_SCALE_ROUTE(loss_bwd_half_half, __half, __half)
B200_LOSS_SCALE_ROUTE(loss_bwd_float_float, float, float)
#undef B200_LOSS_SCALE_ROUTE

static inline void
b200_catclassifier_bwd_half_i32(int n, const __half *x, __half *dx, const int32_t *y,
                                const int32_t *dy, float *loss, unsigned int c, float scale,
                                float host_scale, const float *dscale, cudaStream_t stream)
{
    if(dscale)
        catclassifier_bwd_half_i32_dscale(n, x, dx, y, dy, loss, c, scale, dscale, stream);
    else
        catclassifier_bwd_half_i32(n, x, dx, y, dy, loss, c, scale * host_scale, stream);
}

}  // namespace saga
