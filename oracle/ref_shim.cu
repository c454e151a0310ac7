/*
 * extern "C" doorway into the reference's own Adam kernel launchers, so that
 * the parity tests and the benchmark can drive them through ctypes.
 *
 * TEST INFRASTRUCTURE ONLY.  This file holds no arithmetic of its own: it is
 * compiled together with the reference's unmodified src/cuda/cuda_kernels.cu,
 * taken from the reference checkout where it lies (see oracle/Makefile), into
 * oracle/_ref/libsaga_ref_kernels.so.  The declarations it relies on come from
 * the reference's src/cuda/cuda_kernels.hpp:57-64 and src/cuda/cuda_aux.hpp.
 */
#include <stdint.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include "cuda_kernels.hpp"

extern "C" {

/* aux points at 16 bytes of device-accessible memory: {range, inf, nan, anomaly} */
int
sagaref_adam_mixed(int n, float alpha, void *weights, const void *gradients,
                   float *mvec, float *vvec, float *cvec, float b1t, float b2t,
                   float lr, float l2_lambda, void *aux, void *stream)
{
    saga::adam_mixed(n, alpha, (__half *)weights, (const __half *)gradients,
                     mvec, vvec, cvec, b1t, b2t, lr, l2_lambda,
                     (saga::CudaAux *)aux, (cudaStream_t)stream, 0);
    return (int)cudaGetLastError();
}

int
sagaref_adam_float(int n, float *weights, const float *gradients, float *mvec,
                   float *vvec, float b1t, float b2t, float lr,
                   float l2_lambda, void *aux, void *stream)
{
    saga::adam_float(n, weights, gradients, mvec, vvec, b1t, b2t, lr,
                     l2_lambda, (saga::CudaAux *)aux, (cudaStream_t)stream, 0);
    return (int)cudaGetLastError();
}

}
