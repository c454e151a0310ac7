// NCCL fallback of the step: ncclReduceScatter (in place) -> Adam kernel on the
// local shard -> ncclAllGather (in place) -> ncclAllReduce of the three flag
// words, the sequence Saga's AdamMixed::exec / AdamF32::exec and
// CudaProgram::step issue (src/cuda/cuda_optimizer.cpp:88-112,160-185,
// src/cuda/cuda_program.cpp:282-291 of the Saga tree).  libnccl is opened at
// run time, so the library loads on machines without it.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace b200 {

struct NcclPath;

int nccl_path_unique_id(void *id128);
int nccl_path_create(NcclPath **out, int rank, int nranks, const void *id128,
                     std::string *err);
void nccl_path_destroy(NcclPath *np);

// Sums the gradient buffers over ranks; rank r receives its shard in place
// (fp16 summed in fp16 and fp32 in fp32 by NCCL, as in the reference).
int nccl_path_reduce_scatter(NcclPath *np, uint16_t *g_half, size_t s_half,
                             float *g_float, size_t s_float,
                             cudaStream_t st, std::string *err);
// Gathers the updated weight shards in place and sums `flags3` (three u32 on
// the device) over ranks.
int nccl_path_all_gather_and_flags(NcclPath *np, uint16_t *w_half,
                                   size_t s_half, float *w_float,
                                   size_t s_float, uint32_t *flags3,
                                   cudaStream_t st, std::string *err);

}  // namespace b200
