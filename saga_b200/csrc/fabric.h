// Arenas allocated through CUDA's virtual-memory API, so that they can be
// shared between processes as POSIX file descriptors and bound to an NVSwitch
// multicast object (the memory behind multimem.ld_reduce / multimem.st).
// The driver entry points are resolved at run time through the CUDA runtime:
// the library has no link-time dependency on libcuda and loads on a machine
// without a GPU.
#pragma once

#include <cuda.h>

#include <cstddef>
#include <string>

namespace b200 {

// One mapping of physical memory of some device into this process.
struct FabricMapping {
    CUmemGenericAllocationHandle mem = 0;
    CUdeviceptr va = 0;
    size_t bytes = 0;  // mapped size, a multiple of the granularity in use
    bool owns_mem = false;
};

// A multicast object and this rank's view of it.
struct FabricMulticast {
    CUmemGenericAllocationHandle mc = 0;
    CUdeviceptr va = 0;
    size_t bytes = 0;
    int device = -1;
    bool bound = false;
    bool owns_handle = false;
};

// 0 when every needed driver entry point resolved; otherwise a B200OPT_E*
// status and a text in *err.
int fabric_init(std::string *err);

// Does the device support switch multicast and reduction?
int fabric_multicast_supported(int device, bool *yes, std::string *err);

// Size every arena of a group is rounded up to: the larger of the allocation
// granularity and the multicast granularity for `nranks` devices.
int fabric_granularity(int device, int nranks, bool multicast, size_t *gran,
                       std::string *err);

// Physical memory on `device`, mapped read/write for `device`, zero-filled by
// the caller.  `bytes` must be a multiple of the granularity.
int fabric_alloc(FabricMapping *out, int device, size_t bytes, std::string *err);
// Lets another device of this process access the mapping.
int fabric_grant(const FabricMapping &m, int device, std::string *err);
// A file descriptor other processes can import (the caller closes it).
int fabric_export_fd(CUmemGenericAllocationHandle h, int *fd, std::string *err);
// Maps memory exported by another process for `device`.
int fabric_import(FabricMapping *out, int fd, int device, size_t bytes,
                  std::string *err);
void fabric_unmap(FabricMapping *m);

// Multicast object over `nranks` devices covering `bytes`.
int fabric_mc_create(FabricMulticast *out, int nranks, size_t bytes,
                     std::string *err);
int fabric_mc_import(FabricMulticast *out, int fd, size_t bytes, std::string *err);
int fabric_mc_add_device(FabricMulticast *mc, int device, std::string *err);
// After EVERY device has been added: binds this rank's arena at offset 0 and
// maps the multicast view for `device`.
int fabric_mc_bind(FabricMulticast *mc, const FabricMapping &arena, int device,
                   std::string *err);
// Unmaps the view, unbinds this device's memory and drops the handle.  Every
// rank must have stopped issuing multicast accesses before any rank calls it.
void fabric_mc_release(FabricMulticast *mc);

}  // namespace b200
