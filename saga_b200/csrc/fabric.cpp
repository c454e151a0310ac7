#include "fabric.h"

#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <mutex>

#include "../../include/b200opt.h"

namespace b200 {

namespace {

struct Driver {
    PFN_cuGetErrorString GetErrorString = nullptr;
    PFN_cuDeviceGet DeviceGet = nullptr;
    PFN_cuDeviceGetAttribute DeviceGetAttribute = nullptr;
    PFN_cuMemGetAllocationGranularity MemGetAllocationGranularity = nullptr;
    PFN_cuMemCreate MemCreate = nullptr;
    PFN_cuMemRelease MemRelease = nullptr;
    PFN_cuMemAddressReserve MemAddressReserve = nullptr;
    PFN_cuMemAddressFree MemAddressFree = nullptr;
    PFN_cuMemMap MemMap = nullptr;
    PFN_cuMemUnmap MemUnmap = nullptr;
    PFN_cuMemSetAccess MemSetAccess = nullptr;
    PFN_cuMemExportToShareableHandle MemExportToShareableHandle = nullptr;
    PFN_cuMemImportFromShareableHandle MemImportFromShareableHandle = nullptr;
    PFN_cuMulticastCreate MulticastCreate = nullptr;
    PFN_cuMulticastAddDevice MulticastAddDevice = nullptr;
    PFN_cuMulticastBindMem MulticastBindMem = nullptr;
    PFN_cuMulticastUnbind MulticastUnbind = nullptr;
    PFN_cuMulticastGetGranularity MulticastGetGranularity = nullptr;
    bool ok = false;
    std::string why;
};

Driver &drv()
{
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        bool ok = true;
        auto get = [&](const char *name, void **fn) {
            cudaDriverEntryPointQueryResult q;
            if(cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) !=
                   cudaSuccess ||
               q != cudaDriverEntryPointSuccess || !*fn) {
                cudaGetLastError();
                if(ok)
                    d.why = std::string("driver entry point ") + name +
                            " is not available";
                ok = false;
            }
        };
#define GET(field, name) get(name, reinterpret_cast<void **>(&d.field))
        GET(GetErrorString, "cuGetErrorString");
        GET(DeviceGet, "cuDeviceGet");
        GET(DeviceGetAttribute, "cuDeviceGetAttribute");
        GET(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
        GET(MemCreate, "cuMemCreate");
        GET(MemRelease, "cuMemRelease");
        GET(MemAddressReserve, "cuMemAddressReserve");
        GET(MemAddressFree, "cuMemAddressFree");
        GET(MemMap, "cuMemMap");
        GET(MemUnmap, "cuMemUnmap");
        GET(MemSetAccess, "cuMemSetAccess");
        GET(MemExportToShareableHandle, "cuMemExportToShareableHandle");
        GET(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
        GET(MulticastCreate, "cuMulticastCreate");
        GET(MulticastAddDevice, "cuMulticastAddDevice");
        GET(MulticastBindMem, "cuMulticastBindMem");
        GET(MulticastUnbind, "cuMulticastUnbind");
        GET(MulticastGetGranularity, "cuMulticastGetGranularity");
#undef GET
        d.ok = ok;
    });
    return d;
}

int cu_fail(CUresult r, const char *what, std::string *err)
{
    if(err) {
        const char *s = nullptr;
        if(drv().GetErrorString)
            drv().GetErrorString(r, &s);
        *err = std::string(what) + ": " + (s ? s : "unknown driver error");
    }
    return r == CUDA_ERROR_OUT_OF_MEMORY ? B200OPT_ENOMEM
           : r == CUDA_ERROR_NOT_SUPPORTED ? B200OPT_EUNSUPPORTED
                                           : B200OPT_ECUDA;
}

#define CU(call)                              \
    do {                                      \
        CUresult r_ = drv().call;             \
        if(r_ != CUDA_SUCCESS)                \
            return cu_fail(r_, #call, err);   \
    } while(0)

CUmemAllocationProp alloc_prop(int device)
{
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

CUmulticastObjectProp mc_prop(int nranks, size_t bytes)
{
    CUmulticastObjectProp prop = {};
    prop.numDevices = (unsigned)nranks;
    prop.size = bytes;
    prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    prop.flags = 0;
    return prop;
}

int set_access(CUdeviceptr va, size_t bytes, int device, std::string *err)
{
    CUmemAccessDesc acc = {};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CU(MemSetAccess(va, bytes, &acc, 1));
    return B200OPT_OK;
}

int map_handle(CUmemGenericAllocationHandle h, size_t bytes, int device,
               CUdeviceptr *va_out, std::string *err)
{
    CUdeviceptr va = 0;
    CU(MemAddressReserve(&va, bytes, 0, 0, 0));
    CUresult r = drv().MemMap(va, bytes, 0, h, 0);
    if(r != CUDA_SUCCESS) {
        drv().MemAddressFree(va, bytes);
        return cu_fail(r, "cuMemMap", err);
    }
    const int rc = set_access(va, bytes, device, err);
    if(rc) {
        drv().MemUnmap(va, bytes);
        drv().MemAddressFree(va, bytes);
        return rc;
    }
    *va_out = va;
    return B200OPT_OK;
}

}  // namespace

int fabric_init(std::string *err)
{
    // the runtime must have initialised the driver before entry points resolve
    cudaFree(nullptr);
    Driver &d = drv();
    if(!d.ok) {
        if(err)
            *err = d.why;
        return B200OPT_EUNSUPPORTED;
    }
    return B200OPT_OK;
}

int fabric_multicast_supported(int device, bool *yes, std::string *err)
{
    *yes = false;
    int rc = fabric_init(err);
    if(rc)
        return rc;
    CUdevice dev;
    CU(DeviceGet(&dev, device));
    int v = 0;
    CU(DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev));
    *yes = v != 0;
    return B200OPT_OK;
}

int fabric_granularity(int device, int nranks, bool multicast, size_t *gran,
                       std::string *err)
{
    int rc = fabric_init(err);
    if(rc)
        return rc;
    const CUmemAllocationProp prop = alloc_prop(device);
    size_t g = 0;
    CU(MemGetAllocationGranularity(&g, &prop,
                                   CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    if(multicast) {
        // the size passed here only has to be plausible: the granularity does
        // not depend on it
        const CUmulticastObjectProp mp = mc_prop(nranks, g);
        size_t mg = 0;
        CU(MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
        g = std::max(g, mg);
    }
    *gran = g;
    return B200OPT_OK;
}

int fabric_alloc(FabricMapping *out, int device, size_t bytes, std::string *err)
{
    int rc = fabric_init(err);
    if(rc)
        return rc;
    const CUmemAllocationProp prop = alloc_prop(device);
    CUmemGenericAllocationHandle h = 0;
    CU(MemCreate(&h, bytes, &prop, 0));
    CUdeviceptr va = 0;
    rc = map_handle(h, bytes, device, &va, err);
    if(rc) {
        drv().MemRelease(h);
        return rc;
    }
    out->mem = h;
    out->va = va;
    out->bytes = bytes;
    out->owns_mem = true;
    return B200OPT_OK;
}

int fabric_grant(const FabricMapping &m, int device, std::string *err)
{
    return set_access(m.va, m.bytes, device, err);
}

int fabric_export_fd(CUmemGenericAllocationHandle h, int *fd, std::string *err)
{
    int out = -1;
    CU(MemExportToShareableHandle(&out, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR,
                                  0));
    *fd = out;
    return B200OPT_OK;
}

int fabric_import(FabricMapping *out, int fd, int device, size_t bytes,
                  std::string *err)
{
    int rc = fabric_init(err);
    if(rc)
        return rc;
    CUmemGenericAllocationHandle h = 0;
    CU(MemImportFromShareableHandle(&h, (void *)(uintptr_t)fd,
                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    CUdeviceptr va = 0;
    rc = map_handle(h, bytes, device, &va, err);
    if(rc) {
        drv().MemRelease(h);
        return rc;
    }
    out->mem = h;
    out->va = va;
    out->bytes = bytes;
    out->owns_mem = true;  // an imported handle holds its own reference
    return B200OPT_OK;
}

void fabric_unmap(FabricMapping *m)
{
    if(!m || !drv().ok)
        return;
    if(m->va) {
        drv().MemUnmap(m->va, m->bytes);
        drv().MemAddressFree(m->va, m->bytes);
    }
    if(m->mem && m->owns_mem)
        drv().MemRelease(m->mem);
    *m = FabricMapping();
}

int fabric_mc_create(FabricMulticast *out, int nranks, size_t bytes,
                     std::string *err)
{
    int rc = fabric_init(err);
    if(rc)
        return rc;
    const CUmulticastObjectProp prop = mc_prop(nranks, bytes);
    CUmemGenericAllocationHandle h = 0;
    CU(MulticastCreate(&h, &prop));
    out->mc = h;
    out->bytes = bytes;
    out->owns_handle = true;
    return B200OPT_OK;
}

int fabric_mc_import(FabricMulticast *out, int fd, size_t bytes, std::string *err)
{
    int rc = fabric_init(err);
    if(rc)
        return rc;
    CUmemGenericAllocationHandle h = 0;
    CU(MemImportFromShareableHandle(&h, (void *)(uintptr_t)fd,
                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    out->mc = h;
    out->bytes = bytes;
    out->owns_handle = true;
    return B200OPT_OK;
}

int fabric_mc_add_device(FabricMulticast *mc, int device, std::string *err)
{
    CUdevice dev;
    CU(DeviceGet(&dev, device));
    CU(MulticastAddDevice(mc->mc, dev));
    mc->device = device;
    return B200OPT_OK;
}

int fabric_mc_bind(FabricMulticast *mc, const FabricMapping &arena, int device,
                   std::string *err)
{
    if(arena.bytes != mc->bytes) {
        if(err)
            *err = "arena and multicast object differ in size";
        return B200OPT_EINVAL;
    }
    CU(MulticastBindMem(mc->mc, 0, arena.mem, 0, arena.bytes, 0));
    mc->bound = true;
    mc->device = device;
    CUdeviceptr va = 0;
    const int rc = map_handle(mc->mc, mc->bytes, device, &va, err);
    if(rc)
        return rc;
    mc->va = va;
    return B200OPT_OK;
}

void fabric_mc_release(FabricMulticast *mc)
{
    if(!mc || !drv().ok)
        return;
    if(mc->va) {
        drv().MemUnmap(mc->va, mc->bytes);
        drv().MemAddressFree(mc->va, mc->bytes);
    }
    if(mc->bound) {
        CUdevice dev;
        if(drv().DeviceGet(&dev, mc->device) == CUDA_SUCCESS)
            drv().MulticastUnbind(mc->mc, dev, 0, mc->bytes);
    }
    if(mc->mc && mc->owns_handle)
        drv().MemRelease(mc->mc);
    *mc = FabricMulticast();
}

}  // namespace b200
