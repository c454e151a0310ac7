#include "nccl_path.h"

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "../../include/b200opt.h"

namespace b200 {

namespace {

struct Api {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t,
                                  ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t,
                              ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t,
                              ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

Api &api()
{
    static Api a;
    static std::once_flag once;
    std::call_once(once, [] {
        // a copy already mapped into the process (e.g. by PyTorch) is reused
        a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if(!a.lib)
            a.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
        if(!a.lib)
            return;
#define SYM(field, name) \
    a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.lib, name))
        SYM(GetUniqueId, "ncclGetUniqueId");
        SYM(CommInitRank, "ncclCommInitRank");
        SYM(CommDestroy, "ncclCommDestroy");
        SYM(ReduceScatter, "ncclReduceScatter");
        SYM(AllGather, "ncclAllGather");
        SYM(AllReduce, "ncclAllReduce");
        SYM(GroupStart, "ncclGroupStart");
        SYM(GroupEnd, "ncclGroupEnd");
        SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy &&
               a.ReduceScatter && a.AllGather && a.AllReduce && a.GroupStart &&
               a.GroupEnd && a.GetErrorString;
    });
    return a;
}

int nccl_fail(ncclResult_t r, const char *what, std::string *err)
{
    if(err)
        *err = std::string(what) + ": " + api().GetErrorString(r);
    return B200OPT_ECUDA;
}

#define NK(call)                               \
    do {                                       \
        ncclResult_t r_ = (call);              \
        if(r_ != ncclSuccess)                  \
            return nccl_fail(r_, #call, err);  \
    } while(0)

}  // namespace

struct NcclPath {
    ncclComm_t comm = nullptr;
    int rank = 0, nranks = 1;
};

int nccl_path_unique_id(void *id128)
{
    static_assert(sizeof(ncclUniqueId) == B200OPT_NCCL_ID_BYTES, "id size");
    if(!api().ok)
        return B200OPT_EUNSUPPORTED;
    ncclUniqueId id;
    if(api().GetUniqueId(&id) != ncclSuccess)
        return B200OPT_ECUDA;
    memcpy(id128, &id, sizeof(id));
    return B200OPT_OK;
}

int nccl_path_create(NcclPath **out, int rank, int nranks, const void *id128,
                     std::string *err)
{
    if(!api().ok) {
        if(err)
            *err = "libnccl.so.2 could not be opened";
        return B200OPT_EUNSUPPORTED;
    }
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    NcclPath *np = new NcclPath;
    np->rank = rank;
    np->nranks = nranks;
    ncclResult_t r = api().CommInitRank(&np->comm, nranks, id, rank);
    if(r != ncclSuccess) {
        delete np;
        return nccl_fail(r, "ncclCommInitRank", err);
    }
    *out = np;
    return B200OPT_OK;
}

void nccl_path_destroy(NcclPath *np)
{
    if(!np)
        return;
    if(np->comm)
        api().CommDestroy(np->comm);
    delete np;
}

int nccl_path_reduce_scatter(NcclPath *np, uint16_t *g_half, size_t s_half,
                             float *g_float, size_t s_float, cudaStream_t st,
                             std::string *err)
{
    NK(api().GroupStart());
    if(s_float)
        NK(api().ReduceScatter(g_float, g_float + s_float * np->rank, s_float,
                               ncclFloat32, ncclSum, np->comm, st));
    if(s_half)
        NK(api().ReduceScatter(g_half, g_half + s_half * np->rank, s_half,
                               ncclFloat16, ncclSum, np->comm, st));
    NK(api().GroupEnd());
    return B200OPT_OK;
}

int nccl_path_all_gather_and_flags(NcclPath *np, uint16_t *w_half,
                                   size_t s_half, float *w_float,
                                   size_t s_float, uint32_t *flags3,
                                   cudaStream_t st, std::string *err)
{
    NK(api().GroupStart());
    if(s_float)
        NK(api().AllGather(w_float + s_float * np->rank, w_float, s_float,
                           ncclFloat32, np->comm, st));
    if(s_half)
        NK(api().AllGather(w_half + s_half * np->rank, w_half, s_half,
                           ncclFloat16, np->comm, st));
    NK(api().AllReduce(flags3, flags3, 3, ncclUint32, ncclSum, np->comm, st));
    NK(api().GroupEnd());
    return B200OPT_OK;
}

}  // namespace b200
