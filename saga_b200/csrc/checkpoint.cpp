// Optimizer-state checkpoints in Saga's own tensor file format, so that the
// files can be inspected and loaded with Saga's Tensor::load.
//
// The format (src/tensor.cpp:1382-1552 of the Saga tree): 8 bytes "sagaT001",
// u32 element type (0 = float, 1 = half), u32 rank, rank x u32 dimensions, then
// the elements in row-major order; written to "<path>.tmp" and renamed into
// place.  Saga saves weights only (src/graph.cpp:60-104); m, v, the fp32 master
// copy, the iteration counter and the loss scale are lost there, so a resumed
// run restarts Adam from zero moments.  These files carry exactly that state.
//
// Host code only: device memory is reached through the library's own
// b200opt_export_state / b200opt_import_state.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/b200opt.h"

namespace {

struct DiskHeader {
    uint8_t magic[8];
    uint32_t type;
    uint32_t rank;
} __attribute__((packed));
static_assert(sizeof(DiskHeader) == 16, "Saga's tensor file header is 16 bytes");

const char kMagic[] = "sagaT001";

bool write_all(int fd, const void *buf, size_t n)
{
    const char *p = static_cast<const char *>(buf);
    while(n) {
        const ssize_t w = write(fd, p, n);
        if(w < 0) {
            if(errno == EINTR)
                continue;
            return false;
        }
        p += w;
        n -= (size_t)w;
    }
    return true;
}

bool read_all(int fd, void *buf, size_t n)
{
    char *p = static_cast<char *>(buf);
    while(n) {
        const ssize_t r = read(fd, p, n);
        if(r < 0 && errno == EINTR)
            continue;
        if(r <= 0)
            return false;
        p += r;
        n -= (size_t)r;
    }
    return true;
}

std::string part_path(const char *dir, int rank, int nranks, const char *what)
{
    char buf[64];
    snprintf(buf, sizeof(buf), "/adam.r%dof%d.%s.saga", rank, nranks, what);
    return std::string(dir) + buf;
}

// the scalars of a checkpoint, all exactly representable as float
enum {
    kMetaVersion = 0, kMetaRank, kMetaNranks, kMetaIterLow, kMetaIterHigh, kMetaScale,
    kMetaPolicyState, kMetaCount
};

}  // namespace

extern "C" {

int b200opt_tensor_save(const char *path, int dtype, unsigned rank,
                        const uint32_t *dims, const void *data)
{
    if(!path || rank > 8 || (rank && !dims) ||
       (dtype != B200OPT_HALF && dtype != B200OPT_FLOAT))
        return B200OPT_EINVAL;
    size_t elems = 1;
    for(unsigned i = 0; i < rank; i++)
        elems *= dims[i];
    if(elems && !data)
        return B200OPT_EINVAL;
    const size_t bytes = elems * (dtype == B200OPT_HALF ? 2 : 4);
    DiskHeader hd;
    memcpy(hd.magic, kMagic, 8);
    hd.type = dtype == B200OPT_HALF ? 1u : 0u;
    hd.rank = rank;
    const std::string tmp = std::string(path) + ".tmp";
    const int fd = open(tmp.c_str(), O_CREAT | O_TRUNC | O_WRONLY, 0644);
    if(fd == -1)
        return B200OPT_EINVAL;
    const bool ok = write_all(fd, &hd, sizeof(hd)) &&
                    write_all(fd, dims, sizeof(uint32_t) * rank) &&
                    write_all(fd, data, bytes);
    if(close(fd) != 0 || !ok || rename(tmp.c_str(), path) != 0) {
        unlink(tmp.c_str());
        return B200OPT_EINVAL;
    }
    return B200OPT_OK;
}

int b200opt_tensor_load(const char *path, int *dtype, unsigned *rank,
                        uint32_t dims[8], void *data, size_t capacity_bytes,
                        size_t *bytes)
{
    if(!path)
        return B200OPT_EINVAL;
    const int fd = open(path, O_RDONLY);
    if(fd == -1)
        return B200OPT_EINVAL;
    DiskHeader hd;
    uint32_t d[8] = {};
    int rc = B200OPT_EINVAL;
    do {
        if(!read_all(fd, &hd, sizeof(hd)) || memcmp(hd.magic, kMagic, 8) != 0)
            break;
        if(hd.type > 1 || hd.rank > 8)
            break;
        if(!read_all(fd, d, sizeof(uint32_t) * hd.rank))
            break;
        size_t elems = 1;
        for(unsigned i = 0; i < hd.rank; i++)
            elems *= d[i];
        const size_t need = elems * (hd.type == 1 ? 2 : 4);
        struct stat st;
        if(fstat(fd, &st) != 0 ||
           (size_t)st.st_size < sizeof(hd) + sizeof(uint32_t) * hd.rank + need)
            break;  // file too short
        if(dtype)
            *dtype = hd.type == 1 ? B200OPT_HALF : B200OPT_FLOAT;
        if(rank)
            *rank = hd.rank;
        if(dims)
            memcpy(dims, d, sizeof(d));
        if(bytes)
            *bytes = need;
        if(data) {
            if(capacity_bytes < need || !read_all(fd, data, need))
                break;
        }
        rc = B200OPT_OK;
    } while(0);
    close(fd);
    return rc;
}

int b200opt_checkpoint_save(b200opt_t *h, const char *dir, float scale,
                            int policy_state)
{
    if(!h || !dir)
        return B200OPT_EINVAL;
    int rank = 0, nranks = 1, iter = 0;
    int rc = b200opt_rank_info(h, &rank, &nranks);
    if(!rc)
        rc = b200opt_get_iter(h, &iter);
    if(rc)
        return rc;
    std::vector<float> buf;
    static const char *const names[2][3] = {{"half.m", "half.v", "half.master"},
                                            {"float.m", "float.v", nullptr}};
    for(int dt = 0; dt < 2; dt++) {
        for(int which = 0; which < 3; which++) {
            if(!names[dt][which])
                continue;
            size_t cnt = 0;
            rc = b200opt_export_state(h, dt, which, nullptr, 0, &cnt);
            if(rc)
                return rc;
            if(cnt > 0xFFFFFFFFull)
                return B200OPT_ETOOBIG;
            buf.resize(cnt ? cnt : 1);
            rc = b200opt_export_state(h, dt, which, buf.data(), cnt, &cnt);
            if(rc)
                return rc;
            const uint32_t dims[1] = {(uint32_t)cnt};
            rc = b200opt_tensor_save(part_path(dir, rank, nranks, names[dt][which]).c_str(),
                                     B200OPT_FLOAT, 1, dims, buf.data());
            if(rc)
                return rc;
        }
    }
    float meta[kMetaCount] = {};
    meta[kMetaVersion] = 1;
    meta[kMetaRank] = (float)rank;
    meta[kMetaNranks] = (float)nranks;
    meta[kMetaIterLow] = (float)(iter & 0xFFFF);
    meta[kMetaIterHigh] = (float)((unsigned)iter >> 16);
    meta[kMetaScale] = scale;
    meta[kMetaPolicyState] = (float)policy_state;
    const uint32_t mdims[1] = {kMetaCount};
    // the scalars go last: their presence marks a complete checkpoint
    return b200opt_tensor_save(part_path(dir, rank, nranks, "meta").c_str(),
                               B200OPT_FLOAT, 1, mdims, meta);
}

int b200opt_checkpoint_load(b200opt_t *h, const char *dir, float *scale,
                            int *policy_state)
{
    if(!h || !dir)
        return B200OPT_EINVAL;
    int rank = 0, nranks = 1;
    int rc = b200opt_rank_info(h, &rank, &nranks);
    if(rc)
        return rc;
    float meta[kMetaCount] = {};
    int dtype = -1;
    unsigned trank = 0;
    uint32_t dims[8] = {};
    size_t bytes = 0;
    rc = b200opt_tensor_load(part_path(dir, rank, nranks, "meta").c_str(), &dtype, &trank,
                             dims, meta, sizeof(meta), &bytes);
    if(rc)
        return rc;
    if(dtype != B200OPT_FLOAT || trank != 1 || dims[0] != kMetaCount ||
       meta[kMetaVersion] != 1 || (int)meta[kMetaRank] != rank ||
       (int)meta[kMetaNranks] != nranks)
        return B200OPT_EINVAL;
    std::vector<float> buf;
    static const char *const names[2][3] = {{"half.m", "half.v", "half.master"},
                                            {"float.m", "float.v", nullptr}};
    for(int dt = 0; dt < 2; dt++) {
        for(int which = 0; which < 3; which++) {
            if(!names[dt][which])
                continue;
            size_t cnt = 0;
            rc = b200opt_export_state(h, dt, which, nullptr, 0, &cnt);
            if(rc)
                return rc;
            const std::string path = part_path(dir, rank, nranks, names[dt][which]);
            rc = b200opt_tensor_load(path.c_str(), &dtype, &trank, dims, nullptr, 0, &bytes);
            if(rc)
                return rc;
            if(dtype != B200OPT_FLOAT || trank != 1 || dims[0] != cnt)
                return B200OPT_EINVAL;  // saved from another layout or rank count
            buf.resize(cnt ? cnt : 1);
            rc = b200opt_tensor_load(path.c_str(), nullptr, nullptr, nullptr, buf.data(),
                                     cnt * 4, nullptr);
            if(rc)
                return rc;
            if(cnt) {
                rc = b200opt_import_state(h, dt, which, buf.data(), cnt);
                if(rc)
                    return rc;
            }
        }
    }
    const int iter = (int)meta[kMetaIterLow] | ((int)meta[kMetaIterHigh] << 16);
    rc = b200opt_set_iter(h, iter);
    if(rc)
        return rc;
    if(scale)
        *scale = meta[kMetaScale];
    if(policy_state)
        *policy_state = (int)meta[kMetaPolicyState];
    return B200OPT_OK;
}

}  // extern "C"
