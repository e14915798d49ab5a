// Tensor-parallel communicator: a thin wrapper over NCCL, resolved at run time with dlopen so that the
// library has no link-time dependency on it (a process that already loaded libnccl.so.2, e.g. through
// PyTorch, shares that copy).  The reference has no communication layer at all; collectives exist here
// only where the tensor-parallel path has a real exchange step: one all-reduce after the attention output
// projection, one after the second FeedForward product, and a tiny all-gather of argmax candidates when the
// vocabulary is sharded.  NCCL calls are made on the engine's stream and are captured into its CUDA Graph.
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "runtime.hpp"

namespace fxf {
namespace {

struct NcclId {
    char internal[128];
};
using ncclComm_t = void*;
struct NcclApi {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
    std::string why;
};
constexpr int kNcclFloat32 = 7, kNcclSum = 0, kNcclInt8 = 0;

NcclApi& api() {
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            a.why = std::string("cannot load libnccl.so.2: ") + dlerror();
            return;
        }
        auto sym = [&](const char* name) { return dlsym(h, name); };
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.AllReduce && a.AllGather && a.CommDestroy && a.GetErrorString;
        if (!a.ok) a.why = "libnccl.so.2 lacks a required symbol";
    });
    return a;
}

}  // namespace
}  // namespace fxf

struct fxf_comm {
    void* nccl = nullptr;
    int rank = 0, size = 1, device = 0;
};

namespace fxf {

#define FXF_NCCL(expr)                                                                              \
    do {                                                                                            \
        int _r = (expr);                                                                            \
        if (_r != 0) FXF_FAIL("NCCL error %d (%s) at %s:%d", _r, api().GetErrorString(_r), __FILE__, __LINE__); \
    } while (0)

int tp_all_reduce_sum(float* buf, int64_t n, ExecCtx& ctx) {
    if (ctx.tp_size <= 1 || n == 0) return 0;
    auto* c = static_cast<fxf_comm*>(ctx.comm);
    FXF_CHECK(c != nullptr && c->nccl != nullptr, "tensor-parallel engine has no communicator");
    FXF_NCCL(api().AllReduce(buf, buf, size_t(n), kNcclFloat32, kNcclSum, c->nccl, ctx.stream));
    if (ctx.trace) {
        tag_launch(ctx, "nccl_all_reduce", 0, 4.0 * double(n));
        if (trace_after_launch(ctx)) return 1;
    }
    return 0;
}

int tp_all_gather(const void* send, void* recv, int64_t bytes, ExecCtx& ctx) {
    if (ctx.tp_size <= 1) {
        if (send != recv && bytes) FXF_CUDA(cudaMemcpyAsync(recv, send, size_t(bytes), cudaMemcpyDeviceToDevice, ctx.stream));
        return 0;
    }
    auto* c = static_cast<fxf_comm*>(ctx.comm);
    FXF_CHECK(c != nullptr && c->nccl != nullptr, "tensor-parallel engine has no communicator");
    FXF_NCCL(api().AllGather(send, recv, size_t(bytes), kNcclInt8, c->nccl, ctx.stream));
    return 0;
}

}  // namespace fxf

using namespace fxf;

extern "C" {

FXF_API int fxf_comm_unique_id(void* out_128_bytes) {
    FXF_CHECK(out_128_bytes != nullptr, "fxf_comm_unique_id: NULL argument");
    FXF_CHECK(api().ok, "%s", api().why.c_str());
    FXF_NCCL(api().GetUniqueId(static_cast<NcclId*>(out_128_bytes)));
    return 0;
}

FXF_API int fxf_comm_create(const void* unique_id_128_bytes, int rank, int size, int device_ordinal, fxf_comm** out) {
    FXF_CHECK(unique_id_128_bytes && out, "fxf_comm_create: NULL argument");
    FXF_CHECK(size >= 1 && rank >= 0 && rank < size, "fxf_comm_create: rank %d is outside [0, %d)", rank, size);
    FXF_CHECK(api().ok, "%s", api().why.c_str());
    FXF_CUDA(cudaSetDevice(device_ordinal));
    NcclId id;
    std::memcpy(&id, unique_id_128_bytes, sizeof(id));
    auto c = std::make_unique<fxf_comm>();
    c->rank = rank; c->size = size; c->device = device_ordinal;
    FXF_NCCL(api().CommInitRank(&c->nccl, size, id, rank));
    *out = c.release();
    return 0;
}

FXF_API void fxf_comm_destroy(fxf_comm* c) {
    if (!c) return;
    if (c->nccl && api().ok) api().CommDestroy(c->nccl);
    delete c;
}

FXF_API int fxf_comm_rank(const fxf_comm* c) { return c ? c->rank : -1; }
FXF_API int fxf_comm_size(const fxf_comm* c) { return c ? c->size : -1; }

}  // extern "C"
