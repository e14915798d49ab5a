// Tensor-parallel communicator: a thin wrapper over NCCL, resolved at run time with dlopen so that the
// library has no link-time dependency on it (a process that already loaded libnccl.so.2, e.g. through
// PyTorch, shares that copy).  The reference has no communication layer at all; collectives exist here
// only where the tensor-parallel path has a real exchange step: one all-reduce after the attention output
// projection, one after the second FeedForward product, and a tiny all-gather of argmax candidates when the
// vocabulary is sharded.  The two all-reduces of a layer run as this library's own kernel over peer memory
// (kernels/allreduce_p2p.cu) once the ranks have mapped each other's engine allocations (tp_map_peers below: CUDA IPC
// handles exchanged through NCCL); NCCL's all-reduce remains the fallback and carries the small all-gather.  Everything is
// issued on the engine's stream and captured into its CUDA Graph.
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <vector>

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
    if (p2p_all_reduce_usable(buf, n, ctx)) return launch_p2p_all_reduce(buf, n, ctx);
    auto* c = static_cast<fxf_comm*>(ctx.comm);
    FXF_CHECK(c != nullptr && c->nccl != nullptr, "tensor-parallel engine has no communicator");
    FXF_NCCL(api().AllReduce(buf, buf, size_t(n), kNcclFloat32, kNcclSum, c->nccl, ctx.stream));
    if (ctx.trace) {
        tag_launch(ctx, "nccl_all_reduce", 0, 4.0 * double(n));
        if (trace_after_launch(ctx)) return 1;
    }
    return 0;
}

// Exchanges the CUDA IPC handles of the ranks' engine allocations (64 bytes each, gathered with NCCL through a small
// device buffer) and maps every peer's allocation into this process.  Collective.  Returns non-zero, leaving `out`
// unusable, when peer mapping is not possible (the caller then keeps NCCL for the all-reduce).
int tp_map_peers(void* comm, void* base, PeerMap* out) {
    auto* c = static_cast<fxf_comm*>(comm);
    FXF_CHECK(c != nullptr && c->nccl != nullptr && c->size >= 2 && c->size <= kMaxTpRanks, "peer mapping needs a communicator of 2..%d ranks", kMaxTpRanks);
    // slot layout: [ok flag (int) | 60 bytes padding | 64-byte handle] per rank, so that a failing rank is seen by all
    constexpr size_t kSlot = 128;
    char mine[kSlot] = {};
    cudaIpcMemHandle_t h;
    int ok = cudaIpcGetMemHandle(&h, base) == cudaSuccess ? 1 : 0;
    if (!ok) cudaGetLastError();
    std::memcpy(mine, &ok, sizeof(ok));
    std::memcpy(mine + 64, &h, sizeof(h));
    char* dev = nullptr;
    FXF_CUDA(cudaMalloc(reinterpret_cast<void**>(&dev), kSlot * size_t(c->size + 1)));
    std::vector<char> all(kSlot * size_t(c->size));
    cudaStream_t s = nullptr;
    FXF_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    int rc = 0;
    do {
        if (cudaMemcpyAsync(dev, mine, kSlot, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = 1; break; }
        if (api().AllGather(dev, dev + kSlot, kSlot, kNcclInt8, c->nccl, s) != 0) { rc = 1; break; }
        if (cudaMemcpyAsync(all.data(), dev + kSlot, all.size(), cudaMemcpyDeviceToHost, s) != cudaSuccess) { rc = 1; break; }
        if (cudaStreamSynchronize(s) != cudaSuccess) { rc = 1; break; }
    } while (false);
    cudaStreamDestroy(s);
    cudaFree(dev);
    FXF_CHECK(rc == 0, "peer mapping: exchanging the IPC handles failed");
    for (int r = 0; r < c->size; r++) {
        int peer_ok = 0;
        std::memcpy(&peer_ok, all.data() + kSlot * size_t(r), sizeof(peer_ok));
        FXF_CHECK(peer_ok == 1, "peer mapping: rank %d could not export its allocation", r);
    }
    int opened = 1;
    std::string why;
    for (int r = 0; r < c->size && opened; r++) {
        if (r == c->rank) {
            out->base[r] = static_cast<char*>(base);
            continue;
        }
        cudaIpcMemHandle_t ph;
        std::memcpy(&ph, all.data() + kSlot * size_t(r) + 64, sizeof(ph));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, ph, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            opened = 0;
            why = std::string("cudaIpcOpenMemHandle for rank ") + std::to_string(r) + " failed: " + cudaGetErrorString(e);
        } else {
            out->base[r] = static_cast<char*>(p);
        }
    }
    // every rank must take the same decision: count the ranks that mapped all their peers
    float* agree = nullptr;
    FXF_CUDA(cudaMalloc(reinterpret_cast<void**>(&agree), 256));
    const float mine_ok = float(opened);
    float total = 0.f;
    int arc = 0;
    if (cudaMemcpy(agree, &mine_ok, sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) arc = 1;
    if (!arc && api().AllReduce(agree, agree, 1, kNcclFloat32, kNcclSum, c->nccl, nullptr) != 0) arc = 1;
    if (!arc && cudaDeviceSynchronize() != cudaSuccess) arc = 1;
    if (!arc && cudaMemcpy(&total, agree, sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) arc = 1;
    cudaFree(agree);
    if (arc || int(total + 0.5f) != c->size) {
        for (int r = 0; r < c->size; r++)
            if (r != c->rank && out->base[r]) cudaIpcCloseMemHandle(out->base[r]);
        *out = PeerMap{};
        FXF_FAIL("peer mapping is not available on every rank%s%s", why.empty() ? "" : ": ", why.c_str());
    }
    return 0;
}

// Unmaps the peers.  The tiny all-reduce afterwards keeps any rank from freeing its allocation while a peer still has
// it mapped.
void tp_unmap_peers(void* comm, PeerMap* pm) {
    auto* c = static_cast<fxf_comm*>(comm);
    if (c == nullptr || pm == nullptr) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->size && r < kMaxTpRanks; r++)
        if (r != c->rank && pm->base[r]) cudaIpcCloseMemHandle(pm->base[r]);
    float* d = nullptr;
    if (c->nccl && cudaMalloc(reinterpret_cast<void**>(&d), 256) == cudaSuccess) {
        cudaMemset(d, 0, 256);
        api().AllReduce(d, d, 1, kNcclFloat32, kNcclSum, c->nccl, nullptr);
        cudaDeviceSynchronize();
        cudaFree(d);
    }
    *pm = PeerMap{};
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
