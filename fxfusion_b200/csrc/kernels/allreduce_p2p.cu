// Sum-all-reduce of an activation over the tensor-parallel ranks of ONE node through peer memory (NVLink),
// for the two exchange steps of a tensor-parallel transformer layer (after the attention output projection and
// after the second FeedForward product).  The reference has no communication layer; the alternative here is
// NCCL's all-reduce, which at these sizes (25 MB at GPT-2-small shape) is latency-bound: 76 us on 2 GPUs, 115 us on 4.
//
// Every rank maps the other ranks' engine allocations (CUDA IPC), so a tensor at arena offset X is reachable on every
// rank as base[r] + X.  One kernel per all-reduce, same grid on every rank:
//   1. start barrier   block b of rank r tells block b of every peer "my partial sums are written" and waits for theirs;
//   2. reduce-scatter  rank r owns slice r of the buffer: it loads that slice from every rank (ranks in fixed order
//      + all-gather    0..n-1, so the sum does not depend on timing), adds, and stores the result into slice r of
//                      every rank's buffer — plain ld / st over NVLink, no multimem, no TMA;
//   3. end barrier     "my slice is stored everywhere"; when all peers said so the local buffer is complete.
// Flags live in each rank's allocation ([peer][block] ints); their values are a per-engine epoch that only grows
// (kept in device memory so that a captured CUDA Graph replays correctly).  Waits are bounded: on expiry the kernel
// records error 121 / 122 in the engine's status word and returns (20 s for the start barrier, which also absorbs
// the skew between the ranks' host threads; 2 s for the end barrier).
#include "../runtime.hpp"
#include "sm100.cuh"

namespace fxf {
namespace {

using sm100::global_ns;

constexpr int kP2pThreads = 512;
// The start barrier also absorbs the skew between the ranks' host threads (each launches its own forward), so its
// budget is generous; once all ranks are inside the kernel the end barrier is a matter of microseconds.
constexpr unsigned long long kP2pStartBudgetNs = 20000000000ull, kP2pEndBudgetNs = 2000000000ull;
enum : int { kErrP2pStart = 121, kErrP2pEnd = 122 };

struct P2pParams {
    float* buf[kMaxTpRanks];
    int* flags[kMaxTpRanks];
    int* epoch;        // [0] epoch of the last finished all-reduce, [1] blocks finished in this launch
    int* status;
    int rank, n;
    int64_t count4;    // float4 elements in the whole buffer
    int64_t slice4;    // float4 elements per rank slice
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ float4 ld_peer(const float4* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// Block b of this rank <-> block b of every peer.  Returns false (in every thread) when a wait ran out.
__device__ bool peer_barrier(const P2pParams& p, int value, unsigned long long budget_ns, int* timed_out) {
    __threadfence_system();
    __syncthreads();
    const int t = threadIdx.x;
    if (t < p.n && t != p.rank) {
        st_release_sys(p.flags[t] + p.rank * gridDim.x + blockIdx.x, value);
        const int* mine = p.flags[p.rank] + t * gridDim.x + blockIdx.x;
        const unsigned long long t0 = global_ns();
        while (ld_acquire_sys(mine) - value < 0) {
            if (global_ns() - t0 > budget_ns) {
                *timed_out = 1;
                break;
            }
        }
    }
    __syncthreads();
    return *timed_out == 0;
}

__global__ void __launch_bounds__(kP2pThreads) p2p_all_reduce_kernel(P2pParams p) {
    __shared__ int timed_out;
    if (threadIdx.x == 0) timed_out = 0;
    const int epoch = *reinterpret_cast<volatile int*>(p.epoch);
    __syncthreads();
    bool ok = peer_barrier(p, epoch + 1, kP2pStartBudgetNs, &timed_out);
    if (!ok && threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kErrP2pStart);
    if (ok) {
        const int64_t lo = int64_t(p.rank) * p.slice4;
        const int64_t hi = min(lo + p.slice4, p.count4);
        const int64_t stride = int64_t(gridDim.x) * kP2pThreads;
        constexpr int U = 4;  // independent 16-byte loads per peer in flight per thread
        for (int64_t i0 = lo + int64_t(blockIdx.x) * kP2pThreads + threadIdx.x; i0 < hi; i0 += stride * U) {
            float4 acc[U];
#pragma unroll
            for (int u = 0; u < U; u++) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < p.n; r++) {
                const float4* src = reinterpret_cast<const float4*>(p.buf[r]);
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int64_t i = i0 + u * stride;
                    v[u] = i < hi ? ld_peer(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < U; u++) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
            }
            for (int r = 0; r < p.n; r++) {
                float4* dst = reinterpret_cast<float4*>(p.buf[r]);
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int64_t i = i0 + u * stride;
                    if (i < hi) dst[i] = acc[u];
                }
            }
        }
        ok = peer_barrier(p, epoch + 2, kP2pEndBudgetNs, &timed_out);
        if (!ok && threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kErrP2pEnd);
    }
    // the last block of this launch publishes the new epoch for the next all-reduce
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.epoch + 1, 1) == int(gridDim.x) - 1) {
            p.epoch[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile int*>(p.epoch) = epoch + 2;
        }
    }
}

}  // namespace

bool p2p_all_reduce_usable(const float* buf, int64_t n, const ExecCtx& ctx) {
    const PeerMap* pm = ctx.peers;
    if (pm == nullptr || ctx.tp_size < 2 || ctx.tp_size > kMaxTpRanks) return false;
    const char* b = reinterpret_cast<const char*>(buf);
    const char* base = pm->base[ctx.tp_rank];
    if (b < base || b + n * 4 > base + pm->shared_bytes) return false;  // only tensors at offsets every rank shares
    return n % 4 == 0 && aligned16(buf);
}

int launch_p2p_all_reduce(float* buf, int64_t n, ExecCtx& ctx) {
    const PeerMap* pm = ctx.peers;
    FXF_CHECK(p2p_all_reduce_usable(buf, n, ctx), "peer all-reduce called with a buffer outside the shared region");
    P2pParams p{};
    const size_t off = size_t(reinterpret_cast<char*>(buf) - pm->base[ctx.tp_rank]);
    for (int r = 0; r < ctx.tp_size; r++) {
        p.buf[r] = reinterpret_cast<float*>(pm->base[r] + off);
        p.flags[r] = reinterpret_cast<int*>(pm->base[r] + pm->flags_off);
    }
    p.epoch = reinterpret_cast<int*>(pm->base[ctx.tp_rank] + pm->epoch_off);
    p.status = ctx.status;
    p.rank = ctx.tp_rank; p.n = ctx.tp_size;
    p.count4 = n / 4;
    p.slice4 = (p.count4 + ctx.tp_size - 1) / ctx.tp_size;
    tag_launch(ctx, "p2p_all_reduce", double(n) * (ctx.tp_size - 1), 4.0 * double(n) * 2.0 * (ctx.tp_size - 1) / ctx.tp_size);
    p2p_all_reduce_kernel<<<pm->grid, kP2pThreads, 0, ctx.stream>>>(p);
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace fxf
