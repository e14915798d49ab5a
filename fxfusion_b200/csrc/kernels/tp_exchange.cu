// Exchange steps of the tensor-parallel layout over peer memory (NVLink), one kernel per exchange.  The reference has no
// communication layer; these kernels exist because a tensor-parallel transformer layer has two real exchange steps: the
// partial [M,D] outputs of the attention output projection and of the second FeedForward product must be summed over the
// ranks.  Every rank maps the other ranks' engine allocations (CUDA IPC), so a tensor at arena offset X is reachable on
// every rank as base[r] + X.
//
//   p2p_all_reduce_kernel   in-place sum of a buffer over the ranks:
//       start barrier -> rank r sums slice r over the ranks (fixed order 0..n-1) and stores it into slice r of every
//       rank's buffer -> end barrier.
//   tp_exchange_ln_kernel   the exchange fused with the residual Add and the LayerNorm that follow it in a pre-LN
//       transformer block (Add -> LayerNorm, or AddLayerNorm):
//       start barrier -> rank r owns rows [r*R, (r+1)*R) of the [M,D] activation: per row (one warp) it loads the row's
//       partial sums from every rank (plain peer loads, ranks in fixed order), adds the residual row (local), writes the
//       new residual row (to its own memory only — the residual stream stays row-sharded between exchanges — unless
//       someone outside this scheme reads it), normalises the row in registers and stores the normalised row into
//       EVERY rank's LayerNorm output (plain peer stores) -> end barrier.
//       NVLink traffic per rank is that of an all-reduce: (n-1)/n of the buffer arrives as fetched partial rows and
//       another (n-1)/n as the normalised rows the peers store, and as much leaves.  The separate residual Add, the
//       LayerNorm launch and their HBM round trips disappear, and each rank normalises only M/n rows.
//       Pushed variant: the row-parallel product that precedes the exchange has already stored its partial sums of the
//       rows rank q owns into rank q's exchange window (GemmArgs::push_out: peer stores from the GEMM epilogue, hidden
//       behind the product), at row p*R + (row - q*R) for producer p.  The kernel then finds all n partial rows in its own
//       memory, and only the normalised rows cross NVLink inside the exchange.  The window is a buffer of its own: a
//       producer writes it only after it has left the end barrier of the previous exchange, i.e. after every rank has
//       finished reading it.
//
// Only plain ld / st to peer memory: no multimem, no TMA.  Barriers: block b of rank r tells block b of every peer and
// waits for theirs; flag values are a per-engine epoch that only grows (kept in device memory so that a captured CUDA
// Graph replays correctly).  Every wait is bounded; a rank that gives up records 121 (start barrier) / 122 (end barrier)
// in its status word and raises an abort word on every peer, which makes their waits return at once (status 123).  A
// kernel that starts with a non-zero status or a raised abort word does nothing but keep the epoch in step.  After such a
// failure the engine's results are undefined and it has to be destroyed.
#include <cuda_runtime.h>

#include "../runtime.hpp"
#include "sm100.cuh"

namespace fxf {
namespace {

using sm100::global_ns;

constexpr int kP2pThreads = 512;
constexpr int kXchgWarps = 8, kXchgThreads = kXchgWarps * 32;
enum : int { kErrP2pStart = 121, kErrP2pEnd = 122, kErrP2pPeer = 123 };

// Per rank: flags [peer][block]; ctl[0] epoch of the last finished exchange, ctl[1] blocks finished in this launch,
// ctl[2] abort word (a peer or this rank gave up).  Outside the single-GPU emulation only the own rank's ctl / status
// are used besides the peers' flags and abort words.
struct P2pSync {
    int* flags[kMaxTpRanks];
    int* ctl[kMaxTpRanks];
    int* status[kMaxTpRanks];
    int n;
    unsigned long long start_ns, end_ns;
};

struct P2pParams {
    P2pSync sync;
    int rank;          // < 0: single-GPU emulation, rank = blockIdx.y
    float* buf[kMaxTpRanks];
    int64_t count4;    // float4 elements in the whole buffer
    int64_t slice4;    // float4 elements per rank slice
};

struct XchgParams {
    P2pSync sync;
    int rank;                             // < 0: single-GPU emulation, rank = blockIdx.y
    int skip_rank;                        // emulation only: this rank never arrives (exercises the bounded waits); -1 = none
    const float* part[kMaxTpRanks];       // every rank's partial sums [M, D]; pushed: every rank's exchange window
    int pushed;                           // the products stored their rows into the owners' windows (see below)
    float* y[kMaxTpRanks];                // LayerNorm output of every rank (y[0] == NULL: no LayerNorm)
    float* x[kMaxTpRanks];                // new residual stream; NULL entries are not written
    const float* residual[kMaxTpRanks];   // residual[r] is read by rank r only; NULL = none
    int x_own_only;                       // a rank writes only x[rank] (the residual stream stays row-sharded)
    const float* gamma;
    const float* beta;
    float eps, inv_d;
    int64_t M, rows_per_rank;
    int n4;                               // D / 4
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
__device__ __forceinline__ int ld_volatile(const int* p) { return *reinterpret_cast<const volatile int*>(p); }

// Tells every peer (and this rank's later kernels) that this rank has given up.
__device__ __forceinline__ void raise_abort(const P2pSync& s, int rank) {
    const int t = threadIdx.x;
    if (t < s.n) *reinterpret_cast<volatile int*>(s.ctl[t] + 2) = 1;
    (void)rank;
}

// Block b of this rank <-> block b of every peer.  Returns 0 when all peers arrived, 1 when the budget ran out, 2 when the
// abort word was raised while waiting (same value in every thread).
__device__ int peer_barrier(const P2pSync& s, int rank, int value, unsigned long long budget_ns, int* result) {
    __threadfence_system();
    __syncthreads();
    const int t = threadIdx.x;
    if (t < s.n && t != rank) {
        st_release_sys(s.flags[t] + rank * gridDim.x + blockIdx.x, value);
        const int* mine = s.flags[rank] + t * gridDim.x + blockIdx.x;
        const unsigned long long t0 = global_ns();
        unsigned int spin = 0;
        while (ld_acquire_sys(mine) - value < 0) {
            if ((++spin & 15u) == 0) {
                if (ld_volatile(s.ctl[rank] + 2) != 0) { atomicMax(result, 2); break; }
                if (global_ns() - t0 > budget_ns) { atomicMax(result, 1); break; }
            }
        }
    }
    __syncthreads();
    return *reinterpret_cast<volatile int*>(result);
}

// Status + abort after a failed barrier.
__device__ __forceinline__ void report_failure(const P2pSync& s, int rank, int rc, int code_timeout) {
    if (threadIdx.x == 0 && s.status[rank]) atomicCAS(s.status[rank], 0, rc == 2 ? int(kErrP2pPeer) : code_timeout);
    raise_abort(s, rank);
}

// True (in every thread) when this rank must not take part: an earlier kernel of the engine reported an error, or a peer
// gave up.  The peers are told, so that none of them waits for this rank.
__device__ bool must_stand_down(const P2pSync& s, int rank) {
    __shared__ int down;
    if (threadIdx.x == 0) down = ((s.status[rank] && ld_volatile(s.status[rank]) != 0) || ld_volatile(s.ctl[rank] + 2) != 0) ? 1 : 0;
    __syncthreads();
    const bool d = down != 0;
    if (d) {
        if (threadIdx.x == 0 && s.status[rank]) atomicCAS(s.status[rank], 0, int(kErrP2pPeer));
        raise_abort(s, rank);
    }
    return d;
}

// The last block of this rank's launch publishes the new epoch for the next exchange.
__device__ __forceinline__ void publish_epoch(const P2pSync& s, int rank, int epoch) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        int* ctl = s.ctl[rank];
        if (atomicAdd(ctl + 1, 1) == int(gridDim.x) - 1) {
            ctl[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile int*>(ctl) = epoch + 2;
        }
    }
}

__global__ void __launch_bounds__(kP2pThreads) p2p_all_reduce_kernel(P2pParams p) {
    __shared__ int result;
    const int rank = p.rank < 0 ? int(blockIdx.y) : p.rank;
    if (threadIdx.x == 0) result = 0;
    const int epoch = ld_volatile(p.sync.ctl[rank]);
    __syncthreads();
    if (!must_stand_down(p.sync, rank)) {
        int rc = peer_barrier(p.sync, rank, epoch + 1, p.sync.start_ns, &result);
        if (rc) report_failure(p.sync, rank, rc, kErrP2pStart);
        if (rc == 0) {
            const int64_t lo = int64_t(rank) * p.slice4;
            const int64_t hi = min(lo + p.slice4, p.count4);
            const int64_t stride = int64_t(gridDim.x) * kP2pThreads;
            constexpr int U = 4;  // independent 16-byte loads per peer in flight per thread
            for (int64_t i0 = lo + int64_t(blockIdx.x) * kP2pThreads + threadIdx.x; i0 < hi; i0 += stride * U) {
                float4 acc[U];
#pragma unroll
                for (int u = 0; u < U; u++) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int r = 0; r < p.sync.n; r++) {
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
                for (int r = 0; r < p.sync.n; r++) {
                    float4* dst = reinterpret_cast<float4*>(p.buf[r]);
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int64_t i = i0 + u * stride;
                        if (i < hi) dst[i] = acc[u];
                    }
                }
            }
            rc = peer_barrier(p.sync, rank, epoch + 2, p.sync.end_ns, &result);
            if (rc) report_failure(p.sync, rank, rc, kErrP2pEnd);
        }
    }
    publish_epoch(p.sync, rank, epoch);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ void add4(float4& a, const float4& b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }


// NV = float4 per lane per row (rows of up to 128 * NV floats).
template <int NV>
__global__ void __launch_bounds__(kXchgThreads, 1) tp_exchange_ln_kernel(XchgParams p) {
    __shared__ int result;
    const int rank = p.rank < 0 ? int(blockIdx.y) : p.rank;
    if (threadIdx.x == 0) result = 0;
    const int epoch = ld_volatile(p.sync.ctl[rank]);
    __syncthreads();
    if (rank == p.skip_rank) return;   // emulation of a rank that never reaches the exchange (uniform per block)
    if (!must_stand_down(p.sync, rank)) {
        int rc = peer_barrier(p.sync, rank, epoch + 1, p.sync.start_ns, &result);
        if (rc) report_failure(p.sync, rank, rc, kErrP2pStart);
        if (rc == 0) {
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n = p.sync.n, n4 = p.n4;
            const int64_t r0 = int64_t(rank) * p.rows_per_rank, r1 = min(p.M, r0 + p.rows_per_rank);
            const float4* res = reinterpret_cast<const float4*>(p.residual[rank]);
            const float4* gam = reinterpret_cast<const float4*>(p.gamma);
            const float4* bet = reinterpret_cast<const float4*>(p.beta);
            for (int64_t row = r0 + int64_t(blockIdx.x) * kXchgWarps + warp; row < r1; row += int64_t(gridDim.x) * kXchgWarps) {
                const int64_t off = row * n4;
                float4 v[NV], rr[NV];
                if (res) {
#pragma unroll
                    for (int i = 0; i < NV; i++) {
                        const int c = lane + 32 * i;
                        rr[i] = c < n4 ? res[off + c] : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                // the ranks' partial rows, four ranks at a time: every load of a group is issued before the first add
#pragma unroll 1
                for (int g0 = 0; g0 < n; g0 += 4) {
                    float4 t[4][NV];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        if (g0 + q < n) {
                            const float4* src = p.pushed ? reinterpret_cast<const float4*>(p.part[rank]) + (int64_t(g0 + q) * p.rows_per_rank + (row - r0)) * n4
                                                         : reinterpret_cast<const float4*>(p.part[g0 + q]) + off;
#pragma unroll
                            for (int i = 0; i < NV; i++) {
                                const int c = lane + 32 * i;
                                t[q][i] = c < n4 ? ld_peer(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        if (g0 + q < n) {
#pragma unroll
                            for (int i = 0; i < NV; i++) {
                                if (g0 + q == 0) v[i] = t[q][i];
                                else add4(v[i], t[q][i]);
                            }
                        }
                    }
                }
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    if (res) add4(v[i], rr[i]);
                    if (lane + 32 * i < n4) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                }
                for (int q = 0; q < n; q++) {
                    float4* xo = reinterpret_cast<float4*>(p.x[q]);
                    if (xo == nullptr || (p.x_own_only && q != rank)) continue;
#pragma unroll
                    for (int i = 0; i < NV; i++) {
                        const int c = lane + 32 * i;
                        if (c < n4) xo[off + c] = v[i];
                    }
                }
                if (p.y[0] == nullptr) continue;
                // LayerNorm of the row, same arithmetic as layernorm_warp_kernel: mean, centred sum of squares, one reciprocal
                const float mean = warp_sum(s) * p.inv_d;
                float qs = 0.f;
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    if (lane + 32 * i < n4) {
                        const float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
                        qs += (dx * dx + dy * dy) + (dz * dz + dw * dw);
                    }
                }
                const float var = warp_sum(qs) * p.inv_d;
                const float rstd = 1.0f / sqrtf(var + p.eps);
                const float shift = -rstd * mean;
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    const int c = lane + 32 * i;
                    if (c < n4) {
                        const float4 g = gam[c], bb = bet[c];
                        v[i].x = (v[i].x * rstd + shift) * g.x + bb.x;
                        v[i].y = (v[i].y * rstd + shift) * g.y + bb.y;
                        v[i].z = (v[i].z * rstd + shift) * g.z + bb.z;
                        v[i].w = (v[i].w * rstd + shift) * g.w + bb.w;
                    }
                }
                for (int q = 0; q < n; q++) {
                    float4* yo = reinterpret_cast<float4*>(p.y[q]) + off;
#pragma unroll
                    for (int i = 0; i < NV; i++) {
                        const int c = lane + 32 * i;
                        if (c < n4) yo[c] = v[i];
                    }
                }
            }
            rc = peer_barrier(p.sync, rank, epoch + 2, p.sync.end_ns, &result);
            if (rc) report_failure(p.sync, rank, rc, kErrP2pEnd);
        }
    }
    publish_epoch(p.sync, rank, epoch);
}

void fill_sync(P2pSync* s, const PeerMap* pm, const ExecCtx& ctx) {
    for (int r = 0; r < ctx.tp_size; r++) {
        s->flags[r] = reinterpret_cast<int*>(pm->base[r] + pm->flags_off);
        s->ctl[r] = reinterpret_cast<int*>(pm->base[r] + pm->epoch_off);
        s->status[r] = nullptr;
    }
    s->status[ctx.tp_rank] = ctx.status;
    s->n = ctx.tp_size;
    s->start_ns = pm->start_budget_ns;
    s->end_ns = pm->end_budget_ns;
}

bool in_shared_region(const void* ptr, int64_t bytes, const ExecCtx& ctx) {
    const PeerMap* pm = ctx.peers;
    const char* b = static_cast<const char*>(ptr);
    const char* base = pm->base[ctx.tp_rank];
    return b >= base && b + bytes <= base + pm->shared_bytes;   // only tensors at offsets every rank shares
}

template <int NV>
cudaError_t launch_xchg(const XchgParams& p, dim3 grid, cudaStream_t s, bool cooperative) {
    if (!cooperative) {
        tp_exchange_ln_kernel<NV><<<grid, kXchgThreads, 0, s>>>(p);
        return cudaPeekAtLastError();
    }
    void* args[] = {const_cast<XchgParams*>(&p)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(tp_exchange_ln_kernel<NV>), grid, dim3(kXchgThreads), args, 0, s);
}
cudaError_t launch_xchg_nv(int nv, const XchgParams& p, dim3 grid, cudaStream_t s, bool cooperative) {
    switch (nv) {
        case 1: return launch_xchg<1>(p, grid, s, cooperative);
        case 2: return launch_xchg<2>(p, grid, s, cooperative);
        case 3: return launch_xchg<3>(p, grid, s, cooperative);
        case 4: return launch_xchg<4>(p, grid, s, cooperative);
        case 5: return launch_xchg<5>(p, grid, s, cooperative);
        case 6: return launch_xchg<6>(p, grid, s, cooperative);
        case 7: return launch_xchg<7>(p, grid, s, cooperative);
        default: return launch_xchg<8>(p, grid, s, cooperative);
    }
}

}  // namespace

bool p2p_all_reduce_usable(const float* buf, int64_t n, const ExecCtx& ctx) {
    const PeerMap* pm = ctx.peers;
    if (pm == nullptr || ctx.tp_size < 2 || ctx.tp_size > kMaxTpRanks) return false;
    if (!in_shared_region(buf, n * 4, ctx)) return false;
    return n % 4 == 0 && aligned16(buf);
}

int launch_p2p_all_reduce(float* buf, int64_t n, ExecCtx& ctx) {
    const PeerMap* pm = ctx.peers;
    FXF_CHECK(p2p_all_reduce_usable(buf, n, ctx), "peer all-reduce called with a buffer outside the shared region");
    P2pParams p{};
    fill_sync(&p.sync, pm, ctx);
    const size_t off = size_t(reinterpret_cast<char*>(buf) - pm->base[ctx.tp_rank]);
    for (int r = 0; r < ctx.tp_size; r++) p.buf[r] = reinterpret_cast<float*>(pm->base[r] + off);
    p.rank = ctx.tp_rank;
    p.count4 = n / 4;
    p.slice4 = (p.count4 + ctx.tp_size - 1) / ctx.tp_size;
    tag_launch(ctx, "p2p_all_reduce", double(n) * (ctx.tp_size - 1), 4.0 * double(n) * 2.0 * (ctx.tp_size - 1) / ctx.tp_size);
    p2p_all_reduce_kernel<<<pm->grid, kP2pThreads, 0, ctx.stream>>>(p);
    FXF_LAUNCHED(ctx);
    return 0;
}

bool tp_exchange_usable(const TpExchange& x, const float* partial, int64_t M, int64_t D, const ExecCtx& ctx) {
    if (ctx.peers == nullptr || ctx.tp_size < 2 || ctx.tp_size > kMaxTpRanks) return false;
    if (D % 4 != 0 || D > 1024 || M <= 0) return false;
    const int64_t bytes = M * D * 4;
    if (partial != nullptr && (!aligned16(partial) || !in_shared_region(partial, bytes, ctx))) return false;   // NULL: pushed rows
    if (x.y_out && (!aligned16(x.y_out) || !in_shared_region(x.y_out, bytes, ctx) || !aligned16(x.gamma) || !aligned16(x.beta))) return false;
    if (x.x_out && (!aligned16(x.x_out) || !in_shared_region(x.x_out, bytes, ctx))) return false;
    if (x.residual && !aligned16(x.residual)) return false;
    return x.y_out != nullptr || x.x_out != nullptr;
}

bool tp_push_usable(int64_t M, int64_t D, const ExecCtx& ctx) {
    const PeerMap* pm = ctx.peers;
    if (pm == nullptr || ctx.tp_size < 2 || pm->push_bytes == 0 || M <= 0 || M % ctx.tp_size != 0) return false;
    return (M / ctx.tp_size) % 128 == 0 && size_t(M) * size_t(D) * 4 <= pm->push_bytes;
}

float* tp_push_window(int rank, const ExecCtx& ctx) { return reinterpret_cast<float*>(ctx.peers->base[rank] + ctx.peers->push_off); }

int launch_tp_exchange(const TpExchange& x, const float* partial, int64_t M, int64_t D, ExecCtx& ctx, bool pushed) {
    FXF_CHECK(tp_exchange_usable(x, pushed ? nullptr : partial, M, D, ctx), "tensor-parallel exchange called with operands it cannot serve");
    FXF_CHECK(!pushed || tp_push_usable(M, D, ctx), "tensor-parallel exchange: no exchange window for pushed rows");
    const PeerMap* pm = ctx.peers;
    XchgParams p{};
    fill_sync(&p.sync, pm, ctx);
    p.rank = ctx.tp_rank;
    p.skip_rank = -1;
    const char* mine = pm->base[ctx.tp_rank];
    for (int r = 0; r < ctx.tp_size; r++) {
        p.part[r] = pushed ? tp_push_window(r, ctx) : reinterpret_cast<const float*>(pm->base[r] + (reinterpret_cast<const char*>(partial) - mine));
        p.y[r] = x.y_out ? reinterpret_cast<float*>(pm->base[r] + (reinterpret_cast<char*>(x.y_out) - mine)) : nullptr;
        p.x[r] = (x.x_out && (x.replicate_x || r == ctx.tp_rank)) ? reinterpret_cast<float*>(pm->base[r] + (reinterpret_cast<char*>(x.x_out) - mine)) : nullptr;
        p.residual[r] = nullptr;
    }
    p.residual[ctx.tp_rank] = x.residual;
    p.gamma = x.gamma; p.beta = x.beta; p.eps = x.eps; p.inv_d = 1.0f / float(D);
    p.M = M; p.n4 = int(D / 4);
    p.rows_per_rank = (M + ctx.tp_size - 1) / ctx.tp_size;
    p.x_own_only = x.replicate_x ? 0 : 1;
    p.pushed = pushed ? 1 : 0;
    const double frac = double(ctx.tp_size - 1) / ctx.tp_size;
    // bytes = what ARRIVES at this rank over NVLink during the kernel: the peers' partial rows it fetches (unless pushed) and
    // the normalised / residual rows the peers store into it; the same amount leaves it.  That makes an exchange an
    // NVLink-bound step: 2 * (n-1)/n of the activation per direction, whatever the kernel does with it.
    tag_launch(ctx, "tp_exchange_add_layernorm", double(M) * D + 8.0 * double(M) * D / ctx.tp_size,
               4.0 * double(M) * D * frac * ((pushed ? 0.0 : 1.0) + (x.y_out ? 1.0 : 0.0) + ((x.x_out && x.replicate_x) ? 1.0 : 0.0)));
    cudaError_t e = launch_xchg_nv((p.n4 + 31) / 32, p, dim3(unsigned(pm->grid)), ctx.stream, false);
    FXF_CHECK(e == cudaSuccess, "tensor-parallel exchange: launch failed: %s", cudaGetErrorString(e));
    FXF_LAUNCHED(ctx);
    return 0;
}

// Single-GPU emulation of an n-rank exchange (tests): all ranks' buffers live on one device and ONE cooperative launch
// carries the blocks of every rank (blockIdx.y = rank), so that blocks that wait for one another are resident together.
// `sync_mem`: n_ranks * 8192 zeroed bytes ([0,4096) flags, then three control ints, status word at byte 4160 of each
// rank's region).  skip_rank >= 0 keeps that rank away from the exchange: the others run into their wait budget.
// layout: bit 0 = every rank receives every row of x_out; bit 1 = partial[q] is rank q's exchange window as the pushing
// products leave it (row p*R + l = producer p's partial sums of row q*R + l, R = M / n_ranks).
int tp_exchange_emulated(int n_ranks, const float* const* partial, const float* const* residual, float* const* x_out, float* const* y_out,
                         const float* gamma, const float* beta, float eps, int64_t M, int64_t D, int layout, void* sync_mem, int budget_ms,
                         int skip_rank, cudaStream_t stream) {
    const int replicate_x = layout & 1, pushed = (layout >> 1) & 1;
    FXF_CHECK(!pushed || M % n_ranks == 0, "emulated exchange: pushed rows need M to be a multiple of the rank count");
    FXF_CHECK(n_ranks >= 2 && n_ranks <= kMaxTpRanks, "emulated exchange: 2..%d ranks", kMaxTpRanks);
    FXF_CHECK(partial && sync_mem && D % 4 == 0 && D > 0 && D <= 1024 && M > 0, "emulated exchange: bad arguments");
    FXF_CHECK(budget_ms > 0 && budget_ms <= 2000, "emulated exchange: the wait budget must be 1..2000 ms");
    constexpr int kGridX = 16;   // blocks per rank: n_ranks * 16 blocks of 256 threads are resident together on any B200
    XchgParams p{};
    char* sm = static_cast<char*>(sync_mem);
    for (int r = 0; r < n_ranks; r++) {
        p.sync.flags[r] = reinterpret_cast<int*>(sm + size_t(r) * 8192);
        p.sync.ctl[r] = reinterpret_cast<int*>(sm + size_t(r) * 8192 + 4096);
        p.sync.status[r] = reinterpret_cast<int*>(sm + size_t(r) * 8192 + 4160);
        FXF_CHECK(partial[r] != nullptr, "emulated exchange: NULL partial buffer");
        p.part[r] = partial[r];
        p.residual[r] = residual ? residual[r] : nullptr;
        p.y[r] = y_out ? y_out[r] : nullptr;
        p.x[r] = x_out ? x_out[r] : nullptr;
    }
    FXF_CHECK(p.y[0] == nullptr || (gamma && beta), "emulated exchange: LayerNorm output without weight / bias");
    p.sync.n = n_ranks;
    p.sync.start_ns = p.sync.end_ns = (unsigned long long)budget_ms * 1000000ull;
    p.rank = -1;
    p.skip_rank = skip_rank;
    p.gamma = gamma; p.beta = beta; p.eps = eps; p.inv_d = 1.0f / float(D);
    p.M = M; p.n4 = int(D / 4);
    p.rows_per_rank = (M + n_ranks - 1) / n_ranks;
    p.x_own_only = replicate_x ? 0 : 1;
    p.pushed = pushed;
    cudaError_t e = launch_xchg_nv((p.n4 + 31) / 32, p, dim3(kGridX, unsigned(n_ranks)), stream, true);
    FXF_CHECK(e == cudaSuccess, "emulated exchange: cooperative launch failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace fxf
