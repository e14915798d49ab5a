// fp32 FFMA GEMM with fused bias (+ReLU) epilogue:  out[M,N] = act(x[M,K] · w[N,K]^T + bias[N]).
//
// This is the exact-fp32 contraction behind Linear / LinearRelu / FeedForward / the MHA
// projections (reference: torch::linear, csrc/kernels/cpu/linear.cpp:11, linear_relu.cpp:11,
// feedforward.cpp:13, mha.cpp:22,51) for shapes the tensor-core path does not take: small or
// ragged problems (M, N, K not multiples of the tcgen05 tile) and FXF_GEMM_FP32_SIMT mode.
//
// Both operands are K-major, so tiles are fetched with 128-bit loads along K and stored
// transposed in shared memory ([k][row]); every thread then accumulates a TM x TN register
// tile split into 4-wide chunks so that shared-memory reads are conflict-free float4s.
// Global->register prefetch of the next K-slab overlaps the FFMA loop (double buffering).
// Roofline: fp32 FFMA, 148 SMs x 128 lanes x 2 flop.
#include <algorithm>

#include "../runtime.hpp"

namespace fxf {
namespace {

template <int BM, int BN, int BK, int TM, int TN, bool RELU>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_tn_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ out,
               int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldo, int vec_in, int vec_out) {
    constexpr int T = (BM / TM) * (BN / TN);
    constexpr int VM = TM >= 4 ? 4 : TM, VN = TN >= 4 ? 4 : TN;  // chunk widths
    constexpr int CM = TM / VM, CN = TN / VN;                    // chunks per thread
    constexpr int PAD = 4;
    constexpr int A_F4 = BM * BK / 4, B_F4 = BN * BK / 4;        // float4s per tile
    constexpr int A_PER = (A_F4 + T - 1) / T, B_PER = (B_F4 + T - 1) / T;
    constexpr int KQ = BK / 4;

    __shared__ __align__(16) float As[2][BK][BM + PAD];
    __shared__ __align__(16) float Bs[2][BK][BN + PAD];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int64_t row0 = int64_t(blockIdx.y) * BM, col0 = int64_t(blockIdx.x) * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    float4 ra[A_PER], rb[B_PER];

    auto load_global = [&](int64_t k0) {
#pragma unroll
        for (int i = 0; i < A_PER; i++) {
            int f = tid + i * T;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (f < A_F4) {
                int r = f / KQ, kq = f % KQ;
                int64_t gr = row0 + r, gk = k0 + kq * 4;
                if (gr < M) {
                    const float* p = x + gr * ldx + gk;
                    if (vec_in && gk + 3 < K) {
                        v = *reinterpret_cast<const float4*>(p);
                    } else {
                        if (gk < K) v.x = p[0];
                        if (gk + 1 < K) v.y = p[1];
                        if (gk + 2 < K) v.z = p[2];
                        if (gk + 3 < K) v.w = p[3];
                    }
                }
            }
            ra[i] = v;
        }
#pragma unroll
        for (int i = 0; i < B_PER; i++) {
            int f = tid + i * T;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (f < B_F4) {
                int r = f / KQ, kq = f % KQ;
                int64_t gr = col0 + r, gk = k0 + kq * 4;
                if (gr < N) {
                    const float* p = w + gr * ldw + gk;
                    if (vec_in && gk + 3 < K) {
                        v = *reinterpret_cast<const float4*>(p);
                    } else {
                        if (gk < K) v.x = p[0];
                        if (gk + 1 < K) v.y = p[1];
                        if (gk + 2 < K) v.z = p[2];
                        if (gk + 3 < K) v.w = p[3];
                    }
                }
            }
            rb[i] = v;
        }
    };
    auto store_shared = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER; i++) {
            int f = tid + i * T;
            if (f < A_F4) {
                int r = f / KQ, kq = f % KQ;
                As[buf][kq * 4 + 0][r] = ra[i].x;
                As[buf][kq * 4 + 1][r] = ra[i].y;
                As[buf][kq * 4 + 2][r] = ra[i].z;
                As[buf][kq * 4 + 3][r] = ra[i].w;
            }
        }
#pragma unroll
        for (int i = 0; i < B_PER; i++) {
            int f = tid + i * T;
            if (f < B_F4) {
                int r = f / KQ, kq = f % KQ;
                Bs[buf][kq * 4 + 0][r] = rb[i].x;
                Bs[buf][kq * 4 + 1][r] = rb[i].y;
                Bs[buf][kq * 4 + 2][r] = rb[i].z;
                Bs[buf][kq * 4 + 3][r] = rb[i].w;
            }
        }
    };

    const int64_t n_slabs = (K + BK - 1) / BK;
    load_global(0);
    store_shared(0);
    __syncthreads();

    for (int64_t s = 0; s < n_slabs; s++) {
        int buf = int(s & 1);
        if (s + 1 < n_slabs) load_global((s + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[TM], b[TN];
#pragma unroll
            for (int c = 0; c < CM; c++) {
                const float* p = &As[buf][k][c * (BM / CM) + ty * VM];
                if (VM == 4) {
                    float4 v = *reinterpret_cast<const float4*>(p);
                    a[c * VM + 0] = v.x; a[c * VM + 1] = v.y; a[c * VM + 2] = v.z; a[c * VM + 3] = v.w;
                } else {
#pragma unroll
                    for (int i = 0; i < VM; i++) a[c * VM + i] = p[i];
                }
            }
#pragma unroll
            for (int c = 0; c < CN; c++) {
                const float* p = &Bs[buf][k][c * (BN / CN) + tx * VN];
                if (VN == 4) {
                    float4 v = *reinterpret_cast<const float4*>(p);
                    b[c * VN + 0] = v.x; b[c * VN + 1] = v.y; b[c * VN + 2] = v.z; b[c * VN + 3] = v.w;
                } else {
#pragma unroll
                    for (int i = 0; i < VN; i++) b[c * VN + i] = p[i];
                }
            }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < n_slabs) {
            store_shared(buf ^ 1);
            __syncthreads();
        }
    }

    // epilogue: bias, activation, store
#pragma unroll
    for (int cm = 0; cm < CM; cm++) {
#pragma unroll
        for (int i = 0; i < VM; i++) {
            int64_t gr = row0 + cm * (BM / CM) + ty * VM + i;
            if (gr >= M) continue;
#pragma unroll
            for (int cn = 0; cn < CN; cn++) {
                int64_t gc = col0 + cn * (BN / CN) + tx * VN;
                float v[VN];
#pragma unroll
                for (int j = 0; j < VN; j++) {
                    float t = acc[cm * VM + i][cn * VN + j];
                    if (bias != nullptr && gc + j < N) t += bias[gc + j];
                    if (RELU) t = t > 0.f ? t : (t != t ? t : 0.f);
                    v[j] = t;
                }
                float* p = out + gr * ldo + gc;
                if (VN == 4 && vec_out && gc + 3 < N) {
                    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < VN; j++)
                        if (gc + j < N) p[j] = v[j];
                }
            }
        }
    }
}

// Few-row problems (M <= 64: batch-sized MLP layers).  A 32x32 tile would leave all but a handful of SMs
// idle and make each of them walk the whole K; here a CTA owns 32 rows x 8 columns, so N/8 CTAs stream
// disjoint 8-row slices of the weight while the small activation block is re-read from L2.  One output per
// thread, K staged through shared memory in slabs of 128 with register prefetch of the next slab.
constexpr int SK_BM = 32, SK_BN = 8, SK_BK = 128, SK_PAD = 4;

template <bool RELU>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                          float* __restrict__ out, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldo,
                                                          int vec_in) {
    __shared__ __align__(16) float xs[SK_BM][SK_BK + SK_PAD];
    __shared__ __align__(16) float ws[SK_BN][SK_BK + SK_PAD];
    const int tid = threadIdx.x, tm = tid >> 3, tn = tid & 7;
    const int64_t row0 = int64_t(blockIdx.y) * SK_BM, col0 = int64_t(blockIdx.x) * SK_BN;
    float4 rx[4], rw;
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int f = tid + i * 256, r = f >> 5, c = (f & 31) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int64_t gr = row0 + r, gk = k0 + c;
            if (gr < M) {
                const float* p = x + gr * ldx + gk;
                if (vec_in && gk + 3 < K) v = *reinterpret_cast<const float4*>(p);
                else {
                    if (gk < K) v.x = p[0];
                    if (gk + 1 < K) v.y = p[1];
                    if (gk + 2 < K) v.z = p[2];
                    if (gk + 3 < K) v.w = p[3];
                }
            }
            rx[i] = v;
        }
        {
            int r = tid >> 5, c = (tid & 31) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int64_t gr = col0 + r, gk = k0 + c;
            if (gr < N) {
                const float* p = w + gr * ldw + gk;
                if (vec_in && gk + 3 < K) v = *reinterpret_cast<const float4*>(p);
                else {
                    if (gk < K) v.x = p[0];
                    if (gk + 1 < K) v.y = p[1];
                    if (gk + 2 < K) v.z = p[2];
                    if (gk + 3 < K) v.w = p[3];
                }
            }
            rw = v;
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int f = tid + i * 256, r = f >> 5, c = (f & 31) * 4;
            *reinterpret_cast<float4*>(&xs[r][c]) = rx[i];
        }
        *reinterpret_cast<float4*>(&ws[tid >> 5][(tid & 31) * 4]) = rw;
    };
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    const int64_t slabs = (K + SK_BK - 1) / SK_BK;
    if (slabs > 0) fetch(0);
    for (int64_t s = 0; s < slabs; s++) {
        __syncthreads();
        stash();
        __syncthreads();
        if (s + 1 < slabs) fetch((s + 1) * SK_BK);
#pragma unroll 8
        for (int k = 0; k < SK_BK; k += 4) {
            float4 a = *reinterpret_cast<const float4*>(&xs[tm][k]);
            float4 b = *reinterpret_cast<const float4*>(&ws[tn][k]);
            acc0 = fmaf(a.x, b.x, acc0);
            acc1 = fmaf(a.y, b.y, acc1);
            acc2 = fmaf(a.z, b.z, acc2);
            acc3 = fmaf(a.w, b.w, acc3);
        }
    }
    int64_t gr = row0 + tm, gc = col0 + tn;
    if (gr < M && gc < N) {
        float v = (acc0 + acc1) + (acc2 + acc3);
        if (bias != nullptr) v += bias[gc];
        if (RELU) v = v > 0.f ? v : (v != v ? v : 0.f);
        out[gr * ldo + gc] = v;
    }
}

// Few rows against a LARGE weight (single-position decode steps: M = batch, weights of megabytes).  The time is the
// weight read, so the work is cut into many independent pieces that each put a whole [64 x 128] weight slab (32 KB) in
// flight at once: CTA (n-tile, k-part, m-tile) owns 32 rows x 64 columns and a range of 128-wide K slabs.  With more than
// one k-part the partial tiles go to the GEMM workspace and the LAST CTA to finish a tile (a counter per tile) adds them
// in part order — the sum does not depend on which CTA that is — then applies bias and ReLU.  fp32 FFMA throughout.
constexpr int FR_BM = 32, FR_BN = 64, FR_BK = 128, FR_LD = FR_BK + 4;

__global__ void __launch_bounds__(256) gemm_fewrows_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                           float* __restrict__ out, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldo,
                                                           int vec_in, int relu, int k_parts, int slabs_per_part, float* __restrict__ partial, int* __restrict__ counters) {
    extern __shared__ __align__(16) float fr_smem[];
    float (*xs)[FR_LD] = reinterpret_cast<float (*)[FR_LD]>(fr_smem);
    float (*ws)[FR_LD] = reinterpret_cast<float (*)[FR_LD]>(fr_smem + FR_BM * FR_LD);
    __shared__ int is_last;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;           // thread: rows 2*ty, 2*ty+1; columns tx, tx+16, tx+32, tx+48
    const int64_t col0 = int64_t(blockIdx.x) * FR_BN, row0 = int64_t(blockIdx.z) * FR_BM;
    const int part = blockIdx.y;
    const int64_t total_slabs = (K + FR_BK - 1) / FR_BK;
    const int64_t s0 = int64_t(part) * slabs_per_part, s1 = min(s0 + slabs_per_part, total_slabs);
    float acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    auto load4 = [&](const float* base, int64_t r, int64_t rows, int64_t ld, int64_t gk) -> float4 {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows) {
            const float* p = base + r * ld + gk;
            if (vec_in && gk + 3 < K) v = *reinterpret_cast<const float4*>(p);
            else {
                if (gk < K) v.x = p[0];
                if (gk + 1 < K) v.y = p[1];
                if (gk + 2 < K) v.z = p[2];
                if (gk + 3 < K) v.w = p[3];
            }
        }
        return v;
    };
    float4 rw[8], rx[4];
    auto fetch = [&](int64_t sl) {
        const int64_t k0 = sl * FR_BK;
#pragma unroll
        for (int i = 0; i < 8; i++) {          // weight slab: 64 rows x 32 float4
            int f = tid + i * 256, r = f >> 5, c = (f & 31) * 4;
            rw[i] = load4(w, col0 + r, N, ldw, k0 + c);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {          // activation slab: 32 rows x 32 float4
            int f = tid + i * 256, r = f >> 5, c = (f & 31) * 4;
            rx[i] = load4(x, row0 + r, M, ldx, k0 + c);
        }
    };
    if (s0 < s1) fetch(s0);
    for (int64_t sl = s0; sl < s1; sl++) {
        __syncthreads();                        // the previous slab has been consumed
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int f = tid + i * 256;
            *reinterpret_cast<float4*>(&ws[f >> 5][(f & 31) * 4]) = rw[i];
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int f = tid + i * 256;
            *reinterpret_cast<float4*>(&xs[f >> 5][(f & 31) * 4]) = rx[i];
        }
        __syncthreads();
        if (sl + 1 < s1) fetch(sl + 1);        // the next slab's loads fly while this one is multiplied
#pragma unroll 4
        for (int k = 0; k < FR_BK; k += 4) {
            const float4 a0 = *reinterpret_cast<const float4*>(&xs[2 * ty][k]);
            const float4 a1 = *reinterpret_cast<const float4*>(&xs[2 * ty + 1][k]);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4 b = *reinterpret_cast<const float4*>(&ws[tx + 16 * j][k]);
                acc[0][j] = fmaf(a0.x, b.x, acc[0][j]); acc[0][j] = fmaf(a0.y, b.y, acc[0][j]);
                acc[0][j] = fmaf(a0.z, b.z, acc[0][j]); acc[0][j] = fmaf(a0.w, b.w, acc[0][j]);
                acc[1][j] = fmaf(a1.x, b.x, acc[1][j]); acc[1][j] = fmaf(a1.y, b.y, acc[1][j]);
                acc[1][j] = fmaf(a1.z, b.z, acc[1][j]); acc[1][j] = fmaf(a1.w, b.w, acc[1][j]);
            }
        }
    }
    auto finish = [&](float v, int64_t gr, int64_t gc) {
        if (gr < M && gc < N) {
            if (bias != nullptr) v += bias[gc];
            if (relu) v = v > 0.f ? v : (v != v ? v : 0.f);
            out[gr * ldo + gc] = v;
        }
    };
    if (k_parts == 1) {
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) finish(acc[i][j], row0 + 2 * ty + i, col0 + tx + 16 * j);
        return;
    }
    // partial tile [part][32][64] of this (m-tile, n-tile), then the last arriver reduces in part order
    const int64_t tile = int64_t(blockIdx.z) * gridDim.x + blockIdx.x;
    float* mine = partial + (tile * k_parts + part) * (FR_BM * FR_BN);
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) mine[(2 * ty + i) * FR_BN + tx + 16 * j] = acc[i][j];
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int done = atomicAdd(counters + tile, 1);
        is_last = done == k_parts - 1;
        if (is_last) counters[tile] = 0;   // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* all = partial + tile * k_parts * (FR_BM * FR_BN);
    float sum[2][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) sum[i][j] = 0.f;
    for (int q = 0; q < k_parts; q++) {        // part order; the eight loads of a part are independent
        float t[2][4];
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) t[i][j] = __ldcg(all + q * (FR_BM * FR_BN) + (2 * ty + i) * FR_BN + tx + 16 * j);
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) sum[i][j] += t[i][j];
    }
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) finish(sum[i][j], row0 + 2 * ty + i, col0 + tx + 16 * j);
}

// Few rows and a weight worth splitting: enough pieces to occupy the GPU twice over.
bool fewrows_applies(const GemmArgs& a) { return a.M <= 64 && a.N >= 64 && a.N * a.K >= (int64_t(1) << 20); }

int launch_fewrows(const GemmArgs& a, ExecCtx& ctx) {
    const int64_t n_tiles = (a.N + FR_BN - 1) / FR_BN, m_tiles = (a.M + FR_BM - 1) / FR_BM, slabs = (a.K + FR_BK - 1) / FR_BK;
    int64_t parts = 1;
    if (ctx.gemm_ws != nullptr && ctx.gemm_flags != nullptr && n_tiles * m_tiles <= ctx.gemm_flag_count) {
        const int64_t want = (2 * int64_t(ctx.sm_count) + n_tiles * m_tiles - 1) / (n_tiles * m_tiles);
        parts = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, slabs), 8));
        while (parts > 1 && size_t(n_tiles * m_tiles * parts) * FR_BM * FR_BN * sizeof(float) > ctx.gemm_ws_bytes) parts--;
    }
    const int64_t per = (slabs + parts - 1) / parts;
    parts = (slabs + per - 1) / per;   // no empty part
    const int vec_in = (a.ldx % 4 == 0 && a.ldw % 4 == 0 && aligned16(a.x) && aligned16(a.w)) ? 1 : 0;
    const size_t smem = size_t(FR_BM + FR_BN) * FR_LD * sizeof(float);
    static bool configured[64] = {};
    int dev = 0;
    FXF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        FXF_CUDA(cudaFuncSetAttribute(gemm_fewrows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const dim3 fr_grid{unsigned(n_tiles), unsigned(parts), unsigned(m_tiles)};
    gemm_fewrows_kernel<<<fr_grid, 256, smem, ctx.stream>>>(a.x, a.w, a.bias, a.out, a.M, a.N, a.K, a.ldx, a.ldw, a.ldo, vec_in, a.relu ? 1 : 0, int(parts), int(per),
                                                         ctx.gemm_ws, ctx.gemm_flags);
    FXF_LAUNCHED(ctx);
    return 0;
}

int launch_skinny(const GemmArgs& a, ExecCtx& ctx) {
    dim3 grid(unsigned((a.N + SK_BN - 1) / SK_BN), unsigned((a.M + SK_BM - 1) / SK_BM));
    int vec_in = (a.ldx % 4 == 0 && a.ldw % 4 == 0 && aligned16(a.x) && aligned16(a.w)) ? 1 : 0;
    if (a.relu)
        gemm_skinny_kernel<true><<<grid, 256, 0, ctx.stream>>>(a.x, a.w, a.bias, a.out, a.M, a.N, a.K, a.ldx, a.ldw, a.ldo, vec_in);
    else
        gemm_skinny_kernel<false><<<grid, 256, 0, ctx.stream>>>(a.x, a.w, a.bias, a.out, a.M, a.N, a.K, a.ldx, a.ldw, a.ldo, vec_in);
    FXF_LAUNCHED(ctx);
    return 0;
}

template <int BM, int BN, int BK, int TM, int TN>
int launch_cfg(const GemmArgs& a, ExecCtx& ctx) {
    dim3 grid(unsigned((a.N + BN - 1) / BN), unsigned((a.M + BM - 1) / BM));
    dim3 block((BM / TM) * (BN / TN));
    int vec_in = (a.ldx % 4 == 0 && a.ldw % 4 == 0 && aligned16(a.x) && aligned16(a.w)) ? 1 : 0;
    int vec_out = (a.ldo % 4 == 0 && aligned16(a.out)) ? 1 : 0;
    if (a.relu)
        gemm_tn_kernel<BM, BN, BK, TM, TN, true><<<grid, block, 0, ctx.stream>>>(a.x, a.w, a.bias, a.out, a.M, a.N, a.K, a.ldx, a.ldw, a.ldo, vec_in, vec_out);
    else
        gemm_tn_kernel<BM, BN, BK, TM, TN, false><<<grid, block, 0, ctx.stream>>>(a.x, a.w, a.bias, a.out, a.M, a.N, a.K, a.ldx, a.ldw, a.ldo, vec_in, vec_out);
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace

// 0 = 128x128, 1 = 64x64, 2 = 32x32, 3 = skinny 32x8 (or, for large weights, the K-split few-rows kernel)
int simt_tile_choice(int64_t M, int64_t N, int sm_count) {
    if (M <= 64) return 3;
    int64_t big = ((M + 127) / 128) * ((N + 127) / 128);
    int64_t mid = ((M + 63) / 64) * ((N + 63) / 64);
    if (big >= sm_count) return 0;
    if (mid >= sm_count / 2) return 1;
    return 2;
}

int launch_gemm_simt(const GemmArgs& a, ExecCtx& ctx) {
    if (a.M == 0 || a.N == 0) return 0;
    FXF_CHECK(a.M > 0 && a.N > 0 && a.K >= 0, "gemm: negative dimension");
    static const char* names[] = {"gemm_fp32_simt128x128", "gemm_fp32_simt64x64", "gemm_fp32_simt32x32", "gemm_fp32_skinny32x8"};
    const bool fewrows = simt_tile_choice(a.M, a.N, ctx.sm_count) == 3 && fewrows_applies(a);
    tag_launch(ctx, fewrows ? "gemm_fp32_fewrows32x64_ksplit" : names[simt_tile_choice(a.M, a.N, ctx.sm_count)], 2.0 * double(a.M) * double(a.N) * double(a.K),
               4.0 * (double(a.M) * a.K + double(a.N) * a.K + double(a.N) + double(a.M) * a.N));
    if (fewrows) return launch_fewrows(a, ctx);
    switch (simt_tile_choice(a.M, a.N, ctx.sm_count)) {
        case 3: return launch_skinny(a, ctx);
        case 0: return launch_cfg<128, 128, 16, 8, 8>(a, ctx);
        case 1: return launch_cfg<64, 64, 16, 4, 4>(a, ctx);
        default: return launch_cfg<32, 32, 32, 2, 2>(a, ctx);
    }
}

}  // namespace fxf
