// Tensor-core GEMM for sm_100a:  out[M,N] = act(x[M,K] · w[N,K]^T + bias[N])  with fp32-grade
// accuracy from three TF32 products per logical product ("3xTF32").
//
// The contraction behind Linear / LinearRelu / FeedForward / the MHA projections (reference:
// torch::linear, csrc/kernels/cpu/linear.cpp:11, feedforward.cpp:13, mha.cpp:22,51; the
// reference CUDA kernel is a 32x32 SIMT tile, csrc/kernels/cuda/linear.cu:5-41).
//
// Arithmetic.  x = x_hi + x_lo with x_hi = tf32(x) (round to nearest, 10-bit mantissa) and
// x_lo = tf32(x - x_hi); same for w.  x·w ~= x_lo·w_hi + x_hi·w_lo + x_hi·w_hi, accumulated in
// fp32; the dropped x_lo·w_lo term is ~2^-22 relative.  Weights are constants: they are split
// once when an engine is built (split_tf32) and kept as two arrays.  Activations are split inside the
// kernel, in shared memory, while the tensor core works on the previous stage.
//
// Structure (one CTA = one 128 x BN output tile, 192 threads):
//   warp 0    TMA producer: per K-slab of 32 floats (one 128-byte swizzle row) three
//             cp.async.bulk.tensor loads — x tile [128,32], w_hi and w_lo tiles [BN,32] — land in a
//             STAGES-deep ring of shared-memory stages, completion counted on an mbarrier.
//   warps 2-5 split the x tile in place (hi) and into a twin buffer (lo); being element-wise the
//             128-byte swizzle pattern TMA wrote is preserved.  fence.proxy.async, then arrive.
//   warp 1    one thread issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8): 4 K-steps x 3 products
//             per stage, accumulating in TMEM; tcgen05.commit releases the stage to the producer.
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM lanes), add bias, ReLU,
//             store.
// Every mbarrier wait is bounded by a wall-clock budget; on expiry the CTA records an error in
// the status word, stops issuing work, frees its TMEM and returns.
//
// Bound: tensor pipe (TF32 rate / 3).  Shared-memory bandwidth is the practical limiter for an
// SS-operand MMA with cta_group::1 (operand reads + TMA fills + the split pass share 128 B/clk).
#include <cuda.h>

#include <mutex>

#include "../runtime.hpp"

namespace fxf {
namespace {

constexpr int BM = 128;
constexpr int BK = 32;             // floats per K-slab = 128 bytes = one swizzle row
constexpr int kThreads = 192;      // warp0 TMA, warp1 MMA, warps 2..5 split + epilogue
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;  // 2 s per wait

enum : int { kErrWaitTma = 101, kErrWaitSplit = 102, kErrWaitEmpty = 103, kErrWaitAcc = 104 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false when the budget ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = global_ns();
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitBudgetNs) return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
                 : "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFF) >> 4);   // start address, 16-byte units
    d |= uint64_t(1) << 16;                      // leading byte offset (unused for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= uint64_t(1) << 46;                      // descriptor version for sm_100
    d |= uint64_t(2) << 61;                      // layout type: SWIZZLE_128B
    return d;
}
// kind::tf32, fp32 accumulate, A and B K-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    hi = __uint_as_float(to_tf32(x));
    lo = __uint_as_float(to_tf32(x - hi));
}

template <int BN, int STAGES>
struct alignas(1024) TcSmem {
    float a_hi[STAGES][BM * BK];
    float a_lo[STAGES][BM * BK];
    float b_hi[STAGES][BN * BK];
    float b_lo[STAGES][BN * BK];
    uint64_t full_tma[STAGES];
    uint64_t full_split[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
};

struct TcParams {
    const float* bias;
    float* out;
    int64_t M, N, K, ldo;
    int relu;
    int vec_out;
    int* status;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_whi,
                   const __grid_constant__ CUtensorMap map_wlo, TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    // dynamic shared memory is only guaranteed 16-byte aligned; swizzled tiles need 1024
    TcSmem<BN, STAGES>& s = *reinterpret_cast<TcSmem<BN, STAGES>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x, tile_m = blockIdx.y;
    const int num_k = int((p.K + BK - 1) / BK);
    constexpr uint32_t kStageBytes = uint32_t(BM * BK + 2 * BN * BK) * 4u;
    constexpr uint32_t kIdesc = umma_idesc_tf32(BM, BN);
    volatile int* abort_flag = &s.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(&s.full_tma[i], 1);
            mbar_init(&s.full_split[i], 4);   // one arrival per split warp
            mbar_init(&s.empty[i], 1);
        }
        mbar_init(&s.acc_full, 1);
        s.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation is a warp-wide operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)), "r"(uint32_t(BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = s.tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (int k = 0; k < num_k; k++) {
                int st = k % STAGES;
                if (k >= STAGES && !mbar_wait(&s.empty[st], uint32_t((k / STAGES - 1) & 1), abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; if (p.status) atomicCAS(p.status, 0, kErrWaitEmpty); }
                    break;
                }
                mbar_expect_tx(&s.full_tma[st], kStageBytes);
                tma_load_2d(s.a_hi[st], &map_x, k * BK, tile_m * BM, &s.full_tma[st]);
                tma_load_2d(s.b_hi[st], &map_whi, k * BK, tile_n * BN, &s.full_tma[st]);
                tma_load_2d(s.b_lo[st], &map_wlo, k * BK, tile_n * BN, &s.full_tma[st]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = true;
            for (int k = 0; k < num_k && ok; k++) {
                int st = k % STAGES;
                uint32_t par = uint32_t((k / STAGES) & 1);
                if (!mbar_wait(&s.full_tma[st], par, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; if (p.status) atomicCAS(p.status, 0, kErrWaitTma); }
                    ok = false;
                    break;
                }
                if (!mbar_wait(&s.full_split[st], par, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; if (p.status) atomicCAS(p.status, 0, kErrWaitSplit); }
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint64_t a_hi = umma_desc_k_sw128(smem_u32(s.a_hi[st])), a_lo = umma_desc_k_sw128(smem_u32(s.a_lo[st]));
                uint64_t b_hi = umma_desc_k_sw128(smem_u32(s.b_hi[st])), b_lo = umma_desc_k_sw128(smem_u32(s.b_lo[st]));
#pragma unroll
                for (int kk = 0; kk < BK / 8; kk++) {
                    uint64_t adv = uint64_t((kk * 8 * 4) >> 4);  // 32 bytes per K-step inside the swizzle row
                    umma_tf32(tmem_acc, a_lo + adv, b_hi + adv, kIdesc, (k > 0 || kk > 0) ? 1u : 0u);
                    umma_tf32(tmem_acc, a_hi + adv, b_lo + adv, kIdesc, 1u);
                    umma_tf32(tmem_acc, a_hi + adv, b_hi + adv, kIdesc, 1u);
                }
                umma_commit(&s.empty[st]);  // arrives once the MMAs above have consumed the stage
            }
            if (ok) umma_commit(&s.acc_full);
        }
    } else {
        // ---------------- activation split (hi in place, lo into the twin buffer) ----------------
        const int t = threadIdx.x - 64;  // 0..127
        bool ok = true;
        for (int k = 0; k < num_k; k++) {
            int st = k % STAGES;
            if (!mbar_wait(&s.full_tma[st], uint32_t((k / STAGES) & 1), abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; if (p.status) atomicCAS(p.status, 0, kErrWaitTma); }
                ok = false;
                break;
            }
            float4* hi = reinterpret_cast<float4*>(s.a_hi[st]);
            float4* lo = reinterpret_cast<float4*>(s.a_lo[st]);
#pragma unroll
            for (int i = 0; i < (BM * BK / 4) / 128; i++) {
                float4 v = hi[t + i * 128], h, l;
                split_tf32(v.x, h.x, l.x);
                split_tf32(v.y, h.y, l.y);
                split_tf32(v.z, h.z, l.z);
                split_tf32(v.w, h.w, l.w);
                hi[t + i * 128] = h;
                lo[t + i * 128] = l;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.full_split[st]);
        }
        // ---------------- epilogue ----------------
        if (ok && num_k > 0) {
            if (!mbar_wait(&s.acc_full, 0, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; if (p.status) atomicCAS(p.status, 0, kErrWaitAcc); }
                ok = false;
            }
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quarter = warp & 3;  // a warp may only touch TMEM lanes 32*(warp%4) .. +31
            const int64_t row = int64_t(tile_m) * BM + quarter * 32 + lane;
            const int64_t col0 = int64_t(tile_n) * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t r[32];
                if (num_k > 0) {
                    tmem_ld32(tmem_acc + (uint32_t(quarter * 32) << 16) + uint32_t(c * 32), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) r[j] = 0u;
                }
                int64_t col = col0 + c * 32;
                if (row < p.M && col < p.N) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float x = __uint_as_float(r[j]);
                        if (p.bias != nullptr && col + j < p.N) x += __ldg(p.bias + col + j);
                        if (p.relu) x = x > 0.f ? x : (x != x ? x : 0.f);
                        v[j] = x;
                    }
                    float* dst = p.out + row * p.ldo + col;
                    if (p.vec_out && col + 31 < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col + j < p.N) dst[j] = v[j];
                    }
                }
            }
        }
    }
    // ---------------- teardown (every thread arrives here, whatever happened above) ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(uint32_t(BN)) : "memory");
    }
}

// ---- weight split (once per engine) -----------------------------------------------------------
__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int64_t n) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float h, l;
        split_tf32(w[i], h, l);
        hi[i] = h;
        lo[i] = l;
    }
}

// ---- host side -------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D fp32 row-major [rows, cols] with row pitch `ld` floats; box = [box_rows, 32 floats], 128-byte swizzle.
int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    FXF_CHECK(fn != nullptr, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(ld) * sizeof(float)};
    cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FXF_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (rows %lld cols %lld ld %lld)", int(r), (long long)rows, (long long)cols, (long long)ld);
    return 0;
}

template <int BN, int STAGES>
int launch_tc(const GemmArgs& a, ExecCtx& ctx) {
    CUtensorMap mx, mhi, mlo;
    if (make_map(&mx, a.x, a.M, a.K, a.ldx, BM)) return 1;
    if (make_map(&mhi, a.w_hi, a.N, a.K, a.K, BN)) return 1;
    if (make_map(&mlo, a.w_lo, a.N, a.K, a.K, BN)) return 1;
    TcParams p;
    p.bias = a.bias; p.out = a.out; p.M = a.M; p.N = a.N; p.K = a.K; p.ldo = a.ldo;
    p.relu = a.relu ? 1 : 0;
    p.vec_out = (a.ldo % 4 == 0 && aligned16(a.out)) ? 1 : 0;
    p.status = ctx.status;
    size_t smem = sizeof(TcSmem<BN, STAGES>) + 1024;
    static bool configured[64] = {};
    int dev = 0;
    FXF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        FXF_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    dim3 grid(unsigned((a.N + BN - 1) / BN), unsigned((a.M + BM - 1) / BM));
    tag_launch(ctx, BN == 256 ? "gemm_tf32x3_tcgen05_128x256" : "gemm_tf32x3_tcgen05_128x128", 2.0 * double(a.M) * double(a.N) * double(a.K),
               4.0 * (double(a.M) * a.K + double(a.N) * a.K + double(a.N) + double(a.M) * a.N));
    gemm_tf32x3_kernel<BN, STAGES><<<grid, kThreads, smem, ctx.stream>>>(mx, mhi, mlo, p);
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace

// The tensor-core path needs: pre-split weights, 16-byte aligned bases, row pitches that are
// multiples of 4 floats (TMA strides are multiples of 16 bytes), K a multiple of 4 and a problem
// large enough that 128-row tiles are not mostly padding.
bool gemm_tc_supported(const GemmArgs& a) {
    if (a.w_hi == nullptr || a.w_lo == nullptr) return false;
    if (!gemm_tc_shape_ok(a.M, a.N, a.K)) return false;
    if (a.ldx % 4 != 0 || a.ldx < a.K) return false;
    if (!aligned16(a.x) || !aligned16(a.w_hi) || !aligned16(a.w_lo)) return false;
    return true;
}

bool gemm_tc_shape_ok(int64_t M, int64_t N, int64_t K) {
    return M >= 64 && N >= 64 && K >= 32 && K % 4 == 0 && M < (int64_t(1) << 31) && N < (int64_t(1) << 31) && K < (int64_t(1) << 31);
}

int launch_gemm_tc(const GemmArgs& a, ExecCtx& ctx) {
    FXF_CHECK(gemm_tc_supported(a), "tensor-core GEMM called with an unsupported problem");
    if (a.N > 128) return launch_tc<256, 2>(a, ctx);
    return launch_tc<128, 3>(a, ctx);
}

int launch_split_tf32(const float* w, float* hi, float* lo, int64_t n, ExecCtx& ctx) {
    if (n == 0) return 0;
    int64_t blocks = (n + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
    tag_launch(ctx, "split_tf32", 0, 12.0 * double(n));
    split_tf32_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(w, hi, lo, n);
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace fxf
