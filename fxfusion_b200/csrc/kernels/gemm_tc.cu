// Tensor-core GEMM for sm_100a:  out[M,N] = act(x[M,K] · w[N,K]^T + bias[N])  with fp32-grade
// accuracy from three TF32 products per logical product ("3xTF32").
//
// The contraction behind Linear / LinearRelu / FeedForward / the MHA projections (reference:
// torch::linear, csrc/kernels/cpu/linear.cpp:11, feedforward.cpp:13, mha.cpp:22,51; the
// reference CUDA kernel is a 32x32 SIMT tile, csrc/kernels/cuda/linear.cu:5-41).
//
// Arithmetic.  x = x_hi + x_lo with x_hi the TF32 the tensor core sees and x_lo = tf32(x - x_hi); same
// for w.  x·w ~= x_lo·w_hi + x_hi·w_lo + x_hi·w_hi, accumulated in fp32; the dropped x_lo·w_lo term is
// ~2^-21 relative.  Weights are constants: they are split once when an engine is built
// (split_tf32_kernel, x_hi rounded to nearest) and kept as two arrays.  Activations are split inside
// the kernel while the tensor core works on earlier stages, in one of two ways:
//   A in shared memory (256-wide tiles): a TF32 MMA ignores the 13 low mantissa bits of an fp32 operand,
//     so the tile TMA wrote already is x_hi (x truncated); four warps write only x_lo into a twin buffer.
//   A in tensor memory (192- and 128-wide tiles): one thread per tile row reads its BK floats and stores
//     them (= x_hi) and x_lo with tcgen05.st; the MMAs take A from TMEM and only B (w_hi, w_lo) from
//     shared memory.
//   Either way x_lo = x - trunc_tf32(x) exactly (13 bits), passed on without a conversion: the MMA drops
//   its lowest 3 bits, below 2^-20 of x.
//
// Why two ways.  The kernel is bound by the shared-memory data pipe before the tensor pipe: with both
// operands in shared memory, operand reads and the split pass each took ~46 % of its wavefronts.
// Writing only x_lo removes a third of the split traffic; A in TMEM removes the split stores and the
// A operand reads, but TMEM (512 columns) cannot hold two 256-column accumulators plus A stages.
//
// Optional bf16 mode (FXF_GEMM_BF16, template flag BF16): the same pipeline with ONE product per logical product —
// weights converted to bf16 once per engine, the activation tile converted to packed bf16 pairs on its way into
// tensor memory, tcgen05.mma.kind::f16 (K = 16 per instruction), fp32 accumulation and fp32 output.  Results are
// bf16-grade (about 3e-3 of the output scale); it exists for throughput, not for the parity contract.
//
// Structure: a PERSISTENT kernel, one CTA per SM, each CTA walking a strided list of 128 x BN output
// tiles.  512 threads = four warpgroups whose roles only meet on mbarriers; each role resizes its register
// budget (setmaxnreg) so that the epilogue can keep a tile's running sums in registers:
//   warps 0-7   epilogue.  Warp w owns TMEM lanes 32*(w%4).. and the column half w/4 of the tile.  The
//               K loop of a tile is cut into chunks (TcParams::chunk_slabs K-slabs); the MMA warp
//               accumulates each chunk from zero into one of TWO TMEM accumulators, alternating, and the
//               epilogue warps add every finished chunk to fp32 running sums in registers (round to
//               nearest) while the tensor core works on the next chunk.  After the last chunk: bias, residual
//               and ReLU, staged through shared memory so that global stores are row-contiguous.
//   warps 8-11  the activation split of a landed stage (either way above), then arrive.
//   warp 12     TMA producer: per K-slab three cp.async.bulk.tensor loads — x tile [128,BK], w_hi and
//               w_lo tiles [BN,BK] — into a STAGES-deep ring, completion counted on an mbarrier.
//   warp 13     one thread issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8), 3 products per K-step,
//               accumulating in TMEM; tcgen05.commit hands the stage back to the producer and, after
//               the last slab of a chunk, the accumulator to the epilogue.
//   warps 14-15 idle (they complete the fourth warpgroup, which setmaxnreg needs).
// Why chunks.  The tensor core adds into its fp32 accumulator with truncation, so the error of one long
// accumulation chain grows linearly with K (about 4e-8 * K of the result's scale, measured).  Chains of at
// most `chunk` K-elements summed by CUDA cores bound that error for any K (see kChunkKDense / kChunkKConv).
// TMEM columns: [0, 2*BN) accumulators, then STAGES x (BK hi + BK lo) columns of A.
// Every mbarrier wait is bounded by a wall-clock budget; on expiry the CTA records an error in the
// status word, all roles stop issuing work, the CTA frees its TMEM and returns.
//
// Bound: tensor pipe (TF32 rate / 3).
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "../runtime.hpp"
#include "sm100.cuh"

namespace fxf {
namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int kThreads = 512;
constexpr int kEpiWarps = 8, kSplitWarp0 = 8, kTmaWarp = 12, kMmaWarp = 13;
constexpr int ACC = 2;   // TMEM accumulators, alternating per K chunk

enum : int { kErrWaitTma = 101, kErrWaitSplit = 102, kErrWaitEmpty = 103, kErrWaitAcc = 104, kErrWaitAccEmpty = 105, kErrWaitPartial = 106 };

constexpr int kStagePad = 20;  // floats per staged epilogue row: 16 + 4 keeps float4 rows conflict-free

// Register budgets per role (setmaxnreg, multiples of 8; the four warpgroups of a CTA must fit 64 K registers).  The
// epilogue holds BN / 2 running sums per thread; the split warps hold a row of the A stage when A goes to tensor memory.
template <int BN, int BK, bool TS, bool BF16>
struct RegBudget {
    static constexpr int epi = BN >= 256 ? 208 : (BN >= 224 ? 192 : (BN >= 192 ? 184 : 176));
    static constexpr int split = !TS ? 48 : (BN >= 224 ? 72 : ((BK == 32 && !BF16) ? 104 : 80));
    static constexpr int ctrl = BN >= 192 ? 48 : 56;
    static_assert(2 * 128 * epi + 128 * split + 128 * ctrl <= 65536, "register budgets exceed the register file");
};
template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_set() {   // the kernel starts with 128 registers per thread (512 threads, one CTA per SM)
    if constexpr (N > 128) reg_inc<N>();
    else if constexpr (N < 128) reg_dec<N>();
}

// BNB = weight rows held by this CTA: BN, or BN / 2 when two CTAs share a 256-row tile (each stages half of the weight tile)
template <int BNB, int BK, int STAGES, bool TS, bool BF16>
struct alignas(1024) TcSmem {
    float a[STAGES][BM * BK];             // x tile as TMA wrote it (fp32, swizzled rows of BK floats); x_hi in place when !TS
    float a_lo[TS ? 1 : STAGES][TS ? 256 : BM * BK];  // x_lo twin buffers (mixed: bf16(x_lo) | bf16(x)), only when the MMAs read A from shared memory
    float b_hi[STAGES][BF16 ? BNB * BK / 2 : BNB * BK];   // w_hi tile (fp32), or the whole bf16 weight tile in bf16 mode
    float b_lo[BF16 ? 1 : STAGES][BF16 ? 256 : BNB * BK];   // w_lo tile (fp32); mixed variant: bf16(w_hi) tile | bf16(w_lo) tile
    float stage_out[kEpiWarps][32 * kStagePad];   // one 32 x 16 block per epilogue warp
    uint64_t full_tma[STAGES];
    uint64_t full_b[STAGES];      // CTA pairs only: the weight halves of both CTAs have landed (the leader's copy counts)
    uint64_t full_split[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// Implicit-GEMM geometry of a convolution over a channels-last activation.  A tile's 128 rows are a box of
// output pixels (BW x BH x BNI <= 128; rows beyond the box are ignored); K-slab k is input-channel slab
// (k % c_slabs) of filter tap (k / c_slabs), fetched by one 4-D TMA load whose W/H coordinates are shifted by
// the tap (out-of-range pixels = zero padding).  A strided convolution uses the tensor map's traversal stride:
// the box spans BW*stride input pixels and every stride-th one is fetched.
struct ConvGeom {
    int enabled;
    int c_slabs, KW, WO, HO, N;
    int pad_h, pad_w, dil_h, dil_w, str_h, str_w;
    int BW, BH, BNI, tiles_w, tiles_h;
    uint32_t a_bytes;
};

struct TcParams {
    ConvGeom cv;
    const float* bias;
    const float* residual;   // optional, addressed like `out`
    float* out;
    int64_t M, N, K, ldo;
    int relu;
    int vec_out;
    int tiles_m, tiles_n, m_fastest;
    // Tail split: the first `full_tiles` tiles are computed whole; each of the remaining `tail_tiles` is cut along K
    // into `tail_split` work units that run on different CTAs.  Parts 1.. write their partial accumulator to `ws`
    // (unit-major, 128 x BN floats each) and raise flags[unit*4 + warp]; part 0 adds them in part order (deterministic).
    int full_tiles, tail_tiles, tail_split;
    int chunk_slabs;   // K-slabs per accumulation chain (>= 1)
    float* ws;
    int* flags;
    int* status;
    // Row-pushed output (tensor parallelism, row-parallel product): push_rows > 0 sends the rows [q*push_rows, (q+1)*push_rows)
    // of the result to push_out[q] (rank q's exchange window, possibly peer memory), at row push_rank*push_rows + (row -
    // q*push_rows) of it: after all ranks' launches rank q holds every rank's partial sums of the rows it owns, rank-major.
    // push_rows is a multiple of the 128 rows a CTA stores, so a tile has one destination.
    float* push_out[kMaxTpRanks];
    int64_t push_rows;
    int push_rank;
    int push_owners;   // > 1: row tiles are walked owner-interleaved (tiles_m is a multiple of it)
    // Transposed column range (GemmArgs::vt_*): vt_out != NULL switches it on; vt_col0 is a multiple of the column half of
    // the tile, the half a multiple of 32 (half a head), vt_T a multiple of 32 and no tile is cut along K.
    float* vt_out;
    unsigned char* vt_flags;
    int64_t vt_col0;
    int vt_T, vt_heads, vt_n32;
};

// x - (x with its 13 low mantissa bits cleared): the part of x a TF32 MMA does not see.  The difference is exact in fp32 and
// is handed to the MMA as it is (which again reads its upper 19 bits: what is dropped is below 2^-20 of x), so the
// activation split needs no conversion instruction.
__device__ __forceinline__ float lo_of_truncated(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

struct Unit {
    int tile, k0, k1, part, nparts, u;
};
__device__ __forceinline__ Unit get_unit(const TcParams& p, int unit, int num_k) {
    Unit r;
    if (unit < p.full_tiles) {
        r.tile = unit; r.k0 = 0; r.k1 = num_k; r.part = 0; r.nparts = 1; r.u = 0;
    } else {
        r.u = unit - p.full_tiles;
        r.nparts = p.tail_split;
        r.tile = p.full_tiles + r.u / r.nparts;
        r.part = r.u % r.nparts;
        r.k0 = int(int64_t(num_k) * r.part / r.nparts);
        r.k1 = int(int64_t(num_k) * (r.part + 1) / r.nparts);
    }
    return r;
}

__device__ __forceinline__ void tile_coords(const TcParams& p, int tile, int& tm, int& tn) {
    if (p.m_fastest) {
        tm = tile % p.tiles_m;
        tn = tile / p.tiles_m;
    } else {
        tn = tile % p.tiles_n;
        tm = tile / p.tiles_n;
    }
    // Row-pushed output: consecutive row tiles go to different owners, so that the stores that cross NVLink are spread over
    // the whole launch instead of arriving in one burst (owner-major order would send a rank's remote rows last).
    if (p.push_owners > 1) tm = (tm % p.push_owners) * (p.tiles_m / p.push_owners) + tm / p.push_owners;
}

// origin (ox0, oy0, n0) of the pixel box of M-tile `tm`
__device__ __forceinline__ void conv_tile_origin(const ConvGeom& c, int tm, int& ox0, int& oy0, int& n0) {
    ox0 = (tm % c.tiles_w) * c.BW;
    oy0 = ((tm / c.tiles_w) % c.tiles_h) * c.BH;
    n0 = (tm / (c.tiles_w * c.tiles_h)) * c.BNI;
}
// element offset of output row `r` (0..127) of M-tile `tm`, and whether that row exists
__device__ __forceinline__ int64_t out_row_offset(const TcParams& p, int tm, int r, bool& ok) {
    if (!p.cv.enabled) {
        int64_t row = int64_t(tm) * BM + r;
        ok = row < p.M;
        return row * p.ldo;
    }
    const ConvGeom& c = p.cv;
    int ox0, oy0, n0;
    conv_tile_origin(c, tm, ox0, oy0, n0);
    int w = r % c.BW, h = (r / c.BW) % c.BH, ni = r / (c.BW * c.BH);
    int ox = ox0 + w, oy = oy0 + h, n = n0 + ni;
    ok = ni < c.BNI && ox < c.WO && oy < c.HO && n < c.N;
    return ((int64_t(n) * c.HO + oy) * c.WO + ox) * p.ldo;
}

__device__ __forceinline__ float relu_keep_nan(float v) { return v > 0.f ? v : (v != v ? v : 0.f); }

// One finished accumulation chunk, this thread's row and HALF columns of it: TMEM -> registers, added to the running sums
// (16 columns per load keep the temporaries small: the sums themselves take HALF registers).
template <int HALF>
__device__ __forceinline__ void drain_chunk(uint32_t tacc, float (&sum)[HALF]) {
    static_assert(HALF % 16 == 0, "column halves are drained 16 columns at a time");
#pragma unroll
    for (int c = 0; c < HALF; c += 16) {
        uint32_t r[16];
        tmem_ld16(tacc + uint32_t(c), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; j++) sum[c + j] += __uint_as_float(r[j]);
    }
}

// PAIR: two CTAs of a cluster compute one 256 x BN tile with tcgen05.mma.cta_group::2 — each CTA stages its own 128 rows
// of x and HALF of the weight tile, which cuts the shared-memory traffic per flop (the limiter of this kernel) by a third
// to a half.  The leader (even rank) issues the MMAs for both; every CTA splits its own x rows and drains / stores its own
// 128 accumulator rows.  Barriers that gate the MMA (weight halves landed, x split, accumulator drained) live in the leader
// and are reached by the other CTA through the shared::cluster window; MMA completion is committed to both CTAs.
// VAR selects how the three products of a logical product are formed:
//   0  three TF32 products, A (hi and lo) from shared memory or from tensor memory (TS)
//   1  hybrid: x_hi read from shared memory as delivered, x_lo from tensor memory
//   2  mixed: the main product x_hi * w_hi as TF32 MMAs (x as delivered in shared memory: the MMA truncates it; w_hi the
//      fp32 tile), and BOTH correction products as bf16 MMAs (kind::f16, K = 16 per instruction): bf16(x_lo) * bf16(w_hi)
//      and bf16(x) * bf16(w_lo).  The correction operands are 2^-11 of their products, so their bf16 rounding (2^-9) costs
//      about 2^-20 of a product — the grade of the three-TF32 scheme, whose own accumulation truncates at that level.
//      What it buys: a tcgen05.mma occupies the tensor pipe for the same time whatever its kind (measured: 137 cycles at
//      N = 256, 97 at N <= 128), so 4 instead of 6 instructions per 16-deep K-slab is a third less tensor time.  Bytes
//      through L2 and shared memory are unchanged: per weight element 4 (w_hi) + 2 (bf16 w_hi) + 2 (bf16 w_lo).
//      With CTA pairs the bf16 copies of x_lo and x are written into shared memory by the split warps (rows of 32 bytes,
//      32-byte swizzle, beside each other in the stage's x_lo buffer); narrower tiles pack them into tensor memory.
template <int BN, int BK, int STAGES, bool TS, bool BF16, int VAR, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_whi,
                   const __grid_constant__ CUtensorMap map_wlo, TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    // dynamic shared memory is only guaranteed 16-byte aligned; swizzled tiles need 1024
    static_assert(!BF16 || (TS && BK == 32), "the bf16 mode takes A from tensor memory with 32-float slabs");
    constexpr bool HYB = VAR == 1, MIX = VAR == 2;
    static_assert(!HYB || (TS && !BF16), "hybrid: x_hi is the raw tile in shared memory, x_lo goes to tensor memory");
    static_assert(!MIX || (!BF16 && (TS != PAIR) && (BK == 16 || (BK == 32 && PAIR))), "mixed: A in shared memory for CTA pairs (16- or 32-deep slabs), in tensor memory otherwise (16-deep)");
    static_assert(BN % 32 == 0, "tile width must be a multiple of 32 columns (16 per column half and staging step)");
    static_assert(!PAIR || (!BF16 && VAR != 1), "CTA pairs exist for the plain 3xTF32 and the mixed variants");
    constexpr int BNB = PAIR ? BN / 2 : BN;   // weight rows staged by this CTA
    using Smem = TcSmem<BNB, BK, STAGES, TS, BF16>;
    using Regs = RegBudget<BN, BK, TS, BF16>;
    Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_k = int((p.K + BK - 1) / BK);
    const int num_units = p.full_tiles + p.tail_tiles * p.tail_split;
    const int chunk = p.chunk_slabs > 0 ? p.chunk_slabs : num_k;
    const int rank = PAIR ? int(cluster_ctarank()) : 0;     // position inside the CTA pair; rank 0 issues the MMAs
    const int sched_id = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x), sched_n = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
    constexpr uint32_t kBBytes = BF16 ? uint32_t(BNB * BK) * 2u : uint32_t(2 * BNB * BK) * 4u;   // weight bytes per stage and CTA (mixed: fp32 w_hi + two bf16 tiles)
    constexpr uint32_t kABytes = uint32_t(BM * BK) * 4u;
    constexpr uint32_t kStageBytes = kABytes + kBBytes;
    constexpr uint32_t kIdesc = BF16 ? umma_idesc_bf16(BM, BN) : umma_idesc_tf32(PAIR ? 2 * BM : BM, BN);
    constexpr int kACols = BF16 ? BK / 2 : (MIX ? BK : (HYB ? BK : 2 * BK));   // TMEM columns of one A stage (mixed: bf16(x_lo) | bf16(x), 8 columns each)
    constexpr int kBfTileBytes = BNB * BK * 2;   // one bf16 weight tile of the mixed variant
    constexpr uint32_t kIdescBf = umma_idesc_bf16(PAIR ? 2 * BM : BM, BN);   // the bf16 product of the mixed variant
    constexpr uint32_t kColA = uint32_t(ACC * BN);             // first TMEM column of the A stages
    constexpr uint32_t kColsUsed = kColA + (TS ? uint32_t(STAGES * kACols) : 0u);
    static_assert(kColsUsed <= 512, "accumulators and A stages exceed the 512 TMEM columns");
    constexpr uint32_t kTmemCols = kColsUsed <= 256 ? 256 : 512;  // allocations are powers of two
    volatile int* abort_flag = &s.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(&s.full_tma[i], 1);
            mbar_init(&s.full_b[i], 1);
            mbar_init(&s.full_split[i], PAIR ? 8 : 4);   // one arrival per split warp (of both CTAs of a pair)
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < ACC; i++) {
            mbar_init(&s.acc_full[i], 1);
            mbar_init(&s.acc_empty[i], PAIR ? 2 * kEpiWarps : kEpiWarps);    // one arrival per epilogue warp
        }
        s.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {  // TMEM allocation is a warp-wide operation; a pair allocates in both CTAs together
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync_all();   // the other CTA's barriers exist before anything of this CTA signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s.tmem_base;

    if (warp >= kTmaWarp) {
        reg_set<Regs::ctrl>();
        if (warp == kTmaWarp) {
            // ---------------- TMA producer ----------------
            if (lane == 0) {
                uint32_t it = 0;  // slab counter over all tiles of this CTA
                for (int unit = sched_id; unit < num_units; unit += sched_n) {
                    const Unit un = get_unit(p, unit, num_k);
                    int tm, tn;
                    tile_coords(p, un.tile, tm, tn);
                    if (PAIR) tm = tm * 2 + rank;   // this CTA's 128 rows of the pair's 256-row tile
                    for (int k = un.k0; k < un.k1; k++, it++) {
                        int st = it % STAGES;
                        if (it >= uint32_t(STAGES) && !mbar_wait(&s.empty[st], ((it / STAGES) - 1) & 1, abort_flag)) {
                            give_up(abort_flag, p.status, kErrWaitEmpty);
                            goto producer_done;
                        }
                        if (PAIR) {
                            // x rows: this CTA's own barrier (its split warps wait for it); weight halves: the leader's barrier,
                            // which expects the bytes of both CTAs
                            mbar_expect_tx(&s.full_tma[st], kABytes);
                            tma_load_2d(s.a[st], &map_x, k * BK, tm * BM, &s.full_tma[st]);
                            if (rank == 0) mbar_expect_tx(&s.full_b[st], 2 * kBBytes);
                            tma_load_2d_pair(s.b_hi[st], &map_whi, k * BK, tn * BN + rank * BNB, &s.full_b[st]);
                            if (MIX) {   // rows [0, N) of the bf16 matrix are bf16(w_hi), rows [N, 2N) bf16(w_lo)
                                char* bl = reinterpret_cast<char*>(s.b_lo[BF16 ? 0 : st]);
                                tma_load_2d_pair(bl, &map_wlo, k * BK, tn * BN + rank * BNB, &s.full_b[st]);
                                tma_load_2d_pair(bl + kBfTileBytes, &map_wlo, k * BK, int(p.N) + tn * BN + rank * BNB, &s.full_b[st]);
                            } else {
                                tma_load_2d_pair(s.b_lo[BF16 ? 0 : st], &map_wlo, k * BK, tn * BN + rank * BNB, &s.full_b[st]);
                            }
                            continue;
                        }
                        if (p.cv.enabled) {
                            int ox0, oy0, n0;
                            conv_tile_origin(p.cv, tm, ox0, oy0, n0);
                            const int tap = k / p.cv.c_slabs, cs = k - tap * p.cv.c_slabs, kh = tap / p.cv.KW, kw = tap - kh * p.cv.KW;
                            mbar_expect_tx(&s.full_tma[st], p.cv.a_bytes + kBBytes);
                            tma_load_4d(s.a[st], &map_x, cs * BK, ox0 * p.cv.str_w - p.cv.pad_w + kw * p.cv.dil_w,
                                        oy0 * p.cv.str_h - p.cv.pad_h + kh * p.cv.dil_h, n0, &s.full_tma[st]);
                        } else {
                            mbar_expect_tx(&s.full_tma[st], kStageBytes);
                            tma_load_2d(s.a[st], &map_x, k * BK, tm * BM, &s.full_tma[st]);
                        }
                        tma_load_2d(s.b_hi[st], &map_whi, k * BK, tn * BN, &s.full_tma[st]);
                        if (MIX) {
                            char* bl = reinterpret_cast<char*>(s.b_lo[BF16 ? 0 : st]);
                            tma_load_2d(bl, &map_wlo, k * BK, tn * BN, &s.full_tma[st]);                              // bf16(w_hi)
                            tma_load_2d(bl + kBfTileBytes, &map_wlo, k * BK, int(p.N) + tn * BN, &s.full_tma[st]);    // bf16(w_lo)
                        } else if (!BF16) {
                            tma_load_2d(s.b_lo[BF16 ? 0 : st], &map_wlo, k * BK, tn * BN, &s.full_tma[st]);   // fp32 w_lo
                        }
                    }
                }
            producer_done:;
            }
        } else if (warp == kMmaWarp) {
            // ---------------- MMA issuer ----------------
            if (lane == 0 && rank == 0) {   // in a pair only the leader issues MMAs (for both CTAs)
                uint32_t it = 0, ccount = 0;   // K-slabs and accumulation chunks issued so far by this CTA
                for (int unit = sched_id; unit < num_units; unit += sched_n) {
                    const Unit un = get_unit(p, unit, num_k);
                    for (int kc0 = un.k0; kc0 < un.k1; kc0 += chunk, ccount++) {
                        const int kc1 = min(kc0 + chunk, un.k1);
                        const uint32_t buf = ccount % ACC;
                        if (ccount >= uint32_t(ACC) &&
                            !(PAIR ? mbar_wait_cluster(&s.acc_empty[buf], ((ccount / ACC) - 1) & 1, abort_flag) : mbar_wait(&s.acc_empty[buf], ((ccount / ACC) - 1) & 1, abort_flag))) {
                            give_up(abort_flag, p.status, kErrWaitAccEmpty);
                            goto mma_done;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t tmem_acc = tmem_base + buf * uint32_t(BN);
                        for (int k = kc0; k < kc1; k++, it++) {
                            int st = it % STAGES;
                            uint32_t par = (it / STAGES) & 1;
                            if (!mbar_wait(PAIR ? &s.full_b[st] : &s.full_tma[st], par, abort_flag)) {
                                give_up(abort_flag, p.status, kErrWaitTma);
                                goto mma_done;
                            }
                            if (!(PAIR ? mbar_wait_cluster(&s.full_split[st], par, abort_flag) : mbar_wait(&s.full_split[st], par, abort_flag))) {
                                give_up(abort_flag, p.status, kErrWaitSplit);
                                goto mma_done;
                            }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            if (PAIR) {
                                // 256 x BN over the pair: A (hi / lo) at the same shared- or tensor-memory offsets in both CTAs, the
                                // weight half of each CTA at the same shared-memory offset
                                const uint64_t pb_hi = umma_desc_k_major<BK>(smem_u32(s.b_hi[st])), pb_lo = umma_desc_k_major<BK>(smem_u32(s.b_lo[BF16 ? 0 : st]));
                                if (MIX) {
                                    // bf16(x_lo) * bf16(w_hi) and bf16(x) * bf16(w_lo): one 16-deep bf16 MMA each, all operands in shared
                                    // memory; then x_hi * w_hi as two 8-deep TF32 MMAs on the raw tiles
                                    const uint64_t a_raw = umma_desc_k_major<BK>(smem_u32(s.a[st]));
                                    const uint32_t al = smem_u32(s.a_lo[TS ? 0 : st]), bl = smem_u32(s.b_lo[BF16 ? 0 : st]);
                                    const uint64_t d_xl = umma_desc_k_major_bytes<BK * 2>(al), d_wh = umma_desc_k_major_bytes<BK * 2>(bl);
                                    const uint64_t d_xb = umma_desc_k_major_bytes<BK * 2>(al + uint32_t(BM * BK * 2)), d_wl = umma_desc_k_major_bytes<BK * 2>(bl + uint32_t(kBfTileBytes));
#pragma unroll
                                    for (int kk = 0; kk < BK / 16; kk++) {   // 16 bf16 = 32 bytes per instruction inside the swizzle row
                                        const uint64_t adv = uint64_t((kk * 32) >> 4);
                                        umma_bf16_pair(tmem_acc, d_xl + adv, d_wh + adv, kIdescBf, (k > kc0 || kk > 0) ? 1u : 0u);
                                        umma_bf16_pair(tmem_acc, d_xb + adv, d_wl + adv, kIdescBf, 1u);
                                    }
#pragma unroll
                                    for (int kk = 0; kk < BK / 8; kk++) {
                                        const uint64_t adv = uint64_t((kk * 8 * 4) >> 4);
                                        umma_tf32_pair(tmem_acc, a_raw + adv, pb_hi + adv, kIdesc, 1u);
                                    }
                                } else if (TS) {
                                    const uint32_t a_hi = tmem_base + kColA + uint32_t(st * kACols), a_lo = a_hi + uint32_t(BK);
#pragma unroll
                                    for (int kk = 0; kk < BK / 8; kk++) {
                                        const uint64_t adv = uint64_t((kk * 8 * 4) >> 4);
                                        umma_tf32_ts_pair(tmem_acc, a_lo + uint32_t(kk * 8), pb_hi + adv, kIdesc, (k > kc0 || kk > 0) ? 1u : 0u);
                                        umma_tf32_ts_pair(tmem_acc, a_hi + uint32_t(kk * 8), pb_lo + adv, kIdesc, 1u);
                                        umma_tf32_ts_pair(tmem_acc, a_hi + uint32_t(kk * 8), pb_hi + adv, kIdesc, 1u);
                                    }
                                } else {
                                    const uint64_t a_hi = umma_desc_k_major<BK>(smem_u32(s.a[st])), a_lo = umma_desc_k_major<BK>(smem_u32(s.a_lo[st]));
#pragma unroll
                                    for (int kk = 0; kk < BK / 8; kk++) {
                                        const uint64_t adv = uint64_t((kk * 8 * 4) >> 4);
                                        umma_tf32_pair(tmem_acc, a_lo + adv, pb_hi + adv, kIdesc, (k > kc0 || kk > 0) ? 1u : 0u);
                                        umma_tf32_pair(tmem_acc, a_hi + adv, pb_lo + adv, kIdesc, 1u);
                                        umma_tf32_pair(tmem_acc, a_hi + adv, pb_hi + adv, kIdesc, 1u);
                                    }
                                }
                                umma_commit_pair(&s.empty[st]);   // frees the stage in both CTAs
                                continue;
                            }
                            if (BF16) {
                                const uint32_t a_bf = tmem_base + kColA + uint32_t(st * kACols);   // 8 columns (16 bf16) per K-step
                                const uint64_t b_bf = umma_desc_k_major_bytes<BK * 2>(smem_u32(s.b_hi[st]));
#pragma unroll
                                for (int kk = 0; kk < BK / 16; kk++)
                                    umma_bf16_ts(tmem_acc, a_bf + uint32_t(kk * 8), b_bf + uint64_t((kk * 32) >> 4), kIdesc, (k > kc0 || kk > 0) ? 1u : 0u);
                                umma_commit(&s.empty[st]);
                                continue;
                            }
                            uint64_t b_hi = umma_desc_k_major<BK>(smem_u32(s.b_hi[st])), b_lo = umma_desc_k_major<BK>(smem_u32(s.b_lo[BF16 ? 0 : st]));
                            if (MIX) {
                                // bf16(x_lo) * bf16(w_hi) and bf16(x) * bf16(w_lo), one 16-deep bf16 MMA each (A from tensor memory); then
                                // x_hi * w_hi per 8-deep step (x as delivered in shared memory: the MMA truncates it to TF32)
                                const uint64_t a_raw = umma_desc_k_major<BK>(smem_u32(s.a[st]));
                                const uint32_t a_lb = tmem_base + kColA + uint32_t(st * kACols), a_bf = a_lb + uint32_t(BK / 2);   // [bf16(x_lo): 8 columns | bf16(x): 8 columns]
                                const uint32_t bl = smem_u32(s.b_lo[BF16 ? 0 : st]);
                                umma_bf16_ts(tmem_acc, a_lb, umma_desc_k_major_bytes<BK * 2>(bl), kIdescBf, k > kc0 ? 1u : 0u);
                                umma_bf16_ts(tmem_acc, a_bf, umma_desc_k_major_bytes<BK * 2>(bl + uint32_t(kBfTileBytes)), kIdescBf, 1u);
#pragma unroll
                                for (int kk = 0; kk < BK / 8; kk++) {
                                    const uint64_t adv = uint64_t((kk * 8 * 4) >> 4);
                                    umma_tf32(tmem_acc, a_raw + adv, b_hi + adv, kIdesc, 1u);
                                }
                            } else if (HYB) {
                                // x_hi = the fp32 tile as it lies in shared memory (the MMA truncates it), x_lo from tensor memory
                                const uint32_t a_lo = tmem_base + kColA + uint32_t(st * kACols);
                                const uint64_t a_hi = umma_desc_k_major<BK>(smem_u32(s.a[st]));
#pragma unroll
                                for (int kk = 0; kk < BK / 8; kk++) {
                                    uint64_t adv = uint64_t((kk * 8 * 4) >> 4);
                                    umma_tf32_ts(tmem_acc, a_lo + uint32_t(kk * 8), b_hi + adv, kIdesc, (k > kc0 || kk > 0) ? 1u : 0u);
                                    umma_tf32(tmem_acc, a_hi + adv, b_lo + adv, kIdesc, 1u);
                                    umma_tf32(tmem_acc, a_hi + adv, b_hi + adv, kIdesc, 1u);
                                }
                            } else if (TS) {
                                const uint32_t a_hi = tmem_base + kColA + uint32_t(st * kACols), a_lo = a_hi + uint32_t(BK);  // 8 columns per K-step
#pragma unroll
                                for (int kk = 0; kk < BK / 8; kk++) {
                                    uint64_t adv = uint64_t((kk * 8 * 4) >> 4);  // 32 bytes per K-step inside the swizzle row
                                    umma_tf32_ts(tmem_acc, a_lo + uint32_t(kk * 8), b_hi + adv, kIdesc, (k > kc0 || kk > 0) ? 1u : 0u);
                                    umma_tf32_ts(tmem_acc, a_hi + uint32_t(kk * 8), b_lo + adv, kIdesc, 1u);
                                    umma_tf32_ts(tmem_acc, a_hi + uint32_t(kk * 8), b_hi + adv, kIdesc, 1u);
                                }
                            } else {
                                uint64_t a_hi = umma_desc_k_major<BK>(smem_u32(s.a[st])), a_lo = umma_desc_k_major<BK>(smem_u32(s.a_lo[st]));
#pragma unroll
                                for (int kk = 0; kk < BK / 8; kk++) {
                                    uint64_t adv = uint64_t((kk * 8 * 4) >> 4);
                                    umma_tf32(tmem_acc, a_lo + adv, b_hi + adv, kIdesc, (k > kc0 || kk > 0) ? 1u : 0u);
                                    umma_tf32(tmem_acc, a_hi + adv, b_lo + adv, kIdesc, 1u);
                                    umma_tf32(tmem_acc, a_hi + adv, b_hi + adv, kIdesc, 1u);
                                }
                            }
                            umma_commit(&s.empty[st]);  // arrives once the MMAs above have consumed the stage
                        }
                        if (PAIR) umma_commit_pair(&s.acc_full[buf]);
                        else umma_commit(&s.acc_full[buf]);
                    }
                }
            mma_done:;
            }
        }
    } else if (warp >= kSplitWarp0) {
        reg_set<Regs::split>();
        uint32_t it = 0;
        if (TS) {
            // ---------------- activation split: shared memory -> registers -> TMEM (hi | lo) ----------------
            const int quarter = warp & 3;                 // TMEM lane quarter this warp may address
            const int row = quarter * 32 + lane;          // tile row owned by this thread
            const uint32_t lane_base = uint32_t(quarter * 32) << 16;
            // TMA swizzle: the 16-byte chunks of a row are permuted by the row index (64-byte rows: bits 1-2, 128-byte rows: bits 0-2)
            const int sw = BK == 16 ? ((row >> 1) & 3) : (row & 7);
            for (int unit = sched_id; unit < num_units; unit += sched_n) {
                const Unit un = get_unit(p, unit, num_k);
                for (int k = un.k0; k < un.k1; k++, it++) {
                    int st = it % STAGES;
                    if (!mbar_wait(&s.full_tma[st], (it / STAGES) & 1, abort_flag)) {
                        give_up(abort_flag, p.status, kErrWaitTma);
                        goto split_done;
                    }
                    const float4* src = reinterpret_cast<const float4*>(s.a[st]) + row * (BK / 4);
                    if (BF16) {
                        // bf16 mode: the row's BK floats become BK/2 packed words (element k in the low half of word k/2)
                        uint32_t packed[16];
#pragma unroll
                        for (int c = 0; c < BK / 4 && c < 8; c++) {
                            float4 v = src[c ^ sw];
                            packed[2 * c + 0] = pack_bf16x2(v.x, v.y);
                            packed[2 * c + 1] = pack_bf16x2(v.z, v.w);
                        }
                        tmem_st16(tmem_base + lane_base + kColA + uint32_t(st * kACols), packed);
                        tmem_wait_st();
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&s.full_split[st]);
                        continue;
                    }
                    if (MIX) {
                        // what the TF32 truncation of x drops, and x itself, each as 8 packed bf16 pairs (element k in the low half
                        // of word k/2): columns [0, 8) and [8, 16) of the stage
                        uint32_t packed[16];
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const float4 v = src[c ^ sw];
                            packed[2 * c + 0] = pack_bf16x2(lo_of_truncated(v.x), lo_of_truncated(v.y));
                            packed[2 * c + 1] = pack_bf16x2(lo_of_truncated(v.z), lo_of_truncated(v.w));
                            packed[8 + 2 * c + 0] = pack_bf16x2(v.x, v.y);
                            packed[8 + 2 * c + 1] = pack_bf16x2(v.z, v.w);
                        }
                        const uint32_t a_col = tmem_base + lane_base + kColA + uint32_t(st * kACols);
                        tmem_st16(a_col, packed);
                        tmem_wait_st();
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            if (PAIR) mbar_arrive_leader(&s.full_split[st]);
                            else mbar_arrive(&s.full_split[st]);
                        }
                        continue;
                    }
                    if (HYB) {
                        uint32_t lo_only[BK];
#pragma unroll
                        for (int c = 0; c < BK / 4; c++) {
                            float4 v = src[c ^ sw];
                            lo_only[4 * c + 0] = __float_as_uint(lo_of_truncated(v.x));
                            lo_only[4 * c + 1] = __float_as_uint(lo_of_truncated(v.y));
                            lo_only[4 * c + 2] = __float_as_uint(lo_of_truncated(v.z));
                            lo_only[4 * c + 3] = __float_as_uint(lo_of_truncated(v.w));
                        }
                        tmem_st(tmem_base + lane_base + kColA + uint32_t(st * kACols), lo_only);
                        tmem_wait_st();
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&s.full_split[st]);
                        continue;
                    }
                    // x_hi = x as it is (the MMA truncates), x_lo = what the truncation drops; 16 columns at a time
                    const uint32_t a_col = tmem_base + lane_base + kColA + uint32_t(st * kACols);
#pragma unroll
                    for (int h = 0; h < BK / 16; h++) {
                        uint32_t hi[16], lo[16];
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            float4 v = src[(h * 4 + c) ^ sw];
                            hi[4 * c + 0] = __float_as_uint(v.x); lo[4 * c + 0] = __float_as_uint(lo_of_truncated(v.x));
                            hi[4 * c + 1] = __float_as_uint(v.y); lo[4 * c + 1] = __float_as_uint(lo_of_truncated(v.y));
                            hi[4 * c + 2] = __float_as_uint(v.z); lo[4 * c + 2] = __float_as_uint(lo_of_truncated(v.z));
                            hi[4 * c + 3] = __float_as_uint(v.w); lo[4 * c + 3] = __float_as_uint(lo_of_truncated(v.w));
                        }
                        tmem_st16(a_col + uint32_t(h * 16), hi);
                        tmem_st16(a_col + uint32_t(BK + h * 16), lo);
                    }
                    tmem_wait_st();
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_leader(&s.full_split[st]);
                        else mbar_arrive(&s.full_split[st]);
                    }
                }
            }
        } else {
            // ---------------- activation split in shared memory (hi in place, lo into the twin buffer) ----------------
            const int t = threadIdx.x - kSplitWarp0 * 32;  // 0..127
            for (int unit = sched_id; unit < num_units; unit += sched_n) {
                const Unit un = get_unit(p, unit, num_k);
                for (int k = un.k0; k < un.k1; k++, it++) {
                    int st = it % STAGES;
                    if (!mbar_wait(&s.full_tma[st], (it / STAGES) & 1, abort_flag)) {
                        give_up(abort_flag, p.status, kErrWaitTma);
                        goto split_done;
                    }
                    // The MMA reads only the upper 19 bits of an fp32 operand, so the tile TMA wrote already IS x_hi
                    // (x truncated to TF32); only x_lo = tf32(x - trunc(x)) has to be written.
                    const float4* hi = reinterpret_cast<const float4*>(s.a[st]);
                    float4* lo = reinterpret_cast<float4*>(s.a_lo[st]);
                    if (MIX) {
                        // bf16(x_lo) and bf16(x) tiles, [128 rows x BK] bf16 = rows of 2*BK bytes under the swizzle the MMA descriptor
                        // names (32-byte rows: 16-byte chunk j of row r at j ^ ((r >> 2) & 1); 64-byte rows: at j ^ ((r >> 1) & 3)),
                        // one tile behind the other.  The fp32 source rows are swizzled too (64-byte rows: chunk ^ ((r >> 1) & 3),
                        // 128-byte rows: chunk ^ (r & 7)).
                        char* lob = reinterpret_cast<char*>(s.a_lo[st]);
                        constexpr int CH = BK / 4;   // 16-byte chunks per fp32 row
#pragma unroll
                        for (int i = 0; i < (BM * BK / 4) / 128; i++) {
                            const int f = t + i * 128, row = f / CH;
                            const int c_log = (f % CH) ^ (BK == 16 ? ((row >> 1) & 3) : (row & 7));
                            const float4 v = hi[f];
                            uint2 pl, px;
                            pl.x = pack_bf16x2(lo_of_truncated(v.x), lo_of_truncated(v.y));
                            pl.y = pack_bf16x2(lo_of_truncated(v.z), lo_of_truncated(v.w));
                            px.x = pack_bf16x2(v.x, v.y);
                            px.y = pack_bf16x2(v.z, v.w);
                            const int dsw = BK == 16 ? ((row >> 2) & 1) : ((row >> 1) & 3);
                            const int dst = row * (2 * BK) + (((c_log >> 1) ^ dsw) << 4) + ((c_log & 1) << 3);
                            *reinterpret_cast<uint2*>(lob + dst) = pl;
                            *reinterpret_cast<uint2*>(lob + BM * BK * 2 + dst) = px;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < (BM * BK / 4) / 128; i++) {
                            float4 v = hi[t + i * 128], l;
                            l.x = lo_of_truncated(v.x);
                            l.y = lo_of_truncated(v.y);
                            l.z = lo_of_truncated(v.z);
                            l.w = lo_of_truncated(v.w);
                            lo[t + i * 128] = l;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA (async proxy)
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_leader(&s.full_split[st]);
                        else mbar_arrive(&s.full_split[st]);
                    }
                }
            }
        }
    split_done:;
    } else {
        // ---------------- epilogue (warps 0..7; warp w owns TMEM lanes 32*(w%4).. and column half w/4) ----------------
        reg_set<Regs::epi>();
        constexpr int HALF = BN / 2;
        const int q = warp & 3, chalf = warp >> 2;
        float* stage = s.stage_out[warp];
        const uint32_t lane_base = uint32_t(q * 32) << 16;
        uint32_t ccount = 0;
        for (int unit = sched_id; unit < num_units; unit += sched_n) {
            const Unit un = get_unit(p, unit, num_k);
            int tm, tn;
            tile_coords(p, un.tile, tm, tn);
            if (PAIR) tm = tm * 2 + rank;   // this CTA's 128 rows of the pair's 256-row tile
            const bool writes_partial = un.nparts > 1 && un.part > 0;
            const bool adds_partials = un.nparts > 1 && un.part == 0;
            // partial-tile slot of (unit, CTA of the pair); the parts of one tile are `pstep` slots apart
            const int slot = PAIR ? un.u * 2 + rank : un.u, pstep = PAIR ? 2 : 1;
            float* ws_mine = p.ws + size_t(slot) * size_t(BM * BN);
            // ---- running sums of this thread's row over the K chunks of the unit ----
            float sum[HALF];   // start from zero and always add: one code path keeps the register allocation tight
#pragma unroll
            for (int j = 0; j < HALF; j++) sum[j] = 0.f;
            bool alive = true;
            for (int kc0 = un.k0; kc0 < un.k1; kc0 += chunk, ccount++) {
                const uint32_t buf = ccount % ACC;
                if (!mbar_wait(&s.acc_full[buf], (ccount / ACC) & 1, abort_flag)) {
                    give_up(abort_flag, p.status, kErrWaitAcc);
                    alive = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tacc = tmem_base + buf * uint32_t(BN) + lane_base + uint32_t(chalf * HALF);
                drain_chunk<HALF>(tacc, sum);
                // the chunk is in registers: hand the TMEM buffer back
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_leader(&s.acc_empty[buf]);
                    else mbar_arrive(&s.acc_empty[buf]);
                }
            }
            if (!alive) break;
            if (adds_partials) {
                // the other K-parts of this tile run on other CTAs of this launch; wait for this warp's share of each
                int ok = 1;
                if (lane == 0)
                    for (int pp = 1; pp < un.nparts && ok; pp++) ok = flag_wait(p.flags + (slot + pp * pstep) * kEpiWarps + warp, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    give_up(abort_flag, p.status, kErrWaitPartial);
                    break;
                }
            }
            // ---- store: 16 columns at a time through shared memory, so that global accesses are row-contiguous ----
            const int row0 = q * 32;  // first row of this warp inside the tile
            const int64_t col_base = int64_t(tn) * BN + chalf * HALF;
            const int cq = (lane & 3) * 4, rsub = lane >> 2;  // 4 lanes cover one 64-byte row segment, 8 rows per instruction
            // Per-lane row pointers (rows i*8 + rsub, columns from col_base + cq): a group only adds a compile-time offset.
            float* orow[4];
            const float* rrow[4];
            bool oks[4];
            float* out_base = p.out;
            if (p.push_rows > 0) {
                const int64_t owner = (int64_t(tm) * BM) / p.push_rows;
                out_base = p.push_out[owner] + (int64_t(p.push_rank) - owner) * p.push_rows * p.ldo;
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int64_t off = out_row_offset(p, tm, row0 + i * 8 + rsub, oks[i]) + col_base + cq;
                orow[i] = out_base + off;
                rrow[i] = p.residual + off;   // only dereferenced when p.residual is set
            }
            const float* brow = p.bias + col_base + cq;              // only dereferenced when p.bias is set
            float* wrow = ws_mine + (row0 + rsub) * BN + chalf * HALF + cq;   // this lane's first row of the partial tile
            if (p.vt_out != nullptr && col_base >= p.vt_col0) {
                // ---- the V third of a packed QKV projection: transposed per head, straight from the registers ----
                // lane = row (token t of batch b), register j = column: for a fixed column the 32 lanes write 32 consecutive
                // keys of one V^T row (128 bytes).  A 32-row group never straddles two sequences (vt_T % 32 == 0).
                const int64_t grow = int64_t(tm) * BM + row0 + lane;
                const bool ok = grow < p.M;
                const int64_t b = grow / p.vt_T, t = grow - b * p.vt_T;
#pragma unroll
                for (int hh = 0; hh < HALF / 32; hh++) {               // 32 columns = half a head at a time
                    const int64_t c0 = col_base + hh * 32;             // first column of this piece inside the result
                    if (c0 >= p.N) continue;
                    const int64_t v0 = c0 - p.vt_col0, h = v0 >> 6;
                    const int d0 = int(v0 & 32);                       // 0 or 32: which half of the head
                    float* dst = p.vt_out + ((b * p.vt_heads + h) * 64 + d0) * int64_t(p.vt_T) + t;
                    bool bad = false;
#pragma unroll
                    for (int d = 0; d < 32; d++) {
                        const float v = sum[hh * 32 + d] + (p.bias ? __ldg(p.bias + c0 + d) : 0.f);
                        bad = bad || (v - v != 0.f);   // NaN or infinity
                        if (ok) dst[int64_t(d) * p.vt_T] = v;
                    }
                    const unsigned any_bad = __ballot_sync(0xffffffffu, ok && bad);
                    if (lane == 0 && ok) p.vt_flags[((b * p.vt_heads + h) * 2 + (d0 >> 5)) * p.vt_n32 + (t >> 5)] = any_bad ? 1 : 0;
                }
                continue;
            }
            if (!p.vec_out && !p.cv.enabled && un.nparts == 1 && p.residual == nullptr) {
                // ---- rows that do not start on 16-byte boundaries (a pitch like the 50257-column vocabulary) ----
                // Row r of this warp's 32 x HALF block starts `a` floats past a 16-byte boundary (a depends on the row).  The
                // block is stored as aligned 16-byte pieces shifted by a: the staging rows carry the last four columns of the
                // previous group in front of the current sixteen, so that the four pieces of a group, columns
                // [16g - a + 4q, +4), lie inside one staging row; the 4 - a leading and a trailing columns of the row segment
                // are stored by the row's owner straight from its registers.  Bias and activation are applied in place first.
                if (p.bias) {
#pragma unroll
                    for (int j = 0; j < HALF; j++) {
                        const int64_t c = col_base + j;
                        sum[j] += c < p.N ? __ldg(p.bias + c) : 0.f;   // the same address in every lane: one broadcast load
                    }
                }
                if (p.relu) {
#pragma unroll
                    for (int j = 0; j < HALF; j++) sum[j] = relu_keep_nan(sum[j]);
                }
                const int qq = lane & 3;
                float* rp[4];
                int ra[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int64_t grow = int64_t(tm) * BM + row0 + i * 8 + rsub;
                    rp[i] = out_base + grow * p.ldo + col_base;
                    ra[i] = grow < p.M ? int((reinterpret_cast<uintptr_t>(rp[i]) >> 2) & 3) : -1;   // -1: no such row
                }
#pragma unroll
                for (int g = 0; g < HALF / 16; g++) {
                    if (col_base + g * 16 - 3 >= p.N) continue;   // warp-uniform: nothing of this group (or its carry) is inside
                    if (g > 0) *reinterpret_cast<float4*>(stage + lane * kStagePad) = make_float4(sum[g * 16 - 4], sum[g * 16 - 3], sum[g * 16 - 2], sum[g * 16 - 1]);
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        *reinterpret_cast<float4*>(stage + lane * kStagePad + 4 + j) = make_float4(sum[g * 16 + j], sum[g * 16 + j + 1], sum[g * 16 + j + 2], sum[g * 16 + j + 3]);
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int a = ra[i];
                        if (a < 0 || (g == 0 && qq == 0 && a > 0)) continue;   // the piece left of the block belongs to the neighbour
                        const int c = g * 16 - a + 4 * qq;                      // first column of the piece, relative to col_base
                        const float* sp = stage + (i * 8 + rsub) * kStagePad + 4 - a + 4 * qq;
                        const float4 v = make_float4(sp[0], sp[1], sp[2], sp[3]);
                        const int64_t cabs = col_base + c;
                        if (cabs + 3 < p.N) {
                            *reinterpret_cast<float4*>(rp[i] + c) = v;
                        } else {
                            if (cabs < p.N) rp[i][c] = v.x;
                            if (cabs + 1 < p.N) rp[i][c + 1] = v.y;
                            if (cabs + 2 < p.N) rp[i][c + 2] = v.z;
                        }
                    }
                    __syncwarp();
                }
                {   // the row owner's leading 4 - a and trailing a columns
                    const int64_t grow = int64_t(tm) * BM + row0 + lane;
                    float* op = out_base + grow * p.ldo + col_base;
                    const int a = int((reinterpret_cast<uintptr_t>(op) >> 2) & 3);
                    if (grow < p.M && a > 0) {
#pragma unroll
                        for (int j = 0; j < 3; j++) {
                            if (j < 4 - a && col_base + j < p.N) op[j] = sum[j];
                            if (j < a && col_base + HALF - 1 - j < p.N) op[HALF - 1 - j] = sum[HALF - 1 - j];
                        }
                    }
                }
                continue;
            }
#pragma unroll
            for (int g = 0; g < HALF / 16; g++) {
                const int64_t col = col_base + g * 16;
                if (col >= p.N && !writes_partial) continue;  // warp-uniform
                // thread `lane` holds row (row0 + lane), 16 consecutive columns: stage them row-major
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    *reinterpret_cast<float4*>(stage + lane * kStagePad + j) = make_float4(sum[g * 16 + j], sum[g * 16 + j + 1], sum[g * 16 + j + 2], sum[g * 16 + j + 3]);
                __syncwarp();
                if (writes_partial) {
                    // raw partial sums, 128 x BN row-major; bias and activation belong to part 0
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        *reinterpret_cast<float4*>(wrow + i * 8 * BN + g * 16) = *reinterpret_cast<const float4*>(stage + (i * 8 + rsub) * kStagePad + cq);
                } else if (p.vec_out && col + 15 < p.N) {
                    float4 v[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) v[i] = *reinterpret_cast<const float4*>(stage + (i * 8 + rsub) * kStagePad + cq);
                    if (adds_partials) {
                        // the loads of a part are issued before the first add: one L2 round trip per part and group
                        for (int pp = 1; pp < un.nparts; pp++) {
                            const float* src = wrow + size_t(pp * pstep) * size_t(BM * BN) + g * 16;
                            float4 w[4];
#pragma unroll
                            for (int i = 0; i < 4; i++) w[i] = __ldcg(reinterpret_cast<const float4*>(src + i * 8 * BN));
#pragma unroll
                            for (int i = 0; i < 4; i++) { v[i].x += w[i].x; v[i].y += w[i].y; v[i].z += w[i].z; v[i].w += w[i].w; }
                        }
                    }
                    if (p.bias) {
                        const float4 b4 = *reinterpret_cast<const float4*>(brow + g * 16);
#pragma unroll
                        for (int i = 0; i < 4; i++) { v[i].x += b4.x; v[i].y += b4.y; v[i].z += b4.z; v[i].w += b4.w; }
                    }
                    if (p.residual != nullptr) {
                        // a folded residual Add, (acc + bias) + residual as the two separate nodes do; the loads are issued together
                        float4 r4[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) r4[i] = oks[i] ? *reinterpret_cast<const float4*>(rrow[i] + g * 16) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int i = 0; i < 4; i++) { v[i].x += r4[i].x; v[i].y += r4[i].y; v[i].z += r4[i].z; v[i].w += r4[i].w; }
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float4 o = v[i];
                        if (p.relu) {
                            o.x = relu_keep_nan(o.x); o.y = relu_keep_nan(o.y); o.z = relu_keep_nan(o.z); o.w = relu_keep_nan(o.w);
                        }
                        if (oks[i]) *reinterpret_cast<float4*>(orow[i] + g * 16) = o;
                    }
                } else {
                    // ragged or unaligned output (e.g. a vocabulary of 50257 columns): two rows per instruction, 16 lanes on
                    // consecutive columns
                    const int cl = lane & 15, r2 = lane >> 4;
                    const bool col_ok = col + cl < p.N;
                    const float b = (p.bias && col_ok) ? __ldg(p.bias + col + cl) : 0.f;
                    if (!p.cv.enabled && !adds_partials && p.residual == nullptr) {
                        // dense rows without extras: affine addresses, independent iterations (the stores of consecutive rows pipeline)
                        const int64_t grow = int64_t(tm) * BM + row0 + r2;
                        float* op = out_base + grow * p.ldo + col + cl;
                        const int64_t step = 2 * p.ldo;
#pragma unroll 8
                        for (int i = 0; i < 16; i++) {
                            float v = stage[(i * 2 + r2) * kStagePad + cl] + b;
                            if (p.relu) v = relu_keep_nan(v);
                            if (col_ok && grow + 2 * i < p.M) op[i * step] = v;
                        }
                    } else {
#pragma unroll 1
                        for (int i = 0; i < 16; i++) {
                            const int rr = i * 2 + r2;
                            float v = stage[rr * kStagePad + cl];
                            if (adds_partials)
                                for (int pp = 1; pp < un.nparts; pp++)
                                    v += __ldcg(ws_mine + size_t(pp * pstep) * size_t(BM * BN) + (row0 + rr) * BN + chalf * HALF + g * 16 + cl);
                            v += b;
                            bool row_ok;
                            const int64_t off = out_row_offset(p, tm, row0 + rr, row_ok);
                            if (p.residual && col_ok && row_ok) v += p.residual[off + col + cl];
                            if (p.relu) v = relu_keep_nan(v);
                            if (col_ok && row_ok) out_base[off + col + cl] = v;
                        }
                    }
                }
                __syncwarp();
            }
            if (writes_partial) {
                __threadfence();
                __syncwarp();
                if (lane == 0) flag_set(p.flags + slot * kEpiWarps + warp, 1);
            } else if (adds_partials) {
                __syncwarp();   // every lane has read its partials: lower the flags for the next launch
                if (lane == 0)
                    for (int pp = 1; pp < un.nparts; pp++) flag_set(p.flags + (slot + pp * pstep) * kEpiWarps + warp, 0);
            }
        }
    }
    // ---------------- teardown (every thread arrives here, whatever happened above) ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still touch its memory
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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

// Work split of `tiles` tiles (128 x bn, depth K) over `sms` persistent CTAs: whole tiles first, then the remainder
// R = tiles % sms cut along K into s parts each, so that the last round keeps R*s SMs busy for 1/s of a tile instead
// of R SMs for a whole one.  s minimises  tile_time / s + reduce_time(s)  over 1 <= s <= min(sms / R, 4) with at least
// 64 of K per part; the two times are in microseconds as measured on B200 (0.43 us per 128 x 256 x 16 slab of three
// TF32 products; 3 us + 7 us per extra part for writing, fetching and adding the partial tiles).
struct TailSplit { int64_t full, tail; int parts; double tail_us, tile_us; };
TailSplit plan_tail(int64_t tiles, int64_t K, int bn, int sms, bool allowed) {
    TailSplit t{tiles, 0, 1, 0.0, 0.0};
    t.tile_us = double((K + 15) / 16) * 0.43 * double(bn) / 256.0;
    t.tail_us = tiles % std::max(sms, 1) ? t.tile_us : 0.0;
    if (!allowed || sms <= 1) return t;
    const int64_t R = tiles % sms;
    if (R == 0) return t;
    const int64_t smax = std::min<int64_t>(std::min<int64_t>(sms / R, K / 64), 4);
    for (int64_t s = 2; s <= smax; s++) {
        const double us = t.tile_us / double(s) + 3.0 + 7.0 * double(s - 1);
        if (us < t.tail_us) {
            t.tail_us = us;
            t.full = tiles - R; t.tail = R; t.parts = int(s);
        }
    }
    return t;
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

// 2-D fp32 row-major [rows, cols] with row pitch `ld` floats; box = [box_rows, bk floats], rows one swizzle span wide.
int make_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, int bk) {
    EncodeTiledFn fn = encode_tiled_fn();
    FXF_CHECK(fn != nullptr, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(ld) * sizeof(float)};
    cuuint32_t box[2] = {cuuint32_t(bk), cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FXF_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (rows %lld cols %lld ld %lld)", int(r), (long long)rows, (long long)cols, (long long)ld);
    return 0;
}

// bf16 weight matrix [rows, cols] (row pitch `ld` elements): box [box_rows, bk], rows of bk * 2 bytes = one swizzle span
int make_map_bf16(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, int bk) {
    EncodeTiledFn fn = encode_tiled_fn();
    FXF_CHECK(fn != nullptr, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
    cuuint32_t box[2] = {cuuint32_t(bk), cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FXF_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (bf16) failed with code %d (rows %lld cols %lld ld %lld)", int(r), (long long)rows, (long long)cols, (long long)ld);
    return 0;
}

// channels-last activation [N,H,W,C] as a 4-D map; box = [BNI, BH, BW, bk channels], 64-byte swizzle (bk = 16).
// With a traversal stride s the box extent is given in input pixels (BW * s) and ceil(extent / s) = BW are loaded.
int make_map_nhwc(CUtensorMap* map, const float* base, int N, int H, int W, int C, int bni, int bh, int bw, int bk, int sh, int sw) {
    EncodeTiledFn fn = encode_tiled_fn();
    FXF_CHECK(fn != nullptr, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cuuint64_t dims[4] = {cuuint64_t(C), cuuint64_t(W), cuuint64_t(H), cuuint64_t(N)};
    cuuint64_t strides[3] = {cuuint64_t(C) * 4, cuuint64_t(W) * C * 4, cuuint64_t(H) * W * C * 4};
    cuuint32_t box[4] = {cuuint32_t(bk), cuuint32_t(bw * sw), cuuint32_t(bh * sh), cuuint32_t(bni)};
    cuuint32_t estr[4] = {1, cuuint32_t(sw), cuuint32_t(sh), 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FXF_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (conv) failed with code %d", int(r));
    return 0;
}

// K-elements per accumulation chain.  The tensor core's truncating adds cost about 4e-8 of the result's scale per K-element
// of a chain, and every extra chain costs time (measured on B200 at GPT-2-small shape: +2 % per forward with chains of
// 256, +9 % with 128, +14 % with 64: the drain of a chain competes with the store of the previous tile for the epilogue
// warps).  Dense layers are followed by normalisation and meet max-abs 1e-4 / rel 1e-3 with chains of 1024 (K = 768 is then
// one chain, as many as before); convolution stacks (ResNet-50: 52 in a row, logits of scale 400) need chains of 64 to
// meet the same rule end to end.
constexpr int kChunkKDense = 1024, kChunkKConv = 64;

template <int BN, int BK, int STAGES, bool TS, bool BF16 = false, int VAR = 0, bool PAIR = false>
int launch_tc(const GemmArgs& a, ExecCtx& ctx, const ConvTcArgs* cv = nullptr, const ConvGeom* geom = nullptr) {
    constexpr int BNB = PAIR ? BN / 2 : BN;      // weight rows one CTA stages
    constexpr int TM = PAIR ? 2 * BM : BM;       // rows of a scheduled tile (a CTA pair works on 256)
    FXF_CHECK(!PAIR || cv == nullptr, "CTA pairs are not used for convolutions");
    CUtensorMap mx, mhi, mlo;
    if (cv) {
        if (make_map_nhwc(&mx, cv->x, cv->N, cv->H, cv->W, cv->C, geom->BNI, geom->BH, geom->BW, BK, geom->str_h, geom->str_w)) return 1;
    } else if (make_map(&mx, a.x, a.M, a.K, a.ldx, BM, BK)) return 1;
    if (BF16) {
        if (make_map_bf16(&mhi, a.w_hi, a.N, a.K, a.K, BN, BK)) return 1;
        mlo = mhi;
    } else if (VAR == 2) {
        // mixed: w_lo points to a [2N, K] bf16 matrix, rows [0, N) = bf16(w_hi), rows [N, 2N) = bf16(w - w_hi)
        FXF_CHECK(a.w_mixed, "the mixed GEMM variant needs weights prepared for it");
        if (make_map(&mhi, a.w_hi, a.N, a.K, a.K, BNB, BK)) return 1;
        if (make_map_bf16(&mlo, a.w_lo, 2 * a.N, a.K, a.K, BNB, BK)) return 1;
    } else {
        FXF_CHECK(!a.w_mixed, "weights prepared for the mixed GEMM variant cannot feed the 3xTF32 kernels");
        if (make_map(&mhi, a.w_hi, a.N, a.K, a.K, BNB, BK)) return 1;
        if (make_map(&mlo, a.w_lo, a.N, a.K, a.K, BNB, BK)) return 1;
    }
    TcParams p{};
    if (geom) {
        p.cv = *geom;
        p.cv.enabled = 1;
        p.cv.c_slabs = cv->C / BK;
        p.cv.a_bytes = uint32_t(geom->BW * geom->BH * geom->BNI * BK) * 4u;
    }
    p.bias = a.bias; p.residual = cv ? cv->residual : a.residual; p.out = a.out; p.M = a.M; p.N = a.N; p.K = a.K; p.ldo = a.ldo;
    p.relu = a.relu ? 1 : 0;
    p.vec_out = (a.ldo % 4 == 0 && aligned16(a.out) && (a.bias == nullptr || aligned16(a.bias)) && (p.residual == nullptr || aligned16(p.residual))) ? 1 : 0;
    if (a.vt_out != nullptr) {
        FXF_CHECK(!cv && a.residual == nullptr && !a.relu && a.push_rows == 0 && (BN / 2) % 32 == 0 && a.vt_col0 % (BN / 2) == 0 && (a.N - a.vt_col0) % 64 == 0 &&
                      a.vt_T > 0 && a.vt_T % 32 == 0 && a.M % a.vt_T == 0 && a.vt_flags != nullptr && a.vt_heads * 64 == a.N - a.vt_col0,
                  "gemm: the transposed column range does not fit this kernel variant");
        p.vt_out = a.vt_out; p.vt_flags = a.vt_flags; p.vt_col0 = a.vt_col0; p.vt_T = a.vt_T; p.vt_heads = a.vt_heads; p.vt_n32 = a.vt_n32;
    }
    if (a.push_rows > 0) {
        const int64_t owners = a.M / a.push_rows;
        FXF_CHECK(!cv && a.residual == nullptr && a.push_out != nullptr && a.push_rows % BM == 0 && a.M % a.push_rows == 0 && owners >= 1 &&
                      owners <= kMaxTpRanks && a.push_rank >= 0 && a.push_rank < owners,
                  "gemm: a row-pushed output needs whole 128-row tiles per owner, no residual and at most %d owners", kMaxTpRanks);
        for (int64_t r = 0; r < owners; r++) {
            FXF_CHECK(a.push_out[r] != nullptr, "gemm: row-pushed output with a NULL window");
            p.push_out[r] = a.push_out[r];
            if (!aligned16(a.push_out[r])) p.vec_out = 0;
        }
        p.push_rows = a.push_rows;
        p.push_rank = a.push_rank;
    }
    p.tiles_m = int((a.M + TM - 1) / TM);
    if (a.push_rows > 0 && a.push_rows % TM == 0) p.push_owners = int(a.M / a.push_rows);
    p.tiles_n = int((a.N + BN - 1) / BN);
    // walk tiles so that the operand that does not fit in L2 is the one reused by concurrent CTAs
    p.m_fastest = a.N > a.M ? 1 : 0;
    p.status = ctx.status;
    size_t smem = sizeof(TcSmem<BNB, BK, STAGES, TS, BF16>) + 1024;
    static bool configured[64] = {};
    int dev = 0;
    FXF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        FXF_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<BN, BK, STAGES, TS, BF16, VAR, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n;
    // work units are scheduled over CTAs, or over CTA pairs (each CTA of a pair needs its own partial-tile slot and flags)
    const int workers = PAIR ? ctx.sm_count / 2 : ctx.sm_count, slots_per_unit = PAIR ? 2 : 1;
    TailSplit ts = plan_tail(tiles, a.K, BN, workers, ctx.gemm_ws != nullptr && ctx.gemm_flags != nullptr && a.vt_out == nullptr);
    if (ts.parts > 1 && (size_t(ts.tail) * ts.parts * slots_per_unit * size_t(BM * BN) * sizeof(float) > ctx.gemm_ws_bytes ||
                         ts.tail * ts.parts * slots_per_unit * kEpiWarps > ctx.gemm_flag_count))
        ts = TailSplit{tiles, 0, 1, 0.0, 0.0};
    p.full_tiles = int(ts.full); p.tail_tiles = int(ts.tail); p.tail_split = ts.parts;
    p.chunk_slabs = std::max(1, (ctx.tc_chunk_k > 0 ? ctx.tc_chunk_k : ((cv || a.conv_chain) ? kChunkKConv : kChunkKDense)) / BK);
    p.ws = ctx.gemm_ws; p.flags = ctx.gemm_flags;
    const int64_t units = ts.full + ts.tail * ts.parts;
    int grid = int(units < workers ? units : workers) * slots_per_unit;
    if (cv) {
        const double pix = double(cv->N) * cv->HO * cv->WO;
        tag_launch(ctx, BF16 ? "conv2d_igemm_bf16_tcgen05" : "conv2d_igemm_tf32x3_tcgen05", 2.0 * pix * double(a.N) * double(a.K),
                   4.0 * (double(cv->N) * cv->H * cv->W * cv->C + double(a.N) * a.K + double(a.N) + pix * a.N));
    } else {
        tag_launch(ctx, BF16 ? "gemm_bf16_tcgen05" : (VAR == 2 ? "gemm_tf32_bf16x2_tcgen05" : "gemm_tf32x3_tcgen05"), 2.0 * double(a.M) * double(a.N) * double(a.K),
                   4.0 * (double(a.M) * a.K + double(a.N) * a.K + double(a.N) + double(a.M) * a.N));
    }
    if (PAIR) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(grid));
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx.stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        FXF_CUDA(cudaLaunchKernelEx(&cfg, gemm_tf32x3_kernel<BN, BK, STAGES, TS, BF16, VAR, PAIR>, mx, mhi, mlo, p));
    } else {
        gemm_tf32x3_kernel<BN, BK, STAGES, TS, BF16, VAR, PAIR><<<grid, kThreads, smem, ctx.stream>>>(mx, mhi, mlo, p);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace

// The tensor-core path needs: pre-split weights, 16-byte aligned bases, row pitches that are
// multiples of 4 floats (TMA strides are multiples of 16 bytes), K a multiple of 4 and a problem
// large enough that 128-row tiles are not mostly padding.
bool gemm_tc_supported(const GemmArgs& a, bool allow_few_rows) {
    if (a.w_hi == nullptr || (!a.w_is_bf16 && a.w_lo == nullptr)) return false;
    if (a.w_is_bf16 && a.K % 8 != 0) return false;   // bf16 rows must be 16-byte multiples for TMA
    if (!gemm_tc_shape_ok(allow_few_rows && a.M >= 1 ? std::max<int64_t>(a.M, 64) : a.M, a.N, a.K)) return false;
    if (a.ldx % 4 != 0 || a.ldx < a.K) return false;
    if (!aligned16(a.x) || !aligned16(a.w_hi) || (!a.w_is_bf16 && !aligned16(a.w_lo))) return false;
    return true;
}

bool gemm_tc_shape_ok(int64_t M, int64_t N, int64_t K) {
    return M >= 64 && N >= 64 && K >= 32 && K % 4 == 0 && M < (int64_t(1) << 31) && N < (int64_t(1) << 31) && K < (int64_t(1) << 31);
}

// Tile width.  A persistent CTA runs ceil(tiles / SMs) tiles back to back, so the launch time is that count
// times the tile time (proportional to BN, with a small penalty for narrower tiles whose operand traffic per
// flop is higher).  E.g. M = 8192 on 148 SMs: N = 768 gives 192 tiles of 256 (2 rounds) but 256 tiles of 192
// (also 2 rounds, each 25 % shorter); N = 2304 is best at 256.
int gemm_tc_pick_bn(int64_t M, int64_t N, int sm_count, int64_t K) {
    if (N <= 128) return 128;
    const int64_t tiles_m = (M + BM - 1) / BM;
    // Very large problems whose N wastes < 2 % of a 224-wide tiling take the hybrid variant (x_hi read from shared
    // memory as delivered, x_lo from tensor memory; 224 = the widest tile that leaves TMEM room for x_lo stages):
    // 6 % faster than 256-wide tiles on the 8192 x 50257 x 768 vocabulary projection, slower on mid-size shapes.
    const int64_t n224 = (N + 223) / 224;
    if (K > 0 && tiles_m * n224 >= int64_t(16) * sm_count && double(n224 * 224) <= 1.02 * double(N)) return 224;
    const int cand[3] = {256, 192, 128};
    const double penalty[3] = {1.0, 1.10, 1.25};   // time per flop relative to the 256-wide tile (measured on the GPT-2 shapes)
    int best = 256;
    double best_cost = 0;
    for (int i = 0; i < 3; i++) {
        const int64_t tiles = tiles_m * ((N + cand[i] - 1) / cand[i]);
        const TailSplit t = plan_tail(tiles, K > 0 ? K : 768, cand[i], sm_count, K > 0);
        // rounds of whole tiles, plus the (possibly K-split) last round
        const double cost = (double(t.full / sm_count) * t.tile_us + t.tail_us) * penalty[i];
        if (i == 0 || cost < best_cost * 0.95) {
            best = cand[i];
            best_cost = cost;
        }
    }
    return best;
}

// Kernel variant per tile width.  Where the MMAs take A from decides it: with both operands in shared memory the kernel
// saturates the shared-memory data pipe (192-wide tiles: operand reads 48 % + split loads/stores 48 % of its wavefronts,
// tensor pipe 62 %); from tensor memory the split writes nothing to shared memory and the MMA reads only B there (measured
// on B200: 128-wide tiles gain 40 %, 192-wide 5-7 %).  256-wide tiles keep A in shared memory: TMEM (512 columns) holds the
// two 256-column accumulators and nothing else.  224 = the widest tile that leaves TMEM room for x_lo stages (hybrid).
//   256x256 pair  two CTAs of a cluster per 256-row tile (cta_group::2), A in shared memory, each CTA stages half of the
//        weight tile, BK 16, 6 stages: the default for the widest tiles of plain GEMMs
//   256  A in shared memory (x_hi = the tile as delivered, x_lo twin buffer), BK 16, 4 stages (convolutions; GEMMs with pairs off)
//   224  hybrid: x_hi read from shared memory as delivered, x_lo from tensor memory, BK 16, 4 stages
//   192  A (hi and lo) in tensor memory, BK 16, 4 stages
//   128  A in tensor memory, BK 32, 4 stages;  64: the same with 64-wide tiles for N <= 64
const char* gemm_tc_variant(int64_t M, int64_t N, int64_t K, int sm_count, bool k_split, bool few_rows, int* bn_out, bool pairs) {
    int bn = gemm_tc_pick_bn(M, N, sm_count, k_split ? K : 0);
    if (N <= 128) bn = N <= 64 ? 64 : 128;
    if (few_rows && M < 64) bn = N <= 64 ? 64 : 128;   // a weight-streaming problem: more, narrower tiles keep more SMs loading
    if (bn_out) *bn_out = bn;
    if (pairs && M > BM && sm_count >= 2 && bn >= 224) return "tcgen05-tf32x3-256x256-pair-smemA";
    switch (bn) {
        case 256: return "tcgen05-tf32x3-128x256-smemA";
        case 224: return "tcgen05-tf32x3-128x224-hybridA";
        case 192: return "tcgen05-tf32x3-128x192-tmemA";
        case 128: return "tcgen05-tf32x3-128x128-tmemA";
        default: return "tcgen05-tf32x3-128x64-tmemA";
    }
}

// Variant of the mixed arithmetic (one TF32 product + two bf16 corrections): the dispatch rule of the 3xTF32 kernels, with
// the 256- and 224-wide single-CTA tiles (whose A operand would not fit beside two accumulators in tensor memory) mapped to
// 192-wide ones.
const char* gemm_tc_mixed_variant(int64_t M, int64_t N, int64_t K, int sm_count, bool k_split, bool few_rows, int* bn_out, bool pairs) {
    int bn = 0;
    gemm_tc_variant(M, N, K, sm_count, k_split, few_rows, &bn, false);
    // Pairs take the widest tiles and, with this arithmetic, also 192-wide candidates of deep products (K >= 1024: measured
    // 8192 x 768 x 1536 in 85 us with pairs against 93 us without; at K = 768 and below the 192-wide tiles win).
    const bool pair = pairs && M > BM && sm_count >= 2 && (bn >= 224 || (bn == 192 && K >= 1024 && N >= 512));
    if (!pair && bn > 192) bn = 192;
    if (bn_out) *bn_out = pair ? 256 : bn;
    if (pair) return "tcgen05-tf32+2bf16-256x256-pair-smemA";
    switch (bn) {
        case 192: return "tcgen05-tf32+2bf16-128x192-tmemA";
        case 128: return "tcgen05-tf32+2bf16-128x128-tmemA";
        default: return "tcgen05-tf32+2bf16-128x64-tmemA";
    }
}

bool gemm_tc_vt_ok(const GemmArgs& a, const ExecCtx& ctx) {
    if (a.vt_out == nullptr || a.vt_flags == nullptr || a.residual != nullptr || a.relu || a.push_rows != 0 || a.w_is_bf16) return false;
    if (!gemm_tc_supported(a) || a.vt_T <= 0 || a.vt_T % 32 != 0 || a.M % a.vt_T != 0 || (a.N - a.vt_col0) != int64_t(a.vt_heads) * 64) return false;
    int bn = 0;
    if (a.w_mixed) gemm_tc_mixed_variant(a.M, a.N, a.K, ctx.sm_count, false, false, &bn, ctx.tc_pair != 1);
    else {
        gemm_tc_variant(a.M, a.N, a.K, ctx.sm_count, false, false, &bn, false);
        if (ctx.tc_pair != 1 && a.M > BM && ctx.sm_count >= 2 && bn >= 224) bn = 256;
    }
    if (bn == 224) return false;                       // column halves must be multiples of half a head (32 columns)
    return a.vt_col0 % (bn / 2) == 0;
}

int launch_gemm_tc(const GemmArgs& a, ExecCtx& ctx, bool allow_few_rows) {
    FXF_CHECK(gemm_tc_supported(a, allow_few_rows), "tensor-core GEMM called with an unsupported problem");
    int bn = 0;
    const bool ks = ctx.gemm_ws != nullptr && a.vt_out == nullptr;   // a transposed column range rules out tiles cut along K
    if (a.w_mixed) {
        gemm_tc_mixed_variant(a.M, a.N, a.K, ctx.sm_count, ks, allow_few_rows, &bn, ctx.tc_pair != 1);
        switch (bn) {
            // 32-deep slabs, three stages: the MMA-issuing thread pays its two barrier waits and its commit (about 90 cycles each)
            // per slab, which at 16-deep slabs and four instructions left the tensor pipe waiting for the thread (+9 % measured)
            case 256: return launch_tc<256, 32, 3, false, false, 2, true>(a, ctx);
            case 192: return launch_tc<192, 16, 5, true, false, 2>(a, ctx);
            case 128: return launch_tc<128, 16, 8, true, false, 2>(a, ctx);
            default: return launch_tc<64, 16, 8, true, false, 2>(a, ctx);
        }
    }
    gemm_tc_variant(a.M, a.N, a.K, ctx.sm_count, ks, allow_few_rows, &bn, false);
    if (a.w_is_bf16) {  // bf16 mode: one product per logical product, A converted into tensor memory
        if (bn >= 192 && a.N > 128) return launch_tc<192, 32, 6, true, true>(a, ctx);
        return launch_tc<128, 32, 8, true, true>(a, ctx);
    }
    // Wide tiles go to CTA pairs (256-row tiles, each CTA stages half of the weight tile: 40 % fewer bytes from L2 and six
    // stages instead of four): measured +4 % on the GPT-2-small GEMMs, also against the 224-wide hybrid.  192-wide tiles lose
    // with pairs (tensor memory leaves them four stages, too few for the cross-CTA latency).
    if (ctx.tc_pair != 1 && a.M > BM && ctx.sm_count >= 2 && bn >= 224) return launch_tc<256, 16, 6, false, false, 0, true>(a, ctx);
    switch (bn) {
        case 256: return launch_tc<256, 16, 4, false>(a, ctx);
        case 224: return launch_tc<224, 16, 4, true, false, true>(a, ctx);
        case 192: return launch_tc<192, 16, 4, true>(a, ctx);
        case 128: return launch_tc<128, 32, 4, true>(a, ctx);
        default: return launch_tc<64, 32, 4, true>(a, ctx);
    }
}

// ---- convolution as implicit GEMM ---------------------------------------------------------------------
bool conv_tc_shape_ok(int64_t n_pix, int C, int O) { return C >= 16 && C % 16 == 0 && O >= 64 && n_pix >= 64; }

namespace {
// Pixel box (BW x BH x BNI <= 128) that wastes the fewest rows: ragged tiles at the right/bottom edge and
// rows of the 128-row MMA tile beyond the box both count as waste.
void pick_pixel_box(int N, int HO, int WO, ConvGeom* g) {
    double best = -1;
    for (int bw = 1; bw <= std::min(WO, 128); bw++)
        for (int bh = 1; bh <= std::min(HO, 128 / bw); bh++) {
            int bni = (bw == WO && bh == HO) ? std::max(1, std::min(N, 128 / (bw * bh))) : 1;
            int64_t tiles = int64_t((WO + bw - 1) / bw) * ((HO + bh - 1) / bh) * ((N + bni - 1) / bni);
            double eff = double(WO) * HO * N / (double(tiles) * 128.0);
            if (eff > best + 1e-9) {
                best = eff;
                g->BW = bw; g->BH = bh; g->BNI = bni;
            }
        }
    g->tiles_w = (WO + g->BW - 1) / g->BW;
    g->tiles_h = (HO + g->BH - 1) / g->BH;
}

__global__ void __launch_bounds__(256) conv_weight_split_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int O, int C, int KH, int KW) {
    int64_t total = int64_t(O) * C * KH * KW, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int c = int(i % C);
        int64_t t = i / C;
        int kw = int(t % KW); t /= KW;
        int kh = int(t % KH);
        int o = int(t / KH);
        float h, l;
        split_tf32(w[((int64_t(o) * C + c) * KH + kh) * KW + kw], h, l);
        hi[i] = h;
        lo[i] = l;
    }
}
}  // namespace

int launch_conv_weight_split(const float* w_oihw, float* hi, float* lo, int O, int C, int KH, int KW, ExecCtx& ctx) {
    int64_t total = int64_t(O) * C * KH * KW;
    if (total == 0) return 0;
    int64_t blocks = (total + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
    tag_launch(ctx, "conv_weight_split_tf32", 0, 12.0 * double(total));
    conv_weight_split_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(w_oihw, hi, lo, O, C, KH, KW);
    FXF_LAUNCHED(ctx);
    return 0;
}

int launch_conv_tc(const ConvTcArgs& c, ExecCtx& ctx) {
    FXF_CHECK(c.x && c.w_hi && (c.w_lo || c.w_is_bf16) && c.out, "conv (tensor core): NULL operand");
    FXF_CHECK(c.str_h >= 1 && c.str_h <= 2 && c.str_w >= 1 && c.str_w <= 2, "conv (tensor core): stride must be 1 or 2");
    FXF_CHECK(conv_tc_shape_ok(int64_t(c.N) * c.HO * c.WO, c.C, c.O) && aligned16(c.x) && aligned16(c.w_hi) && (c.w_is_bf16 || aligned16(c.w_lo)),
              "conv (tensor core): unsupported problem");
    ConvGeom g{};
    g.KW = c.KW; g.WO = c.WO; g.HO = c.HO; g.N = c.N;
    g.pad_h = c.pad_h; g.pad_w = c.pad_w; g.dil_h = c.dil_h; g.dil_w = c.dil_w; g.str_h = c.str_h; g.str_w = c.str_w;
    pick_pixel_box(c.N, c.HO, c.WO, &g);
    const int64_t tiles_m = int64_t(g.tiles_w) * g.tiles_h * ((c.N + g.BNI - 1) / g.BNI);
    GemmArgs a;
    a.w_hi = c.w_hi; a.w_lo = c.w_lo; a.bias = c.bias; a.out = c.out;
    a.M = tiles_m * BM;  // rows the kernel schedules; rows outside the image are masked at the store
    a.N = c.O;
    a.K = int64_t(c.KH) * c.KW * c.C;
    a.ldo = c.O;
    a.relu = c.relu;
    int bn = 0;
    gemm_tc_variant(a.M, a.N, a.K, ctx.sm_count, ctx.gemm_ws != nullptr, false, &bn, false);
    if (c.w_is_bf16) {
        a.w_is_bf16 = true;
        FXF_CHECK(c.C % 32 == 0, "conv (tensor core, bf16): input channels must be a multiple of 32");
        if (bn >= 192) return launch_tc<192, 32, 6, true, true>(a, ctx, &c, &g);
        return launch_tc<128, 32, 8, true, true>(a, ctx, &c, &g);
    }
    switch (bn) {
        case 256: return launch_tc<256, 16, 4, false>(a, ctx, &c, &g);
        case 224: return launch_tc<224, 16, 4, true, false, true>(a, ctx, &c, &g);
        case 192: return launch_tc<192, 16, 4, true>(a, ctx, &c, &g);
        case 128: return c.C % 32 == 0 ? launch_tc<128, 32, 4, true>(a, ctx, &c, &g) : launch_tc<128, 16, 8, true>(a, ctx, &c, &g);
        default: return c.C % 32 == 0 ? launch_tc<64, 32, 4, true>(a, ctx, &c, &g) : launch_tc<64, 16, 8, true>(a, ctx, &c, &g);
    }
}

// ---- bf16 mode: weights converted once per engine ---------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) convert_bf16_kernel(const float* __restrict__ w, uint16_t* __restrict__ out, int64_t n) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = uint16_t(pack_bf16x2(w[i], 0.f) & 0xffffu);
}
__global__ void __launch_bounds__(256) conv_weight_bf16_kernel(const float* __restrict__ w, uint16_t* __restrict__ out, int O, int C, int KH, int KW) {
    int64_t total = int64_t(O) * C * KH * KW, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int c = int(i % C);
        int64_t t = i / C;
        int kw = int(t % KW); t /= KW;
        int kh = int(t % KH);
        int o = int(t / KH);
        out[i] = uint16_t(pack_bf16x2(w[((int64_t(o) * C + c) * KH + kh) * KW + kw], 0.f) & 0xffffu);
    }
}
}  // namespace

int launch_convert_bf16(const float* w, void* out, int64_t n, ExecCtx& ctx) {
    if (n == 0) return 0;
    int64_t blocks = (n + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
    tag_launch(ctx, "convert_bf16", 0, 6.0 * double(n));
    convert_bf16_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(w, static_cast<uint16_t*>(out), n);
    FXF_LAUNCHED(ctx);
    return 0;
}

int launch_conv_weight_bf16(const float* w_oihw, void* out, int O, int C, int KH, int KW, ExecCtx& ctx) {
    int64_t total = int64_t(O) * C * KH * KW;
    if (total == 0) return 0;
    int64_t blocks = (total + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
    tag_launch(ctx, "conv_weight_bf16", 0, 6.0 * double(total));
    conv_weight_bf16_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(w_oihw, static_cast<uint16_t*>(out), O, C, KH, KW);
    FXF_LAUNCHED(ctx);
    return 0;
}


namespace {
__global__ void __launch_bounds__(256) split_mixed_kernel(const float* __restrict__ w, float* __restrict__ hi, uint16_t* __restrict__ lo_bf, int64_t n) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float h, l;
        split_tf32(w[i], h, l);   // h = tf32(w) rounded to nearest; the low part is taken exactly below
        hi[i] = h;
        lo_bf[i] = uint16_t(pack_bf16x2(h, 0.f) & 0xffffu);              // rows [0, N): bf16(w_hi)
        lo_bf[n + i] = uint16_t(pack_bf16x2(w[i] - h, 0.f) & 0xffffu);   // rows [N, 2N): bf16(w - w_hi)
        (void)l;
    }
}
}  // namespace

int launch_split_mixed(const float* w, float* hi, void* bf_pair, int64_t n, ExecCtx& ctx) {
    if (n == 0) return 0;
    int64_t blocks = (n + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
    tag_launch(ctx, "split_tf32_bf16", 0, 12.0 * double(n));
    split_mixed_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(w, hi, static_cast<uint16_t*>(bf_pair), n);
    FXF_LAUNCHED(ctx);
    return 0;
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
