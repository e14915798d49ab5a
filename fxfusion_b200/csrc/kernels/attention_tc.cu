// Tensor-core attention core for head_dim 64 on sm_100a:
//     ctx = softmax(mask_fill(Q·K^T / scale_divisor)) · V        per (batch, head)
// with both contractions on tcgen05, fp32-grade: per fp32 product one TF32 product of the high parts plus two bf16
// correction products (bf16(a_lo)·bf16(b) and bf16(a)·bf16(b_lo), fp32 accumulation) — 32 tensor-core instructions per
// block of 64 keys where three TF32 products would take 48; an instruction costs the same whatever its kind.
// Same semantics as attention.cu (reference csrc/kernels/cpu/mha.cpp:38-49): division by the scale,
// -inf where mask == 0, fully masked rows give NaN, masked keys still enter P·V with weight 0 (so a
// non-finite V row poisons the output as 0 * inf does in the reference).  A block of 64 keys is skipped
// only when that cannot change a bit of the result: every mask byte of the block is 0 for all 128 query
// rows of the CTA (its probabilities are exactly 0) and the block's V rows are all finite (0 * V = 0).
// With a causal mask that drops the upper-triangle blocks.
//
// Two kernels:
//   attn_vt_kernel   transposes the V third of the packed projection qkv[B*T, 3D] into V^T [B*H, 64, T]
//                    (keys contiguous) so that the B operand of P·V is K-major.
//   attn_tc_kernel   one CTA per (128 queries, b, h), 384 threads, key blocks of 64, TWO CTAs per SM: a CTA walks
//                    TMA -> split -> S-MMA -> softmax -> P·V-MMA of a block as one dependent chain, so a second resident
//                    CTA is what keeps the tensor pipe and the softmax threads of an SM busy at the same time.  Per CTA
//                    106 KB of shared memory and 256 of the 512 tensor-memory columns:
//                        S [128x64] (P_hi overwrites it in place) | bf16(P_lo), bf16(P) | O [128x64] | bf16(Q_lo), bf16(Q).
//       warp 0, lane 0  TMA loads (Q and K tiles straight out of qkv through a 3-D tensor map, V^T
//                       tiles from the transposed copy; zero fill beyond T) and all MMAs:
//                       S = Q·K_blk^T (main product on the fp32 tiles as delivered, corrections with A from tensor memory),
//                       O_blk = P·V_blk with P read from tensor memory.
//       warps 1-3       write the bf16 copies (x and x_lo) of every landed K / V tile, so the softmax threads never wait
//                       for operands;
//       warps 4-11      softmax, two threads per query row, each owning 32 of the block's 64 keys and 32 of the 64
//                       output columns: first the bf16 copies of their half row of Q into tensor memory; per block
//                       tcgen05.ld of S, scale, mask (staged through shared memory so the global reads are
//                       coalesced), online softmax in the log2 domain (running max m, running sum l), P as fp32
//                       (over S) and as two bf16 copies into TMEM; after the P·V MMA the block's O is folded into
//                       registers (o = o*alpha + O_blk).
//       Registers: the kernel starts with 80 per thread (384 threads x 2 CTAs); setmaxnreg moves warps 0-3 to 48 and
//       the softmax warps to 96.
// Waits are bounded; on expiry the CTA records an error code in the status word and leaves.
#include <cmath>

#include "../runtime.hpp"
#include "sm100.cuh"

namespace fxf {
namespace {

using namespace sm100;

constexpr int HD = 64, BQ = 128, BKEY = 64;
constexpr int kAttnThreads = 384;
constexpr uint32_t kTmemCols = 256;      // S / P_hi | P_lo | O | Q_lo, 64 columns each: two CTAs share an SM's 512 columns
constexpr int kRegsCtrl = 48, kRegsSoft = 96;   // setmaxnreg budgets: warps 0-3 (TMA / MMA / splits) and warps 4-11 (softmax);
                                                // 128 * 48 + 256 * 96 = the 384 * 80 registers a CTA starts with
constexpr int kSoftWarp0 = 4;            // warps 4..11: TMEM lane quarter = warp % 4, key half = (warp - 4) / 4
constexpr int kSplitWarp0 = 1, kSplitWarps = 3;   // warps 1..3 split the landed Q / K / V tiles (off the softmax threads' path)
constexpr int kMaskPitch = 80;           // bytes per staged mask row (64 + 16): 16-byte reads stay conflict-free
constexpr float kLog2e = 1.4426950408889634f;
enum : int { kErrAttnQ = 111, kErrAttnK = 112, kErrAttnV = 113, kErrAttnS = 114, kErrAttnP = 115, kErrAttnO = 116, kErrAttnSplit = 117 };

// 2^x on the special-function unit: 2^-inf = 0, NaN stays NaN (the row-poisoning rules rely on both).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Barrier between the two softmax warps that share a quarter of the query rows (ids 1..4; id 0 is __syncthreads): the row
// statistics they exchange concern only their own 32 rows, so the four pairs need not wait for one another.
__device__ __forceinline__ void soft_sync(int quarter) { asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory"); }

// ---- V transpose -------------------------------------------------------------------------------------
// Also records, per (batch*head, half of the head's 64 columns, 32-key slab), whether any V element is NaN or infinite:
// vflags[(bh * 2 + half) * n32 + slab] (this kernel reports a slab under half 0 and clears half 1).
__global__ void __launch_bounds__(256) attn_vt_kernel(const float* __restrict__ qkv, int64_t ld, int64_t v_off, int T, int H, float* __restrict__ vt,
                                                      unsigned char* __restrict__ vflags, int n32) {
    // one block moves 64 keys x 64 head columns: rows of 256 bytes on both sides
    __shared__ float tile[HD][65];
    const int bh = blockIdx.y, b = bh / H, h = bh % H, t0 = blockIdx.x * 64, tid = threadIdx.x;
    int bad[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int f = tid + i * 256, r = f >> 4, c4 = (f & 15) * 4, t = t0 + r;   // i = 0, 1: keys 0..31 of the block; i = 2, 3: keys 32..63
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < T) v = *reinterpret_cast<const float4*>(qkv + (int64_t(b) * T + t) * ld + v_off + int64_t(h) * HD + c4);
        // x - x is 0 for finite x and NaN for NaN / infinity
        bad[i >> 1] |= ((v.x - v.x) != 0.f) | ((v.y - v.y) != 0.f) | ((v.z - v.z) != 0.f) | ((v.w - v.w) != 0.f);
        tile[c4 + 0][r] = v.x; tile[c4 + 1][r] = v.y; tile[c4 + 2][r] = v.z; tile[c4 + 3][r] = v.w;
    }
    const int bad0 = __syncthreads_or(bad[0]), bad1 = __syncthreads_or(bad[1]);
    if (tid == 0) {
        const int sl = blockIdx.x * 2;
        vflags[int64_t(bh) * 2 * n32 + sl] = bad0 ? 1 : 0;
        vflags[(int64_t(bh) * 2 + 1) * n32 + sl] = 0;
        if (sl + 1 < n32) {
            vflags[int64_t(bh) * 2 * n32 + sl + 1] = bad1 ? 1 : 0;
            vflags[(int64_t(bh) * 2 + 1) * n32 + sl + 1] = 0;
        }
    }
    for (int idx = tid; idx < HD * 64; idx += 256) {
        int d = idx >> 6, tt = idx & 63, t = t0 + tt;
        if (t < T) vt[(int64_t(bh) * HD + d) * T + t] = tile[d][tt];
    }
}

// ---- main kernel -------------------------------------------------------------------------------------
struct alignas(1024) AttnTcSmem {
    float q_hi[2][BQ * 32];                        // two 32-wide slabs of head_dim (the bf16 copies of Q live in tensor memory)
    float k_hi[2][BKEY * 32];                      // K block as delivered: two 32-wide slabs of head_dim
    uint16_t k_bf[BKEY * HD], k_lo_bf[BKEY * HD];  // bf16(k) and bf16(k - tf32(k)): [64 keys x 64] rows of 128 bytes, 128-byte swizzle
    float v_hi[2][HD * 32];                        // V^T block as delivered: two 32-key slabs [64 x 32]
    uint16_t v_bf[HD * BKEY], v_lo_bf[HD * BKEY];  // the same two bf16 copies of V^T [64 head columns x 64 keys]
    unsigned char mask_rows[BQ * kMaskPitch];      // this block's mask bytes, one padded row per query
    float exch[2][BQ];                             // row statistics exchanged between the two threads of a row
    uint64_t bar_q, bar_k, bar_v, bar_qs, bar_ks, bar_vs, bar_s, bar_p, bar_o;
    unsigned long long need_blocks;                // bit blk set: key block blk has to be processed
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(2 * (sizeof(AttnTcSmem) + 2048) <= 228 * 1024, "two CTAs of the attention kernel must fit one SM");

struct AttnTcParams {
    const unsigned char* vflags;   // per (batch*head, column half of the head, 32-key slab): V has a non-finite element
    int n32;                       // slabs per (batch*head)
    const uint8_t* mask;
    float* ctx;
    int B, T, Tk, H;      // T queries and Tk keys per batch
    int q_col, k_col;     // first column of the Q block inside a query row / of the K block inside a key row
    int64_t ld_ctx;
    int64_t mask_sb, mask_sh, mask_sq, mask_sk;
    float scale_divisor;
    float inv_scale;      // 1 / scale_divisor, used only when that is exact
    int scale_is_pow2;
    int mask_vec16;       // mask rows may be fetched as aligned 16-byte words
    int* status;
};

// x - (x with its 13 low mantissa bits cleared): the part of x a TF32 MMA does not see.  The difference is exact in fp32 and
// is handed to the MMA as it is (which again reads its upper 19 bits: what is dropped is below 2^-20 of x), so the split
// needs no conversion instruction.
__device__ __forceinline__ float lo_of_truncated(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
// The MMA reads only the upper 19 bits of an fp32 operand in shared memory, so the tile TMA wrote already is the "hi"
// operand of the main TF32 product.  The two correction products run as bf16 MMAs: this writes their B operands, bf16(x)
// and bf16(x_lo), for a tile of 64 rows x 64 elements delivered as two 32-float slabs (128-byte rows, 16-byte chunk j of row
// r at chunk j ^ (r & 7)); the bf16 tiles have 128-byte rows of 64 elements under the same swizzle.
__device__ __forceinline__ void split_tile_bf16(const float* slabs, uint16_t* x_bf, uint16_t* lo_bf, int t, int n_threads) {
    const float4* src = reinterpret_cast<const float4*>(slabs);
    char* db = reinterpret_cast<char*>(x_bf);
    char* dl = reinterpret_cast<char*>(lo_bf);
    for (int i = t; i < 2 * 64 * 8; i += n_threads) {
        const int sl = i >> 9, r = (i >> 3) & 63, j = (i & 7) ^ (r & 7);   // slab, row, logical 16-byte chunk of the slab row
        const float4 v = src[i];
        uint2 px, pl;
        px.x = pack_bf16x2(v.x, v.y);
        px.y = pack_bf16x2(v.z, v.w);
        pl.x = pack_bf16x2(lo_of_truncated(v.x), lo_of_truncated(v.y));
        pl.y = pack_bf16x2(lo_of_truncated(v.z), lo_of_truncated(v.w));
        const int J = sl * 4 + (j >> 1);                                     // 16-byte chunk of the bf16 row (8 elements)
        const int dst = r * 128 + ((J ^ (r & 7)) << 4) + ((j & 1) << 3);
        *reinterpret_cast<uint2*>(db + dst) = px;
        *reinterpret_cast<uint2*>(dl + dst) = pl;
    }
}
template <int N>
__device__ __forceinline__ void attn_reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void attn_reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__global__ void __launch_bounds__(kAttnThreads, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_vt,
               AttnTcParams p) {
    extern __shared__ unsigned char smem_raw[];
    AttnTcSmem& s = *reinterpret_cast<AttnTcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs are handed out in linear order (x fastest): the last query tile of every (batch, head) goes first.  Under a
    // causal mask the later query tiles keep more key blocks, so the long CTAs start first and the short ones fill the tail.
    const int lin = blockIdx.y * gridDim.x + blockIdx.x, n_bh = gridDim.y;
    const int bh = lin % n_bh, b = bh / p.H, h = bh % p.H, q0 = (int(gridDim.x) - 1 - lin / n_bh) * BQ, T = p.T, Tk = p.Tk;
    const int nblk = (Tk + BKEY - 1) / BKEY;
    volatile int* abort_flag = &s.abort_flag;
    constexpr uint32_t kQBytes = BQ * HD * 4, kKBytes = BKEY * HD * 4, kVBytes = HD * BKEY * 4;
    // tensor-memory columns: S (P_hi replaces it in place) | bf16(P_lo) 32 + bf16(P) 32 | O | bf16(Q_lo) 32 + bf16(Q) 32
    constexpr uint32_t kColS = 0, kColPhi = 0, kColPloB = 64, kColPB = 96, kColO = 128, kColQloB = 192, kColQB = 224;
    constexpr uint32_t kIdesc = umma_idesc_tf32(BQ, 64);     // both contractions produce 128 x 64 tiles (64 keys / 64 head columns)
    constexpr uint32_t kIdescBf = umma_idesc_bf16(BQ, 64);   // the correction products (bf16, K = 16 per instruction)

    if (threadIdx.x == 0) {
        mbar_init(&s.bar_q, 1);
        mbar_init(&s.bar_k, 1);
        mbar_init(&s.bar_v, 1);
        mbar_init(&s.bar_qs, 8);              // one arrival per softmax warp (they write Q_lo into tensor memory)
        mbar_init(&s.bar_ks, kSplitWarps);    // one arrival per split warp
        mbar_init(&s.bar_vs, kSplitWarps);
        mbar_init(&s.bar_s, 1);
        mbar_init(&s.bar_p, 8);
        mbar_init(&s.bar_o, 1);
        s.abort_flag = 0;
        s.need_blocks = 0ull;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s.tmem_base;

    // ---- which key blocks matter to this CTA's 128 query rows ----
    const unsigned long long all_blocks = nblk >= 64 ? ~0ull : ((1ull << nblk) - 1ull);
    if (p.mask_vec16 && nblk <= 64) {
        unsigned long long mine = 0;
        const uint8_t* mh = p.mask + int64_t(b) * p.mask_sb + int64_t(h) * p.mask_sh;
        const int vec_per_row = Tk / 16, rows = min(BQ, T - q0);
        for (int idx = threadIdx.x; idx < rows * vec_per_row; idx += kAttnThreads) {
            const int rr = idx / vec_per_row, vv = idx - rr * vec_per_row;
            const uint4 m16 = *reinterpret_cast<const uint4*>(mh + int64_t(q0 + rr) * p.mask_sq + vv * 16);
            if (m16.x | m16.y | m16.z | m16.w) mine |= 1ull << (vv / (BKEY / 16));
        }
        // a block whose V rows hold NaN or infinity is kept: 0 * inf has to reach the output
        for (int sl = threadIdx.x; sl < p.n32; sl += kAttnThreads)
            if (p.vflags[int64_t(bh) * 2 * p.n32 + sl] | p.vflags[(int64_t(bh) * 2 + 1) * p.n32 + sl]) mine |= 1ull << (sl / (BKEY / 32));
        const unsigned int lo32 = __reduce_or_sync(0xffffffffu, (unsigned int)(mine & 0xffffffffull));
        const unsigned int hi32 = __reduce_or_sync(0xffffffffu, (unsigned int)(mine >> 32));
        mine = (unsigned long long)lo32 | ((unsigned long long)hi32 << 32);
        if (lane == 0 && mine) atomicOr(&s.need_blocks, mine);
        __syncthreads();
    } else {
        if (threadIdx.x == 0) s.need_blocks = all_blocks;
        __syncthreads();
    }
    const unsigned long long need = s.need_blocks & all_blocks;
    const int n_act = __popcll(need);

    if (warp < 4) {
        attn_reg_dec<kRegsCtrl>();
        if (warp == 0) {
            if (lane == 0) {
                auto load_k = [&](int blk) {
                    mbar_expect_tx(&s.bar_k, kKBytes);
                    for (int sl = 0; sl < 2; sl++) tma_load_3d(s.k_hi[sl], &map_k, p.k_col + h * HD + sl * 32, blk * BKEY, b, &s.bar_k);
                };
                auto load_v = [&](int blk) {
                    mbar_expect_tx(&s.bar_v, kVBytes);
                    for (int ks = 0; ks < 2; ks++) tma_load_3d(s.v_hi[ks], &map_vt, blk * BKEY + ks * 32, 0, bh, &s.bar_v);
                };
                unsigned long long rem = need;
                if (n_act > 0) {
                    mbar_expect_tx(&s.bar_q, kQBytes);
                    for (int sl = 0; sl < 2; sl++) tma_load_3d(s.q_hi[sl], &map_qkv, p.q_col + h * HD + sl * 32, q0, b, &s.bar_q);
                    load_k(__ffsll(rem) - 1);
                    load_v(__ffsll(rem) - 1);
                }
                if (n_act > 0 && !mbar_wait(&s.bar_qs, 0, abort_flag)) {
                    give_up(abort_flag, p.status, kErrAttnQ);
                } else {
                    for (int i = 0; i < n_act; i++) {
                        rem &= rem - 1;                                   // `rem` now holds the blocks after this one
                        const int next_blk = rem ? __ffsll(rem) - 1 : -1;
                        const uint32_t par = i & 1;
                        if (!mbar_wait(&s.bar_ks, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnK); break; }
                        tc_fence_after();
                        // S = Q · K_blk^T: q_hi·k_hi as TF32 products (both operands as delivered in shared memory), then the
                        // corrections bf16(q_lo)·bf16(k) and bf16(q)·bf16(k_lo) as bf16 products (A from tensor memory), 16 deep each
#pragma unroll
                        for (int sl = 0; sl < 2; sl++) {
                            const uint64_t qh = umma_desc_k_major<32>(smem_u32(s.q_hi[sl])), kh = umma_desc_k_major<32>(smem_u32(s.k_hi[sl]));
#pragma unroll
                            for (int kk = 0; kk < 4; kk++) {
                                const uint64_t adv = uint64_t((kk * 32) >> 4);
                                umma_tf32(tmem + kColS, qh + adv, kh + adv, kIdesc, (sl > 0 || kk > 0) ? 1u : 0u);
                            }
                        }
                        {
                            const uint64_t kb = umma_desc_k_major_bytes<128>(smem_u32(s.k_bf)), klb = umma_desc_k_major_bytes<128>(smem_u32(s.k_lo_bf));
#pragma unroll
                            for (int kk = 0; kk < 4; kk++) {
                                const uint64_t adv = uint64_t((kk * 32) >> 4);
                                umma_bf16_ts(tmem + kColS, tmem + kColQloB + uint32_t(kk * 8), kb + adv, kIdescBf, 1u);
                                umma_bf16_ts(tmem + kColS, tmem + kColQB + uint32_t(kk * 8), klb + adv, kIdescBf, 1u);
                            }
                        }
                        umma_commit(&s.bar_s);
                        if (next_blk >= 0) {  // K buffer is free once the S MMAs have completed
                            if (!mbar_wait(&s.bar_s, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnS); break; }
                            load_k(next_blk);
                        }
                        if (!mbar_wait(&s.bar_vs, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnV); break; }
                        if (!mbar_wait(&s.bar_p, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnP); break; }
                        tc_fence_after();
                        // O_blk = P · V_blk   (A = P from tensor memory, B = V^T, K-major over keys): p_hi·v_hi as TF32 products, the
                        // corrections bf16(p_lo)·bf16(v) and bf16(p)·bf16(v_lo) as bf16 products
#pragma unroll
                        for (int ks = 0; ks < 2; ks++) {
                            const uint64_t vh = umma_desc_k_major<32>(smem_u32(s.v_hi[ks]));
#pragma unroll
                            for (int kk = 0; kk < 4; kk++) {
                                const uint64_t adv = uint64_t((kk * 32) >> 4);
                                umma_tf32_ts(tmem + kColO, tmem + kColPhi + uint32_t(ks * 32 + kk * 8), vh + adv, kIdesc, (ks > 0 || kk > 0) ? 1u : 0u);
                            }
                        }
                        {
                            const uint64_t vb = umma_desc_k_major_bytes<128>(smem_u32(s.v_bf)), vlb = umma_desc_k_major_bytes<128>(smem_u32(s.v_lo_bf));
#pragma unroll
                            for (int kk = 0; kk < 4; kk++) {
                                const uint64_t adv = uint64_t((kk * 32) >> 4);
                                umma_bf16_ts(tmem + kColO, tmem + kColPloB + uint32_t(kk * 8), vb + adv, kIdescBf, 1u);
                                umma_bf16_ts(tmem + kColO, tmem + kColPB + uint32_t(kk * 8), vlb + adv, kIdescBf, 1u);
                            }
                        }
                        umma_commit(&s.bar_o);
                        if (next_blk >= 0) {  // V buffer is free once the P·V MMAs have completed
                            if (!mbar_wait(&s.bar_o, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnO); break; }
                            load_v(next_blk);
                        }
                    }
                }
            }
        } else {
            // ---------------- operand split: the "lo" twins of every landed K / V block ----------------
            const int t = threadIdx.x - kSplitWarp0 * 32, nt = kSplitWarps * 32;
            for (int i = 0; i < n_act; i++) {
                const uint32_t par = i & 1;
                if (!mbar_wait(&s.bar_k, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnK); break; }
                split_tile_bf16(s.k_hi[0], s.k_bf, s.k_lo_bf, t, nt);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.bar_ks);
                if (!mbar_wait(&s.bar_v, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnV); break; }
                split_tile_bf16(s.v_hi[0], s.v_bf, s.v_lo_bf, t, nt);
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.bar_vs);
            }
        }
    } else {
        // ---------------- softmax: two threads per query row ----------------
        attn_reg_inc<kRegsSoft>();
        const int sw = warp - kSoftWarp0;          // 0..7
        const int quarter = sw & 3, half = sw >> 2;
        const int row = quarter * 32 + lane, qi = q0 + row;
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        const bool row_ok = qi < T;
        const uint8_t* mhead = p.mask + int64_t(b) * p.mask_sb + int64_t(h) * p.mask_sh;
        bool alive = true;   // a thread that gave up keeps walking the loop so that soft_sync() stays matched
        if (n_act > 0) {
            // ---- bf16(q_lo) and bf16(q) of this thread's row of Q (head columns [32*half, 32*half + 32)) go into tensor memory,
            //      two elements per column (element k in the low half of word k/2) ----
            if (!mbar_wait(&s.bar_q, 0, abort_flag)) { give_up(abort_flag, p.status, kErrAttnQ); alive = false; }
            if (alive) {
                const float4* src = reinterpret_cast<const float4*>(s.q_hi[half]) + row * 8;   // 128-byte rows, 16-byte chunks XOR-swizzled by row % 8
                const int swz = row & 7;
                uint32_t ql[16], qx[16];
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const float4 v = src[c ^ swz];
                    ql[2 * c + 0] = pack_bf16x2(lo_of_truncated(v.x), lo_of_truncated(v.y));
                    ql[2 * c + 1] = pack_bf16x2(lo_of_truncated(v.z), lo_of_truncated(v.w));
                    qx[2 * c + 0] = pack_bf16x2(v.x, v.y);
                    qx[2 * c + 1] = pack_bf16x2(v.z, v.w);
                }
                tmem_st16(tmem + kColQloB + lane_base + uint32_t(half * 16), ql);
                tmem_st16(tmem + kColQB + lane_base + uint32_t(half * 16), qx);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.bar_qs);
            }
        }
        float o[32];
#pragma unroll
        for (int j = 0; j < 32; j++) o[j] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;

        unsigned long long rem = need;
        for (int i = 0; i < n_act; i++) {
            const int blk = __ffsll(rem) - 1;
            rem &= rem - 1;
            const uint32_t par = i & 1;
            // ---- stage this warp's share of the mask: rows of its quarter, the 32 keys of its half ----
            const int key0 = blk * BKEY + half * 32;
            if (p.mask_vec16) {
#pragma unroll
                for (int it = 0; it < 2; it++) {
                    const int rr = quarter * 32 + it * 16 + (lane >> 1), kq = key0 + (lane & 1) * 16, qq = q0 + rr;
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (qq < T && kq < Tk) v = *reinterpret_cast<const uint4*>(mhead + int64_t(qq) * p.mask_sq + kq);
                    *reinterpret_cast<uint4*>(s.mask_rows + rr * kMaskPitch + half * 32 + (lane & 1) * 16) = v;
                }
            } else {
                for (int idx = lane; idx < 32 * 32; idx += 32) {
                    const int rr = quarter * 32 + (idx >> 5), kc = key0 + (idx & 31), qq = q0 + rr;
                    unsigned char v = 0;
                    if (qq < T && kc < Tk) v = mhead[int64_t(qq) * p.mask_sq + int64_t(kc) * p.mask_sk];
                    s.mask_rows[rr * kMaskPitch + half * 32 + (idx & 31)] = v;
                }
            }
            __syncwarp();
            uint32_t keep = 0;
            {
                const uint4* mp = reinterpret_cast<const uint4*>(s.mask_rows + row * kMaskPitch + half * 32);
#pragma unroll
                for (int w = 0; w < 2; w++) {
                    const uint4 m16 = mp[w];
                    const uint32_t words[4] = {m16.x, m16.y, m16.z, m16.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        // 0x01 per non-zero byte, gathered into 4 bits by one multiply
                        const uint32_t nz = __vcmpne4(words[k], 0u) & 0x01010101u;
                        keep |= ((nz * 0x01020408u) >> 24 & 0xFu) << (16 * w + 4 * k);
                    }
                }
            }
            __syncwarp();
            // ---- pass 1: scale, mask, log2 domain, partial row maximum; processed scores go back to TMEM ----
            if (alive && !mbar_wait(&s.bar_s, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnS); alive = false; }
            float tmax = -INFINITY;
            const uint32_t scol = tmem + kColS + lane_base + uint32_t(half * 32);
            if (alive) {
                tc_fence_after();
                uint32_t r[32];
                tmem_ld32(scol, r);
                tmem_wait_ld();
                if (p.scale_is_pow2) {
                    // v / 2^k * log2(e) == v * (2^-k * log2(e)) bit for bit: the first factor only shifts the exponent
                    const float cmul = p.inv_scale * kLog2e;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float v = ((keep >> j) & 1u) ? __uint_as_float(r[j]) * cmul : -INFINITY;
                        tmax = fmaxf(tmax, v);  // NaN scores do not move the max; they reach the sum below
                        r[j] = __float_as_uint(v);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float v = __uint_as_float(r[j]) / p.scale_divisor;
                        v = ((keep >> j) & 1u) ? v * kLog2e : -INFINITY;
                        tmax = fmaxf(tmax, v);
                        r[j] = __float_as_uint(v);
                    }
                }
                tmem_st32(scol, r);
                tmem_wait_st();
            }
            s.exch[half][row] = tmax;
            soft_sync(quarter);
            const float m_new = fmaxf(m_run, fmaxf(tmax, s.exch[half ^ 1][row]));
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = fast_exp2(m_run - m_safe);
            // ---- pass 2: probabilities, their partial sum, hi/lo halves into TMEM (P_hi over the scores), 16 keys at a time ----
            float psum = 0.f;
            if (alive) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t r[16], pl[8], px[8];
                    tmem_ld16(scol + uint32_t(c * 16), r);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float p0 = fast_exp2(__uint_as_float(r[j]) - m_safe), p1 = fast_exp2(__uint_as_float(r[j + 1]) - m_safe);
                        psum += p0;
                        psum += p1;
                        // P_hi = p as it is (the TF32 MMA reads only its upper 19 bits); the corrections take bf16(p_lo), the 13
                        // bits it does not see, and bf16(p)
                        r[j] = __float_as_uint(p0);
                        r[j + 1] = __float_as_uint(p1);
                        pl[j >> 1] = pack_bf16x2(lo_of_truncated(p0), lo_of_truncated(p1));
                        px[j >> 1] = pack_bf16x2(p0, p1);
                    }
                    tmem_st16(scol + uint32_t(c * 16), r);
                    tmem_st8(tmem + kColPloB + lane_base + uint32_t(half * 16 + c * 8), pl);
                    tmem_st8(tmem + kColPB + lane_base + uint32_t(half * 16 + c * 8), px);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.bar_p);
            }
            l_run = l_run * alpha + psum;   // this thread's share of the row sum; the two shares are added at the end
            m_run = m_new;
#pragma unroll
            for (int j = 0; j < 32; j++) o[j] *= alpha;
            if (alive && !mbar_wait(&s.bar_o, par, abort_flag)) { give_up(abort_flag, p.status, kErrAttnO); alive = false; }
            if (alive) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t r[16];
                    tmem_ld16(tmem + kColO + lane_base + uint32_t(half * 32 + c * 16), r);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; j++) o[c * 16 + j] += __uint_as_float(r[j]);
                }
                tc_fence_before();
            }
            soft_sync(quarter);   // exch[] is reused by the next block (and by the final sum exchange)
        }
        s.exch[half][row] = l_run;
        soft_sync(quarter);
        const float l_tot = s.exch[0][row] + s.exch[1][row];
        if (alive && row_ok) {
            // one reciprocal per row instead of 32 divisions; a fully masked row has o = 0 and l = 0: 0 * inf = NaN, as the
            // reference softmax gives
            const float inv_l = 1.0f / l_tot;
            float* dst = p.ctx + (int64_t(b) * T + qi) * p.ld_ctx + int64_t(h) * HD + half * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(o[j] * inv_l, o[j + 1] * inv_l, o[j + 2] * inv_l, o[j + 3] * inv_l);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return EncodeTiledFn(nullptr);
    }();
    return fn;
}
// fp32 tensor seen as [n2, n1, n0] with n0 contiguous and byte strides s1 (dim 1), s2 (dim 2);
// box [1, box1, 32 floats], 128-byte swizzle, zero fill outside.
int make_map3(CUtensorMap* map, const float* base, int64_t n0, int64_t n1, int64_t n2, int64_t s1, int64_t s2, int box1) {
    EncodeTiledFn fn = encode_fn();
    FXF_CHECK(fn != nullptr, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cuuint64_t dims[3] = {cuuint64_t(n0), cuuint64_t(n1), cuuint64_t(n2)};
    cuuint64_t strides[2] = {cuuint64_t(s1), cuuint64_t(s2)};
    cuuint32_t box[3] = {32, cuuint32_t(box1), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FXF_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (attention) failed with code %d", int(r));
    return 0;
}

}  // namespace

bool attention_tc_supported(const AttnArgs& a, int gemm_mode) {
    if (gemm_mode == FXF_GEMM_FP32_SIMT) return false;
    const int Tk = a.kv ? a.Tk : a.T;
    if (a.hd != HD || Tk % 4 != 0 || Tk < 16 || a.T < 1) return false;   // V^T rows (Tk floats) must be 16-byte multiples
    if ((Tk + BKEY - 1) / BKEY > 64) return false;   // the kernel tracks its key blocks in one 64-bit word: at most 4096 keys
    if (a.ld_qkv % 4 != 0 || a.ld_ctx % 4 != 0 || (a.q_off | a.k_off | a.v_off) % 4 != 0) return false;
    if (a.kv && (a.ld_kv % 4 != 0 || !aligned16(a.kv))) return false;
    if (!aligned16(a.qkv) || !aligned16(a.ctx)) return false;
    return true;
}

// V^T [B*H, 64, T] followed by one "non-finite" byte per (batch*head, column half of the head, 32-key slab)
size_t attention_tc_scratch_bytes(int64_t B, int64_t T, int64_t H) {
    return size_t(B) * size_t(T) * size_t(H) * HD * sizeof(float) + round_up(size_t(2) * size_t(B) * size_t(H) * size_t((T + 31) / 32), 256);
}

int launch_attention_tc(const AttnArgs& a, float* vt_scratch, ExecCtx& ctx, bool v_transposed) {
    FXF_CHECK(vt_scratch != nullptr && aligned16(vt_scratch), "attention: tensor-core path needs its V^T buffer");
    const int64_t BH = int64_t(a.B) * a.H;
    const int Tk = a.kv ? a.Tk : a.T;                     // keys per batch
    const float* kvp = a.kv ? a.kv : a.qkv;               // where K and V live
    const int64_t ldk = a.kv ? a.ld_kv : a.ld_qkv;
    const int n32 = (Tk + 31) / 32;
    dim3 pgrid(unsigned((Tk + 63) / 64), unsigned(BH));
    unsigned char* vflags = reinterpret_cast<unsigned char*>(vt_scratch + size_t(BH) * size_t(Tk) * HD);
    if (!v_transposed) {   // otherwise the projection's epilogue has written V^T and the flags already
        tag_launch(ctx, "attention_v_transpose", 0, 8.0 * double(BH) * Tk * HD);
        attn_vt_kernel<<<pgrid, 256, 0, ctx.stream>>>(kvp, ldk, a.v_off, Tk, a.H, vt_scratch, vflags, n32);
        FXF_LAUNCHED(ctx);
    }

    CUtensorMap mq, mk, mv;
    // Q and K tiles come straight out of the packed projection: [B, T, ld] with the row pitch of qkv
    if (make_map3(&mq, a.qkv, a.ld_qkv, a.T, a.B, a.ld_qkv * 4, int64_t(a.T) * a.ld_qkv * 4, BQ)) return 1;
    if (make_map3(&mk, kvp, ldk, Tk, a.B, ldk * 4, int64_t(Tk) * ldk * 4, BKEY)) return 1;
    if (make_map3(&mv, vt_scratch, Tk, HD, BH, int64_t(Tk) * 4, int64_t(Tk) * HD * 4, HD)) return 1;
    AttnTcParams p;
    p.vflags = vflags; p.n32 = int((Tk + 31) / 32);
    p.mask = a.mask; p.ctx = a.ctx; p.B = a.B; p.T = a.T; p.Tk = Tk; p.H = a.H; p.ld_ctx = a.ld_ctx;
    p.q_col = int(a.q_off); p.k_col = int(a.k_off);
    p.mask_sb = a.mask_sb; p.mask_sh = a.mask_sh; p.mask_sq = a.mask_sq; p.mask_sk = a.mask_sk;
    p.scale_divisor = a.scale_divisor;
    {
        int e = 0;
        float m = std::frexp(a.scale_divisor, &e);
        p.scale_is_pow2 = (m == 0.5f && a.scale_divisor > 0.f && std::isfinite(a.scale_divisor)) ? 1 : 0;
        p.inv_scale = p.scale_is_pow2 ? 1.0f / a.scale_divisor : 0.f;
    }
    p.mask_vec16 = (a.mask_sk == 1 && Tk % 16 == 0 && a.mask_sb % 16 == 0 && a.mask_sh % 16 == 0 && a.mask_sq % 16 == 0 && aligned16(a.mask)) ? 1 : 0;
    p.status = ctx.status;
    size_t smem = sizeof(AttnTcSmem) + 1024;
    static bool configured[64] = {};
    int dev = 0;
    FXF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        FXF_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        FXF_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, int(cudaSharedmemCarveoutMaxShared)));   // room for two CTAs
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    dim3 grid(unsigned((a.T + BQ - 1) / BQ), unsigned(BH));
    tag_launch(ctx, "attention_tf32_bf16x2_tcgen05", 4.0 * double(a.B) * a.H * double(a.T) * Tk * a.hd,
               4.0 * 2.0 * double(a.B) * (double(a.T) + Tk) * double(a.H) * a.hd + double(a.B) * a.T * Tk);
    attn_tc_kernel<<<grid, kAttnThreads, smem, ctx.stream>>>(mq, mk, mv, p);
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace fxf
