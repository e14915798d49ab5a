// Fused attention core: ctx = softmax(mask_fill(Q·K^T / scale_divisor)) · V, per (batch, head).
//
// Reference semantics (csrc/kernels/cpu/mha.cpp:38-49): scores are DIVIDED by
// scale_divisor, positions where mask == 0 become -inf, softmax over keys, then P·V, and the
// heads are re-interleaved into [B,T,D].  Consequences that this kernel reproduces without
// special cases:
//   * a query row whose keys are all masked yields NaN (exp(-inf - -inf)); here l = 0 and
//     0/0 = NaN at the final normalisation;
//   * masked keys still take part in P·V with weight 0, so a NaN in V poisons the row
//     (0 * NaN = NaN) exactly as torch::matmul does — no key tile is ever skipped, the
//     mask being run-time data;
//   * an unmasked NaN score makes the whole row NaN (expf(NaN) feeds the row sum).
//
// Layout: Q, K, V are column blocks of the packed projection qkv[B*T, ld] (head h at columns
// h*hd..), the mask is addressed through byte strides so [B,1,T,T], [B,1,1,T] and [1,1,T,T]
// all work, ctx is [B*T, ld_ctx] with head h at columns h*hd.
//
// One CTA = 64 query rows of one (b,h); keys are streamed in tiles of 64 with the online
// softmax recurrence (running max m, running sum l, rescale factor alpha), so the [T,T] score
// matrix never exists in memory.  256 threads as 16x16; each thread owns a 4x4 patch of the
// score tile and a 4 x (HD/16) patch of the output.  fp32 FFMA throughout.
#include <cmath>

#include "../runtime.hpp"

namespace fxf {
namespace {

constexpr int kBQ = 64, kBK = 64, kPad = 4;

template <int HD>
struct AttnSmem {
    float q[HD][kBQ + kPad];   // Q tile, transposed: [d][row]
    float k[HD][kBK + kPad];   // K tile, transposed: [d][key]
    float v[kBK][HD + kPad];   // V tile: [key][d]
    float p[kBK][kBQ + kPad];  // probabilities, transposed: [key][row]
};

template <int HD>
__global__ void __launch_bounds__(256) attention_kernel(AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    AttnSmem<HD>& s = *reinterpret_cast<AttnSmem<HD>*>(smem_raw);
    constexpr int TNO = HD / 16;  // output columns per thread
    constexpr int DQ = HD / 4;    // float4s per row of a tile

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int q0 = blockIdx.x * kBQ;
    const int T = a.T, hd = a.hd;                      // T = number of queries per batch
    const int Tk = a.kv ? a.Tk : a.T;                   // number of keys per batch
    const float* kvp = a.kv ? a.kv : a.qkv;
    const int64_t ldk = a.kv ? a.ld_kv : a.ld_qkv;
    const bool vec = (hd % 4 == 0) && (a.ld_qkv % 4 == 0) && (ldk % 4 == 0) && ((a.q_off | a.k_off | a.v_off) % 4 == 0);

    const float* qbase = a.qkv + int64_t(b) * T * a.ld_qkv + a.q_off + int64_t(h) * hd;
    const float* kbase = kvp + int64_t(b) * Tk * ldk + a.k_off + int64_t(h) * hd;
    const float* vbase = kvp + int64_t(b) * Tk * ldk + a.v_off + int64_t(h) * hd;

    auto load_row4 = [&](const float* base, int64_t ld, int rows, int row, int d4) -> float4 {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        int d = d4 * 4;
        if (row < rows && d < hd) {
            const float* p = base + int64_t(row) * ld + d;
            if (vec) {
                v = *reinterpret_cast<const float4*>(p);
            } else {
                v.x = p[0];
                if (d + 1 < hd) v.y = p[1];
                if (d + 2 < hd) v.z = p[2];
                if (d + 3 < hd) v.w = p[3];
            }
        }
        return v;
    };

    // Q tile (zero-padded beyond T rows / hd columns)
    for (int f = tid; f < kBQ * DQ; f += 256) {
        int r = f / DQ, d4 = f % DQ;
        float4 v = load_row4(qbase, a.ld_qkv, T, q0 + r, d4);
        s.q[d4 * 4 + 0][r] = v.x; s.q[d4 * 4 + 1][r] = v.y; s.q[d4 * 4 + 2][r] = v.z; s.q[d4 * 4 + 3][r] = v.w;
    }

    float o[4][TNO];
    float m_run[4], l_run[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int j = 0; j < TNO; j++) o[i][j] = 0.f;
    }

    const uint8_t* mbase = a.mask + int64_t(b) * a.mask_sb + int64_t(h) * a.mask_sh;

    for (int k0 = 0; k0 < Tk; k0 += kBK) {
        __syncthreads();  // previous tile fully consumed (also orders the Q stores on the first pass)
        for (int f = tid; f < kBK * DQ; f += 256) {
            int r = f / DQ, d4 = f % DQ;
            float4 kv = load_row4(kbase, ldk, Tk, k0 + r, d4);
            s.k[d4 * 4 + 0][r] = kv.x; s.k[d4 * 4 + 1][r] = kv.y; s.k[d4 * 4 + 2][r] = kv.z; s.k[d4 * 4 + 3][r] = kv.w;
            float4 vv = load_row4(vbase, ldk, Tk, k0 + r, d4);
            *reinterpret_cast<float4*>(&s.v[r][d4 * 4]) = vv;
        }
        __syncthreads();

        // S patch = Q · K^T
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) sc[i][j] = 0.f;
#pragma unroll 8
        for (int d = 0; d < HD; d++) {
            float4 qa = *reinterpret_cast<const float4*>(&s.q[d][ty * 4]);
            float4 kb = *reinterpret_cast<const float4*>(&s.k[d][tx * 4]);
            float qv[4] = {qa.x, qa.y, qa.z, qa.w}, kv[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) sc[i][j] = fmaf(qv[i], kv[j], sc[i][j]);
        }

        // scale, mask, online softmax
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int qr = q0 + ty * 4 + i;
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int kc = k0 + tx * 4 + j;
                float v = sc[i][j] / a.scale_divisor;
                bool keep = false;
                if (kc < Tk && qr < T) keep = mbase[int64_t(qr) * a.mask_sq + int64_t(kc) * a.mask_sk] != 0;
                v = keep ? v : -INFINITY;
                sc[i][j] = v;
                tmax = fmaxf(tmax, v);  // NaN scores do not move the max; they reach the sum below
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
            float m_new = fmaxf(m_run[i], tmax);
            float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            float alpha = expf(m_run[i] - m_safe);
            float psum = 0.f;
            float pv[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                pv[j] = expf(sc[i][j] - m_safe);
                psum += pv[j];
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
            l_run[i] = l_run[i] * alpha + psum;
            m_run[i] = m_new;
#pragma unroll
            for (int j = 0; j < TNO; j++) o[i][j] *= alpha;
#pragma unroll
            for (int j = 0; j < 4; j++) s.p[tx * 4 + j][ty * 4 + i] = pv[j];
        }
        __syncthreads();

        // O patch += P · V
#pragma unroll 8
        for (int kk = 0; kk < kBK; kk++) {
            float4 pa = *reinterpret_cast<const float4*>(&s.p[kk][ty * 4]);
            float pr[4] = {pa.x, pa.y, pa.z, pa.w};
            float vv[TNO];
#pragma unroll
            for (int j = 0; j < TNO; j++) vv[j] = s.v[kk][tx * TNO + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < TNO; j++) o[i][j] = fmaf(pr[i], vv[j], o[i][j]);
        }
    }

    // normalise and store (0/0 = NaN for a fully masked row, as the reference softmax gives)
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int qr = q0 + ty * 4 + i;
        if (qr >= T) continue;
        float* dst = a.ctx + (int64_t(b) * T + qr) * a.ld_ctx + int64_t(h) * hd;
#pragma unroll
        for (int j = 0; j < TNO; j++) {
            int d = tx * TNO + j;
            if (d < hd) dst[d] = o[i][j] / l_run[i];
        }
    }
}

template <int HD>
int launch_hd(const AttnArgs& a, ExecCtx& ctx) {
    size_t smem = sizeof(AttnSmem<HD>);
    FXF_CUDA(cudaFuncSetAttribute(attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    dim3 grid(unsigned((a.T + kBQ - 1) / kBQ), unsigned(a.B * a.H));
    attention_kernel<HD><<<grid, 256, smem, ctx.stream>>>(a);
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace

int launch_attention(const AttnArgs& a, ExecCtx& ctx) {
    if (a.B == 0 || a.T == 0 || a.H == 0) return 0;
    FXF_CHECK(a.hd >= 1 && a.hd <= 128, "mha: head_dim %d is outside the supported range 1..128", a.hd);
    const double tk = a.kv ? a.Tk : a.T;
    tag_launch(ctx, "attention_fp32_flash", 4.0 * double(a.B) * a.H * double(a.T) * tk * a.hd,
               4.0 * 2.0 * double(a.B) * (double(a.T) + tk) * double(a.H) * a.hd + double(a.B) * a.T * tk);
    if (a.hd <= 16) return launch_hd<16>(a, ctx);
    if (a.hd <= 32) return launch_hd<32>(a, ctx);
    if (a.hd <= 64) return launch_hd<64>(a, ctx);
    return launch_hd<128>(a, ctx);
}

}  // namespace fxf
