// Conv2d / Conv2dRelu (BatchNorm already folded into weight and bias by the compile side) and
// the window-pooling ops.  The graph contract is NCHW float32; between layout-aware nodes the engine may
// keep activations channels-last (NHWC), which it states through the registry strides, so every kernel
// here addresses its tensors through (n, c, h, w) strides and is correct for either layout.
//
// Reference semantics (LibTorch calls):
//   conv2d / conv2d_relu  csrc/kernels/cpu/conv2d.cpp:5-17, conv2d_relu.cpp:5-17
//       ints = [sh, sw, ph, pw, dh, dw, groups, <6 unused launch placeholders>]
//   max_pool2d            csrc/kernels/cpu/max_pool2d.cpp:5-16
//       ints = [kh, kw, sh, sw, ph, pw, dh, dw, ceil_mode, ...]; padding counts as -inf, NaN wins
//   avg_pool2d            csrc/kernels/cpu/avg_pool2d.cpp:5-15
//       ints = [kh, kw, sh, sw, ph, pw, ceil_mode, ...]; count_include_pad = true, the divisor is
//       the window clipped to the padded extent
//   adaptive_avg_pool2d   csrc/kernels/cpu/adaptive_avg_pool2d.cpp:5-12
//       ints = [oh, ow, ...]; window i = [floor(i*H/oh), ceil((i+1)*H/oh))
//
// Convolution paths:
//   * 1x1, stride 1, no padding, channels-last in and out: the convolution IS the GEMM
//     out[pixel, o] = x[pixel, :] · w[o, :] + b[o]  — it runs on the tcgen05 3xTF32 GEMM kernel with the bias
//     and ReLU fused in its epilogue (weights split into TF32 hi/lo once, at engine build).
//   * everything else: an implicit GEMM (rows = output pixels n*Ho*Wo, columns = output channels, depth =
//     Cin/groups*Kh*Kw) on fp32 FFMA tiles of 64x64x16 with the im2col gather done while the A tile is staged.
#include <cfloat>
#include <cmath>

#include "../runtime.hpp"

namespace fxf {
namespace {

struct Strides4 {
    int64_t n, c, h, w;
};
inline Strides4 strides_of(const FxfTensor& t) {  // rank 3 ([C,H,W]) or 4
    if (t.rank == 4) return {t.stride[0], t.stride[1], t.stride[2], t.stride[3]};
    return {0, t.stride[0], t.stride[1], t.stride[2]};
}

struct ConvDesc {
    int N, C, H, W, O, KH, KW, HO, WO;
    int sh, sw, ph, pw, dh, dw, groups;
    int cg, og;   // channels / outputs per group
    int relu;
    Strides4 xs, os;
};

constexpr int CBM = 64, CBN = 64, CBK = 16;

__global__ void __launch_bounds__(256) conv2d_igemm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                           float* __restrict__ out, ConvDesc d) {
    __shared__ __align__(16) float As[CBK][CBM + 4];
    __shared__ __align__(16) float Bs[CBK][CBN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;  // tx -> pixels, ty -> channels
    const int g = blockIdx.z;
    const int64_t pix0 = int64_t(blockIdx.x) * CBM;
    const int oc0 = blockIdx.y * CBN;  // within group
    const int64_t n_pix = int64_t(d.N) * d.HO * d.WO;
    const int Kdepth = d.cg * d.KH * d.KW;

    // A staging: thread loads 4 (pixel, k) pairs: pixel = tid % 64, k = tid / 64 + 4*i
    const int a_pix = tid & 63, a_k0 = tid >> 6;
    int64_t gp = pix0 + a_pix;
    int pn = 0, py = 0, px = 0;
    bool pvalid = gp < n_pix;
    if (pvalid) {
        px = int(gp % d.WO);
        int64_t t = gp / d.WO;
        py = int(t % d.HO);
        pn = int(t / d.HO);
    }
    // B staging: weight row (oc) x 16 k-values; thread loads 4: oc = tid / 4, k = (tid % 4) * 4 + i
    const int b_oc = tid >> 2, b_k0 = (tid & 3) * 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < Kdepth; k0 += CBK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int k = k0 + a_k0 + 4 * i;
            float v = 0.f;
            if (pvalid && k < Kdepth) {
                int kw = k % d.KW;
                int t = k / d.KW;
                int kh = t % d.KH;
                int c = t / d.KH;
                int iy = py * d.sh - d.ph + kh * d.dh, ix = px * d.sw - d.pw + kw * d.dw;
                if (iy >= 0 && iy < d.H && ix >= 0 && ix < d.W)
                    v = x[int64_t(pn) * d.xs.n + int64_t(g * d.cg + c) * d.xs.c + int64_t(iy) * d.xs.h + int64_t(ix) * d.xs.w];
            }
            As[a_k0 + 4 * i][a_pix] = v;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int k = k0 + b_k0 + i, oc = oc0 + b_oc;
            float v = 0.f;
            if (oc < d.og && k < Kdepth) v = w[(int64_t(g) * d.og + oc) * Kdepth + k];
            Bs[b_k0 + i][b_oc] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < CBK; k++) {
            float4 av = *reinterpret_cast<const float4*>(&As[k][tx * 4]);
            float4 bv = *reinterpret_cast<const float4*>(&Bs[k][ty * 4]);
            float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int64_t p = pix0 + tx * 4 + i;
        if (p >= n_pix) continue;
        int ox = int(p % d.WO);
        int64_t t = p / d.WO;
        int oy = int(t % d.HO), n = int(t / d.HO);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int oc = oc0 + ty * 4 + j;
            if (oc >= d.og) continue;
            int o = g * d.og + oc;
            float v = acc[i][j] + bias[o];
            if (d.relu) v = v > 0.f ? v : (v != v ? v : 0.f);
            out[int64_t(n) * d.os.n + int64_t(o) * d.os.c + int64_t(oy) * d.os.h + int64_t(ox) * d.os.w] = v;
        }
    }
}

// ---- pools ----------------------------------------------------------------------------------------
struct PoolDesc {
    int64_t N;
    int C, H, W, HO, WO, kh, kw, sh, sw, ph, pw, dh, dw;
    Strides4 xs, os;
    int cl;  // walk the output channels-fastest (channels-last tensors) instead of width-fastest
};

__device__ __forceinline__ void pool_coords(const PoolDesc& d, int64_t i, int64_t& n, int& c, int& oy, int& ox) {
    if (d.cl) {
        c = int(i % d.C); i /= d.C;
        ox = int(i % d.WO); i /= d.WO;
        oy = int(i % d.HO);
        n = i / d.HO;
    } else {
        ox = int(i % d.WO); i /= d.WO;
        oy = int(i % d.HO); i /= d.HO;
        c = int(i % d.C);
        n = i / d.C;
    }
}

enum PoolOp { kMaxPool = 0, kAvgPool = 1, kAdaptiveAvg = 2 };

template <int OP>
__global__ void __launch_bounds__(256) pool2d_kernel(const float* __restrict__ x, float* __restrict__ out, PoolDesc d) {
    int64_t total = d.N * d.C * d.HO * d.WO, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t n;
        int c, oy, ox;
        pool_coords(d, i, n, c, oy, ox);
        const float* src = x + n * d.xs.n + int64_t(c) * d.xs.c;
        float r;
        if (OP == kMaxPool) {
            float m = -INFINITY;
            for (int a = 0; a < d.kh; a++) {
                int iy = oy * d.sh - d.ph + a * d.dh;
                if (iy < 0 || iy >= d.H) continue;
                for (int b = 0; b < d.kw; b++) {
                    int ix = ox * d.sw - d.pw + b * d.dw;
                    if (ix < 0 || ix >= d.W) continue;
                    float v = src[int64_t(iy) * d.xs.h + int64_t(ix) * d.xs.w];
                    if (v > m || v != v) m = v;
                }
            }
            r = m;
        } else {
            int hs, he, ws, we, count;
            if (OP == kAvgPool) {
                hs = oy * d.sh - d.ph; ws = ox * d.sw - d.pw;
                he = min(hs + d.kh, d.H + d.ph); we = min(ws + d.kw, d.W + d.pw);
                count = (he - hs) * (we - ws);  // count_include_pad
                hs = max(hs, 0); ws = max(ws, 0); he = min(he, d.H); we = min(we, d.W);
            } else {
                hs = int((int64_t(oy) * d.H) / d.HO); he = int((int64_t(oy + 1) * d.H + d.HO - 1) / d.HO);
                ws = int((int64_t(ox) * d.W) / d.WO); we = int((int64_t(ox + 1) * d.W + d.WO - 1) / d.WO);
                count = (he - hs) * (we - ws);
            }
            float s = 0.f;
            for (int iy = hs; iy < he; iy++)
                for (int ix = ws; ix < we; ix++) s += src[int64_t(iy) * d.xs.h + int64_t(ix) * d.xs.w];
            r = s / float(count);
        }
        out[n * d.os.n + int64_t(c) * d.os.c + int64_t(oy) * d.os.h + int64_t(ox) * d.os.w] = r;
    }
}

// Global average of a row-major plane (output 1x1, NCHW input): one warp per (n,c) plane.
__global__ void __launch_bounds__(256) global_avg_pool_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t NC, int HW) {
    int lane = threadIdx.x & 31;
    int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5, nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t p = warp; p < NC; p += nwarps) {
        const float* src = x + p * HW;
        float s = 0.f;
        for (int i = lane; i < HW; i += 32) s += src[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) out[p] = s / float(HW);
    }
}

// ---- stem convolutions (few input channels, stride 2) as a stride-1 convolution over a space-to-depth copy ----------
// A k x k stride-2 convolution over C <= 4 channels cannot feed the tensor-core path (16-channel K slabs).  Rearranging
// the zero-padded input P into S[n, Y, X, (ry*2 + rx)*C + c] = P[n, c, 2Y + ry, 2X + rx] (16 channels, the unused ones
// zero) turns it into a stride-1, unpadded ceil(k/2) x ceil(k/2) convolution over 16 channels with the filters
// rearranged the same way (taps beyond k are zero): out[oy, ox] = sum_{qy,qx,ch} S[oy+qy, ox+qx, ch] * W'[o, qy, qx, ch].
__global__ void __launch_bounds__(256) space_to_depth16_kernel(const float* __restrict__ x, float4* __restrict__ s, int64_t N, int C, int H, int W, int Hs, int Ws,
                                                               int ph, int pw, Strides4 xs) {
    const int64_t total = N * Hs * Ws * 4, stride = int64_t(gridDim.x) * blockDim.x;   // one float4 = 4 of the 16 channels
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int g = int(i & 3);
        int64_t t = i >> 2;
        const int X = int(t % Ws); t /= Ws;
        const int Y = int(t % Hs);
        const int64_t n = t / Hs;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int ch = g * 4 + j, r = ch / C, c = ch - r * C;   // r = ry*2 + rx
            float val = 0.f;
            if (r < 4) {
                const int iy = 2 * Y + (r >> 1) - ph, ix = 2 * X + (r & 1) - pw;
                if (iy >= 0 && iy < H && ix >= 0 && ix < W) val = x[n * xs.n + int64_t(c) * xs.c + int64_t(iy) * xs.h + int64_t(ix) * xs.w];
            }
            v[j] = val;
        }
        s[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// filters OIHW [O, C, KH, KW] -> [O, KH2, KW2, 16] in the space-to-depth channel order, split into TF32 hi / lo
__global__ void __launch_bounds__(256) conv_weight_s2d_split_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int O, int C, int KH,
                                                                    int KW, int KH2, int KW2) {
    const int64_t total = int64_t(O) * KH2 * KW2 * 16, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int ch = int(i & 15);
        int64_t t = i >> 4;
        const int qx = int(t % KW2); t /= KW2;
        const int qy = int(t % KH2);
        const int o = int(t / KH2);
        const int r = ch / C, c = ch - r * C;
        float val = 0.f;
        if (r < 4) {
            const int ky = 2 * qy + (r >> 1), kx = 2 * qx + (r & 1);
            if (ky < KH && kx < KW) val = w[((int64_t(o) * C + c) * KH + ky) * KW + kx];
        }
        const float h = __uint_as_float(__float_as_uint(val) & 0xffffe000u);   // what a TF32 MMA sees of an fp32 operand
        uint32_t lbits;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lbits) : "f"(val - h));
        hi[i] = val;    // the MMA truncates it itself
        lo[i] = __uint_as_float(lbits);
    }
}

// ---- host side ----------------------------------------------------------------------------------------
struct ConvPlan : NodePlan {
    bool gemm_1x1 = false;          // planned for the tensor-core GEMM (still needs channels-last tensors at run time)
    bool bf16 = false;              // bf16 mode: one bf16 copy of the weights instead of the TF32 hi/lo pair
    bool igemm_tc = false;          // k x k or strided 1x1, stride <= 2: planned for the tensor-core implicit GEMM (same run-time condition)
    bool s2d_tc = false;            // <= 4 input channels, stride 2: space-to-depth copy, then a stride-1 tensor-core convolution
    int Hs = 0, Ws = 0, KH2 = 0, KW2 = 0;
    int64_t w_elems = 0;
    const float *w_hi = nullptr, *w_lo = nullptr;
    int prepare(Registry& reg, const TensorIds& in, const TensorIds&, const Params&, ExecCtx& ctx) override {
        if (!gemm_1x1 && !igemm_tc && !s2d_tc) return 0;
        FXF_CHECK(persist != nullptr, "conv plan: persistent memory was not assigned");
        float* h = static_cast<float*>(persist);
        const FxfTensor& w = reg[in[1]];
        if (s2d_tc) {
            const int64_t blocks = (w_elems + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
            tag_launch(ctx, "conv_weight_s2d_split", 0, 12.0 * double(w_elems));
            conv_weight_s2d_split_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(static_cast<const float*>(w.ptr), h, h + w_elems, int(w.shape[0]),
                                                                                                   int(w.shape[1]), int(w.shape[2]), int(w.shape[3]), KH2, KW2);
            FXF_LAUNCHED(ctx);
            w_hi = h;
            w_lo = h + w_elems;
            return 0;
        }
        if (bf16) {
            if (igemm_tc) {
                if (launch_conv_weight_bf16(static_cast<const float*>(w.ptr), h, int(w.shape[0]), int(w.shape[1]), int(w.shape[2]), int(w.shape[3]), ctx)) return 1;
            } else if (launch_convert_bf16(static_cast<const float*>(w.ptr), h, w_elems, ctx)) return 1;
            w_hi = h;
            w_lo = nullptr;
            return 0;
        }
        if (igemm_tc) {
            if (launch_conv_weight_split(static_cast<const float*>(w.ptr), h, h + w_elems, int(w.shape[0]), int(w.shape[1]), int(w.shape[2]), int(w.shape[3]), ctx)) return 1;
        } else if (launch_split_tf32(static_cast<const float*>(w.ptr), h, h + w_elems, w_elems, ctx)) return 1;
        w_hi = h;
        w_lo = h + w_elems;
        return 0;
    }
};

// dense [N*H*W, C] view of a 4-D tensor: channels-last, or any layout when H*W == 1 / C == 1
bool pixel_major(const FxfTensor& t) { return t.rank == 4 && (is_channels_last(t) || (is_contiguous(t) && (t.shape[2] * t.shape[3] == 1 || t.shape[1] == 1))); }

int conv_desc(const FxfTensor& x, const FxfTensor& w, const FxfTensor& b, const FxfTensor& o, const Params& p, ConvDesc* d, const char* who) {
    FXF_CHECK(x.dtype == FXF_F32 && w.dtype == FXF_F32 && o.dtype == FXF_F32, "%s: only float32 is supported", who);
    FXF_CHECK(x.rank == 4 && w.rank == 4 && o.rank == 4, "%s: x, weight and output must be 4-D (NCHW / OIHW)", who);
    FXF_CHECK(is_contiguous(w), "%s: weight must be contiguous OIHW", who);
    d->N = int(x.shape[0]); d->C = int(x.shape[1]); d->H = int(x.shape[2]); d->W = int(x.shape[3]);
    d->O = int(w.shape[0]); d->KH = int(w.shape[2]); d->KW = int(w.shape[3]);
    d->sh = int(p.ints[0]); d->sw = int(p.ints[1]); d->ph = int(p.ints[2]); d->pw = int(p.ints[3]);
    d->dh = int(p.ints[4]); d->dw = int(p.ints[5]); d->groups = int(p.ints[6]);
    FXF_CHECK(d->groups >= 1 && d->C % d->groups == 0 && d->O % d->groups == 0, "%s: channels are not divisible by groups", who);
    d->cg = d->C / d->groups; d->og = d->O / d->groups;
    FXF_CHECK(w.shape[1] == d->cg, "%s: weight input channels do not match x", who);
    FXF_CHECK(numel(b) == d->O, "%s: bias size mismatch", who);
    FXF_CHECK(d->sh > 0 && d->sw > 0 && d->dh > 0 && d->dw > 0, "%s: stride and dilation must be positive", who);
    d->HO = (d->H + 2 * d->ph - d->dh * (d->KH - 1) - 1) / d->sh + 1;
    d->WO = (d->W + 2 * d->pw - d->dw * (d->KW - 1) - 1) / d->sw + 1;
    FXF_CHECK(o.shape[0] == d->N && o.shape[1] == d->O && o.shape[2] == d->HO && o.shape[3] == d->WO, "%s: output shape does not match the convolution geometry", who);
    d->xs = strides_of(x);
    d->os = strides_of(o);
    return 0;
}

inline int pool_grid(int64_t total, const ExecCtx& ctx) {
    int64_t blocks = (total + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
    return int(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

int run_conv(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, bool relu, const NodePlan* plan, ExecCtx& ctx, const char* who) {
    FXF_CHECK(in.size() >= 3 && out.size() >= 1 && p.ints.size() >= 7, "%s: expects [x, weight, bias] and 7 int params", who);
    const FxfTensor &x = reg[in[0]], &w = reg[in[1]], &b = reg[in[2]], &o = reg[out[0]];
    ConvDesc d;
    if (conv_desc(x, w, b, o, p, &d, who)) return 1;
    d.relu = relu ? 1 : 0;
    int64_t n_pix = int64_t(d.N) * d.HO * d.WO;
    if (n_pix == 0 || d.O == 0) return 0;
    const ConvPlan* cp = static_cast<const ConvPlan*>(plan);
    const bool is_1x1 = d.KH == 1 && d.KW == 1 && d.sh == 1 && d.sw == 1 && d.ph == 0 && d.pw == 0 && d.groups == 1;
    if (is_1x1 && pixel_major(x) && pixel_major(o)) {
        GemmArgs g;
        g.x = static_cast<const float*>(x.ptr);
        g.w = static_cast<const float*>(w.ptr);
        if (cp && cp->gemm_1x1) { g.w_hi = cp->w_hi; g.w_lo = cp->w_lo; g.w_is_bf16 = cp->bf16; }
        g.bias = static_cast<const float*>(b.ptr);
        g.out = static_cast<float*>(o.ptr);
        g.M = n_pix; g.N = d.O; g.K = d.C;
        g.ldx = d.C; g.ldw = d.C; g.ldo = d.O;
        g.relu = relu;
        apply_fusion(ctx, g, false);
        g.conv_chain = true;
        return launch_gemm(g, ctx);
    }
    if (cp && cp->s2d_tc && cp->w_hi && is_channels_last(o) && ctx.scratch != nullptr &&
        ctx.scratch_bytes >= size_t(d.N) * size_t(cp->Hs) * size_t(cp->Ws) * 16 * sizeof(float)) {
        float* sbuf = static_cast<float*>(ctx.scratch);
        const int64_t total4 = int64_t(d.N) * cp->Hs * cp->Ws * 4;
        tag_launch(ctx, "space_to_depth16", 0, double(x.nbytes) + 16.0 * double(total4));
        space_to_depth16_kernel<<<pool_grid(total4, ctx), 256, 0, ctx.stream>>>(static_cast<const float*>(x.ptr), reinterpret_cast<float4*>(sbuf), d.N, d.C, d.H, d.W,
                                                                                cp->Hs, cp->Ws, d.ph, d.pw, d.xs);
        FXF_LAUNCHED(ctx);
        ConvTcArgs c;
        c.x = sbuf;
        c.w_hi = cp->w_hi; c.w_lo = cp->w_lo;
        c.bias = static_cast<const float*>(b.ptr);
        c.out = static_cast<float*>(o.ptr);
        c.N = d.N; c.C = 16; c.H = cp->Hs; c.W = cp->Ws; c.O = d.O; c.KH = cp->KH2; c.KW = cp->KW2; c.HO = d.HO; c.WO = d.WO;
        c.pad_h = 0; c.pad_w = 0; c.dil_h = 1; c.dil_w = 1; c.str_h = 1; c.str_w = 1;
        c.relu = relu;
        apply_fusion(ctx, c, false);
        tag_launch(ctx, "conv2d_s2d_igemm_tf32x3_tcgen05", 2.0 * double(n_pix) * d.O * d.C * d.KH * d.KW, double(x.nbytes) + double(w.nbytes) + double(o.nbytes));
        return launch_conv_tc(c, ctx);
    }
    if (cp && cp->igemm_tc && cp->w_hi && is_channels_last(x) && is_channels_last(o) && aligned16(x.ptr)) {
        ConvTcArgs c;
        c.x = static_cast<const float*>(x.ptr);
        c.w_hi = cp->w_hi; c.w_lo = cp->w_lo; c.w_is_bf16 = cp->bf16;
        c.bias = static_cast<const float*>(b.ptr);
        c.out = static_cast<float*>(o.ptr);
        c.N = d.N; c.C = d.C; c.H = d.H; c.W = d.W; c.O = d.O; c.KH = d.KH; c.KW = d.KW; c.HO = d.HO; c.WO = d.WO;
        c.pad_h = d.ph; c.pad_w = d.pw; c.dil_h = d.dh; c.dil_w = d.dw; c.str_h = d.sh; c.str_w = d.sw;
        c.relu = relu;
        apply_fusion(ctx, c, false);
        return launch_conv_tc(c, ctx);
    }
    dim3 grid(unsigned((n_pix + CBM - 1) / CBM), unsigned((d.og + CBN - 1) / CBN), unsigned(d.groups));
    tag_launch(ctx, "conv2d_igemm_fp32_simt64x64", 2.0 * double(n_pix) * d.O * d.cg * d.KH * d.KW,
               double(x.nbytes) + double(w.nbytes) + double(b.nbytes) + double(o.nbytes));
    // a folded residual Add: the FFMA kernel writes the plain convolution into the Add's output, then act(out + residual)
    float* dst = static_cast<float*>(o.ptr);
    const bool fused = ctx.fuse.out != nullptr;
    if (fused) {
        dst = ctx.fuse.out;
        d.relu = 0;
    }
    conv2d_igemm_kernel<<<grid, 256, 0, ctx.stream>>>(static_cast<const float*>(x.ptr), static_cast<const float*>(w.ptr), static_cast<const float*>(b.ptr), dst, d);
    FXF_LAUNCHED(ctx);
    if (fused) {
        ctx.fuse.consumed = true;
        return launch_residual_epilogue(dst, ctx.fuse.residual, numel(o), relu || ctx.fuse.relu, ctx);
    }
    return 0;
}

int pool_desc(const FxfTensor& x, const FxfTensor& o, PoolDesc* d, const char* who) {
    FXF_CHECK(x.dtype == FXF_F32 && o.dtype == FXF_F32, "%s: only float32 is supported", who);
    FXF_CHECK((x.rank == 3 || x.rank == 4) && o.rank == x.rank, "%s: input must be [N,C,H,W] or [C,H,W]", who);
    const int r = x.rank;
    d->N = r == 4 ? x.shape[0] : 1;
    d->C = int(x.shape[r - 3]); d->H = int(x.shape[r - 2]); d->W = int(x.shape[r - 1]);
    d->HO = int(o.shape[r - 2]); d->WO = int(o.shape[r - 1]);
    FXF_CHECK(o.shape[r - 3] == d->C && (r == 3 || o.shape[0] == x.shape[0]), "%s: output batch/channels do not match the input", who);
    d->xs = strides_of(x);
    d->os = strides_of(o);
    d->cl = is_channels_last(o) ? 1 : 0;
    return 0;
}



}  // namespace

int k_conv2d(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan* plan, ExecCtx& ctx) {
    return run_conv(reg, in, out, p, false, plan, ctx, "conv2d");
}
int k_conv2d_relu(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan* plan, ExecCtx& ctx) {
    return run_conv(reg, in, out, p, true, plan, ctx, "conv2d_relu");
}

int k_max_pool2d(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 1 && out.size() >= 1 && p.ints.size() >= 9, "max_pool2d: expects 9 int params");
    PoolDesc d;
    if (pool_desc(reg[in[0]], reg[out[0]], &d, "max_pool2d")) return 1;
    d.kh = int(p.ints[0]); d.kw = int(p.ints[1]); d.sh = int(p.ints[2]); d.sw = int(p.ints[3]);
    d.ph = int(p.ints[4]); d.pw = int(p.ints[5]); d.dh = int(p.ints[6]); d.dw = int(p.ints[7]);
    FXF_CHECK(d.sh > 0 && d.sw > 0, "max_pool2d: stride must be positive");
    int64_t total = d.N * d.C * d.HO * d.WO;
    if (total == 0) return 0;
    pool2d_kernel<kMaxPool><<<pool_grid(total, ctx), 256, 0, ctx.stream>>>(static_cast<const float*>(reg[in[0]].ptr), static_cast<float*>(reg[out[0]].ptr), d);
    FXF_LAUNCHED(ctx);
    return 0;
}

int k_avg_pool2d(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 1 && out.size() >= 1 && p.ints.size() >= 7, "avg_pool2d: expects 7 int params");
    PoolDesc d;
    if (pool_desc(reg[in[0]], reg[out[0]], &d, "avg_pool2d")) return 1;
    d.kh = int(p.ints[0]); d.kw = int(p.ints[1]); d.sh = int(p.ints[2]); d.sw = int(p.ints[3]);
    d.ph = int(p.ints[4]); d.pw = int(p.ints[5]); d.dh = 1; d.dw = 1;
    FXF_CHECK(d.sh > 0 && d.sw > 0, "avg_pool2d: stride must be positive");
    int64_t total = d.N * d.C * d.HO * d.WO;
    if (total == 0) return 0;
    pool2d_kernel<kAvgPool><<<pool_grid(total, ctx), 256, 0, ctx.stream>>>(static_cast<const float*>(reg[in[0]].ptr), static_cast<float*>(reg[out[0]].ptr), d);
    FXF_LAUNCHED(ctx);
    return 0;
}

int k_adaptive_avg_pool2d(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 1 && out.size() >= 1 && p.ints.size() >= 2, "adaptive_avg_pool2d: expects [oh, ow]");
    PoolDesc d;
    if (pool_desc(reg[in[0]], reg[out[0]], &d, "adaptive_avg_pool2d")) return 1;
    FXF_CHECK(d.HO == p.ints[0] && d.WO == p.ints[1], "adaptive_avg_pool2d: output shape does not match output_size");
    d.kh = d.kw = d.sh = d.sw = d.dh = d.dw = 1; d.ph = d.pw = 0;
    int64_t total = d.N * d.C * d.HO * d.WO;
    if (total == 0) return 0;
    if (d.HO == 1 && d.WO == 1 && is_contiguous(reg[in[0]]) && is_contiguous(reg[out[0]])) {
        int64_t nc = d.N * d.C, blocks = (nc * 32 + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
        global_avg_pool_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(static_cast<const float*>(reg[in[0]].ptr), static_cast<float*>(reg[out[0]].ptr), nc, d.H * d.W);
    } else {
        // a channels-last input is walked channels-fastest, which keeps the strided window reads coalesced
        if (is_channels_last(reg[in[0]])) d.cl = 1;
        pool2d_kernel<kAdaptiveAvg><<<pool_grid(total, ctx), 256, 0, ctx.stream>>>(static_cast<const float*>(reg[in[0]].ptr), static_cast<float*>(reg[out[0]].ptr), d);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}

std::unique_ptr<NodePlan> plan_conv(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const PlanEnv& env) {
    auto pl = std::make_unique<ConvPlan>();
    if (in.size() >= 3 && out.size() >= 1 && reg[in[1]].rank == 4 && reg[out[0]].rank == 4 && p.ints.size() >= 7) {
        const FxfTensor &w = reg[in[1]], &o = reg[out[0]];
        pl->flops = 2.0 * double(numel(o)) * double(w.shape[1]) * double(w.shape[2]) * double(w.shape[3]);
        pl->bytes = double(reg[in[0]].nbytes) + double(w.nbytes) + double(reg[in[2]].nbytes) + double(o.nbytes);
        const int64_t M = o.shape[0] * o.shape[2] * o.shape[3], O = w.shape[0], C = w.shape[1];
        const bool is_1x1 = w.shape[2] == 1 && w.shape[3] == 1 && p.ints[0] == 1 && p.ints[1] == 1 && p.ints[2] == 0 && p.ints[3] == 0 && p.ints[6] == 1;
        if (is_1x1 && env.gemm_mode != FXF_GEMM_FP32_SIMT && gemm_tc_shape_ok(M, O, C)) {
            pl->gemm_1x1 = true;
            pl->w_elems = O * C;
            pl->bf16 = env.gemm_mode == FXF_GEMM_BF16 && C % 8 == 0;
            pl->persist_bytes = round_up(size_t(2) * size_t(pl->w_elems) * sizeof(float), 256);
            pl->variant = pl->bf16 ? "1x1 -> tcgen05-bf16 GEMM when channels-last, else igemm-simt64x64" : "1x1 -> tcgen05-tf32x3 GEMM when channels-last, else igemm-simt64x64";
        } else if (!is_1x1 && p.ints[0] >= 1 && p.ints[0] <= 2 && p.ints[1] >= 1 && p.ints[1] <= 2 && p.ints[6] == 1 && env.gemm_mode != FXF_GEMM_FP32_SIMT && conv_tc_shape_ok(M, int(C), int(O)) &&
                   reg[in[0]].rank == 4 && reg[in[0]].shape[1] == C) {
            pl->igemm_tc = true;
            pl->w_elems = O * C * w.shape[2] * w.shape[3];
            pl->bf16 = env.gemm_mode == FXF_GEMM_BF16 && C % 32 == 0;
            pl->persist_bytes = round_up(size_t(2) * size_t(pl->w_elems) * sizeof(float), 256);
            pl->variant = pl->bf16 ? "tcgen05-bf16 implicit GEMM when channels-last, else igemm-simt64x64" : "tcgen05-tf32x3 implicit GEMM when channels-last, else igemm-simt64x64";
        } else if (!is_1x1 && p.ints[0] == 2 && p.ints[1] == 2 && p.ints[4] == 1 && p.ints[5] == 1 && p.ints[6] == 1 && C >= 1 && C <= 4 && O >= 64 &&
                   env.gemm_mode != FXF_GEMM_FP32_SIMT && reg[in[0]].rank == 4 && reg[in[0]].shape[1] == C && M >= 64) {
            // stem: space-to-depth copy (16 channels) in the shared scratch, then a stride-1 tensor-core convolution
            const FxfTensor& x = reg[in[0]];
            pl->s2d_tc = true;
            pl->KH2 = int((w.shape[2] + 1) / 2);
            pl->KW2 = int((w.shape[3] + 1) / 2);
            pl->Hs = int(o.shape[2]) + pl->KH2 - 1;   // rows the unpadded stride-1 convolution reads
            pl->Ws = int(o.shape[3]) + pl->KW2 - 1;
            (void)x;
            pl->w_elems = O * pl->KH2 * pl->KW2 * 16;
            pl->persist_bytes = round_up(size_t(2) * size_t(pl->w_elems) * sizeof(float), 256);
            pl->scratch_bytes = size_t(o.shape[0]) * size_t(pl->Hs) * size_t(pl->Ws) * 16 * sizeof(float);
            pl->variant = "space-to-depth + tcgen05-tf32x3 implicit GEMM when the output is channels-last, else igemm-simt64x64";
        } else {
            pl->variant = "igemm-simt64x64";
        }
    }
    return pl;
}

}  // namespace fxf
