// LayerNorm and Add+LayerNorm over the trailing `N` elements of each of `M` rows.
//
// Reference semantics (LibTorch): out = layer_norm(x [+ z], normalized_shape, weight, bias, eps)
//   csrc/kernels/cpu/layer_norm.cpp:5-16, csrc/kernels/cpu/add_layer_norm.cpp:5-17
// with M and N derived as in csrc/runtime/cache.cpp:39-47 (N = product of normalized_shape,
// M = numel / N).  Variance is the biased one and eps sits inside the square root.
//
// HBM-bound: each row is read once (x, and z for the fused add), kept in registers, reduced
// with warp shuffles (mean first, then centred sum of squares, so no cancellation), and
// written once.  One warp owns one row; 128-bit loads; a block carries 8 warps and the grid
// strides over rows.  Rows wider than 32 lanes x 8 float4 (N > 1024) or not 16-byte aligned
// use a block-per-row kernel that re-reads the row from L2 instead.
#include "../runtime.hpp"

namespace fxf {
namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int NV, bool ADD>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) layernorm_warp_kernel(const float4* __restrict__ x, const float4* __restrict__ z,
                                                                             const float4* __restrict__ w, const float4* __restrict__ b,
                                                                             float4* __restrict__ out, int64_t M, int n4, float inv_n, float eps) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t row_stride = int64_t(gridDim.x) * kWarpsPerBlock;
    for (int64_t row = int64_t(blockIdx.x) * kWarpsPerBlock + warp; row < M; row += row_stride) {
        const float4* xr = x + row * n4;
        const float4* zr = ADD ? z + row * n4 : nullptr;
        float4 v[NV];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int c = lane + 32 * i;
            if (c < n4) {
                v[i] = xr[c];
                if (ADD) {
                    float4 t = zr[c];
                    v[i].x += t.x; v[i].y += t.y; v[i].z += t.z; v[i].w += t.w;
                }
                s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            } else {
                v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float mean = warp_sum(s) * inv_n;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int c = lane + 32 * i;
            if (c < n4) {
                float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
                q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        }
        float var = warp_sum(q) * inv_n;
        float rstd = 1.0f / sqrtf(var + eps);
        float shift = -rstd * mean;
        float4* orow = out + row * n4;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int c = lane + 32 * i;
            if (c < n4) {
                float4 g = w[c], bb = b[c], r;
                r.x = (v[i].x * rstd + shift) * g.x + bb.x;
                r.y = (v[i].y * rstd + shift) * g.y + bb.y;
                r.z = (v[i].z * rstd + shift) * g.z + bb.z;
                r.w = (v[i].w * rstd + shift) * g.w + bb.w;
                orow[c] = r;
            }
        }
    }
}

__device__ float block_sum(float v, float* red) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}

template <bool ADD>
__global__ void __launch_bounds__(256) layernorm_block_kernel(const float* __restrict__ x, const float* __restrict__ z, const float* __restrict__ w,
                                                              const float* __restrict__ b, float* __restrict__ out, int64_t M, int64_t N, float inv_n, float eps) {
    __shared__ float red[32];
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
        const float* xr = x + row * N;
        const float* zr = ADD ? z + row * N : nullptr;
        float s = 0.f;
        for (int64_t c = threadIdx.x; c < N; c += blockDim.x) s += ADD ? xr[c] + zr[c] : xr[c];
        float mean = block_sum(s, red) * inv_n;
        float q = 0.f;
        for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
            float d = (ADD ? xr[c] + zr[c] : xr[c]) - mean;
            q += d * d;
        }
        float var = block_sum(q, red) * inv_n;
        float rstd = 1.0f / sqrtf(var + eps);
        float shift = -rstd * mean;
        for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
            float v = ADD ? xr[c] + zr[c] : xr[c];
            out[row * N + c] = (v * rstd + shift) * w[c] + b[c];
        }
    }
}

struct LayerNormPlan : NodePlan {
    int64_t M = 0, N = 0;
};

template <bool ADD>
int run_layernorm(const float* x, const float* z, const float* w, const float* b, float* out, int64_t M, int64_t N, float eps, ExecCtx& ctx) {
    if (M == 0 || N == 0) return 0;
    float inv_n = 1.0f / float(N);
    bool vec = N % 4 == 0 && N <= 1024 && aligned16(x) && aligned16(w) && aligned16(b) && aligned16(out) && (!ADD || aligned16(z));
    if (vec) {
        int n4 = int(N / 4), nv = (n4 + 31) / 32;
        int64_t blocks = (M + kWarpsPerBlock - 1) / kWarpsPerBlock;
        int64_t cap = int64_t(ctx.sm_count) * 8;
        int grid = int(blocks < cap ? blocks : cap);
        auto X = reinterpret_cast<const float4*>(x);
        auto Z = reinterpret_cast<const float4*>(z);
        auto W = reinterpret_cast<const float4*>(w);
        auto Bv = reinterpret_cast<const float4*>(b);
        auto O = reinterpret_cast<float4*>(out);
        dim3 blk(kWarpsPerBlock * 32);
#define FXF_LN_CASE(NV) case NV: layernorm_warp_kernel<NV, ADD><<<grid, blk, 0, ctx.stream>>>(X, Z, W, Bv, O, M, n4, inv_n, eps); break;
        switch (nv) {
            FXF_LN_CASE(1) FXF_LN_CASE(2) FXF_LN_CASE(3) FXF_LN_CASE(4)
            FXF_LN_CASE(5) FXF_LN_CASE(6) FXF_LN_CASE(7) FXF_LN_CASE(8)
        }
#undef FXF_LN_CASE
    } else {
        int64_t cap = int64_t(ctx.sm_count) * 8;
        int grid = int(M < cap ? M : cap);
        layernorm_block_kernel<ADD><<<grid, 256, 0, ctx.stream>>>(x, z, w, b, out, M, N, inv_n, eps);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}

int rows_cols(const FxfTensor& x, const Params& p, int64_t* M, int64_t* N, const char* who) {
    FXF_CHECK(!p.ints.empty() && !p.floats.empty(), "%s: expects [rank, dims...] and [eps]", who);
    int64_t rank = p.ints[0];
    FXF_CHECK(rank >= 0 && int64_t(p.ints.size()) >= 1 + rank, "%s: normalized_shape truncated", who);
    int64_t n = 1;
    for (int64_t i = 0; i < rank; i++) n *= p.ints[1 + i];
    FXF_CHECK(n > 0, "%s: empty normalized_shape", who);
    int64_t total = numel(x);
    FXF_CHECK(total % n == 0, "%s: input size is not a multiple of normalized_shape", who);
    *N = n;
    *M = total / n;
    return 0;
}

}  // namespace

int k_layer_norm(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 3 && out.size() >= 1, "layer_norm: expects [x, weight, bias]");
    const FxfTensor &x = reg[in[0]], &w = reg[in[1]], &b = reg[in[2]], &o = reg[out[0]];
    FXF_CHECK(x.dtype == FXF_F32 && o.dtype == FXF_F32, "layer_norm: only float32 is supported");
    int64_t M, N;
    if (rows_cols(x, p, &M, &N, "layer_norm")) return 1;
    FXF_CHECK(numel(w) == N && numel(b) == N && numel(o) == M * N, "layer_norm: operand sizes do not match");
    return run_layernorm<false>(static_cast<const float*>(x.ptr), nullptr, static_cast<const float*>(w.ptr), static_cast<const float*>(b.ptr),
                                static_cast<float*>(o.ptr), M, N, p.floats[0], ctx);
}

int k_add_layer_norm(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 4 && out.size() >= 1, "add_layer_norm: expects [a, b, weight, bias]");
    const FxfTensor &a = reg[in[0]], &z = reg[in[1]], &w = reg[in[2]], &b = reg[in[3]], &o = reg[out[0]];
    FXF_CHECK(a.dtype == FXF_F32 && z.dtype == FXF_F32 && o.dtype == FXF_F32, "add_layer_norm: only float32 is supported");
    int64_t M, N;
    if (rows_cols(a, p, &M, &N, "add_layer_norm")) return 1;
    FXF_CHECK(numel(z) == numel(a), "add_layer_norm: the two addends must have equal shapes");
    FXF_CHECK(numel(w) == N && numel(b) == N && numel(o) == M * N, "add_layer_norm: operand sizes do not match");
    return run_layernorm<true>(static_cast<const float*>(a.ptr), static_cast<const float*>(z.ptr), static_cast<const float*>(w.ptr),
                               static_cast<const float*>(b.ptr), static_cast<float*>(o.ptr), M, N, p.floats[0], ctx);
}

std::unique_ptr<NodePlan> plan_layernorm(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const PlanEnv&) {
    auto p = std::make_unique<LayerNormPlan>();
    double b = 0;
    for (auto id : in) b += double(reg[id].nbytes);
    for (auto id : out) b += double(reg[id].nbytes);
    p->bytes = b;
    p->flops = out.empty() ? 0 : 8.0 * double(numel(reg[out[0]]));
    p->variant = "warp-per-row vec128";
    return p;
}

}  // namespace fxf
