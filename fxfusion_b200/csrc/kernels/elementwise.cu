// Bandwidth-bound kernels: Add / AddRelu / Relu / Mul / Size / Narrow / Embedding / Transpose.
//
// All of them are HBM-bound copies with at most one FLOP per element, so the design is the
// same everywhere: 128-bit loads and stores whenever the addresses allow it, consecutive
// threads on consecutive 16-byte words, and a grid-stride loop over a grid sized from the SM
// count so that the launch covers the machine a whole number of times.
//
// Semantics follow the reference CPU kernels (LibTorch calls):
//   add / add_relu  csrc/kernels/cpu/add.cpp:5-10, add_relu.cpp:5-11   (torch broadcasting)
//   relu            csrc/kernels/cpu/relu.cpp:5-9   (output may alias the input buffer)
//   mul             csrc/kernels/cpu/mul.cpp:5-25   (mode 0 tensor*tensor, 1..3 tensor*scalar)
//   size            csrc/kernels/cpu/size.cpp:5-11  (int64 scalar)
//   narrow          csrc/kernels/cpu/narrow.cpp:5-13 (copying slice)
//   embedding       csrc/kernels/cpu/embedding.cpp:5-11
//   transpose       csrc/kernels/cpu/transpose.cpp:5-12 (materialised two-dim swap)
#include "../runtime.hpp"

namespace fxf {
namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t work_items, const ExecCtx& ctx, int per_sm = 8) {
    int64_t blocks = (work_items + kThreads - 1) / kThreads;
    int64_t cap = int64_t(ctx.sm_count) * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return int(blocks);
}

enum BinOp { kAdd = 0, kAddRelu = 1, kMul = 2 };

template <int OP> __device__ __forceinline__ float apply(float a, float b) {
    if (OP == kAdd) return a + b;
    if (OP == kAddRelu) {
        float s = a + b;
        // torch::relu keeps NaN (max semantics that propagate NaN); fmaxf would drop it.
        return s > 0.f ? s : (s != s ? s : 0.f);
    }
    return a * b;
}
template <int OP> __device__ __forceinline__ float4 apply4(float4 a, float4 b) {
    return make_float4(apply<OP>(a.x, b.x), apply<OP>(a.y, b.y), apply<OP>(a.z, b.z), apply<OP>(a.w, b.w));
}

// out[i] = a[i] op b[i % nb]   (nb == n for the equal-shape case), 4 elements per thread.
template <int OP>
__global__ void __launch_bounds__(kThreads) binary_vec4_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                                               float4* __restrict__ out, int64_t n4, int64_t nb4) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 va = a[i];
        float4 vb = b[nb4 == n4 ? i : i % nb4];
        out[i] = apply4<OP>(va, vb);
    }
}

struct BroadcastDesc {
    int rank;
    int64_t shape[FXF_MAX_DIMS];
    int64_t sa[FXF_MAX_DIMS];
    int64_t sb[FXF_MAX_DIMS];
};

template <int OP>
__global__ void __launch_bounds__(kThreads) binary_generic_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                                  float* __restrict__ out, int64_t n, BroadcastDesc d) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t rem = i, oa = 0, ob = 0;
        for (int k = d.rank - 1; k >= 0; k--) {
            int64_t c = rem % d.shape[k];
            rem /= d.shape[k];
            oa += c * d.sa[k];
            ob += c * d.sb[k];
        }
        out[i] = apply<OP>(a[oa], b[ob]);
    }
}

template <int OP>
int run_binary(const FxfTensor& a, const FxfTensor& b, const FxfTensor& out, ExecCtx& ctx) {
    FXF_CHECK(a.dtype == FXF_F32 && b.dtype == FXF_F32 && out.dtype == FXF_F32, "binary op: only float32 is supported");
    int64_t n = numel(out);
    if (n == 0) return 0;
    // right-aligned broadcast strides
    BroadcastDesc d;
    d.rank = out.rank;
    FXF_CHECK(a.rank <= out.rank && b.rank <= out.rank, "binary op: operand rank exceeds output rank");
    for (int k = 0; k < out.rank; k++) {
        d.shape[k] = out.shape[k];
        int ka = k - (out.rank - a.rank), kb = k - (out.rank - b.rank);
        int64_t da = ka >= 0 ? a.shape[ka] : 1, db = kb >= 0 ? b.shape[kb] : 1;
        FXF_CHECK((da == out.shape[k] || da == 1) && (db == out.shape[k] || db == 1),
                  "binary op: shapes are not broadcastable to the output shape");
        d.sa[k] = (ka >= 0 && da != 1) ? a.stride[ka] : 0;
        d.sb[k] = (kb >= 0 && db != 1) ? b.stride[kb] : 0;
    }
    int64_t na = numel(a), nb = numel(b);
    // fast path: a covers the output, b is either equal-shaped or a trailing block of it
    bool b_suffix = is_contiguous(b) && nb > 0 && n % nb == 0;
    if (b_suffix && nb != n) {
        // b must equal the trailing dims of out (after dropping its leading 1s)
        int64_t prod = 1;
        int k = out.rank - 1;
        int kb = b.rank - 1;
        for (; kb >= 0 && prod < nb; kb--, k--) {
            if (b.shape[kb] != out.shape[k]) { b_suffix = false; break; }
            prod *= out.shape[k];
        }
        for (; b_suffix && kb >= 0; kb--) if (b.shape[kb] != 1) b_suffix = false;
        if (prod != nb) b_suffix = false;
    }
    // operands and output in one and the same dense layout (row-major or channels-last): a flat element-wise pass
    const bool flat = same_layout(a, out) && same_layout(b, out) && (is_contiguous(out) || is_channels_last(out));
    if (!flat) FXF_CHECK(is_contiguous(out), "binary op: a channels-last output needs operands in the same layout");
    if (flat) { b_suffix = true; nb = n; na = n; }
    if (na == n && (flat || is_contiguous(a)) && b_suffix && n % 4 == 0 && nb % 4 == 0 && aligned16(a.ptr) && aligned16(b.ptr) && aligned16(out.ptr)) {
        int64_t n4 = n / 4;
        binary_vec4_kernel<OP><<<grid_for(n4, ctx), kThreads, 0, ctx.stream>>>(
            static_cast<const float4*>(a.ptr), static_cast<const float4*>(b.ptr), static_cast<float4*>(out.ptr), n4, nb / 4);
    } else {
        if (flat) {  // identical layouts but not 16-byte friendly: walk storage order with unit strides
            d.rank = 1;
            d.shape[0] = n;
            d.sa[0] = d.sb[0] = 1;
        }
        binary_generic_kernel<OP><<<grid_for(n, ctx), kThreads, 0, ctx.stream>>>(
            static_cast<const float*>(a.ptr), static_cast<const float*>(b.ptr), static_cast<float*>(out.ptr), n, d);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}

// ---- unary: relu, scale -------------------------------------------------------------------
enum UnOp { kRelu = 0, kScale = 1 };
template <int OP> __device__ __forceinline__ float unary(float x, float s) {
    if (OP == kRelu) return x > 0.f ? x : (x != x ? x : 0.f);
    return x * s;
}
template <int OP>
__global__ void __launch_bounds__(kThreads) unary_vec4_kernel(const float4* x, float4* out, int64_t n4, float s) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 v = x[i];
        out[i] = make_float4(unary<OP>(v.x, s), unary<OP>(v.y, s), unary<OP>(v.z, s), unary<OP>(v.w, s));
    }
}
template <int OP>
__global__ void __launch_bounds__(kThreads) unary_kernel(const float* x, float* out, int64_t n, float s) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = unary<OP>(x[i], s);
}
template <int OP>
int run_unary(const FxfTensor& x, const FxfTensor& out, float s, ExecCtx& ctx) {
    FXF_CHECK(x.dtype == FXF_F32 && out.dtype == FXF_F32, "unary op: only float32 is supported");
    int64_t n = numel(out);
    FXF_CHECK(numel(x) == n, "unary op: input/output element counts differ");
    FXF_CHECK(same_layout(x, out) || (is_contiguous(x) && is_contiguous(out)), "unary op: input and output layouts differ");
    if (n == 0) return 0;
    if (n % 4 == 0 && aligned16(x.ptr) && aligned16(out.ptr)) {
        unary_vec4_kernel<OP><<<grid_for(n / 4, ctx), kThreads, 0, ctx.stream>>>(static_cast<const float4*>(x.ptr), static_cast<float4*>(out.ptr), n / 4, s);
    } else {
        unary_kernel<OP><<<grid_for(n, ctx), kThreads, 0, ctx.stream>>>(static_cast<const float*>(x.ptr), static_cast<float*>(out.ptr), n, s);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}

// ---- size ---------------------------------------------------------------------------------
__global__ void fill_i64_kernel(int64_t* out, int64_t v, int64_t n) {
    int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = v;
}

// ---- strided row copy (narrow) --------------------------------------------------------------
// rows x row_bytes, source rows `src_pitch` bytes apart.  16-byte words when aligned.
__global__ void __launch_bounds__(kThreads) rowcopy16_kernel(const uint4* src, uint4* dst, int64_t rows, int64_t row_w, int64_t src_pitch_w) {
    int64_t total = rows * row_w, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t r = i / row_w, c = i - r * row_w;
        dst[i] = src[r * src_pitch_w + c];
    }
}
template <typename T>
__global__ void __launch_bounds__(kThreads) rowcopy_kernel(const T* src, T* dst, int64_t rows, int64_t row_w, int64_t src_pitch_w) {
    int64_t total = rows * row_w, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t r = i / row_w, c = i - r * row_w;
        dst[i] = src[r * src_pitch_w + c];
    }
}

// ---- embedding ----------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) embedding_vec4_kernel(const int64_t* __restrict__ idx, const float4* __restrict__ w, float4* __restrict__ out,
                                                                  int64_t n_idx, int64_t d4, int64_t vocab, int* status) {
    int64_t total = n_idx * d4, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t r = i / d4, c = i - r * d4;
        int64_t row = idx[r];
        if (row < 0 || row >= vocab) {
            if (status) atomicCAS(status, 0, 2);
            out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            out[i] = w[row * d4 + c];
        }
    }
}
__global__ void __launch_bounds__(kThreads) embedding_kernel(const int64_t* __restrict__ idx, const float* __restrict__ w, float* __restrict__ out,
                                                             int64_t n_idx, int64_t d, int64_t vocab, int* status) {
    int64_t total = n_idx * d, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t r = i / d, c = i - r * d;
        int64_t row = idx[r];
        if (row < 0 || row >= vocab) {
            if (status) atomicCAS(status, 0, 2);
            out[i] = 0.f;
        } else {
            out[i] = w[row * d + c];
        }
    }
}

// ---- transpose ------------------------------------------------------------------------------
struct TransposeDesc {
    int rank;
    int64_t out_shape[FXF_MAX_DIMS];
    int64_t in_stride_perm[FXF_MAX_DIMS];  // stride of the input along the dim that feeds output dim k
};
template <typename T>
__global__ void __launch_bounds__(kThreads) transpose_generic_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n, TransposeDesc d) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t rem = i, off = 0;
        for (int k = d.rank - 1; k >= 0; k--) {
            int64_t c = rem % d.out_shape[k];
            rem /= d.out_shape[k];
            off += c * d.in_stride_perm[k];
        }
        out[i] = x[off];
    }
}
// Batched [R, C] -> [C, R] through a 32x33 shared tile: both the read and the write are coalesced.
template <typename T>
__global__ void __launch_bounds__(256) transpose_tile_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t R, int64_t C, int64_t tiles_r, int64_t tiles_c, int64_t n_tiles) {
    __shared__ T tile[32][33];
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        int64_t b = t / (tiles_r * tiles_c);
        int64_t rem = t - b * tiles_r * tiles_c;
        int64_t tr = rem / tiles_c, tc = rem - tr * tiles_c;
        const T* src = x + b * R * C;
        T* dst = out + b * R * C;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            int64_t r = tr * 32 + ty + j, c = tc * 32 + tx;
            if (r < R && c < C) tile[ty + j][tx] = src[r * C + c];
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            int64_t c = tc * 32 + ty + j, r = tr * 32 + tx;
            if (r < R && c < C) dst[c * R + r] = tile[tx][ty + j];
        }
        __syncthreads();
    }
}

template <typename T>
int run_transpose_typed(const FxfTensor& x, const FxfTensor& out, int d0, int d1, ExecCtx& ctx) {
    int64_t n = numel(out);
    if (n == 0) return 0;
    int rank = x.rank;
    if (d0 > d1) std::swap(d0, d1);
    if (is_contiguous(x) && d1 == rank - 1 && d0 == rank - 2) {
        int64_t R = x.shape[d0], C = x.shape[d1], batch = n / (R * C);
        int64_t tr = (R + 31) / 32, tc = (C + 31) / 32, tiles = batch * tr * tc;
        int grid = int(tiles < int64_t(ctx.sm_count) * 8 ? tiles : int64_t(ctx.sm_count) * 8);
        transpose_tile_kernel<T><<<grid, 256, 0, ctx.stream>>>(static_cast<const T*>(x.ptr), static_cast<T*>(out.ptr), R, C, tr, tc, tiles);
    } else {
        TransposeDesc d;
        d.rank = rank;
        for (int k = 0; k < rank; k++) {
            int src = k == d0 ? d1 : (k == d1 ? d0 : k);
            d.out_shape[k] = x.shape[src];
            d.in_stride_perm[k] = x.stride[src];
        }
        transpose_generic_kernel<T><<<grid_for(n, ctx), kThreads, 0, ctx.stream>>>(static_cast<const T*>(x.ptr), static_cast<T*>(out.ptr), n, d);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}

struct SimplePlan : NodePlan {};

std::unique_ptr<NodePlan> plan_elementwise(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const PlanEnv&) {
    auto p = std::make_unique<SimplePlan>();
    double b = 0;
    for (auto id : in) b += double(reg[id].nbytes);
    for (auto id : out) b += double(reg[id].nbytes);
    p->bytes = b;
    p->flops = out.empty() ? 0 : double(numel(reg[out[0]]));
    p->variant = "vec128";
    return p;
}

}  // namespace

// ---- KernelFn entry points -------------------------------------------------------------------
int k_add(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 2 && out.size() >= 1, "add: expects 2 inputs and 1 output");
    return run_binary<kAdd>(reg[in[0]], reg[in[1]], reg[out[0]], ctx);
}
int k_add_relu(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 2 && out.size() >= 1, "add_relu: expects 2 inputs and 1 output");
    return run_binary<kAddRelu>(reg[in[0]], reg[in[1]], reg[out[0]], ctx);
}
int k_relu(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 1 && out.size() >= 1, "relu: expects 1 input and 1 output");
    return run_unary<kRelu>(reg[in[0]], reg[out[0]], 0.f, ctx);
}
int k_mul(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(!p.ints.empty(), "mul: missing mul_mode");
    int64_t mode = p.ints[0];
    if (mode == 0) {
        FXF_CHECK(in.size() >= 2 && out.size() >= 1, "mul: tensor-tensor mode expects 2 inputs");
        return run_binary<kMul>(reg[in[0]], reg[in[1]], reg[out[0]], ctx);
    }
    FXF_CHECK(mode >= 1 && mode <= 3, "mul: unknown mul_mode %lld", (long long)mode);
    FXF_CHECK(!p.floats.empty() && in.size() >= 1 && out.size() >= 1, "mul: scalar mode expects 1 input and 1 float param");
    return run_unary<kScale>(reg[in[0]], reg[out[0]], p.floats[0], ctx);
}
int k_size(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 1 && out.size() >= 1 && !p.ints.empty(), "size: expects 1 input, 1 output and a dim");
    const FxfTensor& x = reg[in[0]];
    FxfTensor& o = reg[out[0]];
    int64_t dim = p.ints[0];
    if (dim < 0) dim += x.rank;
    FXF_CHECK(dim >= 0 && dim < x.rank, "size: dim out of range");
    FXF_CHECK(o.dtype == FXF_I64, "size: output must be int64");
    int64_t n = numel(o);
    fill_i64_kernel<<<int((n + 255) / 256), 256, 0, ctx.stream>>>(static_cast<int64_t*>(o.ptr), x.shape[dim], n);
    FXF_LAUNCHED(ctx);
    return 0;
}
int k_narrow(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 1 && out.size() >= 1 && p.ints.size() >= 3, "narrow: expects [dim,start,length]");
    const FxfTensor& x = reg[in[0]];
    const FxfTensor& o = reg[out[0]];
    int64_t dim = p.ints[0], start = p.ints[1], length = p.ints[2];
    if (dim < 0) dim += x.rank;
    FXF_CHECK(dim >= 0 && dim < x.rank, "narrow: dim out of range");
    FXF_CHECK(is_contiguous(x), "narrow: input must be contiguous");
    // A negative length means "read it from the scalar input" in the reference
    // (narrow.cpp:11, a device->host sync on CUDA).  Shapes are static per compiled graph, so
    // the length is already the extent of the output tensor along `dim`.
    if (length < 0) length = o.shape[dim];
    if (start < 0) start += x.shape[dim];
    FXF_CHECK(o.rank == x.rank && o.shape[dim] == length, "narrow: output shape does not match the slice");
    FXF_CHECK(start >= 0 && start + length <= x.shape[dim], "narrow: slice exceeds the input extent");
    int esz = dtype_size(x.dtype);
    int64_t inner = 1, outer = 1;
    for (int k = int(dim) + 1; k < x.rank; k++) inner *= x.shape[k];
    for (int k = 0; k < dim; k++) outer *= x.shape[k];
    int64_t row_bytes = length * inner * esz, pitch = x.shape[dim] * inner * esz;
    if (outer * row_bytes == 0) return 0;
    const char* src = static_cast<const char*>(x.ptr) + start * inner * esz;
    char* dst = static_cast<char*>(o.ptr);
    if (row_bytes % 16 == 0 && pitch % 16 == 0 && aligned16(src) && aligned16(dst)) {
        rowcopy16_kernel<<<grid_for(outer * row_bytes / 16, ctx), kThreads, 0, ctx.stream>>>(
            reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), outer, row_bytes / 16, pitch / 16);
    } else if (esz == 4) {
        rowcopy_kernel<uint32_t><<<grid_for(outer * row_bytes / 4, ctx), kThreads, 0, ctx.stream>>>(
            reinterpret_cast<const uint32_t*>(src), reinterpret_cast<uint32_t*>(dst), outer, row_bytes / 4, pitch / 4);
    } else {
        rowcopy_kernel<uint8_t><<<grid_for(outer * row_bytes, ctx), kThreads, 0, ctx.stream>>>(
            reinterpret_cast<const uint8_t*>(src), reinterpret_cast<uint8_t*>(dst), outer, row_bytes, pitch);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}
int k_embedding(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 2 && out.size() >= 1, "embedding: expects [indices, weight]");
    const FxfTensor& idx = reg[in[0]];
    const FxfTensor& w = reg[in[1]];
    const FxfTensor& o = reg[out[0]];
    FXF_CHECK(idx.dtype == FXF_I64, "embedding: indices must be int64");
    FXF_CHECK(w.dtype == FXF_F32 && w.rank == 2 && o.dtype == FXF_F32, "embedding: weight must be float32 [V,D]");
    int64_t n_idx = numel(idx), D = w.shape[1], V = w.shape[0];
    FXF_CHECK(numel(o) == n_idx * D, "embedding: output size mismatch");
    if (n_idx * D == 0) return 0;
    if (D % 4 == 0 && aligned16(w.ptr) && aligned16(o.ptr)) {
        embedding_vec4_kernel<<<grid_for(n_idx * D / 4, ctx), kThreads, 0, ctx.stream>>>(
            static_cast<const int64_t*>(idx.ptr), static_cast<const float4*>(w.ptr), static_cast<float4*>(o.ptr), n_idx, D / 4, V, ctx.status);
    } else {
        embedding_kernel<<<grid_for(n_idx * D, ctx), kThreads, 0, ctx.stream>>>(
            static_cast<const int64_t*>(idx.ptr), static_cast<const float*>(w.ptr), static_cast<float*>(o.ptr), n_idx, D, V, ctx.status);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}
int k_transpose(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan*, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 1 && out.size() >= 1 && p.ints.size() >= 2, "transpose: expects [dim0, dim1]");
    const FxfTensor& x = reg[in[0]];
    const FxfTensor& o = reg[out[0]];
    int64_t d0 = p.ints[0], d1 = p.ints[1];
    if (d0 < 0) d0 += x.rank;
    if (d1 < 0) d1 += x.rank;
    FXF_CHECK(d0 >= 0 && d0 < x.rank && d1 >= 0 && d1 < x.rank, "transpose: dims out of range");
    FXF_CHECK(x.rank <= FXF_MAX_DIMS, "transpose dims exceed cache capacity");
    FXF_CHECK(numel(o) == numel(x), "transpose: output size mismatch");
    switch (dtype_size(x.dtype)) {
        case 4: return run_transpose_typed<uint32_t>(x, o, int(d0), int(d1), ctx);
        case 8: return run_transpose_typed<uint64_t>(x, o, int(d0), int(d1), ctx);
        case 2: return run_transpose_typed<uint16_t>(x, o, int(d0), int(d1), ctx);
        case 1: return run_transpose_typed<uint8_t>(x, o, int(d0), int(d1), ctx);
    }
    FXF_FAIL("transpose: unsupported dtype");
}

std::unique_ptr<NodePlan> plan_bandwidth(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const PlanEnv& m) {
    return plan_elementwise(reg, in, out, p, m);
}
// Narrow and Embedding touch only the slice / the gathered rows, not their whole first input.
std::unique_ptr<NodePlan> plan_gather(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const PlanEnv&) {
    auto p = std::make_unique<SimplePlan>();
    double ob = out.empty() ? 0 : double(reg[out[0]].nbytes);
    p->bytes = 2 * ob;
    if (in.size() >= 2 && reg[in[0]].dtype == FXF_I64) p->bytes += double(reg[in[0]].nbytes);
    p->variant = "vec128";
    return p;
}

}  // namespace fxf
