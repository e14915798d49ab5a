// Device-side pieces of the greedy static decode loop
// (reference: py/fxfusion/models/transformer/inference.py:28-45, a Python loop that rebuilds
// the mask with torch ops, runs the engine, and takes torch.argmax of one logits row).
//
//   build_mask      mask[b,0,q,k] = (k < current_len) & (tokens[b,k] != pad) & (k <= q)
//                   — static_prefix_mask & padding_mask & causal
//                   (py/fxfusion/models/transformer/layers/masks.py:98-110, 141-154)
//   argmax_scatter  tokens[b,current_len] = argmax_v logits[b,current_len-1,v]
//                   — first maximal index; NaN compares as the largest value (torch.argmax)
#include <cmath>

#include "../runtime.hpp"

namespace fxf {
namespace {

__global__ void __launch_bounds__(256) build_mask_kernel(const int64_t* __restrict__ tokens, uint8_t* __restrict__ mask, int B, int T, int cur, int64_t pad) {
    int64_t total = int64_t(B) * T * T, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int k = int(i % T);
        int64_t t = i / T;
        int q = int(t % T);
        int b = int(t / T);
        mask[i] = (k < cur && k <= q && tokens[int64_t(b) * T + k] != pad) ? 1 : 0;
    }
}

// 4 keys per thread, one 32-bit store.
__global__ void __launch_bounds__(256) build_mask_vec4_kernel(const int64_t* __restrict__ tokens, uint32_t* __restrict__ mask, int B, int T, int cur, int64_t pad) {
    int T4 = T / 4;
    int64_t total = int64_t(B) * T * T4, stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int k4 = int(i % T4);
        int64_t t = i / T4;
        int q = int(t % T);
        int b = int(t / T);
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int k = k4 * 4 + j;
            uint32_t keep = (k < cur && k <= q && tokens[int64_t(b) * T + k] != pad) ? 1u : 0u;
            word |= keep << (8 * j);
        }
        mask[i] = word;
    }
}

struct Best {
    float v;
    int64_t i;
};
// true if a should replace b as the running argmax
__device__ __forceinline__ bool better(const Best& a, const Best& b) {
    if (b.i < 0) return a.i >= 0;
    if (a.i < 0) return false;
    bool an = a.v != a.v, bn = b.v != b.v;
    if (an || bn) {
        if (an && bn) return a.i < b.i;
        return an;
    }
    if (a.v > b.v) return true;
    if (a.v < b.v) return false;
    return a.i < b.i;
}

__global__ void __launch_bounds__(1024) argmax_scatter_kernel(const float* __restrict__ logits, int64_t row_stride, int64_t row_off, int64_t* __restrict__ tokens, int T, int64_t V, int cur) {
    __shared__ Best red[32];
    int b = blockIdx.x;
    const float* row = logits + int64_t(b) * row_stride + row_off;
    Best best{0.f, -1};
    for (int64_t i = threadIdx.x; i < V; i += blockDim.x) {
        Best c{row[i], i};
        if (better(c, best)) best = c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best c;
        c.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        c.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        if (better(c, best)) best = c;
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = lane < (blockDim.x >> 5) ? red[lane] : Best{0.f, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best c;
            c.v = __shfl_xor_sync(0xffffffffu, best.v, o);
            c.i = __shfl_xor_sync(0xffffffffu, best.i, o);
            if (better(c, best)) best = c;
        }
        if (lane == 0) tokens[int64_t(b) * T + cur] = best.i < 0 ? 0 : best.i;
    }
}

// Vocabulary-sharded variant: every rank scans only its own column block and publishes one candidate per
// sequence; after the all-gather each rank picks the same winner (the comparator prefers the lower index
// on ties, so the result equals an argmax over the whole row).
struct alignas(16) Candidate {
    float v;
    int pad;
    int64_t i;
};

__global__ void __launch_bounds__(1024) argmax_partial_kernel(const float* __restrict__ logits, int64_t row_stride, int64_t row_off, Candidate* __restrict__ cand,
                                                              int64_t col0, int64_t ncols) {
    __shared__ Best red[32];
    int b = blockIdx.x;
    const float* row = logits + int64_t(b) * row_stride + row_off;
    Best best{0.f, -1};
    for (int64_t i = col0 + threadIdx.x; i < col0 + ncols; i += blockDim.x) {
        Best c{row[i], i};
        if (better(c, best)) best = c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best c;
        c.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        c.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        if (better(c, best)) best = c;
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = lane < (blockDim.x >> 5) ? red[lane] : Best{0.f, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best c;
            c.v = __shfl_xor_sync(0xffffffffu, best.v, o);
            c.i = __shfl_xor_sync(0xffffffffu, best.i, o);
            if (better(c, best)) best = c;
        }
        if (lane == 0) cand[b] = Candidate{best.v, 0, best.i};
    }
}

__global__ void argmax_combine_scatter_kernel(const Candidate* __restrict__ all, int64_t* __restrict__ tokens, int B, int T, int cur, int n_ranks) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    Best best{0.f, -1};
    for (int r = 0; r < n_ranks; r++) {
        Candidate c = all[int64_t(r) * B + b];
        Best cb{c.v, c.i};
        if (better(cb, best)) best = cb;
    }
    tokens[int64_t(b) * T + cur] = best.i < 0 ? 0 : best.i;
}

}  // namespace

int decode_argmax_scatter_rows(const float* logits, int64_t row_stride, int64_t row_off, int64_t* tokens, int B, int T, int64_t V, int cur, ExecCtx& ctx);
int decode_argmax_scatter_sharded_rows(const float* logits, int64_t row_stride, int64_t row_off, int64_t* tokens, int B, int T, int64_t V, int cur,
                                       int64_t col0, int64_t ncols, void* cand_local, void* cand_all, ExecCtx& ctx);

// cand_local: B candidates; cand_all: n_ranks * B candidates (16 bytes each)
int decode_argmax_scatter_sharded(const float* logits, int64_t* tokens, int B, int T, int64_t V, int cur, int64_t col0, int64_t ncols,
                                  void* cand_local, void* cand_all, ExecCtx& ctx) {
    return decode_argmax_scatter_sharded_rows(logits, int64_t(T) * V, int64_t(cur - 1) * V, tokens, B, T, V, cur, col0, ncols, cand_local, cand_all, ctx);
}

// Row b of the logits starts at logits + b * row_stride + row_off; the token goes to tokens[b, cur].
int decode_argmax_scatter_sharded_rows(const float* logits, int64_t row_stride, int64_t row_off, int64_t* tokens, int B, int T, int64_t V, int cur,
                                       int64_t col0, int64_t ncols, void* cand_local, void* cand_all, ExecCtx& ctx) {
    FXF_CHECK(cur >= 1 && cur < T, "decode: current_len %d must be in [1, %d)", cur, T);
    if (B == 0) return 0;
    (void)V;
    argmax_partial_kernel<<<B, 1024, 0, ctx.stream>>>(logits, row_stride, row_off, static_cast<Candidate*>(cand_local), col0, ncols);
    FXF_LAUNCHED(ctx);
    if (tp_all_gather(cand_local, cand_all, int64_t(B) * int64_t(sizeof(Candidate)), ctx)) return 1;
    argmax_combine_scatter_kernel<<<(B + 127) / 128, 128, 0, ctx.stream>>>(static_cast<const Candidate*>(cand_all), tokens, B, T, cur, ctx.tp_size);
    FXF_LAUNCHED(ctx);
    return 0;
}

namespace {
// ids[b] = tokens[b, p]; *pos = p  — the inputs of one incremental decode step
__global__ void step_prepare_kernel(const int64_t* __restrict__ tokens, int64_t* __restrict__ ids, int64_t* __restrict__ pos, int B, int T, int p) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) ids[b] = tokens[int64_t(b) * T + p];
    if (b == 0) *pos = p;
}
}  // namespace

int decode_step_prepare(const int64_t* tokens, int64_t* ids, int64_t* pos, int B, int T, int p, ExecCtx& ctx) {
    FXF_CHECK(p >= 0 && p < T, "decode: position %d is outside the static length %d", p, T);
    step_prepare_kernel<<<(B + 127) / 128 > 0 ? (B + 127) / 128 : 1, 128, 0, ctx.stream>>>(tokens, ids, pos, B, T, p);
    FXF_LAUNCHED(ctx);
    return 0;
}

int decode_build_mask(const int64_t* tokens, uint8_t* mask, int B, int T, int cur, int64_t pad, ExecCtx& ctx) {
    FXF_CHECK(B >= 0 && T >= 0 && cur >= 0 && cur <= T, "decode: current_len %d exceeds static length %d", cur, T);
    if (B == 0 || T == 0) return 0;
    int64_t cap = int64_t(ctx.sm_count) * 8;
    if (T % 4 == 0 && (reinterpret_cast<uintptr_t>(mask) & 3) == 0) {
        int64_t total = int64_t(B) * T * (T / 4), blocks = (total + 255) / 256;
        build_mask_vec4_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(tokens, reinterpret_cast<uint32_t*>(mask), B, T, cur, pad);
    } else {
        int64_t total = int64_t(B) * T * T, blocks = (total + 255) / 256;
        build_mask_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(tokens, mask, B, T, cur, pad);
    }
    FXF_LAUNCHED(ctx);
    return 0;
}

int decode_argmax_scatter(const float* logits, int64_t* tokens, int B, int T, int64_t V, int cur, ExecCtx& ctx) {
    return decode_argmax_scatter_rows(logits, int64_t(T) * V, int64_t(cur - 1) * V, tokens, B, T, V, cur, ctx);
}

int decode_argmax_scatter_rows(const float* logits, int64_t row_stride, int64_t row_off, int64_t* tokens, int B, int T, int64_t V, int cur, ExecCtx& ctx) {
    FXF_CHECK(cur >= 1 && cur < T, "decode: current_len %d must be in [1, %d)", cur, T);
    FXF_CHECK(V >= 1, "decode: empty vocabulary");
    if (B == 0) return 0;
    argmax_scatter_kernel<<<B, 1024, 0, ctx.stream>>>(logits, row_stride, row_off, tokens, T, V, cur);
    FXF_LAUNCHED(ctx);
    return 0;
}

}  // namespace fxf
