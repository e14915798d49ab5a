// Dense-contraction ops: Linear, LinearRelu, FeedForward, MHA — single GPU and tensor-parallel.
//
// Reference semantics (LibTorch-delegating CPU kernels):
//   linear       out = x · w^T + b                          csrc/kernels/cpu/linear.cpp:5-12
//   linear_relu  out = relu(x · w^T + b)                    csrc/kernels/cpu/linear_relu.cpp:5-12
//   feedforward  out = (relu(x · w1^T + b1)) · w2^T + b2    csrc/kernels/cpu/feedforward.cpp:5-14
//   mha          packed QKV projection, masked softmax attention, output projection
//                                                            csrc/kernels/cpu/mha.cpp:5-52
// The reference allocates an intermediate per node (csrc/runtime/cache.cpp:28-37, 54-73:
// FeedForward [M,F]; MHA qkv [B,T,3D], scores [B,H,T,T], ctx [B,T,D]).  Here every node
// borrows the engine's single shared scratch region for the duration of its launches, and the
// score matrix is never materialised.
//
// Tensor parallelism (the reference has none).  With tp_size = n ranks, each holding the whole graph file:
//   MHA          heads are sharded: rank r keeps heads [r·H/n, (r+1)·H/n): the matching rows of each of the
//                Q, K, V thirds of the packed weight and bias, and the matching COLUMNS of the output
//                projection.  Its out-projection yields a partial [M,D]; bias only on rank 0; all-reduce.
//   FeedForward  w1 rows / b1 entries [r·F/n, (r+1)·F/n) (column-parallel), ReLU local, the matching
//                columns of w2 (row-parallel) -> partial [M,P]; b2 only on rank 0; all-reduce.
//   final Linear (optional) its rows (vocabulary) are sharded; each rank writes only its column block of
//                the logits, and the decode argmax combines the ranks' candidates.
// Everything else is replicated.  The slices are gathered once, at engine build, into the node's
// persistent memory (and split into TF32 hi/lo there), so a forward never touches the unsharded weights.
#include <algorithm>

#include "../runtime.hpp"

namespace fxf {

// FXF_GEMM_AUTO takes the cheapest fp32-grade arithmetic the tensor cores offer: one TF32 product plus two bf16 corrections
// (weights whose rows are not multiples of 8 elements, and convolutions, stay with three TF32 products).
static bool mixed_arithmetic(int gemm_mode) { return gemm_mode == FXF_GEMM_TF32_BF16X2 || gemm_mode == FXF_GEMM_AUTO; }

static bool use_tc(const GemmArgs& a, int gemm_mode) {
    if (gemm_mode == FXF_GEMM_FP32_SIMT) return false;
    return gemm_tc_supported(a);
}

namespace {
__global__ void __launch_bounds__(256) residual_epilogue_kernel(float* __restrict__ out, const float* __restrict__ res, int64_t n, int relu) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = out[i] + res[i];
        if (relu) v = v > 0.f ? v : (v != v ? v : 0.f);
        out[i] = v;
    }
}
}  // namespace

int launch_residual_epilogue(float* out, const float* residual, int64_t n, bool relu, ExecCtx& ctx) {
    if (n == 0) return 0;
    int64_t blocks = (n + 255) / 256, cap = int64_t(ctx.sm_count) * 8;
    tag_launch(ctx, "residual_epilogue", double(n), 12.0 * double(n));
    residual_epilogue_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx.stream>>>(out, residual, n, relu ? 1 : 0);
    FXF_LAUNCHED(ctx);
    return 0;
}

int launch_gemm(const GemmArgs& a, ExecCtx& ctx) {
    if (a.M == 0 || a.N == 0) return 0;
    if (use_tc(a, ctx.gemm_mode)) return launch_gemm_tc(a, ctx);
    FXF_CHECK(a.push_rows == 0, "gemm: a row-pushed output needs the tensor-core kernels");
    if (a.residual != nullptr) {
        // the FFMA kernels have no residual epilogue: plain GEMM, then act(out + residual) in place (dense rows only)
        FXF_CHECK(a.ldo == a.N, "gemm: a fused residual needs a dense output on the fp32 FFMA path");
        GemmArgs plain = a;
        plain.residual = nullptr;
        plain.relu = false;
        if (launch_gemm(plain, ctx)) return 1;
        return launch_residual_epilogue(a.out, a.residual, a.M * a.N, a.relu, ctx);
    }
    FXF_CHECK(ctx.gemm_mode != FXF_GEMM_TF32X3, "gemm: FXF_GEMM_TF32X3 was requested but the shape M=%lld N=%lld K=%lld (or its alignment) is not supported by the tensor-core kernel",
              (long long)a.M, (long long)a.N, (long long)a.K);
    return launch_gemm_simt(a, ctx);
}

std::string gemm_variant_name(const GemmArgs& a, int gemm_mode, int sm_count, bool pairs) {
    if (gemm_mode == FXF_GEMM_BF16 && gemm_tc_shape_ok(a.M, a.N, a.K) && a.K % 8 == 0) return std::string("tcgen05-bf16-128x") + (a.N > 128 ? "192" : "128");
    if (mixed_arithmetic(gemm_mode) && gemm_tc_shape_ok(a.M, a.N, a.K) && a.K % 8 == 0) return gemm_tc_mixed_variant(a.M, a.N, a.K, sm_count, true, false, nullptr, pairs);
    if (gemm_mode != FXF_GEMM_FP32_SIMT && gemm_tc_shape_ok(a.M, a.N, a.K)) return gemm_tc_variant(a.M, a.N, a.K, sm_count, true, false, nullptr, pairs);
    static const char* names[] = {"simt128x128", "simt64x64", "simt32x32", "skinny32x8"};
    return names[simt_tile_choice(a.M, a.N, sm_count)];
}

namespace {

// A dense fp32 matrix [rows, cols] (a vector when cols == 1), assembled from up to three row
// ranges and one column range of a graph tensor.  `whole` slices use the tensor in place.
struct Slice {
    int input = -1;                 // position of the source tensor in the node's input_ids
    int n_ranges = 0;
    int64_t row0[3] = {0, 0, 0}, nrow[3] = {0, 0, 0};
    int64_t col0 = 0, ncol = 0;     // column window
    int64_t src_ld = 0;             // row pitch of the source (elements)
    bool whole = true;              // the slice is the entire tensor: no copy
    bool split = false;             // TF32 hi/lo copies wanted (tensor-core GEMM operand)
    bool bf16 = false;              // bf16 mode: one bf16 copy instead (hi points to it, lo stays NULL)
    bool mixed = false;             // mixed mode: hi = TF32 high part (fp32), lo -> bf16(w - hi)
    bool drop = false;              // replaced by "no bias" (rank != 0 of a row-parallel product)
    size_t off_copy = 0, off_split = 0;  // byte offsets inside the plan's persistent memory
    const float *ptr = nullptr, *hi = nullptr, *lo = nullptr;  // resolved by prepare()
    int64_t rows() const { return nrow[0] + nrow[1] + nrow[2]; }
    int64_t elems() const { return rows() * ncol; }
};

struct DensePlan : NodePlan {
    Slice s[6];  // meaning depends on the op (see the plan builders)
    int n = 0;
    // dims the kernels need again
    int64_t M = 0, heads_local = 0, head0 = 0, n_local = 0, col_off = 0;
    size_t cache_off = 0;   // CachedMHA: byte offset of the K/V cache inside the persistent memory
    bool prepared = false;
    bool bf16_mode = false;   // set by the plan builders from the engine's GEMM mode
    bool mixed_mode = false;  // likewise: FXF_GEMM_TF32_BF16X2

    Slice& add(int input, int64_t rows, int64_t cols) {
        Slice& x = s[n++];
        x.input = input;
        x.n_ranges = 1;
        x.row0[0] = 0; x.nrow[0] = rows;
        x.col0 = 0; x.ncol = cols; x.src_ld = cols;
        return x;
    }
    void reserve(Slice& x, bool want_split) {
        if (x.drop) return;
        if (!x.whole) {
            x.off_copy = persist_bytes;
            persist_bytes += round_up(size_t(x.elems()) * sizeof(float), 256);
        }
        if (want_split) {
            x.split = true;
            x.bf16 = bf16_mode && x.ncol % 8 == 0;
            x.mixed = mixed_mode && x.ncol % 8 == 0;   // bf16 rows must be 16-byte multiples for TMA; same bytes as a hi/lo pair
            x.off_split = persist_bytes;
            persist_bytes += round_up(x.bf16 ? size_t(x.elems()) * 2 : size_t(2) * size_t(x.elems()) * sizeof(float), 256);
        }
    }
    int prepare(Registry& reg, const TensorIds& in, const TensorIds&, const Params&, ExecCtx& ctx) override {
        for (int i = 0; i < n; i++) {
            Slice& x = s[i];
            if (x.drop) continue;
            const float* src = static_cast<const float*>(reg[in[x.input]].ptr);
            if (x.whole) {
                x.ptr = src;
            } else {
                FXF_CHECK(persist != nullptr, "dense plan: persistent memory was not assigned");
                float* dst = reinterpret_cast<float*>(static_cast<char*>(persist) + x.off_copy);
                int64_t done = 0;
                for (int r = 0; r < x.n_ranges; r++) {
                    if (x.nrow[r] == 0) continue;
                    FXF_CUDA(cudaMemcpy2DAsync(dst + done * x.ncol, size_t(x.ncol) * 4, src + x.row0[r] * x.src_ld + x.col0, size_t(x.src_ld) * 4,
                                               size_t(x.ncol) * 4, size_t(x.nrow[r]), cudaMemcpyDeviceToDevice, ctx.stream));
                    done += x.nrow[r];
                }
                x.ptr = dst;
            }
            if (x.split) {
                FXF_CHECK(persist != nullptr, "dense plan: persistent memory was not assigned");
                float* h = reinterpret_cast<float*>(static_cast<char*>(persist) + x.off_split);
                if (x.bf16) {
                    if (launch_convert_bf16(x.ptr, h, x.elems(), ctx)) return 1;
                    x.hi = h;
                    x.lo = nullptr;
                } else if (x.mixed) {
                    if (launch_split_mixed(x.ptr, h, h + x.elems(), x.elems(), ctx)) return 1;
                    x.hi = h;
                    x.lo = h + x.elems();
                } else {
                    if (launch_split_tf32(x.ptr, h, h + x.elems(), x.elems(), ctx)) return 1;
                    x.hi = h;
                    x.lo = h + x.elems();
                }
            }
        }
        prepared = true;
        return 0;
    }
};
inline const DensePlan* dense(const NodePlan* p) { return static_cast<const DensePlan*>(p); }

// M < 64 (batch-sized layers, single-position decode steps) never takes the tensor-core path: those problems are weight
// reads, served by the fp32 FFMA few-rows kernels from the fp32 weights (half the bytes of a hi/lo pair).
bool want_tc(const PlanEnv& env, int64_t M, int64_t N, int64_t K) { return env.gemm_mode != FXF_GEMM_FP32_SIMT && gemm_tc_shape_ok(M, N, K); }

void fill_gemm(GemmArgs& g, const float* x, const Slice& w, const Slice* bias, float* out, int64_t M, int64_t ldx, int64_t ldo, bool relu) {
    g.x = x; g.w = w.ptr; g.w_hi = w.hi; g.w_lo = w.lo; g.w_is_bf16 = w.bf16; g.w_mixed = w.mixed;
    g.bias = (bias && !bias->drop) ? bias->ptr : nullptr;
    g.out = out; g.M = M; g.N = w.rows(); g.K = w.ncol;
    g.ldx = ldx; g.ldw = w.ncol; g.ldo = ldo; g.relu = relu;
}

int64_t leading_rows(const FxfTensor& x) {
    int64_t m = 1;
    for (int k = 0; k + 1 < x.rank; k++) m *= x.shape[k];
    return m;
}

// ---- Linear / LinearRelu ------------------------------------------------------------------------------
// slices: s[0] = weight rows kept by this rank, s[1] = matching bias entries
int run_linear(Registry& reg, const TensorIds& in, const TensorIds& out, bool relu, const NodePlan* plan, ExecCtx& ctx, const char* who) {
    FXF_CHECK(in.size() >= 3 && out.size() >= 1, "%s: expects [x, weight, bias]", who);
    const FxfTensor &x = reg[in[0]], &w = reg[in[1]], &b = reg[in[2]], &o = reg[out[0]];
    FXF_CHECK(x.dtype == FXF_F32 && w.dtype == FXF_F32 && b.dtype == FXF_F32 && o.dtype == FXF_F32, "%s: only float32 is supported", who);
    FXF_CHECK(w.rank == 2 && x.rank >= 1, "%s: weight must be [N,K] and x at least 1-D", who);
    const int64_t K = x.shape[x.rank - 1], N = w.shape[0], M = leading_rows(x);
    FXF_CHECK(w.shape[1] == K, "%s: x inner size %lld does not match weight K %lld", who, (long long)K, (long long)w.shape[1]);
    FXF_CHECK(numel(b) == N, "%s: bias size does not match weight rows", who);
    FXF_CHECK(numel(o) == M * N, "%s: output size mismatch", who);
    const DensePlan* pl = dense(plan);
    FXF_CHECK(pl != nullptr && pl->n == 2 && pl->prepared, "%s: the node was not prepared", who);
    GemmArgs g;
    fill_gemm(g, static_cast<const float*>(x.ptr), pl->s[0], &pl->s[1], static_cast<float*>(o.ptr) + pl->col_off, M, K, N, relu);
    if (pl->col_off == 0 && pl->s[0].rows() == N) apply_fusion(ctx, g, false);   // never with a column-sharded output
    return launch_gemm(g, ctx);
}

}  // namespace

int k_linear(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan* plan, ExecCtx& ctx) {
    return run_linear(reg, in, out, false, plan, ctx, "linear");
}

int linear_on_rows(const NodePlan* plan, const float* x_rows, int64_t M, int64_t ldx, float* out, int64_t ldo, ExecCtx& ctx) {
    const DensePlan* pl = dense(plan);
    FXF_CHECK(pl != nullptr && pl->n == 2 && pl->prepared, "linear (rows): the node was not prepared");
    if (M == 0 || pl->s[0].rows() == 0) return 0;
    GemmArgs g;
    fill_gemm(g, x_rows, pl->s[0], &pl->s[1], out + pl->col_off, M, ldx, ldo, false);
    // few rows against a large weight: the tensor-core kernel streams the pre-split weight once; rows beyond M are zero fill
    if (ctx.gemm_mode != FXF_GEMM_FP32_SIMT && gemm_tc_supported(g, true)) return launch_gemm_tc(g, ctx, true);
    return launch_gemm_simt(g, ctx);
}
int k_linear_relu(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan* plan, ExecCtx& ctx) {
    return run_linear(reg, in, out, true, plan, ctx, "linear_relu");
}

std::unique_ptr<NodePlan> plan_linear(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const PlanEnv& env) {
    auto p = std::make_unique<DensePlan>();
    p->bf16_mode = env.gemm_mode == FXF_GEMM_BF16;
    p->mixed_mode = mixed_arithmetic(env.gemm_mode);
    if (in.size() < 3 || out.size() < 1) return p;
    const FxfTensor &x = reg[in[0]], &w = reg[in[1]];
    if (w.rank != 2 || x.rank < 1) return p;
    const int64_t K = x.shape[x.rank - 1], N = w.shape[0], M = leading_rows(x);
    Slice& ws = p->add(1, N, K);
    Slice& bs = p->add(2, N, 1);
    p->n_local = N;
    if (env.shard_output_cols && env.tp_size > 1) {
        // vocabulary-parallel head: rank r owns rows [r*c, min(N, (r+1)*c)) with c = ceil(N / n)
        int64_t c = (N + env.tp_size - 1) / env.tp_size, r0 = std::min<int64_t>(N, c * env.tp_rank), r1 = std::min<int64_t>(N, r0 + c);
        ws.row0[0] = r0; ws.nrow[0] = r1 - r0; ws.whole = false;
        bs.row0[0] = r0; bs.nrow[0] = r1 - r0; bs.whole = false;
        p->col_off = r0;
        p->n_local = r1 - r0;
    }
    p->reserve(ws, want_tc(env, M, p->n_local, K));
    p->reserve(bs, false);
    p->M = M;
    p->flops = 2.0 * double(M) * double(p->n_local) * double(K);
    p->bytes = 4.0 * (double(M) * K + double(p->n_local) * K + double(p->n_local) + double(M) * p->n_local);
    GemmArgs g;
    g.M = M; g.N = p->n_local; g.K = K;
    p->variant = gemm_variant_name(g, env.gemm_mode, 148, env.tc_pairs);
    return p;
}

// Last step of a row-parallel product (the second GEMM of MHA / CrossMHA / FeedForward).  Single GPU or a node that is
// replicated on every rank: the GEMM with a folded residual Add, if any.  Sharded node: the GEMM leaves this rank's
// partial sums in the node's own output tensor, then either ONE fused exchange (sum over the ranks + residual + LayerNorm,
// kernels/tp_exchange.cu) when the engine folded the following nodes into it, or the plain all-reduce.
static int finish_row_parallel(GemmArgs& g2, int64_t M, int64_t N, bool sharded, ExecCtx& ctx) {
    if (sharded && ctx.tp_size > 1 && ctx.xchg.enabled) {
        FXF_CHECK(g2.ldo == N && tp_exchange_usable(ctx.xchg, g2.out, M, N, ctx), "tensor-parallel exchange: the folded nodes cannot be served");
        // On the tensor-core kernels the product stores each row straight into its owner's exchange window (peer stores from
        // the epilogue, behind the product's own time): the exchange then reads local memory only.
        float* windows[kMaxTpRanks] = {};
        const bool pushed = g2.residual == nullptr && use_tc(g2, ctx.gemm_mode) && tp_push_usable(M, N, ctx);
        if (pushed) {
            for (int r = 0; r < ctx.tp_size; r++) windows[r] = tp_push_window(r, ctx);
            g2.push_out = windows;
            g2.push_rows = M / ctx.tp_size;
            g2.push_rank = ctx.tp_rank;
        }
        if (launch_gemm(g2, ctx)) return 1;
        ctx.xchg.consumed = true;
        return launch_tp_exchange(ctx.xchg, g2.out, M, N, ctx, pushed);
    }
    apply_fusion(ctx, g2, sharded);
    if (launch_gemm(g2, ctx)) return 1;
    return sharded ? tp_all_reduce_sum(g2.out, M * N, ctx) : 0;
}

// ---- FeedForward ------------------------------------------------------------------------------
// slices: s[0] = w1 rows of this rank [Fl, D], s[1] = b1 entries [Fl], s[2] = w2 columns of this rank [P, Fl], s[3] = b2
int k_feedforward(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan* plan, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 5 && out.size() >= 1, "feedforward: expects [x, w1, b1, w2, b2]");
    const FxfTensor &x = reg[in[0]], &w1 = reg[in[1]], &b1 = reg[in[2]], &w2 = reg[in[3]], &b2 = reg[in[4]], &o = reg[out[0]];
    FXF_CHECK(x.dtype == FXF_F32 && o.dtype == FXF_F32, "feedforward: only float32 is supported");
    FXF_CHECK(w1.rank == 2 && w2.rank == 2 && x.rank >= 1, "feedforward: weights must be 2-D");
    const int64_t K = x.shape[x.rank - 1], F = w1.shape[0], P = w2.shape[0], M = leading_rows(x);
    FXF_CHECK(w1.shape[1] == K && w2.shape[1] == F, "feedforward: weight shapes do not chain (x[..,%lld], w1[%lld,%lld], w2[%lld,%lld])",
              (long long)K, (long long)w1.shape[0], (long long)w1.shape[1], (long long)w2.shape[0], (long long)w2.shape[1]);
    FXF_CHECK(numel(b1) == F && numel(b2) == P, "feedforward: bias sizes do not match");
    FXF_CHECK(numel(o) == M * P, "feedforward: output size mismatch");
    const DensePlan* pl = dense(plan);
    FXF_CHECK(pl != nullptr && pl->n == 4 && pl->prepared, "feedforward: the node was not prepared");
    const int64_t Fl = pl->s[0].rows();
    size_t need = size_t(M) * size_t(Fl) * sizeof(float);
    FXF_CHECK(ctx.scratch_bytes >= need && (need == 0 || ctx.scratch != nullptr), "feedforward: scratch too small (%zu < %zu bytes)", ctx.scratch_bytes, need);
    float* hidden = static_cast<float*>(ctx.scratch);
    GemmArgs g1, g2;
    fill_gemm(g1, static_cast<const float*>(x.ptr), pl->s[0], &pl->s[1], hidden, M, K, Fl, true);
    if (launch_gemm(g1, ctx)) return 1;
    fill_gemm(g2, hidden, pl->s[2], &pl->s[3], static_cast<float*>(o.ptr), M, Fl, P, false);
    return finish_row_parallel(g2, M, P, pl->tp_sharded, ctx);
}

std::unique_ptr<NodePlan> plan_feedforward(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const PlanEnv& env) {
    auto p = std::make_unique<DensePlan>();
    p->bf16_mode = env.gemm_mode == FXF_GEMM_BF16;
    p->mixed_mode = mixed_arithmetic(env.gemm_mode);
    if (in.size() < 5 || out.size() < 1) return p;
    const FxfTensor &x = reg[in[0]], &w1 = reg[in[1]], &w2 = reg[in[3]];
    if (w1.rank != 2 || w2.rank != 2 || x.rank < 1) return p;
    const int64_t K = x.shape[x.rank - 1], F = w1.shape[0], P = w2.shape[0], M = leading_rows(x);
    const int n = env.tp_size > 1 && F % env.tp_size == 0 ? env.tp_size : 1;  // hidden width must divide evenly, else replicate
    const int64_t Fl = F / n, f0 = (n > 1 ? env.tp_rank : 0) * Fl;
    Slice& s_w1 = p->add(1, F, K);
    Slice& s_b1 = p->add(2, F, 1);
    Slice& s_w2 = p->add(3, P, F);
    Slice& s_b2 = p->add(4, P, 1);
    p->tp_sharded = n > 1;
    if (n > 1) {
        s_w1.row0[0] = f0; s_w1.nrow[0] = Fl; s_w1.whole = false;
        s_b1.row0[0] = f0; s_b1.nrow[0] = Fl; s_b1.whole = false;
        s_w2.col0 = f0; s_w2.ncol = Fl; s_w2.whole = false;
        s_b2.drop = env.tp_rank != 0;
    } else if (env.tp_size > 1) {
        p->variant = "replicated ";
    }
    p->reserve(s_w1, want_tc(env, M, Fl, K));
    p->reserve(s_b1, false);
    p->reserve(s_w2, want_tc(env, M, P, Fl));
    p->reserve(s_b2, false);
    p->M = M;
    p->scratch_bytes = size_t(M) * size_t(Fl) * sizeof(float);
    p->flops = 2.0 * double(M) * double(Fl) * double(K) + 2.0 * double(M) * double(P) * double(Fl);
    p->bytes = 4.0 * (double(M) * K + double(Fl) * K + Fl + double(P) * Fl + P + double(M) * P);
    GemmArgs g1, g2;
    g1.M = M; g1.N = Fl; g1.K = K;
    g2.M = M; g2.N = P; g2.K = Fl;
    p->variant += gemm_variant_name(g1, env.gemm_mode, 148, env.tc_pairs) + "+" + gemm_variant_name(g2, env.gemm_mode, 148, env.tc_pairs);
    return p;
}

// ---- MHA ----------------------------------------------------------------------------------------
// slices: s[0] = packed QKV rows of the local heads [3*Dl, D], s[1] = their bias [3*Dl],
//         s[2] = output-projection columns of the local heads [D, Dl], s[3] = output bias [D]
int k_mha(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan* plan, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 6 && out.size() >= 1, "mha: expects [x, mask, qkv_weight, qkv_bias, out_weight, out_bias]");
    FXF_CHECK(p.ints.size() >= 4 && p.floats.size() >= 1, "mha: expects ints [H, head_dim, d_model, qkv_dim] and floats [scale_divisor]");
    const FxfTensor &x = reg[in[0]], &mask = reg[in[1]], &wq = reg[in[2]], &bq = reg[in[3]], &wo = reg[in[4]], &bo = reg[in[5]], &o = reg[out[0]];
    FXF_CHECK(x.rank == 3, "mha: x must be [B,T,D]");
    const int64_t B = x.shape[0], T = x.shape[1], H = p.ints[0], hd = p.ints[1], D = p.ints[2], QKV = p.ints[3], M = B * T;
    FXF_CHECK(H > 0 && hd > 0 && H * hd == D && QKV == 3 * D, "mha: inconsistent head parameters");
    FXF_CHECK(x.shape[2] == D, "mha: x inner size does not match d_model");
    FXF_CHECK(wq.rank == 2 && wq.shape[0] == QKV && wq.shape[1] == D && numel(bq) == QKV, "mha: packed QKV weight/bias shape mismatch");
    FXF_CHECK(wo.rank == 2 && wo.shape[0] == D && wo.shape[1] == D && numel(bo) == D, "mha: output projection shape mismatch");
    FXF_CHECK(numel(o) == M * D, "mha: output size mismatch");
    FXF_CHECK(x.dtype == FXF_F32 && o.dtype == FXF_F32, "mha: only float32 activations are supported");
    FXF_CHECK(mask.dtype == FXF_BOOL, "mha: mask must be a bool tensor");
    FXF_CHECK(mask.rank <= 4, "mha: mask rank must be <= 4");
    // broadcast the mask to [B,H,T,T]: right-align its dims, stride 0 where its extent is 1
    int64_t want[4] = {B, H, T, T}, ms[4] = {0, 0, 0, 0};
    for (int k = 0; k < mask.rank; k++) {
        int tgt = 4 - mask.rank + k;
        FXF_CHECK(mask.shape[k] == want[tgt] || mask.shape[k] == 1, "mha: mask shape is not broadcastable to [B,H,T,T]");
        ms[tgt] = mask.shape[k] == 1 ? 0 : mask.stride[k];
    }
    const DensePlan* pl = dense(plan);
    FXF_CHECK(pl != nullptr && pl->n == 4 && pl->prepared, "mha: the node was not prepared");
    const int64_t Hl = pl->heads_local, Dl = Hl * hd, QKVl = 3 * Dl;
    size_t need = size_t(M) * size_t(QKVl + Dl) * sizeof(float);
    FXF_CHECK(ctx.scratch_bytes >= need && (need == 0 || ctx.scratch != nullptr), "mha: scratch too small (%zu < %zu bytes)", ctx.scratch_bytes, need);
    float* qkv = static_cast<float*>(ctx.scratch);
    float* cx = qkv + M * QKVl;
    float* vt = cx + M * Dl;  // only present when the plan reserved it
    const bool have_vt = ctx.scratch_bytes >= need + attention_tc_scratch_bytes(B, T, Hl);

    GemmArgs g;
    fill_gemm(g, static_cast<const float*>(x.ptr), pl->s[0], &pl->s[1], qkv, M, D, QKVl, false);
    // Where the projection runs on a tensor-core variant whose column halves are multiples of half a head, its epilogue writes the V third
    // transposed (and the finite flags of V) straight into the attention kernel's V^T buffer: no transpose launch.
    bool v_transposed = false;
    if (have_vt && hd == 64 && ctx.gemm_mode != FXF_GEMM_FP32_SIMT && use_tc(g, ctx.gemm_mode)) {
        g.vt_out = vt;
        g.vt_flags = reinterpret_cast<unsigned char*>(vt + size_t(B) * size_t(Hl) * size_t(T) * 64);
        g.vt_col0 = 2 * Dl;
        g.vt_T = int(T); g.vt_heads = int(Hl); g.vt_n32 = int((T + 31) / 32);
        v_transposed = gemm_tc_vt_ok(g, ctx);
        if (!v_transposed) { g.vt_out = nullptr; g.vt_flags = nullptr; }
    }
    if (launch_gemm(g, ctx)) return 1;

    AttnArgs a;
    a.qkv = qkv; a.ctx = cx;
    a.mask = static_cast<const uint8_t*>(mask.ptr) + pl->head0 * ms[1];  // local head 0 is global head `head0`
    a.B = int(B); a.T = int(T); a.H = int(Hl); a.hd = int(hd);
    a.ld_qkv = QKVl; a.q_off = 0; a.k_off = Dl; a.v_off = 2 * Dl; a.ld_ctx = Dl;
    a.mask_sb = ms[0]; a.mask_sh = ms[1]; a.mask_sq = ms[2]; a.mask_sk = ms[3];
    a.scale_divisor = p.floats[0];
    if (have_vt && attention_tc_supported(a, ctx.gemm_mode)) {
        if (launch_attention_tc(a, vt, ctx, v_transposed)) return 1;
    } else {
        FXF_CHECK(!v_transposed, "mha: the projection wrote V transposed but the tensor-core attention kernel cannot run");
        if (launch_attention(a, ctx)) return 1;
    }

    GemmArgs g2;
    fill_gemm(g2, cx, pl->s[2], &pl->s[3], static_cast<float*>(o.ptr), M, Dl, D, false);
    return finish_row_parallel(g2, M, D, pl->tp_sharded, ctx);
}

std::unique_ptr<NodePlan> plan_mha(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const PlanEnv& env) {
    auto pl = std::make_unique<DensePlan>();
    pl->bf16_mode = env.gemm_mode == FXF_GEMM_BF16;
    pl->mixed_mode = mixed_arithmetic(env.gemm_mode);
    if (in.size() < 6 || out.size() < 1 || p.ints.size() < 4 || reg[in[0]].rank != 3) return pl;
    const FxfTensor& x = reg[in[0]];
    const int64_t B = x.shape[0], T = x.shape[1], H = p.ints[0], hd = p.ints[1], D = p.ints[2], QKV = p.ints[3], M = B * T;
    if (H <= 0 || hd <= 0) return pl;
    const int n = env.tp_size > 1 && H % env.tp_size == 0 ? env.tp_size : 1;  // heads must divide evenly, else replicate
    const int64_t Hl = H / n, h0 = (n > 1 ? env.tp_rank : 0) * Hl, Dl = Hl * hd;
    pl->heads_local = Hl;
    pl->head0 = h0;
    pl->tp_sharded = n > 1;
    Slice& s_wq = pl->add(2, QKV, D);
    Slice& s_bq = pl->add(3, QKV, 1);
    Slice& s_wo = pl->add(4, D, D);
    Slice& s_bo = pl->add(5, D, 1);
    if (n > 1) {
        for (Slice* s : {&s_wq, &s_bq}) {
            s->n_ranges = 3;
            for (int third = 0; third < 3; third++) {
                s->row0[third] = third * D + h0 * hd;
                s->nrow[third] = Dl;
            }
            s->whole = false;
        }
        s_wo.col0 = h0 * hd; s_wo.ncol = Dl; s_wo.whole = false;
        s_bo.drop = env.tp_rank != 0;
    } else if (env.tp_size > 1) {
        pl->variant = "replicated ";
    }
    pl->reserve(s_wq, want_tc(env, M, 3 * Dl, D));
    pl->reserve(s_bq, false);
    pl->reserve(s_wo, want_tc(env, M, D, Dl));
    pl->reserve(s_bo, false);
    pl->M = M;
    pl->scratch_bytes = size_t(M) * size_t(3 * Dl + Dl) * sizeof(float);
    const bool tc_attn = env.gemm_mode != FXF_GEMM_FP32_SIMT && hd == 64 && T % 4 == 0 && T >= 16 && T <= 4096 && Dl % 4 == 0;   // the tcgen05 kernel covers at most 32 blocks of 128 keys
    if (tc_attn) pl->scratch_bytes += attention_tc_scratch_bytes(B, T, Hl);
    pl->flops = 2.0 * M * double(3 * Dl) * D + 4.0 * double(B) * Hl * double(T) * T * hd + 2.0 * double(M) * D * Dl;
    pl->bytes = 4.0 * (2.0 * double(M) * D + double(3 * Dl) * D + 3 * Dl + double(D) * Dl + D) + double(reg[in[1]].nbytes);
    GemmArgs g1, g2;
    g1.M = M; g1.N = 3 * Dl; g1.K = D;
    g2.M = M; g2.N = D; g2.K = Dl;
    pl->variant += gemm_variant_name(g1, env.gemm_mode, 148, env.tc_pairs) + (tc_attn ? "+attn-tcgen05-tf32+2bf16+" : "+flash-fp32+") + gemm_variant_name(g2, env.gemm_mode, 148, env.tc_pairs);
    return pl;
}

// ---- CrossMHA (no counterpart in the reference runtime) --------------------------------------------------
// Attention whose queries come from one sequence and whose keys / values from another — the decoder's second
// attention of an encoder-decoder Transformer (reference model: layers/attention.py:19-33 called as
// cross_attn(norm2(x), encoder_output, encoder_output, src_mask), blocks/decoder_block.py:22).  The reference's QKV
// packing needs three Linear siblings on ONE input (matchers.py:615-621), so its compile passes cannot lower this
// call; this opcode is an extension with the same arithmetic as MHA:
//     q = x·Wq^T + bq   [B,Tq,D];   k | v = memory·Wkv^T + bkv   [B,Tk,2D]  (K rows 0..D, V rows D..2D of Wkv)
//     out = softmax(mask_fill(q·k^T / scale_divisor)) · v, heads re-interleaved, then ·Wo^T + bo.
// inputs [x, memory, mask, Wq[D,D], bq[D], Wkv[2D,D], bkv[2D], Wo[D,D], bo[D]]; ints [H, head_dim, D, 2D]; floats [scale_divisor].
// slices: s[0] = Wq rows of the local heads, s[1] = their bias, s[2] = Wkv rows of the local heads (K block, V block),
//         s[3] = their bias, s[4] = Wo columns of the local heads, s[5] = bo
int k_cross_mha(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan* plan, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 9 && out.size() >= 1, "cross_mha: expects [x, memory, mask, q_weight, q_bias, kv_weight, kv_bias, out_weight, out_bias]");
    FXF_CHECK(p.ints.size() >= 4 && p.floats.size() >= 1, "cross_mha: expects ints [H, head_dim, d_model, kv_dim] and floats [scale_divisor]");
    const FxfTensor &x = reg[in[0]], &mem = reg[in[1]], &mask = reg[in[2]], &wq = reg[in[3]], &bq = reg[in[4]], &wkv = reg[in[5]], &bkv = reg[in[6]],
                    &wo = reg[in[7]], &bo = reg[in[8]], &o = reg[out[0]];
    FXF_CHECK(x.rank == 3 && mem.rank == 3, "cross_mha: x must be [B,Tq,D] and memory [B,Tk,D]");
    const int64_t B = x.shape[0], Tq = x.shape[1], Tk = mem.shape[1], H = p.ints[0], hd = p.ints[1], D = p.ints[2], KV = p.ints[3];
    const int64_t Mq = B * Tq, Mk = B * Tk;
    FXF_CHECK(H > 0 && hd > 0 && H * hd == D && KV == 2 * D, "cross_mha: inconsistent head parameters");
    FXF_CHECK(x.shape[2] == D && mem.shape[2] == D && mem.shape[0] == B, "cross_mha: x / memory shapes do not match d_model or each other");
    FXF_CHECK(wq.rank == 2 && wq.shape[0] == D && wq.shape[1] == D && numel(bq) == D, "cross_mha: query projection shape mismatch");
    FXF_CHECK(wkv.rank == 2 && wkv.shape[0] == KV && wkv.shape[1] == D && numel(bkv) == KV, "cross_mha: packed KV weight/bias shape mismatch");
    FXF_CHECK(wo.rank == 2 && wo.shape[0] == D && wo.shape[1] == D && numel(bo) == D, "cross_mha: output projection shape mismatch");
    FXF_CHECK(numel(o) == Mq * D, "cross_mha: output size mismatch");
    FXF_CHECK(x.dtype == FXF_F32 && mem.dtype == FXF_F32 && o.dtype == FXF_F32, "cross_mha: only float32 activations are supported");
    FXF_CHECK(mask.dtype == FXF_BOOL && mask.rank <= 4, "cross_mha: mask must be a bool tensor of rank <= 4");
    int64_t want[4] = {B, H, Tq, Tk}, ms[4] = {0, 0, 0, 0};
    for (int k = 0; k < mask.rank; k++) {
        int tgt = 4 - mask.rank + k;
        FXF_CHECK(mask.shape[k] == want[tgt] || mask.shape[k] == 1, "cross_mha: mask shape is not broadcastable to [B,H,Tq,Tk]");
        ms[tgt] = mask.shape[k] == 1 ? 0 : mask.stride[k];
    }
    const DensePlan* pl = dense(plan);
    FXF_CHECK(pl != nullptr && pl->n == 6 && pl->prepared, "cross_mha: the node was not prepared");
    const int64_t Hl = pl->heads_local, Dl = Hl * hd;
    size_t need = (size_t(Mq) * size_t(2 * Dl) + size_t(Mk) * size_t(2 * Dl)) * sizeof(float);
    FXF_CHECK(ctx.scratch_bytes >= need && (need == 0 || ctx.scratch != nullptr), "cross_mha: scratch too small (%zu < %zu bytes)", ctx.scratch_bytes, need);
    float* q = static_cast<float*>(ctx.scratch);   // [Mq, Dl]
    float* kv = q + Mq * Dl;                        // [Mk, 2*Dl]
    float* cx = kv + Mk * 2 * Dl;                   // [Mq, Dl]
    float* vt = cx + Mq * Dl;                       // only present when the plan reserved it
    const bool have_vt = ctx.scratch_bytes >= need + attention_tc_scratch_bytes(B, Tk, Hl);

    GemmArgs g;
    fill_gemm(g, static_cast<const float*>(x.ptr), pl->s[0], &pl->s[1], q, Mq, D, Dl, false);
    if (launch_gemm(g, ctx)) return 1;
    GemmArgs gk;
    fill_gemm(gk, static_cast<const float*>(mem.ptr), pl->s[2], &pl->s[3], kv, Mk, D, 2 * Dl, false);
    if (launch_gemm(gk, ctx)) return 1;

    if (Tk == 0) {  // softmax over no keys: the context is an empty sum
        if (Mq * Dl > 0) FXF_CUDA(cudaMemsetAsync(cx, 0, size_t(Mq) * size_t(Dl) * sizeof(float), ctx.stream));
    } else {
        AttnArgs a;
        a.qkv = q; a.ld_qkv = Dl; a.q_off = 0;
        a.kv = kv; a.ld_kv = 2 * Dl; a.k_off = 0; a.v_off = Dl; a.Tk = int(Tk);
        a.ctx = cx; a.ld_ctx = Dl;
        a.mask = static_cast<const uint8_t*>(mask.ptr) + pl->head0 * ms[1];
        a.B = int(B); a.T = int(Tq); a.H = int(Hl); a.hd = int(hd);
        a.mask_sb = ms[0]; a.mask_sh = ms[1]; a.mask_sq = ms[2]; a.mask_sk = ms[3];
        a.scale_divisor = p.floats[0];
        if (have_vt && attention_tc_supported(a, ctx.gemm_mode)) {
            if (launch_attention_tc(a, vt, ctx)) return 1;
        } else {
            if (launch_attention(a, ctx)) return 1;
        }
    }

    GemmArgs g2;
    fill_gemm(g2, cx, pl->s[4], &pl->s[5], static_cast<float*>(o.ptr), Mq, Dl, D, false);
    return finish_row_parallel(g2, Mq, D, pl->tp_sharded, ctx);
}

std::unique_ptr<NodePlan> plan_cross_mha(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const PlanEnv& env) {
    auto pl = std::make_unique<DensePlan>();
    pl->bf16_mode = env.gemm_mode == FXF_GEMM_BF16;
    pl->mixed_mode = mixed_arithmetic(env.gemm_mode);
    if (in.size() < 9 || out.size() < 1 || p.ints.size() < 4 || reg[in[0]].rank != 3 || reg[in[1]].rank != 3) return pl;
    const FxfTensor &x = reg[in[0]], &mem = reg[in[1]];
    const int64_t B = x.shape[0], Tq = x.shape[1], Tk = mem.shape[1], H = p.ints[0], hd = p.ints[1], D = p.ints[2], KV = p.ints[3];
    const int64_t Mq = B * Tq, Mk = B * Tk;
    if (H <= 0 || hd <= 0) return pl;
    const int n = env.tp_size > 1 && H % env.tp_size == 0 ? env.tp_size : 1;
    const int64_t Hl = H / n, h0 = (n > 1 ? env.tp_rank : 0) * Hl, Dl = Hl * hd;
    pl->heads_local = Hl;
    pl->head0 = h0;
    pl->tp_sharded = n > 1;
    Slice& s_wq = pl->add(3, D, D);
    Slice& s_bq = pl->add(4, D, 1);
    Slice& s_wkv = pl->add(5, KV, D);
    Slice& s_bkv = pl->add(6, KV, 1);
    Slice& s_wo = pl->add(7, D, D);
    Slice& s_bo = pl->add(8, D, 1);
    if (n > 1) {
        for (Slice* s : {&s_wq, &s_bq}) {
            s->row0[0] = h0 * hd; s->nrow[0] = Dl;
            s->whole = false;
        }
        for (Slice* s : {&s_wkv, &s_bkv}) {
            s->n_ranges = 2;
            for (int half = 0; half < 2; half++) {
                s->row0[half] = half * D + h0 * hd;
                s->nrow[half] = Dl;
            }
            s->whole = false;
        }
        s_wo.col0 = h0 * hd; s_wo.ncol = Dl; s_wo.whole = false;
        s_bo.drop = env.tp_rank != 0;
    } else if (env.tp_size > 1) {
        pl->variant = "replicated ";
    }
    pl->reserve(s_wq, want_tc(env, Mq, Dl, D));
    pl->reserve(s_bq, false);
    pl->reserve(s_wkv, want_tc(env, Mk, 2 * Dl, D));
    pl->reserve(s_bkv, false);
    pl->reserve(s_wo, want_tc(env, Mq, D, Dl));
    pl->reserve(s_bo, false);
    pl->M = Mq;
    pl->scratch_bytes = (size_t(Mq) * size_t(2 * Dl) + size_t(Mk) * size_t(2 * Dl)) * sizeof(float);
    const bool tc_attn = env.gemm_mode != FXF_GEMM_FP32_SIMT && hd == 64 && Tk % 4 == 0 && Tk >= 16 && Tk <= 4096 && Dl % 4 == 0;
    if (tc_attn) pl->scratch_bytes += attention_tc_scratch_bytes(B, Tk, Hl);
    pl->flops = 2.0 * double(Mq) * Dl * D + 2.0 * double(Mk) * 2 * Dl * D + 4.0 * double(B) * Hl * double(Tq) * Tk * hd + 2.0 * double(Mq) * D * Dl;
    pl->bytes = 4.0 * (2.0 * double(Mq) * D + double(Mk) * D + 2.0 * double(Dl) * D + 2.0 * double(Dl) * D + 3 * Dl + D) + double(reg[in[2]].nbytes);
    GemmArgs g1, g2, g3;
    g1.M = Mq; g1.N = Dl; g1.K = D;
    g2.M = Mk; g2.N = 2 * Dl; g2.K = D;
    g3.M = Mq; g3.N = D; g3.K = Dl;
    pl->variant += gemm_variant_name(g1, env.gemm_mode, 148, env.tc_pairs) + "+" + gemm_variant_name(g2, env.gemm_mode, 148, env.tc_pairs) +
                   (tc_attn ? "+attn-tcgen05-tf32+2bf16+" : "+flash-fp32+") + gemm_variant_name(g3, env.gemm_mode, 148, env.tc_pairs);
    return pl;
}

// ---- CachedMHA (no counterpart in the reference runtime) ---------------------------------------------------
// Self-attention of ONE new position per sequence against keys / values kept from earlier positions — the building
// block of incremental ("KV cache") greedy decoding, which the reference lists as future work (README.md:183) and
// replaces by recomputing the whole static buffer every step (inference.py:27-45).  Arithmetic per position is that of
// MHA (csrc/kernels/cpu/mha.cpp:5-52) restricted to query row `pos` under the static decoder mask
// (layers/masks.py:141-154): key j takes part iff j <= pos and tokens[b, j] != pad.
//   inputs [x [B,1,D], tokens int64 [B,T], pos int64 [1] (0-based position of x), Wqkv[3D,D], bqkv[3D], Wo[D,D], bo[D]]
//   ints [H, head_dim, D, 3D, pad_idx]; floats [scale_divisor]; output [B,1,D].
// State: the node's persistent memory holds K and V of every position seen so far, [B, T, 2D]; a call first stores
// row `pos`, then attends over rows 0..pos.  Positions must be fed in order starting at 0.
// slices: s[0] = Wqkv, s[1] = bqkv, s[2] = Wo, s[3] = bo   (replicated under tensor parallelism)
namespace {

constexpr int kCachedAttnThreads = 256;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        float o = __shfl_xor_sync(0xffffffffu, v, off);
        v = is_max ? fmaxf(v, o) : v + o;
    }
    __syncthreads();   // `red` may still be read from a previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < kCachedAttnThreads / 32; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// One block per (head, sequence).  Phase 1: one key per thread (independent 16-byte loads of whole key rows keep many
// requests in flight), scores to shared memory; phase 2: probabilities; phase 3: threads = (output dim, key residue class),
// value rows read coalesced.  Dynamic shared memory: T scores.
__global__ void __launch_bounds__(kCachedAttnThreads) cached_attn_kernel(const float* __restrict__ qkv, float* __restrict__ cache, const int64_t* __restrict__ tokens,
                                                                         const int64_t* __restrict__ pos_ptr, float* __restrict__ ctxo, int T, int D, int hd,
                                                                         float scale_divisor, int64_t pad, int* status) {
    extern __shared__ float scores[];
    __shared__ float red[kCachedAttnThreads / 32], qs[128], part_o[kCachedAttnThreads];
    const int h = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
    const int64_t pos64 = *pos_ptr;
    if (pos64 < 0 || pos64 >= T) {   // uniform: a position outside the cache is reported, nothing is written
        if (t == 0 && status) atomicCAS(status, 0, 3);
        return;
    }
    const int pos = int(pos64), n_keys = pos + 1;
    float* rows = cache + int64_t(b) * T * 2 * D;
    const float* qrow = qkv + int64_t(b) * 3 * D;
    if (t < hd) {
        rows[int64_t(pos) * 2 * D + h * hd + t] = qrow[D + h * hd + t];
        rows[int64_t(pos) * 2 * D + D + h * hd + t] = qrow[2 * D + h * hd + t];
        qs[t] = qrow[h * hd + t];
    }
    __syncthreads();
    // ---- phase 1: scores ----
    const bool vec = (hd % 4 == 0) && (D % 4 == 0);
    float tmax = -INFINITY;
    for (int j = t; j < n_keys; j += kCachedAttnThreads) {
        const float* kj = rows + int64_t(j) * 2 * D + h * hd;
        float dot = 0.f;
        if (vec) {
            for (int d = 0; d < hd; d += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(kj + d);
                dot = fmaf(qs[d], kv.x, dot); dot = fmaf(qs[d + 1], kv.y, dot); dot = fmaf(qs[d + 2], kv.z, dot); dot = fmaf(qs[d + 3], kv.w, dot);
            }
        } else {
            for (int d = 0; d < hd; d++) dot = fmaf(qs[d], kj[d], dot);
        }
        const float sc = tokens[int64_t(b) * T + j] != pad ? dot / scale_divisor : -INFINITY;
        scores[j] = sc;
        tmax = fmaxf(tmax, sc);   // a NaN score does not move the maximum; it reaches the sum below
    }
    const float m_all = block_reduce(tmax, red, true);
    const float m_safe = m_all == -INFINITY ? 0.f : m_all;
    // ---- phase 2: probabilities and their sum ----
    float tsum = 0.f;
    for (int j = t; j < n_keys; j += kCachedAttnThreads) {
        const float pj = expf(scores[j] - m_safe);
        scores[j] = pj;
        tsum += pj;
    }
    const float l_all = block_reduce(tsum, red, false);   // its barriers also publish the probabilities
    // ---- phase 3: context = sum_j p_j * v_j ----
    int hd_pad = 32;
    while (hd_pad < hd) hd_pad <<= 1;
    const int parts = kCachedAttnThreads / hd_pad, d = t % hd_pad, part = t / hd_pad;
    float acc = 0.f;
    if (d < hd) {
        const float* vcol = rows + D + h * hd + d;
        int j = part;
        for (; j + 3 * parts < n_keys; j += 4 * parts) {   // four independent value loads in flight
            const float v0 = vcol[int64_t(j) * 2 * D], v1 = vcol[int64_t(j + parts) * 2 * D], v2 = vcol[int64_t(j + 2 * parts) * 2 * D],
                        v3 = vcol[int64_t(j + 3 * parts) * 2 * D];
            acc = fmaf(scores[j], v0, acc);
            acc = fmaf(scores[j + parts], v1, acc);
            acc = fmaf(scores[j + 2 * parts], v2, acc);
            acc = fmaf(scores[j + 3 * parts], v3, acc);
        }
        for (; j < n_keys; j += parts) acc = fmaf(scores[j], vcol[int64_t(j) * 2 * D], acc);
    }
    part_o[t] = acc;
    __syncthreads();
    if (t < hd) {
        float o = 0.f;
        for (int q = 0; q < parts; q++) o += part_o[q * hd_pad + t];
        ctxo[int64_t(b) * D + h * hd + t] = o / l_all;   // 0/0 = NaN when every key is masked
    }
}

}  // namespace

int k_cached_mha(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan* plan, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 7 && out.size() >= 1, "cached_mha: expects [x, tokens, pos, qkv_weight, qkv_bias, out_weight, out_bias]");
    FXF_CHECK(p.ints.size() >= 5 && p.floats.size() >= 1, "cached_mha: expects ints [H, head_dim, d_model, qkv_dim, pad_idx] and floats [scale_divisor]");
    const FxfTensor &x = reg[in[0]], &tok = reg[in[1]], &pos = reg[in[2]], &wq = reg[in[3]], &bq = reg[in[4]], &wo = reg[in[5]], &bo = reg[in[6]], &o = reg[out[0]];
    FXF_CHECK(x.rank == 3 && x.shape[1] == 1, "cached_mha: x must be [B,1,D]");
    FXF_CHECK(tok.rank == 2 && tok.dtype == FXF_I64 && tok.shape[0] == x.shape[0], "cached_mha: tokens must be int64 [B,T]");
    FXF_CHECK(pos.dtype == FXF_I64 && numel(pos) == 1, "cached_mha: pos must be one int64");
    const int64_t B = x.shape[0], T = tok.shape[1], H = p.ints[0], hd = p.ints[1], D = p.ints[2], QKV = p.ints[3];
    FXF_CHECK(H > 0 && hd > 0 && hd <= 128 && H * hd == D && QKV == 3 * D && x.shape[2] == D, "cached_mha: inconsistent head parameters");
    FXF_CHECK(wq.rank == 2 && wq.shape[0] == QKV && wq.shape[1] == D && numel(bq) == QKV, "cached_mha: packed QKV weight/bias shape mismatch");
    FXF_CHECK(wo.rank == 2 && wo.shape[0] == D && wo.shape[1] == D && numel(bo) == D, "cached_mha: output projection shape mismatch");
    FXF_CHECK(numel(o) == B * D && x.dtype == FXF_F32 && o.dtype == FXF_F32, "cached_mha: output must be float32 [B,1,D]");
    const DensePlan* pl = dense(plan);
    FXF_CHECK(pl != nullptr && pl->n == 4 && pl->prepared && pl->persist != nullptr, "cached_mha: the node was not prepared");
    size_t need = size_t(B) * size_t(4 * D) * sizeof(float);
    FXF_CHECK(ctx.scratch_bytes >= need && ctx.scratch != nullptr, "cached_mha: scratch too small (%zu < %zu bytes)", ctx.scratch_bytes, need);
    float* qkv = static_cast<float*>(ctx.scratch);
    float* cx = qkv + B * 3 * D;
    float* cache = reinterpret_cast<float*>(static_cast<char*>(pl->persist) + pl->cache_off);
    if (B == 0) return 0;
    GemmArgs g;
    fill_gemm(g, static_cast<const float*>(x.ptr), pl->s[0], &pl->s[1], qkv, B, D, QKV, false);
    if (launch_gemm(g, ctx)) return 1;
    tag_launch(ctx, "cached_attention_fp32", 4.0 * double(B) * H * double(T) * hd, 4.0 * 2.0 * double(B) * T * D);
    FXF_CHECK(T * sizeof(float) <= 160 * 1024, "cached_mha: static length %lld is too long for the score buffer", (long long)T);
    if (size_t(T) * sizeof(float) > 40 * 1024) FXF_CUDA(cudaFuncSetAttribute(cached_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(T * sizeof(float))));
    cached_attn_kernel<<<dim3(unsigned(H), unsigned(B)), kCachedAttnThreads, size_t(T) * sizeof(float), ctx.stream>>>(
        qkv, cache, static_cast<const int64_t*>(tok.ptr), static_cast<const int64_t*>(pos.ptr), cx, int(T), int(D), int(hd), p.floats[0], p.ints[4], ctx.status);
    FXF_LAUNCHED(ctx);
    GemmArgs g2;
    fill_gemm(g2, cx, pl->s[2], &pl->s[3], static_cast<float*>(o.ptr), B, D, D, false);
    return launch_gemm(g2, ctx);
}

std::unique_ptr<NodePlan> plan_cached_mha(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const PlanEnv& env) {
    auto pl = std::make_unique<DensePlan>();
    pl->bf16_mode = env.gemm_mode == FXF_GEMM_BF16;
    pl->mixed_mode = mixed_arithmetic(env.gemm_mode);
    if (in.size() < 7 || out.size() < 1 || p.ints.size() < 5 || reg[in[0]].rank != 3 || reg[in[1]].rank != 2) return pl;
    const int64_t B = reg[in[0]].shape[0], T = reg[in[1]].shape[1], H = p.ints[0], hd = p.ints[1], D = p.ints[2], QKV = p.ints[3];
    if (H <= 0 || hd <= 0) return pl;
    pl->heads_local = H;
    Slice& s_wq = pl->add(3, QKV, D);
    Slice& s_bq = pl->add(4, QKV, 1);
    Slice& s_wo = pl->add(5, D, D);
    Slice& s_bo = pl->add(6, D, 1);
    pl->reserve(s_wq, want_tc(env, B, QKV, D));
    pl->reserve(s_bq, false);
    pl->reserve(s_wo, want_tc(env, B, D, D));
    pl->reserve(s_bo, false);
    pl->cache_off = pl->persist_bytes;
    pl->persist_bytes += round_up(size_t(B) * size_t(T) * size_t(2 * D) * sizeof(float), 256);
    pl->M = B;
    pl->scratch_bytes = size_t(B) * size_t(4 * D) * sizeof(float);
    pl->flops = 2.0 * double(B) * QKV * D + 4.0 * double(B) * H * double(T) * hd + 2.0 * double(B) * D * D;
    pl->bytes = 4.0 * (double(QKV) * D + double(D) * D + 2.0 * double(B) * T * D);
    GemmArgs g1;
    g1.M = B; g1.N = QKV; g1.K = D;
    pl->variant = std::string(env.tp_size > 1 ? "replicated " : "") + gemm_variant_name(g1, env.gemm_mode, 148, env.tc_pairs) + "+cached-attn-fp32";
    return pl;
}

}  // namespace fxf
