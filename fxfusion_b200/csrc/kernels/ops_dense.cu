// Dense-contraction ops: Linear, LinearRelu, FeedForward, MHA.
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
#include "../runtime.hpp"

namespace fxf {

static bool use_tc(const GemmArgs& a, int gemm_mode) {
    if (gemm_mode == FXF_GEMM_FP32_SIMT) return false;
    return gemm_tc_supported(a);
}

int launch_gemm(const GemmArgs& a, ExecCtx& ctx) {
    if (a.M == 0 || a.N == 0) return 0;
    if (use_tc(a, ctx.gemm_mode)) return launch_gemm_tc(a, ctx);
    FXF_CHECK(ctx.gemm_mode != FXF_GEMM_TF32X3, "gemm: FXF_GEMM_TF32X3 was requested but the shape M=%lld N=%lld K=%lld (or its alignment) is not supported by the tensor-core kernel",
              (long long)a.M, (long long)a.N, (long long)a.K);
    return launch_gemm_simt(a, ctx);
}

std::string gemm_variant_name(const GemmArgs& a, int gemm_mode, int sm_count) {
    if (gemm_mode != FXF_GEMM_FP32_SIMT && gemm_tc_shape_ok(a.M, a.N, a.K)) return a.N > 128 ? "tcgen05-tf32x3-128x256" : "tcgen05-tf32x3-128x128";
    static const char* names[] = {"simt128x128", "simt64x64", "simt32x32"};
    return names[simt_tile_choice(a.M, a.N, sm_count)];
}

namespace {

// Holds up to two weights pre-split into TF32 hi/lo halves inside the node's persistent memory.
struct DensePlan : NodePlan {
    struct Split {
        int input = -1;      // position in input_ids of the weight
        int64_t n = 0;       // elements
        size_t offset = 0;   // byte offset of the hi half inside `persist`; lo follows
    };
    Split splits[2];
    int n_splits = 0;
    void want_split(int input, int64_t N, int64_t K, int64_t M, int gemm_mode) {
        if (gemm_mode == FXF_GEMM_FP32_SIMT || !gemm_tc_shape_ok(M, N, K)) return;
        Split& sp = splits[n_splits++];
        sp.input = input;
        sp.n = N * K;
        sp.offset = persist_bytes;
        persist_bytes += round_up(size_t(2) * size_t(sp.n) * sizeof(float), 256);
    }
    const float* hi(int input) const {
        for (int i = 0; i < n_splits; i++)
            if (splits[i].input == input && persist) return reinterpret_cast<const float*>(static_cast<const char*>(persist) + splits[i].offset);
        return nullptr;
    }
    const float* lo(int input) const {
        for (int i = 0; i < n_splits; i++)
            if (splits[i].input == input && persist) return hi(input) + splits[i].n;
        return nullptr;
    }
    int prepare(Registry& reg, const TensorIds& in, const TensorIds&, const Params&, ExecCtx& ctx) override {
        for (int i = 0; i < n_splits; i++) {
            const FxfTensor& w = reg[in[splits[i].input]];
            FXF_CHECK(persist != nullptr && numel(w) == splits[i].n, "dense plan: persistent memory was not assigned");
            float* h = reinterpret_cast<float*>(static_cast<char*>(persist) + splits[i].offset);
            if (launch_split_tf32(static_cast<const float*>(w.ptr), h, h + splits[i].n, splits[i].n, ctx)) return 1;
        }
        return 0;
    }
};
inline const DensePlan* dense(const NodePlan* p) { return static_cast<const DensePlan*>(p); }

struct LinearDims {
    int64_t M, N, K;
};

int linear_dims(const FxfTensor& x, const FxfTensor& w, const FxfTensor& b, const FxfTensor& o, LinearDims* d, const char* who) {
    FXF_CHECK(x.dtype == FXF_F32 && w.dtype == FXF_F32 && b.dtype == FXF_F32 && o.dtype == FXF_F32, "%s: only float32 is supported", who);
    FXF_CHECK(w.rank == 2 && x.rank >= 1, "%s: weight must be [N,K] and x at least 1-D", who);
    int64_t K = x.shape[x.rank - 1];
    FXF_CHECK(w.shape[1] == K, "%s: x inner size %lld does not match weight K %lld", who, (long long)K, (long long)w.shape[1]);
    FXF_CHECK(numel(b) == w.shape[0], "%s: bias size does not match weight rows", who);
    d->K = K;
    d->N = w.shape[0];
    d->M = 1;
    for (int k = 0; k + 1 < x.rank; k++) d->M *= x.shape[k];
    FXF_CHECK(numel(o) == d->M * d->N, "%s: output size mismatch", who);
    return 0;
}

int run_linear(Registry& reg, const TensorIds& in, const TensorIds& out, bool relu, const NodePlan* plan, ExecCtx& ctx, const char* who) {
    FXF_CHECK(in.size() >= 3 && out.size() >= 1, "%s: expects [x, weight, bias]", who);
    const FxfTensor &x = reg[in[0]], &w = reg[in[1]], &b = reg[in[2]], &o = reg[out[0]];
    LinearDims d;
    if (linear_dims(x, w, b, o, &d, who)) return 1;
    GemmArgs g;
    g.x = static_cast<const float*>(x.ptr);
    g.w = static_cast<const float*>(w.ptr);
    if (plan) { g.w_hi = dense(plan)->hi(1); g.w_lo = dense(plan)->lo(1); }
    g.bias = static_cast<const float*>(b.ptr);
    g.out = static_cast<float*>(o.ptr);
    g.M = d.M; g.N = d.N; g.K = d.K;
    g.ldx = d.K; g.ldw = d.K; g.ldo = d.N;
    g.relu = relu;
    return launch_gemm(g, ctx);
}

}  // namespace

int k_linear(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan* plan, ExecCtx& ctx) {
    return run_linear(reg, in, out, false, plan, ctx, "linear");
}
int k_linear_relu(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan* plan, ExecCtx& ctx) {
    return run_linear(reg, in, out, true, plan, ctx, "linear_relu");
}

std::unique_ptr<NodePlan> plan_linear(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, int gemm_mode) {
    auto p = std::make_unique<DensePlan>();
    if (in.size() >= 3 && out.size() >= 1) {
        const FxfTensor &x = reg[in[0]], &w = reg[in[1]];
        if (w.rank == 2 && x.rank >= 1 && x.shape[x.rank - 1] > 0) {
            GemmArgs g;
            g.K = x.shape[x.rank - 1]; g.N = w.shape[0]; g.M = numel(x) / g.K;
            g.ldx = g.K; g.ldw = g.K; g.ldo = g.N;
            g.x = static_cast<const float*>(x.ptr); g.w = static_cast<const float*>(w.ptr); g.out = static_cast<float*>(reg[out[0]].ptr);
            p->flops = 2.0 * double(g.M) * double(g.N) * double(g.K);
            p->bytes = 4.0 * (double(g.M) * g.K + double(g.N) * g.K + double(g.N) + double(g.M) * g.N);
            p->variant = gemm_variant_name(g, gemm_mode, 148);
            p->want_split(1, g.N, g.K, g.M, gemm_mode);
        }
    }
    return p;
}

// ---- FeedForward ------------------------------------------------------------------------------
int k_feedforward(Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, const NodePlan* plan, ExecCtx& ctx) {
    FXF_CHECK(in.size() >= 5 && out.size() >= 1, "feedforward: expects [x, w1, b1, w2, b2]");
    const FxfTensor &x = reg[in[0]], &w1 = reg[in[1]], &b1 = reg[in[2]], &w2 = reg[in[3]], &b2 = reg[in[4]], &o = reg[out[0]];
    FXF_CHECK(x.dtype == FXF_F32 && o.dtype == FXF_F32, "feedforward: only float32 is supported");
    FXF_CHECK(w1.rank == 2 && w2.rank == 2 && x.rank >= 1, "feedforward: weights must be 2-D");
    int64_t K = x.shape[x.rank - 1], F = w1.shape[0], P = w2.shape[0];
    FXF_CHECK(w1.shape[1] == K && w2.shape[1] == F, "feedforward: weight shapes do not chain (x[..,%lld], w1[%lld,%lld], w2[%lld,%lld])",
              (long long)K, (long long)w1.shape[0], (long long)w1.shape[1], (long long)w2.shape[0], (long long)w2.shape[1]);
    FXF_CHECK(numel(b1) == F && numel(b2) == P, "feedforward: bias sizes do not match");
    int64_t M = 1;
    for (int k = 0; k + 1 < x.rank; k++) M *= x.shape[k];
    FXF_CHECK(numel(o) == M * P, "feedforward: output size mismatch");
    size_t need = size_t(M) * size_t(F) * sizeof(float);
    FXF_CHECK(ctx.scratch_bytes >= need && (need == 0 || ctx.scratch != nullptr), "feedforward: scratch too small (%zu < %zu bytes)", ctx.scratch_bytes, need);
    float* hidden = static_cast<float*>(ctx.scratch);
    GemmArgs g1;
    g1.x = static_cast<const float*>(x.ptr); g1.w = static_cast<const float*>(w1.ptr); g1.bias = static_cast<const float*>(b1.ptr);
    g1.out = hidden; g1.M = M; g1.N = F; g1.K = K; g1.ldx = K; g1.ldw = K; g1.ldo = F; g1.relu = true;
    if (plan) { g1.w_hi = dense(plan)->hi(1); g1.w_lo = dense(plan)->lo(1); }
    if (launch_gemm(g1, ctx)) return 1;
    GemmArgs g2;
    g2.x = hidden; g2.w = static_cast<const float*>(w2.ptr); g2.bias = static_cast<const float*>(b2.ptr);
    g2.out = static_cast<float*>(o.ptr); g2.M = M; g2.N = P; g2.K = F; g2.ldx = F; g2.ldw = F; g2.ldo = P; g2.relu = false;
    if (plan) { g2.w_hi = dense(plan)->hi(3); g2.w_lo = dense(plan)->lo(3); }
    return launch_gemm(g2, ctx);
}

std::unique_ptr<NodePlan> plan_feedforward(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params&, int gemm_mode) {
    auto p = std::make_unique<DensePlan>();
    if (in.size() >= 5 && out.size() >= 1) {
        const FxfTensor &x = reg[in[0]], &w1 = reg[in[1]], &w2 = reg[in[3]];
        if (w1.rank == 2 && w2.rank == 2 && x.rank >= 1 && x.shape[x.rank - 1] > 0) {
            int64_t K = x.shape[x.rank - 1], F = w1.shape[0], P = w2.shape[0], M = numel(x) / K;
            p->scratch_bytes = size_t(M) * size_t(F) * sizeof(float);
            p->flops = 2.0 * double(M) * double(F) * double(K) + 2.0 * double(M) * double(P) * double(F);
            p->bytes = 4.0 * (double(M) * K + double(F) * K + F + double(P) * F + P + double(M) * P);
            GemmArgs g1; g1.M = M; g1.N = F; g1.K = K; g1.ldx = K; g1.ldw = K; g1.ldo = F;
            GemmArgs g2; g2.M = M; g2.N = P; g2.K = F; g2.ldx = F; g2.ldw = F; g2.ldo = P;
            p->variant = gemm_variant_name(g1, gemm_mode, 148) + "+" + gemm_variant_name(g2, gemm_mode, 148);
            p->want_split(1, F, K, M, gemm_mode);
            p->want_split(3, P, F, M, gemm_mode);
        }
    }
    return p;
}

// ---- MHA ----------------------------------------------------------------------------------------
namespace {
struct MhaDims {
    int64_t B, T, H, hd, D, QKV, M;
};
int mha_dims(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, MhaDims* d) {
    FXF_CHECK(in.size() >= 6 && out.size() >= 1, "mha: expects [x, mask, qkv_weight, qkv_bias, out_weight, out_bias]");
    FXF_CHECK(p.ints.size() >= 4 && p.floats.size() >= 1, "mha: expects ints [H, head_dim, d_model, qkv_dim] and floats [scale_divisor]");
    const FxfTensor& x = reg[in[0]];
    FXF_CHECK(x.rank == 3, "mha: x must be [B,T,D]");
    d->B = x.shape[0]; d->T = x.shape[1];
    d->H = p.ints[0]; d->hd = p.ints[1]; d->D = p.ints[2]; d->QKV = p.ints[3];
    d->M = d->B * d->T;
    FXF_CHECK(d->H > 0 && d->hd > 0 && d->H * d->hd == d->D && d->QKV == 3 * d->D, "mha: inconsistent head parameters");
    FXF_CHECK(x.shape[2] == d->D, "mha: x inner size does not match d_model");
    const FxfTensor &wq = reg[in[2]], &bq = reg[in[3]], &wo = reg[in[4]], &bo = reg[in[5]];
    FXF_CHECK(wq.rank == 2 && wq.shape[0] == d->QKV && wq.shape[1] == d->D && numel(bq) == d->QKV, "mha: packed QKV weight/bias shape mismatch");
    FXF_CHECK(wo.rank == 2 && wo.shape[0] == d->D && wo.shape[1] == d->D && numel(bo) == d->D, "mha: output projection shape mismatch");
    FXF_CHECK(numel(reg[out[0]]) == d->M * d->D, "mha: output size mismatch");
    return 0;
}
}  // namespace

int k_mha(Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, const NodePlan* plan, ExecCtx& ctx) {
    MhaDims d;
    if (mha_dims(reg, in, out, p, &d)) return 1;
    const FxfTensor &x = reg[in[0]], &mask = reg[in[1]], &wq = reg[in[2]], &bq = reg[in[3]], &wo = reg[in[4]], &bo = reg[in[5]], &o = reg[out[0]];
    FXF_CHECK(x.dtype == FXF_F32 && o.dtype == FXF_F32, "mha: only float32 activations are supported");
    FXF_CHECK(mask.dtype == FXF_BOOL, "mha: mask must be a bool tensor");
    FXF_CHECK(mask.rank <= 4, "mha: mask rank must be <= 4");
    // broadcast the mask to [B,H,T,T]: right-align its dims, stride 0 where its extent is 1
    int64_t want[4] = {d.B, d.H, d.T, d.T}, ms[4] = {0, 0, 0, 0};
    for (int k = 0; k < mask.rank; k++) {
        int tgt = 4 - mask.rank + k;
        FXF_CHECK(mask.shape[k] == want[tgt] || mask.shape[k] == 1, "mha: mask shape is not broadcastable to [B,H,T,T]");
        ms[tgt] = mask.shape[k] == 1 ? 0 : mask.stride[k];
    }
    size_t need = size_t(d.M) * size_t(d.QKV + d.D) * sizeof(float);
    FXF_CHECK(ctx.scratch_bytes >= need && (need == 0 || ctx.scratch != nullptr), "mha: scratch too small (%zu < %zu bytes)", ctx.scratch_bytes, need);
    float* qkv = static_cast<float*>(ctx.scratch);
    float* cx = qkv + d.M * d.QKV;
    float* split = cx + d.M * d.D;  // only present when the plan reserved it
    const bool have_split = ctx.scratch_bytes >= need + attention_tc_scratch_bytes(d.B, d.T, d.H);

    GemmArgs g;
    g.x = static_cast<const float*>(x.ptr); g.w = static_cast<const float*>(wq.ptr); g.bias = static_cast<const float*>(bq.ptr);
    g.out = qkv; g.M = d.M; g.N = d.QKV; g.K = d.D; g.ldx = d.D; g.ldw = d.D; g.ldo = d.QKV;
    if (plan) { g.w_hi = dense(plan)->hi(2); g.w_lo = dense(plan)->lo(2); }
    if (launch_gemm(g, ctx)) return 1;

    AttnArgs a;
    a.qkv = qkv; a.mask = static_cast<const uint8_t*>(mask.ptr); a.ctx = cx;
    a.B = int(d.B); a.T = int(d.T); a.H = int(d.H); a.hd = int(d.hd);
    a.ld_qkv = d.QKV; a.q_off = 0; a.k_off = d.D; a.v_off = 2 * d.D; a.ld_ctx = d.D;
    a.mask_sb = ms[0]; a.mask_sh = ms[1]; a.mask_sq = ms[2]; a.mask_sk = ms[3];
    a.scale_divisor = p.floats[0];
    if (have_split && attention_tc_supported(a, ctx.gemm_mode)) {
        if (launch_attention_tc(a, split, ctx)) return 1;
    } else {
        if (launch_attention(a, ctx)) return 1;
    }

    GemmArgs g2;
    g2.x = cx; g2.w = static_cast<const float*>(wo.ptr); g2.bias = static_cast<const float*>(bo.ptr);
    g2.out = static_cast<float*>(o.ptr); g2.M = d.M; g2.N = d.D; g2.K = d.D; g2.ldx = d.D; g2.ldw = d.D; g2.ldo = d.D;
    if (plan) { g2.w_hi = dense(plan)->hi(4); g2.w_lo = dense(plan)->lo(4); }
    return launch_gemm(g2, ctx);
}

std::unique_ptr<NodePlan> plan_mha(const Registry& reg, const TensorIds& in, const TensorIds& out, const Params& p, int gemm_mode) {
    auto pl = std::make_unique<DensePlan>();
    if (in.size() >= 6 && out.size() >= 1 && p.ints.size() >= 4 && reg[in[0]].rank == 3) {
        const FxfTensor& x = reg[in[0]];
        int64_t B = x.shape[0], T = x.shape[1], H = p.ints[0], hd = p.ints[1], D = p.ints[2], QKV = p.ints[3], M = B * T;
        pl->scratch_bytes = size_t(M) * size_t(QKV + D) * sizeof(float);
        const bool tc_attn = gemm_mode != FXF_GEMM_FP32_SIMT && hd == 64 && T % 4 == 0 && T >= 16 && D % 4 == 0;
        if (tc_attn) pl->scratch_bytes += attention_tc_scratch_bytes(B, T, H);
        pl->flops = 2.0 * M * double(QKV) * D + 4.0 * double(B) * H * double(T) * T * hd + 2.0 * double(M) * D * D;
        pl->bytes = 4.0 * (2.0 * double(M) * D + double(QKV) * D + QKV + double(D) * D + D) + double(reg[in[1]].nbytes);
        GemmArgs g1; g1.M = M; g1.N = QKV; g1.K = D; g1.ldx = D; g1.ldw = D; g1.ldo = QKV;
        GemmArgs g2; g2.M = M; g2.N = D; g2.K = D; g2.ldx = D; g2.ldw = D; g2.ldo = D;
        pl->variant = gemm_variant_name(g1, gemm_mode, 148) + (tc_attn ? "+attn-tcgen05-tf32x3+" : "+flash-fp32+") + gemm_variant_name(g2, gemm_mode, 148);
        pl->want_split(2, QKV, D, M, gemm_mode);
        pl->want_split(4, D, D, M, gemm_mode);
    }
    return pl;
}

}  // namespace fxf
