// Runtime contracts of the B200 backend: registry, params, per-node plan and the KernelFn
// function-pointer type.  They keep the shape of the reference's contracts
// (csrc/include/runtime/tensor_registry.hpp:8-26) with LibTorch removed:
//   TensorRegistry  vector<torch::Tensor>      -> vector<FxfTensor> (raw device pointers)
//   Cache           per-node torch::empty bufs -> NodePlan: launch geometry computed once at
//                                                 build + byte counts of the shared scratch /
//                                                 persistent memory the node wants
//   KernelFn        void(*)(reg,in,out,params,cache) -> int(*)(reg,in,out,params,plan,ctx)
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/fxf_b200.h"

namespace fxf {

using Registry = std::vector<FxfTensor>;
using TensorIds = std::vector<uint32_t>;

struct Params {
    std::vector<int64_t> ints;
    std::vector<float> floats;
};

// One traced kernel launch (profiling mode only).
struct LaunchRecord {
    const char* name;      // kernel family, e.g. "gemm_simt128x128", "attention_fp32"
    int node;              // index of the graph node that issued it
    double flops, bytes;   // algorithmic work of this launch
    cudaEvent_t done;      // recorded right after the launch
};

// Everything a launch needs besides the registry.
// The engine allocations of all tensor-parallel ranks of a node as mapped into this process (CUDA IPC).
constexpr int kMaxTpRanks = 8;
struct PeerMap {
    char* base[kMaxTpRanks] = {};   // base[r]: rank r's allocation (own rank: the local pointer)
    size_t shared_bytes = 0;        // offsets below this mean the same tensor on every rank (the planner's arena)
    size_t flags_off = 0;           // barrier flags [peer][block] of the peer all-reduce, same offset on every rank
    size_t epoch_off = 0;           // two ints: epoch, finished-block counter
    int grid = 0;                   // blocks of the peer exchange kernels (fixes the flag layout)
    // Exchange window: a buffer outside the planner's arena (same offset on every rank, never reused for anything else) into
    // which the peers' row-parallel products store their partial sums of this rank's rows.  0 bytes: no window.
    size_t push_off = 0, push_bytes = 0;
    // wait budgets of the two peer barriers of an exchange; the first also absorbs the skew between the ranks' host threads
    unsigned long long start_budget_ns = 20000000000ull, end_budget_ns = 2000000000ull;
};

// The exchange step of a row-parallel product under tensor parallelism, fused with what follows it in a pre-LN transformer
// block: the ranks' partial [M,D] outputs are summed, the residual is added and the rows are normalised by ONE kernel over
// peer memory (kernels/tp_exchange.cu).  Set by the engine around a sharded MHA / CrossMHA / FeedForward node whose
// following Add (+ LayerNorm) or AddLayerNorm nodes were folded into it.
struct TpExchange {
    bool enabled = false;
    const float* residual = nullptr;   // the other operand of the folded Add (this rank's rows of it are read)
    float* x_out = nullptr;            // output of the folded Add: the new residual stream (NULL for AddLayerNorm)
    float* y_out = nullptr;            // output of the folded LayerNorm / AddLayerNorm (NULL: a plain Add was folded)
    const float* gamma = nullptr;
    const float* beta = nullptr;
    float eps = 0.f;
    bool replicate_x = false;          // x_out is read outside this scheme: every rank gets every row of it
    bool consumed = false;
};

// A residual Add / AddRelu node folded into the contraction that precedes it: the owner of that node's final GEMM writes
// act(acc + bias + residual) straight into the Add's output tensor.
struct EpilogueFusion {
    const float* residual = nullptr;
    float* out = nullptr;
    bool relu = false;
    bool consumed = false;
};

struct ExecCtx {
    cudaStream_t stream = nullptr;
    void* scratch = nullptr;       // shared by all nodes of an engine; nodes run one at a time
    size_t scratch_bytes = 0;
    int* status = nullptr;         // sticky device status word (0 = ok)
    int sm_count = 148;
    int gemm_mode = FXF_GEMM_AUTO;
    int launches = 0;              // incremented by every kernel launch (host-side count)
    int tp_rank = 0, tp_size = 1;  // tensor-parallel position; tp_size > 1 needs `comm`
    void* comm = nullptr;          // fxf_comm* (NCCL communicator wrapper), owned by the caller
    const PeerMap* peers = nullptr;  // set when the ranks' allocations are mapped into each other: all-reduce over peer memory
    EpilogueFusion fuse;             // set by the engine around a node whose following Add was folded into it
    TpExchange xchg;                 // set by the engine around a sharded node whose exchange absorbs the following Add / LayerNorm
    // workspace of the tensor-core GEMM's K-split last round: partial tiles and their ready flags (zero between
    // launches).  Without it every tile is computed whole.
    float* gemm_ws = nullptr;
    size_t gemm_ws_bytes = 0;
    int* gemm_flags = nullptr;
    int gemm_flag_count = 0;
    int tc_chunk_k = 0;            // K-elements per tensor-core accumulation chain (0 = the kernel's default)
    int tc_pair = 0;               // 0: 256-wide tensor-core GEMM tiles are computed by CTA pairs (tcgen05 cta_group::2); 1: never
    // profiling: when `trace` is set every launch appends a record carrying the current tag
    std::vector<LaunchRecord>* trace = nullptr;
    int cur_node = -1;
    const char* tag_name = "kernel";
    double tag_flops = 0, tag_bytes = 0;
};
inline void tag_launch(ExecCtx& c, const char* name, double flops, double bytes) {
    c.tag_name = name;
    c.tag_flops = flops;
    c.tag_bytes = bytes;
}
int trace_after_launch(ExecCtx& ctx);
// Called by the op that owns the final GEMM of a node: redirects the output and attaches the residual of a folded Add.
// `partial`: the node is sharded over the tensor-parallel ranks and its outputs are summed afterwards, so only rank 0 adds
// the residual (like the bias); a node that is replicated on every rank adds it everywhere.
template <class Args>
inline void apply_fusion(ExecCtx& ctx, Args& g, bool partial) {
    if (ctx.fuse.out == nullptr) return;
    g.out = ctx.fuse.out;
    g.residual = (!partial || ctx.tp_rank == 0) ? ctx.fuse.residual : nullptr;
    g.relu = g.relu || ctx.fuse.relu;
    ctx.fuse.consumed = true;
}
// out = act(out + residual) over n contiguous floats: the fallback when a GEMM without a fused epilogue ran
int launch_residual_epilogue(float* out, const float* residual, int64_t n, bool relu, ExecCtx& ctx);

struct NodePlan {
    virtual ~NodePlan() = default;
    size_t scratch_bytes = 0;   // shared scratch wanted at execute time
    size_t persist_bytes = 0;   // memory that must survive across runs (e.g. re-laid-out weights)
    void* persist = nullptr;    // assigned by the engine before prepare()
    double flops = 0, bytes = 0;  // algorithmic work of the node
    std::string variant;        // which kernel variant was chosen (for describe / profiling)
    bool tp_sharded = false;    // the node computes a partial result on each tensor-parallel rank (summed by an exchange)
    // Called once after device memory exists (constants uploaded).  May launch kernels.
    virtual int prepare(Registry&, const TensorIds&, const TensorIds&, const Params&, ExecCtx&) { return 0; }
};

// What a plan builder needs to know about the engine it plans for.
struct PlanEnv {
    int gemm_mode = FXF_GEMM_AUTO;
    int tp_rank = 0, tp_size = 1;     // tensor-parallel position of this engine
    bool shard_output_cols = false;   // this node is the graph's final Linear and its columns are sharded over the ranks
    bool tc_pairs = true;             // the engine lets CTA pairs compute the widest GEMM tiles (reported in variant names)
};

using KernelFn = int (*)(Registry&, const TensorIds&, const TensorIds&, const Params&, const NodePlan*, ExecCtx&);
using PlanFn = std::unique_ptr<NodePlan> (*)(const Registry&, const TensorIds&, const TensorIds&, const Params&, const PlanEnv&);

struct OpEntry {
    const char* name = nullptr;
    KernelFn kernel = nullptr;
    PlanFn plan = nullptr;
};

// OpCode -> {kernel, plan builder}.  Counterpart of OpRegistry (csrc/runtime/op_registry.cpp:16-106);
// there is one kernel set only — CUDA — and no CPU fallback.
const OpEntry& op_entry(int op_code);

// ---- error plumbing -------------------------------------------------------------------
void set_last_error(const std::string& msg);
const std::string& last_error();

inline std::string strfmt(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    return std::string(buf);
}

#define FXF_FAIL(...)                                   \
    do {                                                \
        ::fxf::set_last_error(::fxf::strfmt(__VA_ARGS__)); \
        return 1;                                       \
    } while (0)

#define FXF_CHECK(cond, ...)          \
    do {                              \
        if (!(cond)) FXF_FAIL(__VA_ARGS__); \
    } while (0)

#define FXF_CUDA(expr)                                                                       \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess) FXF_FAIL("CUDA error %s at %s:%d (%s)", cudaGetErrorString(_e), __FILE__, __LINE__, #expr); \
    } while (0)

// Checks the launch that has just been issued and counts it.
#define FXF_LAUNCHED(ctx)                                                                     \
    do {                                                                                      \
        cudaError_t _e = cudaPeekAtLastError();                                               \
        if (_e != cudaSuccess) FXF_FAIL("kernel launch failed: %s at %s:%d", cudaGetErrorString(_e), __FILE__, __LINE__); \
        (ctx).launches++;                                                                     \
        if ((ctx).trace && ::fxf::trace_after_launch(ctx)) return 1;                          \
    } while (0)

// ---- tensor helpers ---------------------------------------------------------------------
inline int64_t numel(const FxfTensor& t) {
    int64_t n = 1;
    for (int i = 0; i < t.rank; i++) n *= t.shape[i];
    return n;
}
inline int dtype_size(int dt) {
    switch (dt) {
        case FXF_F32: return 4;
        case FXF_F16: return 2;
        case FXF_I32: return 4;
        case FXF_I64: return 8;
        case FXF_BOOL: return 1;
        default: return 0;
    }
}
inline void set_contiguous(FxfTensor& t) {
    int64_t s = 1;
    for (int i = t.rank - 1; i >= 0; i--) {
        t.stride[i] = s;
        s *= t.shape[i];
    }
}
inline bool is_contiguous(const FxfTensor& t) {
    int64_t s = 1;
    for (int i = t.rank - 1; i >= 0; i--) {
        if (t.shape[i] != 1 && t.stride[i] != s) return false;
        s *= t.shape[i];
    }
    return true;
}
// Channels-last ("NHWC") physical layout of a logical [N,C,H,W] tensor: strides (H*W*C, 1, W*C, C).  The graph
// contract is NCHW; the engine may keep intermediate activations between layout-aware nodes channels-last
// and says so through the registry strides, the way torch's channels_last memory format does.
inline void set_channels_last(FxfTensor& t) {
    const int64_t C = t.shape[1], H = t.shape[2], W = t.shape[3];
    t.stride[0] = H * W * C;
    t.stride[1] = 1;
    t.stride[2] = W * C;
    t.stride[3] = C;
}
inline bool is_channels_last(const FxfTensor& t) {
    if (t.rank != 4 || is_contiguous(t)) return false;
    const int64_t C = t.shape[1], H = t.shape[2], W = t.shape[3];
    return (t.shape[0] == 1 || t.stride[0] == H * W * C) && (C == 1 || t.stride[1] == 1) && (H == 1 || t.stride[2] == W * C) && (W == 1 || t.stride[3] == C);
}
inline bool same_layout(const FxfTensor& a, const FxfTensor& b) {
    if (a.rank != b.rank) return false;
    for (int i = 0; i < a.rank; i++)
        if (a.shape[i] != b.shape[i] || (a.shape[i] != 1 && a.stride[i] != b.stride[i])) return false;
    return true;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- kernels shared between ops (defined in the .cu files) -------------------------------
// out[M,N] = act(x[M,K] · w[N,K]^T + bias[N]); row strides in elements (ldx, ldw, ldo).
// `w_hi` / `w_lo`: the weight pre-split into TF32 high and low parts for the tensor-core path
// (both null when no split exists; the fp32 SIMT kernel is used then).
struct GemmArgs {
    const float* x = nullptr;
    const float* w = nullptr;
    const float* w_hi = nullptr;
    const float* w_lo = nullptr;
    bool w_is_bf16 = false;   // bf16 mode: w_hi points to the weight as bf16 [N,K] (w_lo unused)
    bool w_mixed = false;     // mixed mode: w_hi is the TF32 high part (fp32), w_lo points to a bf16 matrix [2N,K]: bf16(w_hi) rows, then bf16(w - w_hi) rows
    const float* bias = nullptr;
    const float* residual = nullptr;   // optional [M,N] with the pitch of `out`, added after the bias and before the ReLU
    float* out = nullptr;
    int64_t M = 0, N = 0, K = 0;
    int64_t ldx = 0, ldw = 0, ldo = 0;
    bool relu = false;
    bool conv_chain = false;   // a convolution written as a GEMM: use the (shorter) accumulation chains of convolutions
    // Row-pushed output of a row-parallel product under tensor parallelism (tensor-core kernels only): rows
    // [q*push_rows, (q+1)*push_rows) of the result go to push_out[q] (rank q's exchange window, peer memory for q != rank) at
    // row push_rank*push_rows + (row - q*push_rows); `out` is not written.  push_rows == 0: the plain output.
    float* const* push_out = nullptr;
    int64_t push_rows = 0;
    int push_rank = 0;
    // Transposed column range (the V third of a packed QKV projection, tensor-core kernels only): columns [vt_col0, N) of
    // the result are not written to `out`; column vt_col0 + 64*h + d of row b*vt_T + t goes to vt_out[((b*vt_heads + h)*64 + d)
    // * vt_T + t] (V^T per batch and head, keys contiguous: the B operand of the attention's second product), and
    // vt_flags[((b*vt_heads + h)*2 + d/32)*vt_n32 + t/32] tells whether any of those values of a 32-row group and half a
    // head is NaN or infinite.
    // Ask gemm_tc_vt_ok() first.
    float* vt_out = nullptr;
    unsigned char* vt_flags = nullptr;
    int64_t vt_col0 = 0;
    int vt_T = 0, vt_heads = 0, vt_n32 = 0;
};
// Whether launch_gemm would serve the transposed column range of `a` (fields vt_* filled in) on this context.
bool gemm_tc_vt_ok(const GemmArgs& a, const ExecCtx& ctx);
int launch_gemm(const GemmArgs& a, ExecCtx& ctx);
int launch_gemm_simt(const GemmArgs& a, ExecCtx& ctx);
int launch_gemm_tc(const GemmArgs& a, ExecCtx& ctx, bool allow_few_rows = false);
// allow_few_rows: accept M < 64 (a weight-streaming problem: most rows of the 128-row tile are padding, the time is the weight read)
bool gemm_tc_supported(const GemmArgs& a, bool allow_few_rows = false);
bool gemm_tc_shape_ok(int64_t M, int64_t N, int64_t K);
// K > 0: the launch may cut the tiles of its last round along K (needs the context's GEMM workspace)
int gemm_tc_pick_bn(int64_t M, int64_t N, int sm_count, int64_t K = 0);
// Name of the tensor-core kernel variant launch_gemm_tc takes for a problem (and its tile width): the one dispatch rule.
const char* gemm_tc_variant(int64_t M, int64_t N, int64_t K, int sm_count, bool k_split, bool few_rows, int* bn_out, bool pairs = true);
const char* gemm_tc_mixed_variant(int64_t M, int64_t N, int64_t K, int sm_count, bool k_split, bool few_rows, int* bn_out, bool pairs = true);
int launch_split_tf32(const float* w, float* hi, float* lo, int64_t n, ExecCtx& ctx);
// mixed mode: hi = tf32(w) as fp32 [n], lo_bf16 = bf16(hi) [n] followed by bf16(w - hi) [n]
int launch_split_mixed(const float* w, float* hi, void* lo_bf16, int64_t n, ExecCtx& ctx);
int simt_tile_choice(int64_t M, int64_t N, int sm_count);
std::string gemm_variant_name(const GemmArgs& a, int gemm_mode, int sm_count, bool pairs = true);

// Convolution (stride 1 or 2) as an implicit GEMM on the tensor cores: channels-last activation x [N,H,W,C], weights
// repacked to [O, KH*KW*C] (tap-major, channel-minor) and split into TF32 hi/lo, channels-last output [N,HO,WO,O].
struct ConvTcArgs {
    const float* x = nullptr;
    const float *w_hi = nullptr, *w_lo = nullptr;
    bool w_is_bf16 = false;   // bf16 mode: w_hi points to the repacked filters as bf16
    const float* bias = nullptr;
    const float* residual = nullptr;   // optional, laid out like `out`
    float* out = nullptr;
    int N = 0, C = 0, H = 0, W = 0, O = 0, KH = 0, KW = 0, HO = 0, WO = 0;
    int pad_h = 0, pad_w = 0, dil_h = 1, dil_w = 1, str_h = 1, str_w = 1;
    bool relu = false;
};
bool conv_tc_shape_ok(int64_t n_pix, int C, int O);
// The Linear of a planned node applied to M rows that start at x_rows and lie ldx floats apart; row m of the result
// goes to out + m * ldo (+ the column offset of this rank's block when the node's output columns are sharded).
int linear_on_rows(const NodePlan* plan, const float* x_rows, int64_t M, int64_t ldx, float* out, int64_t ldo, ExecCtx& ctx);
int launch_conv_tc(const ConvTcArgs& a, ExecCtx& ctx);
// w_oihw [O,C,KH,KW] -> TF32 hi/lo halves laid out [O,KH,KW,C]
int launch_convert_bf16(const float* w, void* out_bf16, int64_t n, ExecCtx& ctx);
int launch_conv_weight_bf16(const float* w_oihw, void* out_bf16_ohwi, int O, int C, int KH, int KW, ExecCtx& ctx);
int launch_conv_weight_split(const float* w_oihw, float* hi, float* lo, int O, int C, int KH, int KW, ExecCtx& ctx);

// Attention core on packed qkv [B,T,3D] (Q | K | V thirds, head h at columns h*hd) -> ctx [B,T,D].
struct AttnArgs {
    const float* qkv = nullptr;
    // Cross-attention: keys and values come from `kv` (rows of ld_kv floats, Tk rows per batch) while the queries
    // stay in `qkv`; self-attention leaves kv NULL and K/V are read from `qkv` with T rows.
    const float* kv = nullptr;
    int64_t ld_kv = 0;
    int Tk = 0;
    const uint8_t* mask = nullptr;
    float* ctx = nullptr;
    int B = 0, T = 0, H = 0, hd = 0;
    int64_t ld_qkv = 0;   // row stride of qkv (= 3*D of the full model, or of the local shard)
    int64_t q_off = 0, k_off = 0, v_off = 0;  // column offsets of the Q/K/V blocks inside a row
    int64_t ld_ctx = 0;
    int64_t mask_sb = 0, mask_sh = 0, mask_sq = 0, mask_sk = 0;  // mask strides (bytes): batch, head, query, key
    float scale_divisor = 1.f;
};
int launch_attention(const AttnArgs& a, ExecCtx& ctx);
// Sum `n` floats in place over the tensor-parallel ranks (NCCL all-reduce on ctx.stream); no-op for tp_size 1.
int tp_all_reduce_sum(float* buf, int64_t n, ExecCtx& ctx);
// Peer-memory exchanges (kernels/tp_exchange.cu) and the IPC exchange that sets them up (tp_comm.cpp).
bool p2p_all_reduce_usable(const float* buf, int64_t n, const ExecCtx& ctx);
int launch_p2p_all_reduce(float* buf, int64_t n, ExecCtx& ctx);
// sum of the ranks' partial [M,D] + residual -> x_out (own rows or all), LayerNorm of the rows -> y_out on every rank
bool tp_exchange_usable(const TpExchange& x, const float* partial, int64_t M, int64_t D, const ExecCtx& ctx);
int launch_tp_exchange(const TpExchange& x, const float* partial, int64_t M, int64_t D, ExecCtx& ctx, bool pushed = false);
// Pushed exchange: the product stores its rows straight into the owners' exchange windows (GemmArgs::push_out); `partial`
// is then unused.  Usable when the engine has a window of M*D floats and every rank owns a whole number of 128-row tiles.
bool tp_push_usable(int64_t M, int64_t D, const ExecCtx& ctx);
float* tp_push_window(int rank, const ExecCtx& ctx);
int tp_exchange_emulated(int n_ranks, const float* const* partial, const float* const* residual, float* const* x_out, float* const* y_out,
                         const float* gamma, const float* beta, float eps, int64_t M, int64_t D, int replicate_x, void* sync_mem, int budget_ms,
                         int skip_rank, cudaStream_t stream);
int tp_map_peers(void* comm, void* base, PeerMap* out);     // collective: every rank passes its own allocation
void tp_unmap_peers(void* comm, PeerMap* pm);               // collective as well
// Gather `bytes` from every rank into recv[rank * bytes ...] (NCCL all-gather on ctx.stream).
int tp_all_gather(const void* send, void* recv, int64_t bytes, ExecCtx& ctx);
// tcgen05 path (head_dim 64): needs 6*B*T*H*64 floats of scratch for the split, per-head operand copies
bool attention_tc_supported(const AttnArgs& a, int gemm_mode);
size_t attention_tc_scratch_bytes(int64_t B, int64_t T, int64_t H);
// v_transposed: V^T and its finite flags are already in the scratch (written by the projection's epilogue)
int launch_attention_tc(const AttnArgs& a, float* split_scratch, ExecCtx& ctx, bool v_transposed = false);

}  // namespace fxf
