// ExecutionEngine for B200: graph file -> one device arena -> node list -> (CUDA Graph) replay.
//
// Counterpart of the reference runtime core, with LibTorch removed:
//   ExecutionEngine  csrc/runtime/execution_engine.cpp:12-43
//   MemoryManager    csrc/runtime/memory_manager.cpp:30-123   (arena, registry, alias binding)
//   RuntimeGraph     csrc/runtime/runtime_graph.cpp:8-24      (NoOp dropped, kernel resolved once)
//   RuntimeNode      csrc/runtime/runtime_node.cpp:8-45       (ids/params copied out of the file)
//
// Memory: ONE cudaMalloc per engine, laid out as
//   [ activations at the planner's offsets | constants | static input slots | per-node
//     persistent memory | shared scratch | status word ]
// every region 256-byte aligned.  The reference gives each FeedForward/MHA node its own
// torch::empty intermediates (csrc/runtime/cache.cpp:28-73); nodes execute strictly one after
// another, so a single scratch region sized for the hungriest node serves all of them.
//
// Inputs live in static slots (the caller's buffers are copied in on the run's stream), which
// keeps every pointer inside a captured CUDA Graph stable and also makes an Alias/Output of an
// Input see the data of the current run.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

#include "fbs_reader.hpp"
#include "runtime.hpp"

namespace fxf {

// ---- error plumbing -------------------------------------------------------------------
static thread_local std::string g_last_error;
void set_last_error(const std::string& msg) { g_last_error = msg; }
const std::string& last_error() { return g_last_error; }

int decode_build_mask(const int64_t* tokens, uint8_t* mask, int B, int T, int cur, int64_t pad, ExecCtx& ctx);
int decode_argmax_scatter(const float* logits, int64_t* tokens, int B, int T, int64_t V, int cur, ExecCtx& ctx);
int decode_argmax_scatter_sharded(const float* logits, int64_t* tokens, int B, int T, int64_t V, int cur, int64_t col0, int64_t ncols,
                                  void* cand_local, void* cand_all, ExecCtx& ctx);
int decode_step_prepare(const int64_t* tokens, int64_t* ids, int64_t* pos, int B, int T, int p, ExecCtx& ctx);
int decode_argmax_scatter_rows(const float* logits, int64_t row_stride, int64_t row_off, int64_t* tokens, int B, int T, int64_t V, int cur, ExecCtx& ctx);
int decode_argmax_scatter_sharded_rows(const float* logits, int64_t row_stride, int64_t row_off, int64_t* tokens, int B, int T, int64_t V, int cur,
                                       int64_t col0, int64_t ncols, void* cand_local, void* cand_all, ExecCtx& ctx);

int trace_after_launch(ExecCtx& ctx) {
    LaunchRecord r{ctx.tag_name, ctx.cur_node, ctx.tag_flops, ctx.tag_bytes, nullptr};
    FXF_CUDA(cudaEventCreate(&r.done));
    FXF_CUDA(cudaEventRecord(r.done, ctx.stream));
    ctx.trace->push_back(r);
    return 0;
}

namespace {

enum Kind { kInput = 0, kConstant = 1, kActivation = 2, kAlias = 3, kOutput = 4 };
constexpr size_t kAlign = 256;

struct Node {
    int op = 0;
    TensorIds in, out;
    Params params;
    std::unique_ptr<NodePlan> plan;
    KernelFn fn = nullptr;
    int launches = 0;
    // epilogue fusion: this contraction also performs the residual Add / AddRelu that follows it ...
    int fuse_res = -1, fuse_out = -1;   // tensor ids of the residual operand and of the Add's output
    bool fuse_relu = false;
    bool folded = false;                // ... and this Add / AddRelu node launches nothing
    // tensor parallelism: the exchange after this sharded contraction also performs the residual Add and the LayerNorm that
    // follow it (tensor ids; -1 = not part of the fold).  The folded nodes launch nothing.
    bool xchg = false, xchg_replicate_x = false;
    int xchg_res = -1, xchg_x = -1, xchg_y = -1, xchg_gamma = -1, xchg_beta = -1;
    float xchg_eps = 0.f;
};

}  // namespace
}  // namespace fxf

using namespace fxf;

struct fxf_comm;
extern "C" int fxf_comm_rank(const fxf_comm*);
extern "C" int fxf_comm_size(const fxf_comm*);

struct fxf_engine {
    int device = 0;
    std::string name;
    FxfEngineOptions opts{};
    Registry reg;
    std::vector<Node> nodes;
    std::vector<uint32_t> input_ids, output_ids;
    std::vector<size_t> input_off;
    uint8_t* base = nullptr;
    size_t total_bytes = 0, arena_bytes = 0, const_bytes = 0, input_bytes = 0, persist_bytes = 0, scratch_bytes = 0;
    size_t scratch_off = 0, status_off = 0;
    size_t gemm_ws_off = 0, gemm_ws_bytes = 0, gemm_flags_off = 0, gemm_flags_bytes = 0;
    size_t push_off = 0, push_bytes = 0;   // exchange window of the row-parallel products (tensor parallelism)
    ExecCtx ctx;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    cudaStream_t capture_stream = nullptr;
    int launches_per_run = 0;
    // tensor parallelism
    fxf_comm* comm = nullptr;          // borrowed; must outlive the engine
    bool head_sharded = false;         // the final Linear writes only this rank's column block of the logits
    int64_t head_col0 = 0, head_ncols = 0;
    size_t cand_off = 0, cand_bytes = 0;  // argmax candidates: [local | all ranks]
    // peer-memory all-reduce: flags + epoch inside this allocation (same offset on every rank), peers' allocations mapped
    size_t p2p_off = 0;
    PeerMap peers;
    bool peers_mapped = false;
    // decode that evaluates the final Linear only at the position whose logits are read
    int tail_node = -1;                // index of that Linear (the last node), -1 when the graph does not end in one
    size_t lastrow_off = 0, lastrow_bytes = 0;  // its [B,V] output
    cudaGraph_t body_graph = nullptr;  // all nodes before tail_node
    cudaGraphExec_t body_exec = nullptr;

    ~fxf_engine() {
        if (graph_exec) cudaGraphExecDestroy(graph_exec);
        if (graph) cudaGraphDestroy(graph);
        if (body_exec) cudaGraphExecDestroy(body_exec);
        if (body_graph) cudaGraphDestroy(body_graph);
        if (capture_stream) cudaStreamDestroy(capture_stream);
        if (peers_mapped) tp_unmap_peers(comm, &peers);   // collective: every rank destroys its engine
        if (base) cudaFree(base);
    }
};

namespace fxf {
namespace {

// One node, with the epilogue fusion decided at build time: a folded Add launches nothing, the contraction before it gets
// the residual and the Add's output through the context.
int run_node(fxf_engine* e, size_t i) {
    Node& n = e->nodes[i];
    const int before = e->ctx.launches;
    e->ctx.cur_node = int(i);
    if (n.folded) {
        n.launches = 0;
        return 0;
    }
    tag_launch(e->ctx, op_entry(n.op).name, n.plan->flops, n.plan->bytes);
    e->ctx.fuse = EpilogueFusion{};
    if (n.fuse_out >= 0) {
        e->ctx.fuse.residual = static_cast<const float*>(e->reg[size_t(n.fuse_res)].ptr);
        e->ctx.fuse.out = static_cast<float*>(e->reg[size_t(n.fuse_out)].ptr);
        e->ctx.fuse.relu = n.fuse_relu;
    }
    e->ctx.xchg = TpExchange{};
    if (n.xchg) {
        auto fp = [&](int id) { return id >= 0 ? static_cast<float*>(e->reg[size_t(id)].ptr) : nullptr; };
        e->ctx.xchg.enabled = true;
        e->ctx.xchg.residual = fp(n.xchg_res);
        e->ctx.xchg.x_out = fp(n.xchg_x);
        e->ctx.xchg.y_out = fp(n.xchg_y);
        e->ctx.xchg.gamma = fp(n.xchg_gamma);
        e->ctx.xchg.beta = fp(n.xchg_beta);
        e->ctx.xchg.eps = n.xchg_eps;
        e->ctx.xchg.replicate_x = n.xchg_replicate_x;
    }
    if (n.fn(e->reg, n.in, n.out, n.params, n.plan.get(), e->ctx)) return 1;
    if (n.fuse_out >= 0) {
        FXF_CHECK(e->ctx.fuse.consumed, "node %zu (%s): the folded residual Add was not performed by the kernel", i, op_entry(n.op).name);
        e->ctx.fuse = EpilogueFusion{};
    }
    if (n.xchg) {
        FXF_CHECK(e->ctx.xchg.consumed, "node %zu (%s): the folded exchange was not performed by the kernel", i, op_entry(n.op).name);
        e->ctx.xchg = TpExchange{};
    }
    n.launches = e->ctx.launches - before;
    return 0;
}

int run_nodes(fxf_engine* e, cudaStream_t stream, int count = -1) {
    e->ctx.stream = stream;
    for (size_t i = 0; i < e->nodes.size(); i++) {
        if (count >= 0 && int(i) >= count) break;
        if (run_node(e, i)) return 1;
    }
    return 0;
}

int ensure_device(const fxf_engine* e) {
    int cur = -1;
    FXF_CUDA(cudaGetDevice(&cur));
    if (cur != e->device) FXF_CUDA(cudaSetDevice(e->device));
    return 0;
}

int build(fxf_engine* e, const uint8_t* bytes, size_t nbytes) {
    fbs::Buffer buf{bytes, nbytes};
    FXF_CHECK(nbytes >= 8, "graph file is too small to hold a graph (%zu bytes)", nbytes);
    fbs::Table g = fbs::root(&buf);
    e->name = g.str(fbs::GraphF::name);
    uint64_t arena = g.scalar<uint64_t>(fbs::GraphF::arena_size, 0);
    FXF_CHECK(arena <= (uint64_t(1) << 40), "Arena size is implausible: %llu bytes", (unsigned long long)arena);
    e->arena_bytes = size_t(arena);
    uint32_t n_tensors = g.table_vec_size(fbs::GraphF::tensors);
    uint32_t n_nodes = g.table_vec_size(fbs::GraphF::nodes);
    FXF_CHECK(n_tensors > 0, "Execution graph is not loaded: the file holds no tensors");

    struct Meta {
        int kind = 0;
        int64_t offset = -1;
        int alias_of = -1;
        const uint8_t* data = nullptr;
        size_t data_len = 0;
        size_t region_off = 0;
        bool seen = false;
    };
    std::vector<Meta> meta(n_tensors);
    std::vector<uint32_t> order;  // registry ids in file order
    e->reg.assign(n_tensors, FxfTensor{});

    size_t const_cursor = round_up(e->arena_bytes, kAlign);
    const size_t const_begin = const_cursor;
    for (uint32_t i = 0; i < n_tensors; i++) {
        fbs::Table t = g.table_at(fbs::GraphF::tensors, i);
        uint32_t id = t.scalar<uint32_t>(fbs::TensorF::id, 0);
        FXF_CHECK(id < n_tensors, "tensor id %u exceeds the tensor table size %u", id, n_tensors);
        FXF_CHECK(!meta[id].seen, "tensor id %u appears twice", id);
        Meta& m = meta[id];
        m.seen = true;
        m.kind = t.scalar<int8_t>(fbs::TensorF::kind, 0);
        m.offset = t.scalar<int64_t>(fbs::TensorF::offset, -1);
        m.alias_of = t.scalar<int32_t>(fbs::TensorF::alias_of, -1);
        FxfTensor& r = e->reg[id];
        r.dtype = t.scalar<int8_t>(fbs::TensorF::dtype, 0);
        FXF_CHECK(dtype_size(r.dtype) > 0, "Unsupported DType in FlatBuffer (tensor %u, dtype %d)", id, r.dtype);
        auto shape = t.vec<int64_t>(fbs::TensorF::shape);
        FXF_CHECK(shape.size() <= FXF_MAX_DIMS, "tensor %u has rank %u; at most %d dims are supported", id, shape.size(), FXF_MAX_DIMS);
        r.rank = int(shape.size());
        for (int k = 0; k < r.rank; k++) {
            r.shape[k] = shape[k];
            FXF_CHECK(r.shape[k] >= 0, "tensor %u has a negative extent", id);
        }
        set_contiguous(r);
        r.nbytes = numel(r) * dtype_size(r.dtype);
        auto data = t.vec<uint8_t>(fbs::TensorF::data);
        m.data = data.base;
        m.data_len = data.size();
        FXF_CHECK(m.kind >= kInput && m.kind <= kOutput, "Unsupported TensorKind in FlatBuffer (tensor %u, kind %d)", id, m.kind);
        if (m.kind == kConstant) {
            FXF_CHECK(m.data != nullptr, "Constant tensor missing data (tensor %u)", id);
            FXF_CHECK(m.data_len >= size_t(r.nbytes), "Constant tensor %u carries %zu bytes but its shape needs %lld", id, m.data_len, (long long)r.nbytes);
            m.region_off = const_cursor;
            const_cursor = round_up(const_cursor + size_t(r.nbytes), kAlign);
        }
        order.push_back(id);
    }
    e->const_bytes = const_cursor - const_begin;
    size_t cursor = const_cursor;
    for (uint32_t id : order) {
        if (meta[id].kind != kInput) continue;
        e->input_ids.push_back(id);
        meta[id].region_off = cursor;
        e->input_off.push_back(cursor);
        cursor = round_up(cursor + size_t(e->reg[id].nbytes), kAlign);
    }
    e->input_bytes = cursor - const_cursor;

    // ---- nodes: ids and params are copied out; the file buffer is not needed after build ----
    std::vector<bool> feeds_output(n_tensors, false);
    for (uint32_t id : order)
        if (meta[id].kind == kOutput) {
            feeds_output[id] = true;
            if (meta[id].alias_of >= 0 && uint32_t(meta[id].alias_of) < n_tensors) feeds_output[meta[id].alias_of] = true;
        }
    PlanEnv env;
    env.gemm_mode = e->opts.gemm_mode;
    env.tp_rank = e->opts.tp_rank;
    env.tp_size = e->opts.tp_size;
    env.tc_pairs = e->opts.tc_pair != 1;
    for (uint32_t i = 0; i < n_nodes; i++) {
        fbs::Table nt = g.table_at(fbs::GraphF::nodes, i);
        int op = nt.scalar<int8_t>(fbs::NodeF::op_code, 0);
        if (op == FXF_OP_NOOP) continue;
        FXF_CHECK(op > 0 && op < FXF_OP_COUNT, "Unsupported OpCode: %d", op);
        const OpEntry& entry = op_entry(op);
        FXF_CHECK(entry.kernel != nullptr, "Unregistered OpCode: %d", op);
        Node n;
        n.op = op;
        n.fn = entry.kernel;
        auto in = nt.vec<uint32_t>(fbs::NodeF::input_ids);
        auto out = nt.vec<uint32_t>(fbs::NodeF::output_ids);
        auto ints = nt.vec<int64_t>(fbs::NodeF::int_params);
        auto floats = nt.vec<float>(fbs::NodeF::float_params);
        for (uint32_t k = 0; k < in.size(); k++) n.in.push_back(in[k]);
        for (uint32_t k = 0; k < out.size(); k++) n.out.push_back(out[k]);
        for (uint32_t k = 0; k < ints.size(); k++) n.params.ints.push_back(ints[k]);
        for (uint32_t k = 0; k < floats.size(); k++) n.params.floats.push_back(floats[k]);
        for (auto id : n.in) FXF_CHECK(id < n_tensors, "node %u (%s) reads tensor id %u which does not exist", i, entry.name, id);
        for (auto id : n.out) FXF_CHECK(id < n_tensors, "node %u (%s) writes tensor id %u which does not exist", i, entry.name, id);
        FXF_CHECK(!n.out.empty(), "node %u (%s) has no output", i, entry.name);
        e->nodes.push_back(std::move(n));
    }

    // ---- layout pass: keep 4-D activations channels-last between layout-aware nodes ------------------
    // Convolutions may write channels-last (their 1x1 form is then a plain GEMM on the tensor cores); pools and
    // same-shape Add / AddRelu follow their operands.  A tensor stays NCHW if anything else reads it, if it is
    // aliased (views, outputs) or if it is a graph input/output: the file's NCHW contract holds at every boundary.
    {
        std::vector<char> cl(n_tensors, 0);
        auto differs = [&](uint32_t id) {  // layouts are distinguishable only for C > 1 and H*W > 1
            const FxfTensor& t = e->reg[id];
            return t.rank == 4 && t.dtype == FXF_F32 && t.shape[1] > 1 && t.shape[2] * t.shape[3] > 1;
        };
        auto same_shape = [&](uint32_t a, uint32_t b) {
            const FxfTensor &x = e->reg[a], &y = e->reg[b];
            if (x.rank != y.rank) return false;
            for (int k = 0; k < x.rank; k++)
                if (x.shape[k] != y.shape[k]) return false;
            return true;
        };
        for (auto& n : e->nodes)
            if ((n.op == FXF_OP_CONV2D || n.op == FXF_OP_CONV2D_RELU) && differs(n.out[0]) && meta[n.out[0]].kind == kActivation) cl[n.out[0]] = 1;
        for (auto& n : e->nodes) {  // optimistic propagation through pools and element-wise nodes
            const bool pool = n.op == FXF_OP_MAX_POOL2D || n.op == FXF_OP_AVG_POOL2D || n.op == FXF_OP_ADAPTIVE_AVG_POOL2D;
            const bool ew = n.op == FXF_OP_ADD || n.op == FXF_OP_ADD_RELU;
            if (!(pool || ew) || !differs(n.out[0]) || meta[n.out[0]].kind != kActivation) continue;
            bool all = !n.in.empty();
            for (auto id : n.in) all = all && cl[id] && (pool || same_shape(id, n.out[0]));
            if (all) cl[n.out[0]] = 1;
        }
        for (bool changed = true; changed;) {
            changed = false;
            auto demote = [&](uint32_t id) {
                if (cl[id]) { cl[id] = 0; changed = true; }
            };
            for (uint32_t id : order)
                if ((meta[id].kind == kAlias || meta[id].kind == kOutput) && meta[id].alias_of >= 0 && uint32_t(meta[id].alias_of) < n_tensors)
                    demote(uint32_t(meta[id].alias_of));
            for (auto& n : e->nodes) {
                const bool conv = n.op == FXF_OP_CONV2D || n.op == FXF_OP_CONV2D_RELU;
                const bool pool = n.op == FXF_OP_MAX_POOL2D || n.op == FXF_OP_AVG_POOL2D || n.op == FXF_OP_ADAPTIVE_AVG_POOL2D;
                const bool ew = n.op == FXF_OP_ADD || n.op == FXF_OP_ADD_RELU;
                if (conv) continue;  // reads and writes either layout
                if (pool) {
                    if (differs(n.out[0]) && cl[n.in[0]] != cl[n.out[0]]) { demote(n.in[0]); demote(n.out[0]); }
                    continue;
                }
                if (ew) {
                    bool uniform = true;
                    for (auto id : n.in) uniform = uniform && same_shape(id, n.out[0]) && cl[id] == cl[n.out[0]];
                    if (!uniform) {
                        for (auto id : n.in) demote(id);
                        demote(n.out[0]);
                    }
                    continue;
                }
                for (auto id : n.in) demote(id);
            }
        }
        for (uint32_t id = 0; id < n_tensors; id++)
            if (cl[id]) set_channels_last(e->reg[id]);
    }

    // ---- plans (they see the final layouts) ---------------------------------------------------------
    for (auto& n : e->nodes) {
        const int op = n.op;
        const OpEntry& entry = op_entry(op);
        env.shard_output_cols = false;
        if (e->opts.tp_size > 1 && e->opts.tp_shard_output && op == FXF_OP_LINEAR && feeds_output[n.out[0]] && n.in.size() >= 2 &&
            e->reg[n.in[1]].rank == 2 && !e->head_sharded) {
            env.shard_output_cols = true;
            e->head_sharded = true;
            int64_t N = e->reg[n.in[1]].shape[0], c = (N + e->opts.tp_size - 1) / e->opts.tp_size;
            e->head_col0 = std::min<int64_t>(N, c * e->opts.tp_rank);
            e->head_ncols = std::min<int64_t>(N, e->head_col0 + c) - e->head_col0;
        }
        n.plan = entry.plan(e->reg, n.in, n.out, n.params, env);
        e->scratch_bytes = std::max(e->scratch_bytes, n.plan->scratch_bytes);
        e->persist_bytes += round_up(n.plan->persist_bytes, kAlign);
    }
    constexpr size_t kP2pRegion = 8192;  // [0, 4096): flags [rank][block]; [4096, ..): epoch, block counter
    if (e->comm != nullptr && e->opts.tp_size > 1) {
        // placed before everything whose size may differ between ranks, so that its offset is the same everywhere
        e->p2p_off = cursor;
        cursor += kP2pRegion;
        // exchange window of the row-parallel products (their largest output): same size and offset on every rank
        if (e->opts.tp_push) {
            for (auto& n : e->nodes)
                if (n.plan && n.plan->tp_sharded && (n.op == FXF_OP_MHA || n.op == FXF_OP_CROSS_MHA || n.op == FXF_OP_FEEDFORWARD) && !n.out.empty())
                    e->push_bytes = std::max(e->push_bytes, round_up(size_t(e->reg[n.out[0]].nbytes), kAlign));
            e->push_off = cursor;
            cursor += e->push_bytes;
        }
    }
    size_t persist_off = cursor;
    cursor += e->persist_bytes;
    e->scratch_off = cursor;
    cursor = round_up(cursor + e->scratch_bytes, kAlign);
    e->status_off = cursor;
    cursor += kAlign;
    if (e->opts.gemm_mode != FXF_GEMM_FP32_SIMT) {
        // K-split workspace of the tensor-core GEMM: one 128 x 256 partial tile and eight flags (one per epilogue warp) per SM
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, e->device);
        e->gemm_ws_off = cursor;
        e->gemm_ws_bytes = round_up(size_t(sms) * 128 * 256 * sizeof(float), kAlign);
        cursor += e->gemm_ws_bytes;
        e->gemm_flags_off = cursor;
        e->gemm_flags_bytes = round_up(size_t(sms) * 8 * sizeof(int), kAlign);
        cursor += e->gemm_flags_bytes;
    }
    if (e->head_sharded && !e->input_ids.empty() && e->reg[e->input_ids[0]].rank >= 1) {
        e->cand_off = cursor;
        e->cand_bytes = round_up(size_t(e->opts.tp_size + 1) * size_t(e->reg[e->input_ids[0]].shape[0]) * 16, kAlign);
        cursor += e->cand_bytes;
    }
    // a graph that ends in Linear([B,T,D]) -> output 0 can decode with that Linear evaluated on one position only
    uint32_t first_output = n_tensors;  // output 0 = the first output tensor in file order (as the binding below numbers them)
    for (uint32_t id : order)
        if (meta[id].kind == kOutput) { first_output = id; break; }
    if (!e->nodes.empty() && first_output < n_tensors) {
        int last = int(e->nodes.size()) - 1;
        while (last > 0 && e->nodes[size_t(last)].op == 0) last--;  // trailing no-op (output / constant) nodes launch nothing
        const Node& t = e->nodes[size_t(last)];
        if (t.op == FXF_OP_LINEAR && t.in.size() >= 3 && t.out.size() == 1 &&
            (t.out[0] == first_output || (meta[first_output].alias_of >= 0 && uint32_t(meta[first_output].alias_of) == t.out[0]))) {
            const FxfTensor &x = e->reg[t.in[0]], &w = e->reg[t.in[1]], &o = e->reg[t.out[0]];
            if (x.rank == 3 && o.rank == 3 && w.rank == 2 && x.dtype == FXF_F32 && w.dtype == FXF_F32 && x.shape[2] == w.shape[1] && o.shape[2] == w.shape[0]) {
                e->tail_node = last;
                e->lastrow_off = cursor;
                e->lastrow_bytes = round_up(size_t(o.shape[0]) * size_t(o.shape[2]) * sizeof(float), kAlign);
                cursor += e->lastrow_bytes;
            }
        }
    }
    e->total_bytes = cursor;

    // ---- the one device allocation -----------------------------------------------------------
    FXF_CUDA(cudaSetDevice(e->device));
    cudaDeviceProp prop;
    FXF_CUDA(cudaGetDeviceProperties(&prop, e->device));
    FXF_CHECK(prop.major == 10, "this library is built for sm_100a only (B200); device %d is sm_%d%d", e->device, prop.major, prop.minor);
    e->ctx.sm_count = prop.multiProcessorCount;
    e->ctx.gemm_mode = e->opts.gemm_mode;
    e->ctx.tc_chunk_k = e->opts.tc_chunk_k;
    e->ctx.tc_pair = e->opts.tc_pair;
    e->ctx.tp_rank = e->opts.tp_rank;
    e->ctx.tp_size = e->opts.tp_size;
    e->ctx.comm = e->comm;
    void* p = nullptr;
    cudaError_t err = cudaMalloc(&p, e->total_bytes);
    if (err != cudaSuccess) FXF_FAIL("Arena tensor is not allocated: cudaMalloc(%zu bytes) failed: %s", e->total_bytes, cudaGetErrorString(err));
    e->base = static_cast<uint8_t*>(p);
    FXF_CUDA(cudaMemset(e->base, 0, e->arena_bytes));
    FXF_CUDA(cudaMemset(e->base + e->status_off, 0, kAlign));
    e->ctx.scratch = e->base + e->scratch_off;
    e->ctx.scratch_bytes = e->scratch_bytes;
    e->ctx.status = reinterpret_cast<int*>(e->base + e->status_off);
    if (e->p2p_off) {
        FXF_CUDA(cudaMemset(e->base + e->p2p_off, 0, kP2pRegion));
        FXF_CUDA(cudaDeviceSynchronize());
        // FXF_TP_ALLREDUCE=nccl keeps NCCL for the two all-reduces of a layer (debugging / comparison)
        const char* mode = std::getenv("FXF_TP_ALLREDUCE");
        if (!(mode && mode[0] == 'n')) {
            if (tp_map_peers(e->comm, e->base, &e->peers) == 0) {
                e->peers.shared_bytes = e->arena_bytes;
                e->peers.flags_off = e->p2p_off;
                e->peers.epoch_off = e->p2p_off + 4096;
                e->peers.push_off = e->push_off;
                e->peers.push_bytes = e->push_bytes;
                e->peers.grid = 128;  // 8 ranks x 128 blocks x 4 bytes = 4 KB of flags
                if (e->opts.p2p_grid >= 1 && e->opts.p2p_grid <= 128) e->peers.grid = e->opts.p2p_grid;
                e->peers_mapped = true;
                e->ctx.peers = &e->peers;
            } else {
                set_last_error("");   // not an error: the all-reduce stays with NCCL
            }
        }
    }
    if (e->gemm_ws_bytes) {
        e->ctx.gemm_ws = reinterpret_cast<float*>(e->base + e->gemm_ws_off);
        e->ctx.gemm_ws_bytes = e->gemm_ws_bytes;
        e->ctx.gemm_flags = reinterpret_cast<int*>(e->base + e->gemm_flags_off);
        e->ctx.gemm_flag_count = int(e->gemm_flags_bytes / sizeof(int));
        FXF_CUDA(cudaMemset(e->ctx.gemm_flags, 0, e->gemm_flags_bytes));
    }

    // ---- fusion of the nodes that follow a dense contraction (decided here: whether the peers are mapped is known) ------
    {
        auto root = [&](uint32_t id) {
            for (int guard = 0; guard < 64 && meta[id].alias_of >= 0 && uint32_t(meta[id].alias_of) < n_tensors; guard++) id = uint32_t(meta[id].alias_of);
            return id;
        };
        auto same_shape = [&](uint32_t a, uint32_t b) {
            const FxfTensor &x = e->reg[a], &y = e->reg[b];
            if (x.rank != y.rank) return false;
            for (int k = 0; k < x.rank; k++)
                if (x.shape[k] != y.shape[k]) return false;
            return true;
        };
        std::vector<int> producer(n_tensors, -1), n_readers(n_tensors, 0);
        std::vector<char> escapes(n_tensors, 0);
        for (size_t i = 0; i < e->nodes.size(); i++) {
            for (auto id : e->nodes[i].out) producer[root(id)] = int(i);
            for (auto id : e->nodes[i].in) n_readers[root(id)]++;
        }
        for (uint32_t id = 0; id < n_tensors; id++)
            if (meta[id].kind == kOutput) escapes[root(id)] = 1;
        auto arena_range = [&](uint32_t id, int64_t* lo, int64_t* hi) {   // false: not in the arena (constant, input)
            const uint32_t r = root(id);
            if (meta[r].kind == kConstant || meta[r].kind == kInput || meta[r].offset < 0) return false;
            *lo = meta[r].offset;
            *hi = meta[r].offset + int64_t(e->reg[r].nbytes);
            return true;
        };

        // -- tensor parallelism: [sharded contraction -> Add -> LayerNorm] or [sharded contraction -> AddLayerNorm] becomes the
        // contraction plus ONE exchange kernel over peer memory that sums the ranks' partial outputs, adds the residual and
        // normalises (kernels/tp_exchange.cu).  Rank r owns rows [r*R, (r+1)*R): it alone computes them, keeps the new residual
        // rows for itself and stores the normalised rows on every rank.  Conditions: the peers are mapped; the contraction's
        // result is read by the Add only; no broadcasting; the LayerNorm normalises the last dimension (<= 1024 floats); every
        // tensor the kernel writes lies in the arena, apart from or exactly on top of each tensor it reads (rows have one owner,
        // so exact overlap is harmless) and apart from the other output.
        if (e->peers_mapped && !e->opts.no_tp_fused_exchange) {
            auto is_plain_f32 = [&](uint32_t id) { return e->reg[id].dtype == FXF_F32 && is_contiguous(e->reg[id]); };
            auto compatible = [&](uint32_t w, uint32_t r) {   // written tensor w vs read tensor r: disjoint or identical
                int64_t wl = 0, wh = 0, rl = 0, rh = 0;
                if (!arena_range(w, &wl, &wh)) return false;
                if (!arena_range(r, &rl, &rh)) return true;
                return wh <= rl || rh <= wl || (wl == rl && wh == rh);
            };
            for (size_t ai = 0; ai + 1 < e->nodes.size(); ai++) {
                Node& A = e->nodes[ai];
                if ((A.op != FXF_OP_FEEDFORWARD && A.op != FXF_OP_MHA && A.op != FXF_OP_CROSS_MHA) || !A.plan->tp_sharded || A.out.size() != 1) continue;
                Node& B = e->nodes[ai + 1];
                const bool add = B.op == FXF_OP_ADD && B.in.size() == 2, addln = B.op == FXF_OP_ADD_LAYER_NORM && B.in.size() == 4;
                if ((!add && !addln) || B.out.size() != 1) continue;
                const uint32_t t = root(A.out[0]);
                const int which = root(B.in[0]) == t ? 0 : (root(B.in[1]) == t ? 1 : -1);
                if (which < 0) continue;
                const uint32_t r = B.in[1 - which], o = B.out[0];
                if (root(r) == t || n_readers[t] != 1 || escapes[t]) continue;
                if (!is_plain_f32(A.out[0]) || !is_plain_f32(r) || !is_plain_f32(o) || !same_shape(A.out[0], r) || !same_shape(A.out[0], o)) continue;
                if (producer[root(r)] >= int(ai)) continue;   // the residual exists before the contraction runs
                const FxfTensor& ta = e->reg[A.out[0]];
                if (ta.rank < 1) continue;
                const int64_t D = ta.shape[ta.rank - 1];
                if (D <= 0 || D % 4 != 0 || D > 1024 || numel(ta) == 0) continue;
                int64_t lo = 0, hi = 0;
                if (!arena_range(A.out[0], &lo, &hi) || !arena_range(o, &lo, &hi) || meta[o].alias_of >= 0) continue;
                auto ln_over_last_dim = [&](const Node& n, size_t w_at) {
                    return n.params.ints.size() >= 2 && n.params.ints[0] == 1 && n.params.ints[1] == D && !n.params.floats.empty() &&
                           numel(e->reg[n.in[w_at]]) == D && numel(e->reg[n.in[w_at + 1]]) == D && e->reg[n.in[w_at]].dtype == FXF_F32 &&
                           e->reg[n.in[w_at + 1]].dtype == FXF_F32;
                };
                if (addln) {
                    if (!ln_over_last_dim(B, 2)) continue;
                    if (!compatible(o, A.out[0]) || !compatible(o, r)) continue;
                    A.xchg = true;
                    A.xchg_res = int(r); A.xchg_y = int(o); A.xchg_gamma = int(B.in[2]); A.xchg_beta = int(B.in[3]); A.xchg_eps = B.params.floats[0];
                    B.folded = true;
                    continue;
                }
                if (!compatible(o, A.out[0]) || !compatible(o, r)) continue;
                A.xchg = true;
                A.xchg_res = int(r); A.xchg_x = int(o);
                A.xchg_replicate_x = true;   // until the second pass has looked at the readers
                B.folded = true;
                if (ai + 2 < e->nodes.size()) {
                    Node& Cn = e->nodes[ai + 2];
                    if (Cn.op == FXF_OP_LAYER_NORM && Cn.in.size() == 3 && Cn.out.size() == 1 && root(Cn.in[0]) == root(o) && ln_over_last_dim(Cn, 1) &&
                        is_plain_f32(Cn.out[0]) && same_shape(Cn.out[0], o) && meta[Cn.out[0]].alias_of < 0 && arena_range(Cn.out[0], &lo, &hi) &&
                        compatible(Cn.out[0], A.out[0]) && compatible(Cn.out[0], r)) {
                        int64_t yl = 0, yh = 0, xl = 0, xh = 0;
                        arena_range(Cn.out[0], &yl, &yh);
                        arena_range(o, &xl, &xh);
                        if (yh <= xl || xh <= yl) {
                            A.xchg_y = int(Cn.out[0]); A.xchg_gamma = int(Cn.in[1]); A.xchg_beta = int(Cn.in[2]); A.xchg_eps = Cn.params.floats[0];
                            Cn.folded = true;
                        }
                    }
                }
            }
            // second pass: the new residual stream may stay row-sharded (each rank holds only the rows it owns) when every reader
            // of it is inside the scheme: the LayerNorm folded into the same exchange, or the residual operand of a later
            // exchange with the same row partition.  Anything else (another node, a graph output) needs every row everywhere.
            for (size_t ai = 0; ai < e->nodes.size(); ai++) {
                Node& A = e->nodes[ai];
                if (!A.xchg || A.xchg_x < 0) continue;
                const uint32_t X = root(uint32_t(A.xchg_x));
                bool inside = !escapes[X];
                for (size_t bi = 0; bi < e->nodes.size() && inside; bi++) {
                    const Node& R = e->nodes[bi];
                    bool reads = false;
                    for (auto id : R.in) reads = reads || root(id) == X;
                    if (!reads) continue;
                    if (R.folded && bi == ai + 2 && A.xchg_y >= 0) continue;   // the LayerNorm folded into this exchange
                    bool ok = false;
                    if (R.folded && bi >= 1) {
                        const Node& P = e->nodes[bi - 1];   // the contraction this Add / AddLayerNorm was folded into
                        ok = P.xchg && P.xchg_res >= 0 && root(uint32_t(P.xchg_res)) == X && numel(e->reg[P.out[0]]) == numel(e->reg[A.out[0]]) &&
                             e->reg[P.out[0]].shape[e->reg[P.out[0]].rank - 1] == e->reg[A.out[0]].shape[e->reg[A.out[0]].rank - 1];
                        // X must be that Add's residual operand only, not also its other operand
                        int uses = 0;
                        for (auto id : R.in) uses += root(id) == X ? 1 : 0;
                        ok = ok && uses == 1;
                    }
                    inside = ok;
                }
                A.xchg_replicate_x = !inside;
            }
        }

        // -- a residual Add / AddRelu right after a dense contraction is folded into that contraction's epilogue: it writes
        // act(acc + bias + residual) straight into the Add's output (bit-identical to the two nodes run separately: the same
        // two fp32 additions in the same order).  Conditions: the two nodes are adjacent; the contraction's result (through
        // aliases) is read by nothing else and is not a graph output; shapes, dtypes and layouts agree without broadcasting;
        // the residual exists before the contraction runs; and the Add's output does not share arena bytes with any operand
        // the writing GEMM still reads (the planner may have given it the slot of a tensor that dies at the contraction).
        for (size_t bi = 1; !e->opts.no_epilogue_fusion && bi < e->nodes.size(); bi++) {
            Node &A = e->nodes[bi - 1], &B = e->nodes[bi];
            if ((B.op != FXF_OP_ADD && B.op != FXF_OP_ADD_RELU) || B.in.size() != 2 || B.out.size() != 1 || B.folded || A.xchg) continue;
            // Convolutions are left alone: their layers are bandwidth-bound with short K loops, and the residual read in the
            // GEMM epilogue (16 KB in flight per SM) is slower than the separate AddRelu kernel (measured on ResNet-50).
            if (A.op != FXF_OP_LINEAR && A.op != FXF_OP_FEEDFORWARD && A.op != FXF_OP_MHA && A.op != FXF_OP_CROSS_MHA) continue;
            if (A.fuse_out >= 0 || A.out.size() != 1) continue;
            if (B.op == FXF_OP_ADD_RELU && A.plan->tp_sharded) continue;   // the ReLU would have to follow the all-reduce
            if (A.op == FXF_OP_LINEAR && e->opts.tp_size > 1 && e->opts.tp_shard_output) continue;
            const uint32_t t = root(A.out[0]);
            const int which = root(B.in[0]) == t ? 0 : (root(B.in[1]) == t ? 1 : -1);
            if (which < 0) continue;
            const uint32_t r = B.in[1 - which], o = B.out[0];
            if (root(r) == t || n_readers[t] != 1 || escapes[t]) continue;
            const FxfTensor &ta = e->reg[A.out[0]], &tr = e->reg[r], &to = e->reg[o];
            if (ta.dtype != FXF_F32 || tr.dtype != FXF_F32 || to.dtype != FXF_F32) continue;
            if (!same_shape(A.out[0], r) || !same_shape(A.out[0], o)) continue;
            if (!same_layout(ta, tr) || !same_layout(ta, to)) continue;
            const int pr = producer[root(r)];
            if (pr >= int(bi) - 1) continue;   // the residual must exist before the contraction runs (inputs / constants: -1)
            int64_t olo = 0, ohi = 0;
            if (!arena_range(o, &olo, &ohi) || meta[o].alias_of >= 0) continue;
            bool clash = false;
            // MHA / CrossMHA / FeedForward read their activation inputs in their first GEMM; the final GEMM, which does the
            // writing, reads only scratch and weights.  A plain Linear reads its input while it writes.
            if (A.op == FXF_OP_LINEAR)
                for (auto id : A.in) {
                    int64_t lo = 0, hi = 0;
                    if (arena_range(id, &lo, &hi) && lo < ohi && olo < hi) clash = true;
                }
            int64_t rlo = 0, rhi = 0;
            if (arena_range(r, &rlo, &rhi) && rlo < ohi && olo < rhi) clash = true;
            if (clash) continue;
            A.fuse_res = int(r);
            A.fuse_out = int(o);
            A.fuse_relu = B.op == FXF_OP_ADD_RELU;
            B.folded = true;
        }
    }

    // ---- registry binding, in file order (an alias binds to an already-built source) --------
    std::vector<bool> bound(n_tensors, false);
    for (uint32_t id : order) {
        Meta& m = meta[id];
        FxfTensor& r = e->reg[id];
        switch (m.kind) {
            case kConstant:
                r.ptr = e->base + m.region_off;
                if (r.nbytes) FXF_CUDA(cudaMemcpy(r.ptr, m.data, size_t(r.nbytes), cudaMemcpyHostToDevice));
                break;
            case kInput:
                r.ptr = e->base + m.region_off;
                if (r.nbytes) FXF_CUDA(cudaMemset(r.ptr, 0, size_t(r.nbytes)));
                break;
            case kActivation:
                FXF_CHECK(m.offset >= 0, "Arena-backed tensor has invalid offset (tensor %u)", id);
                FXF_CHECK(size_t(m.offset) + size_t(r.nbytes) <= e->arena_bytes, "tensor %u [%lld, +%lld) lies outside the arena of %zu bytes", id,
                          (long long)m.offset, (long long)r.nbytes, e->arena_bytes);
                r.ptr = e->base + m.offset;
                break;
            case kAlias:
            case kOutput:
                if (m.offset >= 0) {
                    FXF_CHECK(size_t(m.offset) + size_t(r.nbytes) <= e->arena_bytes, "tensor %u [%lld, +%lld) lies outside the arena of %zu bytes", id,
                              (long long)m.offset, (long long)r.nbytes, e->arena_bytes);
                    r.ptr = e->base + m.offset;
                } else {
                    int src = m.alias_of;
                    FXF_CHECK(src >= 0 && uint32_t(src) < n_tensors, "Invalid alias source ID (tensor %u aliases %d)", id, src);
                    FXF_CHECK(bound[src], "Alias source tensor is not defined (tensor %u aliases %d)", id, src);
                    FXF_CHECK(numel(e->reg[src]) == numel(r),
                              "Alias numel mismatch for tensor id %u — runtime-shape-changing ops must not be marked as Alias kind", id);
                    r.ptr = e->reg[src].ptr;
                }
                if (m.kind == kOutput) e->output_ids.push_back(id);
                break;
        }
        bound[id] = true;
    }

    // ---- per-node persistent memory + one-off preparation -----------------------------------
    size_t pcur = persist_off;
    for (auto& n : e->nodes) {
        if (n.plan->persist_bytes) {
            n.plan->persist = e->base + pcur;
            pcur += round_up(n.plan->persist_bytes, kAlign);
        }
        if (n.plan->prepare(e->reg, n.in, n.out, n.params, e->ctx)) return 1;
    }
    FXF_CUDA(cudaDeviceSynchronize());

    // ---- warm-up run (validates every node's arguments), then capture ------------------------
    FXF_CUDA(cudaStreamCreateWithFlags(&e->capture_stream, cudaStreamNonBlocking));
    e->ctx.launches = 0;
    if (run_nodes(e, e->capture_stream)) return 1;
    e->launches_per_run = e->ctx.launches;
    FXF_CUDA(cudaStreamSynchronize(e->capture_stream));
    // The warm-up above ran with the default (generous) peer-wait budgets: the ranks reach it with whatever skew their
    // builds had.  The caller's budgets apply from here on (they are kernel arguments, so they are set before the capture).
    if (e->peers_mapped) {
        if (e->opts.p2p_start_budget_ms > 0) e->peers.start_budget_ns = (unsigned long long)e->opts.p2p_start_budget_ms * 1000000ull;
        if (e->opts.p2p_end_budget_ms > 0) e->peers.end_budget_ns = (unsigned long long)e->opts.p2p_end_budget_ms * 1000000ull;
    }
    if (e->opts.use_cuda_graph && !e->nodes.empty()) {
        FXF_CUDA(cudaStreamBeginCapture(e->capture_stream, cudaStreamCaptureModeThreadLocal));
        int rc = run_nodes(e, e->capture_stream);
        cudaError_t ce = cudaStreamEndCapture(e->capture_stream, &e->graph);
        if (rc) return 1;
        if (ce != cudaSuccess) FXF_FAIL("CUDA Graph capture failed: %s", cudaGetErrorString(ce));
        FXF_CUDA(cudaGraphInstantiate(&e->graph_exec, e->graph, 0));
        if (e->tail_node > 0) {
            FXF_CUDA(cudaStreamBeginCapture(e->capture_stream, cudaStreamCaptureModeThreadLocal));
            rc = run_nodes(e, e->capture_stream, e->tail_node);
            ce = cudaStreamEndCapture(e->capture_stream, &e->body_graph);
            if (rc) return 1;
            if (ce != cudaSuccess) FXF_FAIL("CUDA Graph capture (decode body) failed: %s", cudaGetErrorString(ce));
            FXF_CUDA(cudaGraphInstantiate(&e->body_exec, e->body_graph, 0));
        }
    }
    // the warm-up ran on zeroed inputs; leave the arena clean
    FXF_CUDA(cudaMemset(e->base, 0, e->arena_bytes));
    FXF_CUDA(cudaMemset(e->base + e->status_off, 0, kAlign));
    FXF_CUDA(cudaDeviceSynchronize());
    return 0;
}

int create_from_bytes(const uint8_t* bytes, size_t nbytes, int device, const FxfEngineOptions* opts, fxf_comm* comm, fxf_engine** out) {
    FXF_CHECK(out != nullptr, "fxf_engine_create: out_engine is NULL");
    *out = nullptr;
    auto e = std::make_unique<fxf_engine>();
    e->device = device;
    e->opts.struct_size = sizeof(FxfEngineOptions);
    e->opts.use_cuda_graph = 1;
    e->opts.gemm_mode = FXF_GEMM_AUTO;
    e->opts.tp_size = 1;
    if (opts) {
        size_t n = std::min<size_t>(sizeof(FxfEngineOptions), opts->struct_size > 0 ? size_t(opts->struct_size) : sizeof(FxfEngineOptions));
        std::memcpy(&e->opts, opts, n);
        if (e->opts.tp_size < 1) e->opts.tp_size = 1;
    }
    if (comm != nullptr) {
        e->comm = comm;
        e->opts.tp_rank = fxf_comm_rank(comm);
        e->opts.tp_size = fxf_comm_size(comm);
    } else {
        FXF_CHECK(e->opts.tp_size == 1, "a tensor-parallel engine (tp_size %d) needs a communicator: use fxf_engine_create_tp", e->opts.tp_size);
        e->opts.tp_rank = 0;
    }
    int count = 0;
    FXF_CUDA(cudaGetDeviceCount(&count));
    FXF_CHECK(device >= 0 && device < count, "device ordinal %d is out of range (%d CUDA devices)", device, count);
    try {
        if (build(e.get(), bytes, nbytes)) return 1;
    } catch (const std::exception& ex) {
        FXF_FAIL("%s", ex.what());
    }
    *out = e.release();
    return 0;
}

}  // namespace
}  // namespace fxf

// =============================================================================================
// C ABI
// =============================================================================================
extern "C" {

const char* fxf_last_error(void) { return fxf::last_error().c_str(); }

const char* fxf_version(void) { return "fxf_b200 19 ops sm_100a"; }

int fxf_engine_create_tp(const char* graph_path, int device_ordinal, const FxfEngineOptions* opts, fxf_comm* comm, fxf_engine** out_engine) {
    FXF_CHECK(graph_path != nullptr, "fxf_engine_create: graph_path is NULL");
    std::ifstream f(graph_path, std::ios::binary | std::ios::ate);
    if (!f.is_open()) FXF_FAIL("ExecutionEngine failed to open: %s", graph_path);
    std::streamsize size = f.tellg();
    f.seekg(0, std::ios::beg);
    std::vector<uint8_t> bytes(size > 0 ? size_t(size) : 0);
    if (size > 0 && !f.read(reinterpret_cast<char*>(bytes.data()), size)) FXF_FAIL("ExecutionEngine failed to read: %s", graph_path);
    return create_from_bytes(bytes.data(), bytes.size(), device_ordinal, opts, comm, out_engine);
}

int fxf_engine_create(const char* graph_path, int device_ordinal, const FxfEngineOptions* opts, fxf_engine** out_engine) {
    return fxf_engine_create_tp(graph_path, device_ordinal, opts, nullptr, out_engine);
}

int fxf_engine_create_from_memory(const void* bytes, size_t nbytes, int device_ordinal, const FxfEngineOptions* opts, fxf_engine** out_engine) {
    FXF_CHECK(bytes != nullptr, "fxf_engine_create_from_memory: bytes is NULL");
    return create_from_bytes(static_cast<const uint8_t*>(bytes), nbytes, device_ordinal, opts, nullptr, out_engine);
}

void fxf_engine_destroy(fxf_engine* e) {
    if (!e) return;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != e->device) cudaSetDevice(e->device);
    cudaDeviceSynchronize();
    const int dev = e->device;
    delete e;
    if (cur >= 0 && cur != dev) cudaSetDevice(cur);
}

int fxf_engine_num_inputs(const fxf_engine* e) { return e ? int(e->input_ids.size()) : -1; }
int fxf_engine_num_outputs(const fxf_engine* e) { return e ? int(e->output_ids.size()) : -1; }
int fxf_engine_num_nodes(const fxf_engine* e) { return e ? int(e->nodes.size()) : -1; }
int64_t fxf_engine_arena_bytes(const fxf_engine* e) { return e ? int64_t(e->arena_bytes) : -1; }
int64_t fxf_engine_device_bytes(const fxf_engine* e) { return e ? int64_t(e->total_bytes) : -1; }
int fxf_engine_launches_per_run(const fxf_engine* e) { return e ? e->launches_per_run : -1; }

int fxf_engine_input_desc(const fxf_engine* e, int i, FxfTensor* out) {
    FXF_CHECK(e && out, "fxf_engine_input_desc: NULL argument");
    FXF_CHECK(i >= 0 && size_t(i) < e->input_ids.size(), "input index %d out of range", i);
    *out = e->reg[e->input_ids[i]];
    return 0;
}
int fxf_engine_output_desc(const fxf_engine* e, int i, FxfTensor* out) {
    FXF_CHECK(e && out, "fxf_engine_output_desc: NULL argument");
    FXF_CHECK(i >= 0 && size_t(i) < e->output_ids.size(), "output index %d out of range", i);
    *out = e->reg[e->output_ids[i]];
    return 0;
}

static int launch_forward(fxf_engine* e, cudaStream_t s) {
    if (e->graph_exec) {
        FXF_CUDA(cudaGraphLaunch(e->graph_exec, s));
        return 0;
    }
    return run_nodes(e, s);
}

int fxf_engine_run(fxf_engine* e, const void* const* device_inputs, int n_inputs, void* stream) {
    FXF_CHECK(e != nullptr, "fxf_engine_run: engine is NULL");
    FXF_CHECK(size_t(n_inputs) == e->input_ids.size(), "Input count mismatch: the graph has %zu inputs, %d were given", e->input_ids.size(), n_inputs);
    if (ensure_device(e)) return 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < n_inputs; i++) {
        FxfTensor& slot = e->reg[e->input_ids[i]];
        FXF_CHECK(device_inputs && device_inputs[i], "input %d is NULL", i);
        if (device_inputs[i] != slot.ptr && slot.nbytes)
            FXF_CUDA(cudaMemcpyAsync(slot.ptr, device_inputs[i], size_t(slot.nbytes), cudaMemcpyDeviceToDevice, s));
    }
    return launch_forward(e, s);
}

int fxf_engine_run_host(fxf_engine* e, const void* const* host_inputs, int n_inputs, void* const* host_outputs, int n_outputs, void* stream) {
    FXF_CHECK(e != nullptr, "fxf_engine_run_host: engine is NULL");
    FXF_CHECK(size_t(n_inputs) == e->input_ids.size(), "Input count mismatch: the graph has %zu inputs, %d were given", e->input_ids.size(), n_inputs);
    if (ensure_device(e)) return 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < n_inputs; i++) {
        FxfTensor& slot = e->reg[e->input_ids[i]];
        FXF_CHECK(host_inputs && host_inputs[i], "input %d is NULL", i);
        if (slot.nbytes) FXF_CUDA(cudaMemcpyAsync(slot.ptr, host_inputs[i], size_t(slot.nbytes), cudaMemcpyHostToDevice, s));
    }
    if (launch_forward(e, s)) return 1;
    if (host_outputs) {
        FXF_CHECK(size_t(n_outputs) == e->output_ids.size(), "Output count mismatch: the graph has %zu outputs, %d buffers were given", e->output_ids.size(), n_outputs);
        for (int i = 0; i < n_outputs; i++) {
            const FxfTensor& o = e->reg[e->output_ids[i]];
            if (host_outputs[i] && o.nbytes) FXF_CUDA(cudaMemcpyAsync(host_outputs[i], o.ptr, size_t(o.nbytes), cudaMemcpyDeviceToHost, s));
        }
        FXF_CUDA(cudaStreamSynchronize(s));
    }
    return 0;
}

int fxf_engine_device_status(fxf_engine* e, void* stream, int* status_out) {
    FXF_CHECK(e && status_out, "fxf_engine_device_status: NULL argument");
    if (ensure_device(e)) return 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    FXF_CUDA(cudaMemcpyAsync(status_out, e->ctx.status, sizeof(int), cudaMemcpyDeviceToHost, s));
    FXF_CUDA(cudaStreamSynchronize(s));
    return 0;
}

int fxf_engine_describe(const fxf_engine* e, char* out, size_t out_bytes) {
    FXF_CHECK(e && out && out_bytes > 0, "fxf_engine_describe: NULL argument");
    std::ostringstream os;
    os << "graph '" << e->name << "' device " << e->device << " nodes " << e->nodes.size() << " tensors " << e->reg.size() << "\n";
    os << "device allocation " << e->total_bytes << " B = arena " << e->arena_bytes << " + constants " << e->const_bytes << " + input slots " << e->input_bytes
       << " + persistent " << e->persist_bytes << " + scratch " << e->scratch_bytes << " + status 256";
    if (e->push_bytes) os << " + exchange window " << e->push_bytes;
    os << "\n";
    os << "cuda_graph " << (e->graph_exec ? "yes" : "no") << " launches/run " << e->launches_per_run << "\n";
    for (size_t i = 0; i < e->nodes.size(); i++) {
        const Node& n = e->nodes[i];
        os << i << " " << op_entry(n.op).name << " in[";
        for (auto id : n.in) os << id << " ";
        os << "] out[";
        for (auto id : n.out) os << id << "@" << (static_cast<uint8_t*>(e->reg[id].ptr) - e->base) << (is_channels_last(e->reg[id]) ? "[nhwc] " : " ");
        os << "] launches " << n.launches << " variant " << n.plan->variant << " scratch " << n.plan->scratch_bytes;
        if (n.fuse_out >= 0) os << " +" << (n.fuse_relu ? "AddRelu" : "Add") << "(residual " << n.fuse_res << ") -> out " << n.fuse_out;
        if (n.xchg)
            os << " +exchange(residual " << n.xchg_res << ") -> x " << n.xchg_x << (n.xchg_x >= 0 ? (n.xchg_replicate_x ? " [all rows on every rank]" : " [own rows]") : "")
               << " y " << n.xchg_y;
        if (n.folded) os << " folded into an earlier node";
        os << "\n";
    }
    std::string s = os.str();
    size_t n = std::min(out_bytes - 1, s.size());
    std::memcpy(out, s.data(), n);
    out[n] = 0;
    return 0;
}

int fxf_engine_node_info(const fxf_engine* e, int node, int* op_code, double* flops, double* bytes, char* variant, size_t variant_bytes) {
    FXF_CHECK(e != nullptr, "fxf_engine_node_info: engine is NULL");
    FXF_CHECK(node >= 0 && size_t(node) < e->nodes.size(), "node index %d out of range", node);
    const Node& n = e->nodes[node];
    if (op_code) *op_code = n.op;
    if (flops) *flops = n.plan->flops;
    if (bytes) *bytes = n.plan->bytes;
    if (variant && variant_bytes) {
        size_t k = std::min(variant_bytes - 1, n.plan->variant.size());
        std::memcpy(variant, n.plan->variant.data(), k);
        variant[k] = 0;
    }
    return 0;
}

int fxf_engine_time_nodes(fxf_engine* e, float* ms_out, int n, void* stream) {
    FXF_CHECK(e && ms_out, "fxf_engine_time_nodes: NULL argument");
    FXF_CHECK(size_t(n) >= e->nodes.size(), "fxf_engine_time_nodes: buffer holds %d values, %zu needed", n, e->nodes.size());
    if (ensure_device(e)) return 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::vector<cudaEvent_t> ev(e->nodes.size() + 1);
    for (auto& x : ev) FXF_CUDA(cudaEventCreate(&x));
    e->ctx.stream = s;
    FXF_CUDA(cudaEventRecord(ev[0], s));
    int rc = 0;
    for (size_t i = 0; i < e->nodes.size() && !rc; i++) {
        rc = run_node(e, i);
        cudaEventRecord(ev[i + 1], s);
    }
    cudaStreamSynchronize(s);
    if (!rc)
        for (size_t i = 0; i < e->nodes.size(); i++) cudaEventElapsedTime(&ms_out[i], ev[i], ev[i + 1]);
    for (auto& x : ev) cudaEventDestroy(x);
    return rc;
}

int fxf_engine_profile_launches(fxf_engine* e, void* stream, FxfLaunchInfo* out, int capacity, int* n_out) {
    FXF_CHECK(e && out && n_out, "fxf_engine_profile_launches: NULL argument");
    if (ensure_device(e)) return 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::vector<LaunchRecord> trace;
    trace.reserve(size_t(e->launches_per_run) + 8);
    cudaEvent_t start;
    FXF_CUDA(cudaEventCreate(&start));
    e->ctx.trace = &trace;
    FXF_CUDA(cudaEventRecord(start, s));
    int rc = run_nodes(e, s);
    e->ctx.trace = nullptr;
    cudaStreamSynchronize(s);
    int n = 0;
    cudaEvent_t prev = start;
    for (auto& r : trace) {
        if (!rc && n < capacity) {
            FxfLaunchInfo& o = out[n];
            std::memset(&o, 0, sizeof(o));
            std::strncpy(o.kernel, r.name, sizeof(o.kernel) - 1);
            o.node = r.node;
            o.flops = r.flops;
            o.bytes = r.bytes;
            cudaEventElapsedTime(&o.ms, prev, r.done);
            n++;
        }
        if (prev != start) cudaEventDestroy(prev);
        prev = r.done;
    }
    if (prev != start) cudaEventDestroy(prev);
    cudaEventDestroy(start);
    *n_out = n;
    FXF_CHECK(rc || size_t(n) == trace.size(), "fxf_engine_profile_launches: %zu launches but capacity %d", trace.size(), capacity);
    return rc;
}

// ---- single kernels -----------------------------------------------------------------------------
static int make_call(int op_code, const FxfTensor* reg, int n_reg, const uint32_t* in_ids, int n_in, const uint32_t* out_ids, int n_out,
                     const int64_t* ints, int n_ints, const float* floats, int n_floats, Registry* r, TensorIds* in, TensorIds* out, Params* p) {
    FXF_CHECK(op_code > 0 && op_code < FXF_OP_COUNT, "Unsupported OpCode: %d", op_code);
    FXF_CHECK(reg != nullptr && n_reg > 0, "kernel call: empty registry");
    r->assign(reg, reg + n_reg);
    for (int i = 0; i < n_in; i++) {
        FXF_CHECK(in_ids[i] < uint32_t(n_reg), "kernel call: input id %u out of range", in_ids[i]);
        in->push_back(in_ids[i]);
    }
    for (int i = 0; i < n_out; i++) {
        FXF_CHECK(out_ids[i] < uint32_t(n_reg), "kernel call: output id %u out of range", out_ids[i]);
        out->push_back(out_ids[i]);
    }
    FXF_CHECK(!out->empty(), "kernel call: no output id");
    if (n_ints > 0) p->ints.assign(ints, ints + n_ints);
    if (n_floats > 0) p->floats.assign(floats, floats + n_floats);
    for (auto& t : *r) FXF_CHECK(t.rank >= 0 && t.rank <= FXF_MAX_DIMS, "kernel call: tensor rank out of range");
    return 0;
}

// A single kernel call that may reach the tensor-core GEMM (its plan keeps split weights) also carries that kernel's
// K-split workspace behind its scratch: partial tiles for up to kCallWsSms SMs, then the flags.
constexpr size_t kCallWsSms = 160, kCallWsTile = size_t(128) * 256 * sizeof(float), kCallFlagBytes = 8192;
static size_t call_ws_bytes(const NodePlan& plan, int gemm_mode) {
    return (gemm_mode != FXF_GEMM_FP32_SIMT && plan.persist_bytes > 0) ? kCallWsSms * kCallWsTile + kCallFlagBytes : 0;
}

int64_t fxf_kernel_scratch_bytes(int op_code, const FxfTensor* reg, int n_reg, const uint32_t* in_ids, int n_in, const uint32_t* out_ids, int n_out,
                                 const int64_t* ints, int n_ints, const float* floats, int n_floats, int gemm_mode) {
    Registry r;
    TensorIds in, out;
    Params p;
    if (make_call(op_code, reg, n_reg, in_ids, n_in, out_ids, n_out, ints, n_ints, floats, n_floats, &r, &in, &out, &p)) return -1;
    PlanEnv env;
    env.gemm_mode = gemm_mode;
    auto plan = op_entry(op_code).plan(r, in, out, p, env);
    return int64_t(round_up(plan->scratch_bytes, 256) + round_up(plan->persist_bytes, 256) + call_ws_bytes(*plan, gemm_mode));
}

int fxf_kernel_invoke(int op_code, const FxfTensor* reg, int n_reg, const uint32_t* in_ids, int n_in, const uint32_t* out_ids, int n_out,
                      const int64_t* ints, int n_ints, const float* floats, int n_floats, void* scratch, int64_t scratch_bytes, int gemm_mode,
                      void* stream) {
    Registry r;
    TensorIds in, out;
    Params p;
    if (make_call(op_code, reg, n_reg, in_ids, n_in, out_ids, n_out, ints, n_ints, floats, n_floats, &r, &in, &out, &p)) return 1;
    const OpEntry& entry = op_entry(op_code);
    PlanEnv env;
    env.gemm_mode = gemm_mode;
    auto plan = entry.plan(r, in, out, p, env);
    const size_t ws_bytes = call_ws_bytes(*plan, gemm_mode);
    size_t need = round_up(plan->scratch_bytes, 256) + round_up(plan->persist_bytes, 256) + ws_bytes;
    FXF_CHECK(need == 0 || (scratch != nullptr && scratch_bytes >= int64_t(need)), "kernel call: scratch too small (%lld < %zu bytes)", (long long)scratch_bytes, need);
    FXF_CHECK(need == 0 || (reinterpret_cast<uintptr_t>(scratch) & 255) == 0, "kernel call: scratch must be 256-byte aligned");
    ExecCtx ctx;
    ctx.stream = static_cast<cudaStream_t>(stream);
    ctx.scratch = scratch;
    ctx.scratch_bytes = plan->scratch_bytes;
    ctx.gemm_mode = gemm_mode;
    if (plan->persist_bytes) plan->persist = static_cast<char*>(scratch) + round_up(plan->scratch_bytes, 256);
    if (ws_bytes) {
        char* ws = static_cast<char*>(scratch) + round_up(plan->scratch_bytes, 256) + round_up(plan->persist_bytes, 256);
        ctx.gemm_ws = reinterpret_cast<float*>(ws);
        ctx.gemm_ws_bytes = kCallWsSms * kCallWsTile;
        ctx.gemm_flags = reinterpret_cast<int*>(ws + kCallWsSms * kCallWsTile);
        ctx.gemm_flag_count = int(kCallFlagBytes / sizeof(int));
        FXF_CUDA(cudaMemsetAsync(ctx.gemm_flags, 0, kCallFlagBytes, ctx.stream));
    }
    int dev = 0;
    FXF_CUDA(cudaGetDevice(&dev));
    int sms = 0;
    FXF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    ctx.sm_count = sms;
    if (plan->prepare(r, in, out, p, ctx)) return 1;
    return entry.kernel(r, in, out, p, plan.get(), ctx);
}

int fxf_gemm_variant(int64_t M, int64_t N, int64_t K, int gemm_mode, int sm_count, char* out, size_t out_bytes) {
    FXF_CHECK(out != nullptr && out_bytes > 0, "fxf_gemm_variant: NULL argument");
    GemmArgs a;
    a.M = M; a.N = N; a.K = K;
    std::string v = gemm_variant_name(a, gemm_mode, sm_count > 0 ? sm_count : 148);
    size_t k = std::min(out_bytes - 1, v.size());
    std::memcpy(out, v.data(), k);
    out[k] = 0;
    return 0;
}

int fxf_tp_exchange_emulated(int n_ranks, const float* const* partial, const float* const* residual, float* const* x_out, float* const* y_out,
                             const float* gamma, const float* beta, float eps, int64_t M, int64_t D, int layout, void* sync_mem, int64_t sync_bytes,
                             int budget_ms, int skip_rank, void* stream) {
    FXF_CHECK(n_ranks >= 2 && sync_mem != nullptr && sync_bytes >= int64_t(n_ranks) * 8192, "fxf_tp_exchange_emulated: sync_mem must hold n_ranks * 8192 zeroed bytes");
    return tp_exchange_emulated(n_ranks, partial, residual, x_out, y_out, gamma, beta, eps, M, D, layout, sync_mem, budget_ms, skip_rank,
                                static_cast<cudaStream_t>(stream));
}

// The row-pushed product of the tensor-parallel layout outside an engine (one GPU can play every producer in turn).
int64_t fxf_linear_pushed_scratch_bytes(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0) return -1;
    return int64_t(2 * round_up(size_t(N) * size_t(K) * sizeof(float), 256) + kCallWsSms * kCallWsTile + kCallFlagBytes);
}

int fxf_linear_pushed(const float* x, const float* w, const float* bias, float* const* windows, int n_ranks, int rank, int64_t M, int64_t N, int64_t K,
                      void* scratch, int64_t scratch_bytes, void* stream) {
    FXF_CHECK(x && w && windows && scratch, "fxf_linear_pushed: NULL argument");
    FXF_CHECK(n_ranks >= 1 && n_ranks <= kMaxTpRanks && rank >= 0 && rank < n_ranks, "fxf_linear_pushed: 1..%d ranks", kMaxTpRanks);
    FXF_CHECK(M > 0 && M % n_ranks == 0 && (M / n_ranks) % 128 == 0, "fxf_linear_pushed: every rank must own a whole number of 128-row tiles");
    FXF_CHECK(scratch_bytes >= fxf_linear_pushed_scratch_bytes(N, K) && (reinterpret_cast<uintptr_t>(scratch) & 255) == 0,
              "fxf_linear_pushed: scratch too small or not 256-byte aligned");
    ExecCtx ctx;
    ctx.stream = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    FXF_CUDA(cudaGetDevice(&dev));
    FXF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    ctx.sm_count = sms;
    const size_t wb = round_up(size_t(N) * size_t(K) * sizeof(float), 256);
    char* s = static_cast<char*>(scratch);
    float *hi = reinterpret_cast<float*>(s), *lo = reinterpret_cast<float*>(s + wb);
    ctx.gemm_ws = reinterpret_cast<float*>(s + 2 * wb);
    ctx.gemm_ws_bytes = kCallWsSms * kCallWsTile;
    ctx.gemm_flags = reinterpret_cast<int*>(s + 2 * wb + kCallWsSms * kCallWsTile);
    ctx.gemm_flag_count = int(kCallFlagBytes / sizeof(int));
    FXF_CUDA(cudaMemsetAsync(ctx.gemm_flags, 0, kCallFlagBytes, ctx.stream));
    if (launch_split_tf32(w, hi, lo, N * K, ctx)) return 1;
    GemmArgs a;
    a.x = x; a.w = w; a.w_hi = hi; a.w_lo = lo; a.bias = bias; a.out = windows[rank];
    a.M = M; a.N = N; a.K = K; a.ldx = K; a.ldw = K; a.ldo = N;
    a.push_out = windows; a.push_rows = M / n_ranks; a.push_rank = rank;
    FXF_CHECK(gemm_tc_supported(a), "fxf_linear_pushed: the shape M=%lld N=%lld K=%lld is not served by the tensor-core kernels", (long long)M, (long long)N, (long long)K);
    return launch_gemm_tc(a, ctx);
}

// ---- greedy static decode ---------------------------------------------------------------------
int fxf_decode_build_mask(const int64_t* tokens, uint8_t* mask, int B, int T, int current_len, int64_t pad_idx, void* stream) {
    FXF_CHECK(tokens && mask, "fxf_decode_build_mask: NULL argument");
    ExecCtx ctx;
    ctx.stream = static_cast<cudaStream_t>(stream);
    return decode_build_mask(tokens, mask, B, T, current_len, pad_idx, ctx);
}

int fxf_decode_argmax_scatter(const float* logits, int64_t* tokens, int B, int T, int64_t V, int current_len, void* stream) {
    FXF_CHECK(logits && tokens, "fxf_decode_argmax_scatter: NULL argument");
    ExecCtx ctx;
    ctx.stream = static_cast<cudaStream_t>(stream);
    return decode_argmax_scatter(logits, tokens, B, T, V, current_len, ctx);
}

int fxf_engine_argmax_scatter(fxf_engine* e, int64_t* tokens, int current_len, void* stream) {
    FXF_CHECK(e && tokens, "fxf_engine_argmax_scatter: NULL argument");
    FXF_CHECK(!e->output_ids.empty(), "fxf_engine_argmax_scatter: the graph has no output");
    const FxfTensor& logits = e->reg[e->output_ids[0]];
    FXF_CHECK(logits.dtype == FXF_F32 && logits.rank == 3, "fxf_engine_argmax_scatter: output 0 must be float32 [B,T,V]");
    if (ensure_device(e)) return 1;
    const int B = int(logits.shape[0]), T = int(logits.shape[1]);
    ExecCtx ctx;
    ctx.stream = static_cast<cudaStream_t>(stream);
    ctx.sm_count = e->ctx.sm_count;
    ctx.tp_rank = e->ctx.tp_rank;
    ctx.tp_size = e->ctx.tp_size;
    ctx.comm = e->ctx.comm;
    if (!e->head_sharded) return decode_argmax_scatter(static_cast<const float*>(logits.ptr), tokens, B, T, logits.shape[2], current_len, ctx);
    FXF_CHECK(e->cand_bytes >= size_t(e->ctx.tp_size + 1) * size_t(B) * 16, "fxf_engine_argmax_scatter: candidate buffer too small");
    char* cand = reinterpret_cast<char*>(e->base + e->cand_off);
    return decode_argmax_scatter_sharded(static_cast<const float*>(logits.ptr), tokens, B, T, logits.shape[2], current_len, e->head_col0,
                                         e->head_ncols, cand, cand + size_t(B) * 16, ctx);
}

static int decode_loop(fxf_engine* e, int64_t* tokens_io, int initial_len, int64_t pad_idx, void* stream, bool last_row);

int fxf_decode_static(fxf_engine* e, int64_t* tokens_io, int initial_len, int64_t pad_idx, void* stream) {
    return decode_loop(e, tokens_io, initial_len, pad_idx, stream, false);
}

int fxf_decode_static_last_row(fxf_engine* e, int64_t* tokens_io, int initial_len, int64_t pad_idx, void* stream) {
    FXF_CHECK(e, "fxf_decode_static_last_row: NULL argument");
    FXF_CHECK(e->tail_node >= 0, "fxf_decode_static_last_row: the graph does not end in a Linear node that produces output 0");
    return decode_loop(e, tokens_io, initial_len, pad_idx, stream, true);
}

int fxf_engine_supports_last_row(const fxf_engine* e) { return e && e->tail_node >= 0 ? 1 : 0; }

// Incremental greedy decode: `e` is a single-position step graph (inputs ids int64 [B,1], pos int64 [1], tokens int64 [B,T];
// output logits [B,1,V]; its attention nodes are CachedMHA).  Position p = 0 .. T-2 is fed in order: the step reads
// tokens[:, p], and from p + 1 >= initial_len on its argmax becomes tokens[:, p + 1].  No host synchronisation.
int fxf_decode_cached(fxf_engine* e, int64_t* tokens_io, int initial_len, void* stream) {
    FXF_CHECK(e && tokens_io, "fxf_decode_cached: NULL argument");
    FXF_CHECK(e->input_ids.size() == 3 && e->output_ids.size() >= 1, "fxf_decode_cached: the graph must take (ids, pos, tokens) and return logits");
    if (ensure_device(e)) return 1;
    const FxfTensor &ids = e->reg[e->input_ids[0]], &pos = e->reg[e->input_ids[1]], &tok = e->reg[e->input_ids[2]], &logits = e->reg[e->output_ids[0]];
    FXF_CHECK(tok.dtype == FXF_I64 && tok.rank == 2, "fxf_decode_cached: input 2 must be int64 [B,T]");
    const int B = int(tok.shape[0]), T = int(tok.shape[1]);
    FXF_CHECK(ids.dtype == FXF_I64 && numel(ids) == B, "fxf_decode_cached: input 0 must be int64 [B,1]");
    FXF_CHECK(pos.dtype == FXF_I64 && numel(pos) == 1, "fxf_decode_cached: input 1 must be one int64");
    FXF_CHECK(logits.dtype == FXF_F32 && logits.rank == 3 && logits.shape[0] == B && logits.shape[1] == 1, "fxf_decode_cached: output 0 must be float32 [B,1,V]");
    FXF_CHECK(initial_len >= 1 && initial_len <= T, "fxf_decode_cached: initial_len %d must be in [1, %d]", initial_len, T);
    FXF_CHECK(!e->head_sharded, "fxf_decode_cached: the step graph's final Linear is sharded over the vocabulary; build the engine without tp_shard_output");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int64_t* slot = static_cast<int64_t*>(tok.ptr);
    if (tokens_io != slot) FXF_CUDA(cudaMemcpyAsync(slot, tokens_io, size_t(tok.nbytes), cudaMemcpyDeviceToDevice, s));
    ExecCtx ctx;
    ctx.stream = s;
    ctx.sm_count = e->ctx.sm_count;
    const int64_t V = logits.shape[2];
    for (int p = 0; p + 1 < T; p++) {
        if (decode_step_prepare(slot, static_cast<int64_t*>(ids.ptr), static_cast<int64_t*>(pos.ptr), B, T, p, ctx)) return 1;
        if (launch_forward(e, s)) return 1;
        if (p + 1 >= initial_len && decode_argmax_scatter_rows(static_cast<const float*>(logits.ptr), V, 0, slot, B, T, V, p + 1, ctx)) return 1;
    }
    if (tokens_io != slot) FXF_CUDA(cudaMemcpyAsync(tokens_io, slot, size_t(tok.nbytes), cudaMemcpyDeviceToDevice, s));
    return 0;
}

// The final Linear on row (current_len - 1) of every sequence -> [B,V] buffer, then argmax + token scatter.
static int last_row_head(fxf_engine* e, int64_t* tokens, int cur, ExecCtx& ctx) {
    const Node& t = e->nodes[size_t(e->tail_node)];
    const FxfTensor &x = e->reg[t.in[0]], &w = e->reg[t.in[1]];
    const int B = int(x.shape[0]), T = int(x.shape[1]);
    const int64_t D = x.shape[2], V = w.shape[0];
    const int64_t col0 = e->head_sharded ? e->head_col0 : 0, ncols = e->head_sharded ? e->head_ncols : V;
    float* rows = reinterpret_cast<float*>(e->base + e->lastrow_off);
    ctx.gemm_mode = e->ctx.gemm_mode;
    ctx.tc_chunk_k = e->ctx.tc_chunk_k;
    ctx.tc_pair = e->ctx.tc_pair;
    ctx.status = e->ctx.status;
    ctx.gemm_ws = e->ctx.gemm_ws; ctx.gemm_ws_bytes = e->ctx.gemm_ws_bytes;
    ctx.gemm_flags = e->ctx.gemm_flags; ctx.gemm_flag_count = e->ctx.gemm_flag_count;
    if (linear_on_rows(t.plan.get(), static_cast<const float*>(x.ptr) + int64_t(cur - 1) * D, B, int64_t(T) * D, rows, V, ctx)) return 1;
    if (!e->head_sharded) return decode_argmax_scatter_rows(rows, V, 0, tokens, B, T, V, cur, ctx);
    char* cand = reinterpret_cast<char*>(e->base + e->cand_off);
    return decode_argmax_scatter_sharded_rows(rows, V, 0, tokens, B, T, V, cur, col0, ncols, cand, cand + size_t(B) * 16, ctx);
}

static int decode_loop(fxf_engine* e, int64_t* tokens_io, int initial_len, int64_t pad_idx, void* stream, bool last_row) {
    FXF_CHECK(e && tokens_io, "fxf_decode_static: NULL argument");
    FXF_CHECK(e->input_ids.size() == 2 && e->output_ids.size() >= 1, "fxf_decode_static: the graph must take (tokens, mask) and return logits");
    if (ensure_device(e)) return 1;
    FxfTensor& tok = e->reg[e->input_ids[0]];
    FxfTensor& mask = e->reg[e->input_ids[1]];
    const FxfTensor& logits = e->reg[e->output_ids[0]];
    FXF_CHECK(tok.dtype == FXF_I64 && tok.rank == 2, "fxf_decode_static: input 0 must be int64 [B,T]");
    int B = int(tok.shape[0]), T = int(tok.shape[1]);
    FXF_CHECK(mask.dtype == FXF_BOOL && mask.rank == 4 && mask.shape[0] == B && mask.shape[1] == 1 && mask.shape[2] == T && mask.shape[3] == T,
              "fxf_decode_static: input 1 must be bool [B,1,T,T]");
    FXF_CHECK(logits.dtype == FXF_F32 && logits.rank == 3 && logits.shape[0] == B && logits.shape[1] == T, "fxf_decode_static: output 0 must be float32 [B,T,V]");
    FXF_CHECK(initial_len >= 1 && initial_len <= T, "fxf_decode_static: initial_len %d must be in [1, %d]", initial_len, T);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int64_t* slot = static_cast<int64_t*>(tok.ptr);
    if (tokens_io != slot) FXF_CUDA(cudaMemcpyAsync(slot, tokens_io, size_t(tok.nbytes), cudaMemcpyDeviceToDevice, s));
    ExecCtx ctx;
    ctx.stream = s;
    ctx.sm_count = e->ctx.sm_count;
    ctx.tp_rank = e->ctx.tp_rank;
    ctx.tp_size = e->ctx.tp_size;
    ctx.comm = e->ctx.comm;
    for (int cur = initial_len; cur < T; cur++) {
        if (decode_build_mask(slot, static_cast<uint8_t*>(mask.ptr), B, T, cur, pad_idx, ctx)) return 1;
        if (last_row) {
            if (e->body_exec) {
                FXF_CUDA(cudaGraphLaunch(e->body_exec, s));
            } else if (run_nodes(e, s, e->tail_node)) return 1;
            if (last_row_head(e, slot, cur, ctx)) return 1;
        } else {
            if (launch_forward(e, s)) return 1;
            if (fxf_engine_argmax_scatter(e, slot, cur, stream)) return 1;
        }
    }
    if (tokens_io != slot) FXF_CUDA(cudaMemcpyAsync(tokens_io, slot, size_t(tok.nbytes), cudaMemcpyDeviceToDevice, s));
    return 0;
}

}  // extern "C"
