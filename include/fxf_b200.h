/*
 * fxf_b200.h — C ABI of the B200 (sm_100a) CUDA backend for the FXFusion runtime.
 *
 * Everything here is plain C: pointers, sizes and status codes.  No LibTorch type crosses
 * this boundary.  Each entry point names the reference interface it stands in for
 * (paths relative to the reference project).
 *
 * Status convention: 0 = success, non-zero = failure; fxf_last_error() returns the
 * thread-local message of the most recent failure (the reference throws c10::Error /
 * std::runtime_error at the same points, e.g. csrc/runtime/memory_manager.cpp:14,87-90,103,114).
 */
#ifndef FXF_B200_H_
#define FXF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FXF_API __attribute__((visibility("default")))
#else
#define FXF_API
#endif

#define FXF_MAX_DIMS 8

/* DType values of the graph file (schema/graph.fbs:11-17). */
enum { FXF_F32 = 0, FXF_F16 = 1, FXF_I32 = 2, FXF_I64 = 3, FXF_BOOL = 4 };

/* OpCode values of the graph file (schema/graph.fbs:19-40).  Values above 19 do not exist in the reference schema:
 * FXF_OP_CROSS_MHA is attention with queries from one sequence and keys/values from another (the decoder's second
 * attention of an encoder-decoder model), which the reference's QKV packing cannot lower.
 * inputs [x, memory, mask, Wq[D,D], bq[D], Wkv[2D,D], bkv[2D], Wo[D,D], bo[D]], ints [H, head_dim, D, 2D], floats [scale_divisor].
 * FXF_OP_CACHED_MHA is self-attention of one new position per sequence against the keys/values of the positions fed before
 * (kept in the node's persistent memory): the step of an incremental greedy decode, see fxf_decode_cached.
 * inputs [x [B,1,D], tokens int64 [B,T], pos int64 [1], Wqkv[3D,D], bqkv[3D], Wo[D,D], bo[D]], ints [H, head_dim, D, 3D, pad_idx],
 * floats [scale_divisor]. */
enum {
    FXF_OP_NOOP = 0, FXF_OP_CONV2D = 1, FXF_OP_CONV2D_RELU = 2, FXF_OP_LINEAR = 3,
    FXF_OP_LINEAR_RELU = 4, FXF_OP_ADD = 5, FXF_OP_ADD_RELU = 6, FXF_OP_RELU = 7,
    FXF_OP_MUL = 8, FXF_OP_MAX_POOL2D = 9, FXF_OP_AVG_POOL2D = 10,
    FXF_OP_ADAPTIVE_AVG_POOL2D = 11, FXF_OP_TRANSPOSE = 12, FXF_OP_SIZE = 13,
    FXF_OP_NARROW = 14, FXF_OP_EMBEDDING = 15, FXF_OP_LAYER_NORM = 16,
    FXF_OP_ADD_LAYER_NORM = 17, FXF_OP_MHA = 18, FXF_OP_FEEDFORWARD = 19, FXF_OP_CROSS_MHA = 20, FXF_OP_CACHED_MHA = 21, FXF_OP_COUNT = 22
};

/* One registry slot.  Replaces the torch::Tensor elements of the reference TensorRegistry
 * (csrc/include/runtime/tensor_registry.hpp:8).  Strides are in elements. */
typedef struct FxfTensor {
    void*   ptr;
    int32_t dtype;
    int32_t rank;
    int64_t shape[FXF_MAX_DIMS];
    int64_t stride[FXF_MAX_DIMS];
    int64_t nbytes;
} FxfTensor;

/* GEMM arithmetic used by Linear / LinearRelu / FeedForward / MHA projections. */
enum {
    FXF_GEMM_AUTO = 0,      /* fp32-grade on the tensor cores where the shape allows it (FXF_GEMM_TF32_BF16X2 for dense layers
                               whose K is a multiple of 8, FXF_GEMM_TF32X3 otherwise and for convolutions), else fp32 SIMT */
    FXF_GEMM_FP32_SIMT = 1, /* fp32 FFMA tiles only */
    FXF_GEMM_TF32X3 = 2,    /* tcgen05 kind::tf32 with hi/lo operand split (fp32-grade result) */
    FXF_GEMM_BF16 = 3,      /* optional reduced-precision mode: weights and activations rounded to bf16 for the tensor-core
                               products (one product per logical product), fp32 accumulation and fp32 tensors everywhere
                               else; results within about 1e-2 relative of the fp32 path, decode tokens may differ */
    FXF_GEMM_TF32_BF16X2 = 4 /* fp32-grade like FXF_GEMM_TF32X3 (x = x_hi + x_lo, w = w_hi + w_lo): the main product
                               x_hi*w_hi in TF32, both correction products bf16(x_lo)*bf16(w_hi) and bf16(x)*bf16(w_lo) as
                               bf16 tensor-core products with fp32 accumulation.  The corrections are 2^-11 of a product, so
                               their bf16 rounding costs about 2^-20 of it.  Four tensor-core instructions per 16 K-elements
                               instead of six (an instruction takes the same time whatever its kind) */
};

typedef struct FxfEngineOptions {
    int32_t struct_size;     /* sizeof(FxfEngineOptions), for forward compatibility */
    int32_t use_cuda_graph;  /* 1: capture one CUDA Graph per forward and replay it */
    int32_t gemm_mode;       /* FXF_GEMM_* */
    int32_t tp_rank;         /* tensor-parallel rank of this engine (0 when tp_size == 1) */
    int32_t tp_size;         /* number of tensor-parallel ranks (1 = none); both are taken from the communicator */
    int32_t tp_shard_output; /* 1: also shard the rows (vocabulary) of the final Linear over the ranks; each rank then
                                writes only its column block of the output and fxf_engine_argmax_scatter combines them */
    int32_t no_epilogue_fusion;    /* 1: never fold a residual Add into the epilogue of the contraction before it */
    int32_t no_tp_fused_exchange;  /* 1: tensor parallelism keeps all-reduce + Add + LayerNorm as separate launches */
    int32_t p2p_start_budget_ms;   /* wait budget of an exchange's first peer barrier (0 = 20000: it absorbs host-side skew) */
    int32_t p2p_end_budget_ms;     /* wait budget of its second peer barrier (0 = 2000) */
    int32_t p2p_grid;              /* blocks of the peer exchange kernels, 1..128 (0 = 128); must agree on all ranks */
    int32_t tc_chunk_k;            /* K-elements per tensor-core accumulation chain before the partial sums are added in fp32
                                      by CUDA cores (0 = 1024 for dense layers, 64 for convolutions); larger = fewer
                                      drains, more truncation bias per chain (about 4e-8 of the result's scale per element) */
    int32_t tc_pair;               /* 0: the widest tensor-core GEMM tiles (256 columns) are computed by pairs of CTAs
                                      (tcgen05 cta_group::2: 256-row tiles, each CTA stages half of the weight tile);
                                      1: never */
    int32_t tp_push;               /* 0: under tensor parallelism the row-parallel products keep their partial sums local and
                                      the exchange kernel fetches them from the peers; 1: the products store each row
                                      into its owner's exchange window (peer stores from the GEMM epilogue), the exchange
                                      kernel then reads local memory only */
    int32_t reserved[2];
} FxfEngineOptions;

typedef struct fxf_engine fxf_engine;

/* Message of the last failure on the calling thread ("" if none). */
FXF_API const char* fxf_last_error(void);

/* Library build id: "fxf_b200 <n kernels> sm_100a". */
FXF_API const char* fxf_version(void);

/* ExecutionEngine(graph_path, device) — csrc/runtime/execution_engine.cpp:12-29.
 * Reads the graph file, places every tensor in ONE cudaMalloc'd device arena (activations at
 * the planner's offsets, then constants, input slots and shared scratch), binds aliases the
 * way csrc/runtime/memory_manager.cpp:30-111 does and resolves one kernel per node
 * (csrc/runtime/runtime_graph.cpp:8-18).  `opts` may be NULL. */
FXF_API int fxf_engine_create(const char* graph_path, int device_ordinal, const FxfEngineOptions* opts,
                      fxf_engine** out_engine);
/* Tensor-parallel engine (no counterpart in the reference, which is single-device).  Every rank loads the
 * same graph file; MHA nodes keep H/n heads, FeedForward nodes F/n hidden units, their partial outputs are
 * summed with one all-reduce each (on the run's stream, captured into the CUDA Graph); all other nodes
 * are replicated.  `comm` must outlive the engine.  Creation is collective: all ranks call it together.
 * The exchange is this library's own kernel over peer memory: at creation the ranks exchange CUDA IPC handles of their
 * engine allocations and map each other's memory (GPUs of one node with peer access).  Where a residual Add and a LayerNorm
 * (or an AddLayerNorm) follow the sharded node, one kernel sums the ranks' partial outputs, adds the residual and
 * normalises: each rank does that for M / n rows and stores the normalised rows on every rank.  Where peer mapping is not
 * possible, or with FXF_TP_ALLREDUCE=nccl in the environment, NCCL's all-reduce is used and the other nodes stay separate.
 * Device status 121 / 122 = a peer did not reach an exchange within its budget (p2p_start_budget_ms / p2p_end_budget_ms
 * of the options: 20 s for the first barrier, which absorbs host-side skew, 2 s for the second); 123 = a peer reported
 * that it had given up.  After any of them every later exchange of the engine returns at once (on every rank: the rank
 * that gave up tells its peers), results are undefined and the engine has to be destroyed. */
typedef struct fxf_comm fxf_comm;
FXF_API int fxf_comm_unique_id(void* out_128_bytes);           /* rank 0; ship the 128 bytes to the others */
FXF_API int fxf_comm_create(const void* unique_id_128_bytes, int rank, int size, int device_ordinal, fxf_comm** out);
FXF_API void fxf_comm_destroy(fxf_comm* c);
FXF_API int fxf_comm_rank(const fxf_comm* c);
FXF_API int fxf_comm_size(const fxf_comm* c);
FXF_API int fxf_engine_create_tp(const char* graph_path, int device_ordinal, const FxfEngineOptions* opts, fxf_comm* comm,
                                 fxf_engine** out_engine);
/* The exchange step of the tensor-parallel layout, emulated on ONE GPU (no counterpart in the reference; meant for tests
 * where fewer GPUs than ranks are available): the buffers of all n_ranks ranks live on the current device and one
 * cooperative launch carries the blocks of every rank.  For rank r and its rows [r*R, (r+1)*R), R = ceil(M / n_ranks):
 *   x = sum_q partial[q][row] (q = 0..n-1 in order) + residual[r][row];   x_out[r][row] = x  (every x_out[q] when layout & 1);
 *   y_out[q][row] = LayerNorm(x) * gamma + beta over the D columns, for every q.
 * residual, x_out, y_out may be NULL (then gamma / beta may be NULL too).  sync_mem: n_ranks * 8192 zeroed device bytes;
 * afterwards the int at byte r * 8192 + 4160 is rank r's status word (0, or 121 / 122 / 123 as for fxf_engine_create_tp).
 * budget_ms (1..2000) bounds each peer wait; skip_rank >= 0 keeps that rank away from the exchange, so the other ranks'
 * waits run out and report it — the call still returns and the device stays usable.
 * layout bit 1 (value 2): partial[q] is rank q's exchange window as the row-pushed products leave it (M a multiple of
 * n_ranks): row p*R + l of it holds producer p's partial sums of row q*R + l, so rank q reads only its own buffer. */
FXF_API int fxf_tp_exchange_emulated(int n_ranks, const float* const* partial, const float* const* residual,
                                     float* const* x_out, float* const* y_out, const float* gamma, const float* beta,
                                     float eps, int64_t M, int64_t D, int layout, void* sync_mem,
                                     int64_t sync_bytes, int budget_ms, int skip_rank, void* stream);
/* The row-parallel product of the tensor-parallel layout with a row-pushed output, outside an engine (no counterpart in
 * the reference; one GPU can play every producer in turn): producer `rank` of n_ranks computes x[M,K] @ w[N,K]^T (+ bias
 * [N], may be NULL) on the tensor cores and stores row g of the result, owned by rank q = g / R (R = M / n_ranks, a
 * multiple of 128), into windows[q] at row rank*R + (g - q*R); each window holds M*N floats.  scratch: 256-byte aligned,
 * fxf_linear_pushed_scratch_bytes(N, K) bytes (split weights + the kernel's K-split workspace). */
FXF_API int64_t fxf_linear_pushed_scratch_bytes(int64_t N, int64_t K);
FXF_API int fxf_linear_pushed(const float* x, const float* w, const float* bias, float* const* windows, int n_ranks,
                              int rank, int64_t M, int64_t N, int64_t K, void* scratch, int64_t scratch_bytes,
                              void* stream);
/* tokens[b, current_len] = argmax_v output0[b, current_len-1, v] for this engine, whether the vocabulary is
 * sharded (candidates of all ranks are gathered and every rank writes the same token) or not. */
FXF_API int fxf_engine_argmax_scatter(fxf_engine* e, int64_t* tokens, int current_len, void* stream);
/* Same, from bytes already in memory (the engine copies what it needs). */
FXF_API int fxf_engine_create_from_memory(const void* bytes, size_t nbytes, int device_ordinal,
                                  const FxfEngineOptions* opts, fxf_engine** out_engine);
/* Frees the engine.  A tensor-parallel engine whose ranks mapped each other's memory (see fxf_engine_create_tp) must be
 * destroyed on every rank, before the communicator: the call unmaps the peers and then meets the other ranks once, so
 * that no rank frees memory a peer still has mapped. */
FXF_API void fxf_engine_destroy(fxf_engine* e);

/* Counts and descriptors of graph inputs / outputs (memory_manager.cpp:92-111).  Input
 * descriptors point at the engine's static input slots; output descriptors at arena memory
 * that stays valid (and is overwritten) across runs, like the views execution_engine.cpp:42
 * returns. */
FXF_API int fxf_engine_num_inputs(const fxf_engine* e);
FXF_API int fxf_engine_num_outputs(const fxf_engine* e);
FXF_API int fxf_engine_input_desc(const fxf_engine* e, int i, FxfTensor* out);
FXF_API int fxf_engine_output_desc(const fxf_engine* e, int i, FxfTensor* out);
FXF_API int fxf_engine_num_nodes(const fxf_engine* e);
FXF_API int64_t fxf_engine_arena_bytes(const fxf_engine* e);    /* planner arena_size */
FXF_API int64_t fxf_engine_device_bytes(const fxf_engine* e);   /* whole device allocation */
/* Number of kernel launches one forward issues (graph replay or not). */
FXF_API int fxf_engine_launches_per_run(const fxf_engine* e);

/* ExecutionEngine::run — execution_engine.cpp:31-43, inputs resident on the device.
 * `device_inputs[i]` is a contiguous device buffer of the i-th input's dtype/shape; it is
 * copied into the static slot on `stream` (a cudaStream_t, may be NULL = legacy stream), then
 * the forward is enqueued on the same stream.  Asynchronous: no host sync inside. */
FXF_API int fxf_engine_run(fxf_engine* e, const void* const* device_inputs, int n_inputs, void* stream);
/* Same with HOST buffers: host->device copies of the inputs on `stream`, forward, and (if
 * host_outputs != NULL) device->host copies of every output followed by a stream sync. */
FXF_API int fxf_engine_run_host(fxf_engine* e, const void* const* host_inputs, int n_inputs,
                        void* const* host_outputs, int n_outputs, void* stream);
/* Reads the sticky device status word (0 = no kernel reported a problem); syncs `stream`. */
FXF_API int fxf_engine_device_status(fxf_engine* e, void* stream, int* status_out);
/* Human-readable dump of nodes, offsets, scratch and the kernel variant chosen per node. */
FXF_API int fxf_engine_describe(const fxf_engine* e, char* buf, size_t buf_bytes);
/* Per-node CUDA-event timing of one forward (graph replay disabled for the measurement).
 * ms_out receives fxf_engine_num_nodes() values. */
FXF_API int fxf_engine_time_nodes(fxf_engine* e, float* ms_out, int n, void* stream);
FXF_API int fxf_engine_node_info(const fxf_engine* e, int node, int* op_code, double* flops, double* bytes,
                         char* variant, size_t variant_bytes);

/* One forward with a CUDA event after every kernel launch (graph replay disabled): per launch the
 * kernel family, the graph node that issued it, its device time (gap to the previous launch's
 * end on the same stream) and its algorithmic flops / bytes.  Synchronises `stream`. */
typedef struct FxfLaunchInfo {
    char    kernel[48];
    int32_t node;
    float   ms;
    double  flops;
    double  bytes;
} FxfLaunchInfo;
FXF_API int fxf_engine_profile_launches(fxf_engine* e, void* stream, FxfLaunchInfo* out, int capacity, int* n_out);

/* One kernel, outside any engine: the KernelFn contract of
 * csrc/include/runtime/tensor_registry.hpp:20-26 (registry, input ids, output ids, Params)
 * with the per-node Cache (csrc/runtime/cache.cpp:5-73) replaced by caller-provided scratch.
 * `reg` holds device pointers.  fxf_kernel_scratch_bytes tells how much scratch the op needs. */
FXF_API int64_t fxf_kernel_scratch_bytes(int op_code, const FxfTensor* reg, int n_reg,
                                 const uint32_t* in_ids, int n_in, const uint32_t* out_ids, int n_out,
                                 const int64_t* ints, int n_ints, const float* floats, int n_floats,
                                 int gemm_mode);
FXF_API int fxf_kernel_invoke(int op_code, const FxfTensor* reg, int n_reg,
                      const uint32_t* in_ids, int n_in, const uint32_t* out_ids, int n_out,
                      const int64_t* ints, int n_ints, const float* floats, int n_floats,
                      void* scratch, int64_t scratch_bytes, int gemm_mode, void* stream);

/* Name of the GEMM kernel variant the dispatch rule picks for out[M,N] = x[M,K] . w[N,K]^T in an engine with `sm_count`
 * SMs (0 = 148): "tcgen05-tf32x3-128x<width>-<where A is read from>", "tcgen05-bf16-...", or one of the fp32 FFMA
 * kernels ("simt128x128", "simt64x64", "simt32x32", "skinny32x8").  Pure host code (no counterpart in the reference, whose
 * CUDA linear kernel has one 32x32 tile); tests use it to make sure every variant is exercised. */
FXF_API int fxf_gemm_variant(int64_t M, int64_t N, int64_t K, int gemm_mode, int sm_count, char* out, size_t out_bytes);

/* Greedy static decode on the device — the loop of
 * py/fxfusion/models/transformer/inference.py:28-45 with the mask rule of
 * py/fxfusion/models/transformer/layers/masks.py:141-154.
 *
 * fxf_decode_build_mask: mask[b,0,q,k] = (k < current_len) && (tokens[b,k] != pad) && (k <= q),
 *   tokens int64 [B,T], mask bool [B,1,T,T].
 * fxf_decode_argmax_scatter: tokens[b, current_len] = argmax_v logits[b, current_len-1, v]
 *   (first maximum wins, NaN counts as maximum, like torch.argmax); logits fp32 [B,T,V].
 * fxf_decode_static: whole loop for an engine whose inputs are (tokens int64 [B,T],
 *   mask bool [B,1,T,T]) and whose output 0 is logits [B,T,V]: tokens_io (device, [B,T], prompt
 *   in columns < initial_len, pad elsewhere) is completed in place up to column T-1.  No host
 *   synchronisation is performed. */
FXF_API int fxf_decode_build_mask(const int64_t* tokens, uint8_t* mask, int B, int T, int current_len,
                          int64_t pad_idx, void* stream);
FXF_API int fxf_decode_argmax_scatter(const float* logits, int64_t* tokens, int B, int T, int64_t V,
                              int current_len, void* stream);
FXF_API int fxf_decode_static(fxf_engine* e, int64_t* tokens_io, int initial_len, int64_t pad_idx,
                      void* stream);
/* The same loop and the same tokens, for a graph whose last node is the Linear that produces output 0
 * ([B,T,D] -> [B,T,V], the vocabulary projection): each step runs every node but that one, then evaluates
 * the projection only on row current_len-1 of each sequence — the only row the loop reads
 * (inference.py:38-40, `logits[:, current_len - 1, :]`) — into a [B,V] buffer inside the engine, in fp32
 * FFMA arithmetic.  Output 0 of the engine is NOT updated by this call; no counterpart in the reference,
 * whose loop always runs the whole graph.  fxf_engine_supports_last_row tells whether the graph qualifies. */
FXF_API int fxf_engine_supports_last_row(const fxf_engine* e);
/* Incremental ("KV cache") greedy decode, which the reference names as future work (README.md:183).  `e` runs a
 * single-position step graph — inputs ids int64 [B,1], pos int64 [1], tokens int64 [B,T]; output logits [B,1,V]; attention
 * nodes of kind FXF_OP_CACHED_MHA (fxfusion_b200.lowering.gpt_step_graph builds it from the same weights).  Positions
 * 0 .. T-2 are fed in order; prompt positions only fill the caches, from initial_len-1 on the argmax of a step becomes the
 * next token.  tokens_io as for fxf_decode_static.  The arithmetic per position is that of the full-recompute loop, so the
 * tokens agree with fxf_decode_static except where two logits are tied to within rounding. */
FXF_API int fxf_decode_cached(fxf_engine* e, int64_t* tokens_io, int initial_len, void* stream);
FXF_API int fxf_decode_static_last_row(fxf_engine* e, int64_t* tokens_io, int initial_len, int64_t pad_idx,
                               void* stream);

/* FeedForward without any allocation (no counterpart in the reference: its CUDA feedforward takes
 * its hidden buffer from a per-node torch::empty).  For callers that cannot call cudaMalloc — the device
 * is owned by their own pool, or an allocation's implicit synchronisation is not acceptable.  The
 * [M,F] hidden activation is kept in a fixed array inside the library (fxf_feedforward_static_max_bytes()
 * bytes, 8 MiB, held on every GPU that loads the library until the process exits); M*F*4 beyond that is
 * refused with an error.  out[M,P] = relu(x[M,D]·w1[F,D]^T + b1)·w2[P,F]^T + b2, fp32 FFMA kernels; all
 * pointers are device pointers, row-major, dense.  All calls on a GPU share the array: calls that can
 * overlap on the GPU race and must be serialised by the caller.  The first call on a device resolves the
 * array's address; make it before any stream capture. */
FXF_API int64_t fxf_feedforward_static_max_bytes(void);
FXF_API int fxf_feedforward_static(const float* x, const float* w1, const float* b1, const float* w2,
                                   const float* b2, float* out, int64_t M, int64_t D, int64_t F, int64_t P,
                                   void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FXF_B200_H_ */
