// OpCode -> kernel table.  Counterpart of OpRegistry / KernelSet
// (reference csrc/runtime/op_registry.cpp:16-106, csrc/include/runtime/op_registry.hpp:11-31):
// a flat vector indexed by OpCode, filled once.  Only a CUDA kernel set exists here; asking
// for an opcode without a kernel is an error, never a fallback to another backend.
#include "runtime.hpp"

namespace fxf {

#define FXF_DECL_KERNEL(name) int name(Registry&, const TensorIds&, const TensorIds&, const Params&, const NodePlan*, ExecCtx&)
#define FXF_DECL_PLAN(name) std::unique_ptr<NodePlan> name(const Registry&, const TensorIds&, const TensorIds&, const Params&, const PlanEnv&)

FXF_DECL_KERNEL(k_conv2d);
FXF_DECL_KERNEL(k_conv2d_relu);
FXF_DECL_KERNEL(k_linear);
FXF_DECL_KERNEL(k_linear_relu);
FXF_DECL_KERNEL(k_add);
FXF_DECL_KERNEL(k_add_relu);
FXF_DECL_KERNEL(k_relu);
FXF_DECL_KERNEL(k_mul);
FXF_DECL_KERNEL(k_max_pool2d);
FXF_DECL_KERNEL(k_avg_pool2d);
FXF_DECL_KERNEL(k_adaptive_avg_pool2d);
FXF_DECL_KERNEL(k_transpose);
FXF_DECL_KERNEL(k_size);
FXF_DECL_KERNEL(k_narrow);
FXF_DECL_KERNEL(k_embedding);
FXF_DECL_KERNEL(k_layer_norm);
FXF_DECL_KERNEL(k_add_layer_norm);
FXF_DECL_KERNEL(k_mha);
FXF_DECL_KERNEL(k_feedforward);
FXF_DECL_KERNEL(k_cross_mha);
FXF_DECL_KERNEL(k_cached_mha);

FXF_DECL_PLAN(plan_bandwidth);
FXF_DECL_PLAN(plan_gather);
FXF_DECL_PLAN(plan_layernorm);
FXF_DECL_PLAN(plan_linear);
FXF_DECL_PLAN(plan_feedforward);
FXF_DECL_PLAN(plan_mha);
FXF_DECL_PLAN(plan_conv);
FXF_DECL_PLAN(plan_cross_mha);
FXF_DECL_PLAN(plan_cached_mha);

const OpEntry& op_entry(int op_code) {
    static const OpEntry table[FXF_OP_COUNT] = {
        {"NoOp", nullptr, nullptr},
        {"Conv2d", k_conv2d, plan_conv},
        {"Conv2dRelu", k_conv2d_relu, plan_conv},
        {"Linear", k_linear, plan_linear},
        {"LinearRelu", k_linear_relu, plan_linear},
        {"Add", k_add, plan_bandwidth},
        {"AddRelu", k_add_relu, plan_bandwidth},
        {"Relu", k_relu, plan_bandwidth},
        {"Mul", k_mul, plan_bandwidth},
        {"MaxPool2d", k_max_pool2d, plan_bandwidth},
        {"AvgPool2d", k_avg_pool2d, plan_bandwidth},
        {"AdaptiveAvgPool2d", k_adaptive_avg_pool2d, plan_bandwidth},
        {"Transpose", k_transpose, plan_bandwidth},
        {"Size", k_size, plan_gather},
        {"Narrow", k_narrow, plan_gather},
        {"Embedding", k_embedding, plan_gather},
        {"LayerNorm", k_layer_norm, plan_layernorm},
        {"AddLayerNorm", k_add_layer_norm, plan_layernorm},
        {"MHA", k_mha, plan_mha},
        {"FeedForward", k_feedforward, plan_feedforward},
        {"CrossMHA", k_cross_mha, plan_cross_mha},   // extension, not in the reference schema
        {"CachedMHA", k_cached_mha, plan_cached_mha},   // extension: one new position against cached keys / values
    };
    static const OpEntry none{"?", nullptr, nullptr};
    if (op_code < 0 || op_code >= FXF_OP_COUNT) return none;
    return table[op_code];
}

}  // namespace fxf
