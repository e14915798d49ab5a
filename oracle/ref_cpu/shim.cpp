// TEST INFRASTRUCTURE — exposes the reference's unmodified CPU kernels to Python.
//
// Compiled together with the reference's own csrc/kernels/cpu/*.cpp and csrc/runtime/cache.cpp
// (taken from where the reference checkout lies; no reference source is copied into this
// repository).  `call(op_code, registry, in_ids, out_ids, ints, floats)` invokes the KernelFn the
// reference registers for that opcode (csrc/runtime/op_registry.cpp:57-75) with the same
// argument contract (csrc/include/runtime/tensor_registry.hpp:20-26); the kernels write into
// registry[out_ids[0]] in place.  The CPU kernels ignore their Cache argument, so none is built.
#include <torch/extension.h>

#include "kernels.hpp"

using namespace fxfusion;

static void call(int64_t op_code, std::vector<torch::Tensor> reg, std::vector<int64_t> in_ids, std::vector<int64_t> out_ids,
                 std::vector<int64_t> ints, std::vector<double> floats) {
    static const KernelFn table[] = {
        nullptr,
        kernels::cpu::conv2d, kernels::cpu::conv2d_relu, kernels::cpu::linear, kernels::cpu::linear_relu,
        kernels::cpu::add, kernels::cpu::add_relu, kernels::cpu::relu, kernels::cpu::mul,
        kernels::cpu::max_pool2d, kernels::cpu::avg_pool2d, kernels::cpu::adaptive_avg_pool2d,
        kernels::cpu::transpose, kernels::cpu::size, kernels::cpu::narrow, kernels::cpu::embedding,
        kernels::cpu::layer_norm, kernels::cpu::add_layer_norm, kernels::cpu::mha, kernels::cpu::feedforward,
    };
    TORCH_CHECK(op_code > 0 && op_code < int64_t(sizeof(table) / sizeof(table[0])), "Unsupported OpCode: ", op_code);
    TensorIds ii(in_ids.begin(), in_ids.end()), oo(out_ids.begin(), out_ids.end());
    Params p;
    p.ints = ints;
    p.floats.assign(floats.begin(), floats.end());
    table[op_code](reg, ii, oo, p, nullptr);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) { m.def("call", &call); }
