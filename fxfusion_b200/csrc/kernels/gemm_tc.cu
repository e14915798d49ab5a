// Tensor-core GEMM entry points (tcgen05 kind::tf32, 3xTF32 operand split).
#include "../runtime.hpp"

namespace fxf {

bool gemm_tc_supported(const GemmArgs&) { return false; }

int launch_gemm_tc(const GemmArgs&, ExecCtx&) { FXF_FAIL("tensor-core GEMM is not available in this build"); }

}  // namespace fxf
