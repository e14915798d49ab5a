// fxf_feedforward_static — FeedForward for callers that must not allocate device memory.
//
// Some hosts cannot call cudaMalloc when they want to run an op: a serving process that handed the
// whole device to its own pool at start-up, a latency-critical loop that cannot afford the implicit
// device-wide synchronisation an allocation may cause, or a plugin that is simply not allowed to own
// memory.  The engine path sizes and allocates its scratch when an engine is created, and
// fxf_kernel_invoke asks the caller for scratch; this entry point needs neither.  The [M, F] hidden
// activation lives in a fixed array that is part of the library image, so loading the library on a
// GPU reserves it (kStaticScratchBytes, until the process exits) and a call allocates nothing — no
// cudaMalloc, no cudaFree, no library routine that allocates.
//
// Consequences the caller has to live with:
//   * M * F * 4 bytes must fit kStaticScratchBytes; larger problems are refused with an error.
//   * Every call on a GPU uses the same array.  Calls that may overlap on that GPU (different
//     streams, different threads) race on it; serialise them.  The array keeps whatever the last call
//     left behind; this op overwrites all M x F values it later reads, so nothing has to be cleared.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
//     caches it.  Make that first call outside any stream capture.
//
// Arithmetic: the fp32 FFMA GEMM (the kernel FXF_GEMM_FP32_SIMT selects), bias and ReLU fused, i.e.
//   out[M,P] = relu(x[M,D] · w1[F,D]^T + b1) · w2[P,F]^T + b2      (reference feedforward.cpp:5-14).
#include <mutex>

#include "../runtime.hpp"

namespace fxf {
namespace {

constexpr size_t kStaticScratchBytes = size_t(8) << 20;  // 8 MiB: e.g. 512 rows x 4096 hidden floats
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_ff_scratch[kStaticScratchBytes];

// Host code must not pass `g_ff_scratch` to a kernel: on the host that name is only a handle for the
// runtime.  The real device address is obtained once per device, with that device current.
std::mutex g_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

int scratch_for_current_device(float** out) {
    int dev = -1;
    FXF_CUDA(cudaGetDevice(&dev));
    FXF_CHECK(dev >= 0 && dev < kMaxDevices, "fxf_feedforward_static: device ordinal %d is not supported", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_ff_scratch);
        if (e != cudaSuccess || p == nullptr)
            FXF_FAIL("fxf_feedforward_static: cannot resolve the static scratch array on device %d: %s", dev, cudaGetErrorString(e));
        g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

}  // namespace
}  // namespace fxf

using namespace fxf;

extern "C" FXF_API int64_t fxf_feedforward_static_max_bytes(void) { return int64_t(kStaticScratchBytes); }

extern "C" FXF_API int fxf_feedforward_static(const float* x, const float* w1, const float* b1, const float* w2, const float* b2, float* out,
                                      int64_t M, int64_t D, int64_t F, int64_t P, void* stream) {
    FXF_CHECK(M >= 0 && D >= 0 && F >= 0 && P >= 0, "fxf_feedforward_static: negative dimension");
    // an operand without elements (a zero extent) may be passed as NULL
    FXF_CHECK((x || M * D == 0) && (w1 || F * D == 0) && (b1 || F == 0) && (w2 || P * F == 0) && (b2 || P == 0) && (out || M * P == 0),
              "fxf_feedforward_static: NULL argument");
    // F <= max / (4 M) written without overflow
    FXF_CHECK(M == 0 || F == 0 || uint64_t(F) <= kStaticScratchBytes / sizeof(float) / uint64_t(M),
              "fxf_feedforward_static: the hidden activation needs M*F*4 = %lld x %lld x 4 bytes, more than the %zu-byte static scratch; "
              "use an engine or fxf_kernel_invoke for this size",
              (long long)M, (long long)F, kStaticScratchBytes);
    if (M == 0 || P == 0) return 0;
    float* hidden = nullptr;
    if (scratch_for_current_device(&hidden)) return 1;
    ExecCtx ctx;
    ctx.stream = static_cast<cudaStream_t>(stream);
    ctx.gemm_mode = FXF_GEMM_FP32_SIMT;
    int dev = 0, sms = 0;
    FXF_CUDA(cudaGetDevice(&dev));
    FXF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    ctx.sm_count = sms;
    GemmArgs g1;
    g1.x = x; g1.w = w1; g1.bias = b1; g1.out = hidden;
    g1.M = M; g1.N = F; g1.K = D; g1.ldx = D; g1.ldw = D; g1.ldo = F; g1.relu = true;
    if (F > 0 && launch_gemm_simt(g1, ctx)) return 1;
    GemmArgs g2;
    g2.x = hidden; g2.w = w2; g2.bias = b2; g2.out = out;
    g2.M = M; g2.N = P; g2.K = F; g2.ldx = F; g2.ldw = F; g2.ldo = P; g2.relu = false;
    return launch_gemm_simt(g2, ctx);
}
