// fp8lin_linear_static_scratch: the decode-sized linear for callers that cannot
// hand the library a scratch buffer of their own.
//
// Who needs this: a serving process that has already given every spare byte of
// HBM to its KV-cache pool, so a later cudaMalloc for split-K scratch would
// fail; and code on a latency-critical path (a decode loop, a callback) where
// an allocation may stall behind a device-wide synchronisation.  For them the
// scratch lives inside the library image: one fixed array per GPU.  CUDA loads
// the module that holds it lazily, so a GPU sets its copy aside at the FIRST
// call of this entry point on that GPU (the cudaGetSymbolAddress below) and
// keeps it until the process exits.  Make that first call early -- one tiny
// warm-up call per GPU is enough -- before the process hands the remaining HBM
// to its pool, and outside any stream capture; if the memory is already gone
// the call reports FP8LIN_ERR_WORKSPACE.
//
// The array is shared by every call on that GPU and keeps whatever the last
// call left in it.  The only part that has to start at zero -- the split-K
// arrival counters -- is cleared on the caller's stream before each launch.
// Two calls that can run at the same time on one GPU (different streams,
// different threads) would both write the array and corrupt each other:
// serialise them.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace fp8lin {

// Built-in scratch: the counter header plus room for the split-K partial sums
// of one decode-sized call (M <= 64).  16 MiB covers every 7B-class layer shape
// at M <= 64 (the largest, down_proj 18944 -> 3584 at M = 64, needs 9.7 MiB).
constexpr size_t kStaticBodyBytes = 16u << 20;
constexpr size_t kStaticBytes = FP8LIN_WS_HEADER_BYTES + kStaticBodyBytes;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
static unsigned char* g_scratch_ptr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

// Device address of this GPU's copy of the array.  `g_static_scratch` itself is
// only a host-side handle; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
static cudaError_t static_scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_ptr[dev];
    return cudaSuccess;
}

}  // namespace fp8lin

using namespace fp8lin;

extern "C" int fp8lin_linear_static_scratch(int scheme, const void* x, int64_t ldx, const void* w_nk,
                                            const float* w_scale, const float* input_scale, const void* bias,
                                            void* y, int64_t ldy, int64_t M, int64_t K, int64_t N, void* stream) {
    if (scheme != FP8LIN_W8A16 && scheme != FP8LIN_W8A8_STATIC)
        return set_error(FP8LIN_ERR_ARG, "unknown scheme %d", scheme);
    if (M < 0 || K <= 0 || N <= 0 || K % 16 != 0)
        return set_error(FP8LIN_ERR_SHAPE, "bad shape M=%lld K=%lld N=%lld (K must be a positive multiple of 16)",
                         (long long)M, (long long)K, (long long)N);
    if (M == 0) return FP8LIN_OK;
    if (M > 64)
        return set_error(FP8LIN_ERR_WORKSPACE,
                         "M=%lld is beyond the built-in scratch limit of 64 rows; use fp8lin_w8a8/fp8lin_w8a16 "
                         "with a caller-owned workspace", (long long)M);
    if (!x || !w_nk || !w_scale || !y || (scheme == FP8LIN_W8A8_STATIC && !input_scale))
        return set_error(FP8LIN_ERR_NULL, "x, w_nk, w_scale, y (and input_scale for W8A8) must not be NULL");
    if (ldx < K || ldy < N)
        return set_error(FP8LIN_ERR_SHAPE, "ldx=%lld < K or ldy=%lld < N", (long long)ldx, (long long)ldy);
    if (ldx % 8 != 0) return set_error(FP8LIN_ERR_ALIGN, "ldx=%lld must be a multiple of 8 elements", (long long)ldx);
    auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!a16(x) || !a16(w_nk) || !a16(w_scale) || (bias && !a16(bias)))
        return set_error(FP8LIN_ERR_ALIGN, "x, w_nk, w_scale and bias must be 16-byte aligned");
    if (!device_is_sm100()) return set_error(FP8LIN_ERR_ARCH, "fp8lin kernels are built for sm_100a only");

    const StreamPlan pl = plan_stream(scheme, M, K, N, -1);
    if (pl.partial_bytes > kStaticBodyBytes)
        return set_error(FP8LIN_ERR_WORKSPACE,
                         "this shape needs %zu bytes of split-K scratch, more than the built-in %zu bytes; use "
                         "fp8lin_w8a8/fp8lin_w8a16 with a caller-owned workspace", pl.partial_bytes, kStaticBodyBytes);

    unsigned char* scratch = nullptr;
    cudaError_t e = static_scratch_for_current_device(&scratch);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return set_error(FP8LIN_ERR_WORKSPACE,
                         "no device memory left for the built-in %zu-byte scratch array: make the first call on each "
                         "GPU before the process gives the remaining HBM away", kStaticBytes);
    }
    if (e != cudaSuccess) return set_error(FP8LIN_ERR_LAUNCH, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    cudaStream_t st = (cudaStream_t)stream;
    WsView ws = ws_view(scratch, kStaticBytes);
    if (pl.splits > 1) {
        // the counters this launch will use must read zero, whatever an earlier call left behind
        e = cudaMemsetAsync(ws.counters, 0, sizeof(int) * (size_t)pl.n_tiles * pl.m_passes, st);
        if (e != cudaSuccess) return set_error(FP8LIN_ERR_LAUNCH, "clearing counters: %s", cudaGetErrorString(e));
    }
    StreamArgs a;
    a.x = (const __nv_bfloat16*)x; a.w = (const unsigned char*)w_nk; a.w_scale = w_scale;
    a.input_scale = scheme == FP8LIN_W8A8_STATIC ? input_scale : nullptr;
    a.bias = (const __nv_bfloat16*)bias; a.y = (__nv_bfloat16*)y;
    a.partial = (float*)ws.body; a.counters = ws.counters;
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.ldx = (int)ldx; a.ldy = (int)ldy; a.k_per_split = pl.k_per_split;
    e = launch_stream(scheme, pl, a, st);
    if (e != cudaSuccess) return set_error(FP8LIN_ERR_LAUNCH, "stream kernel launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}
