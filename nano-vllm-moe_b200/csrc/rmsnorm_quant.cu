// RMSNorm fused with the static e4m3 activation quantiser: the producer of a W8A8 linear's input.
//
//   v   = x [+ residual]                          (fp32)
//   res = bf16(v)                                 (written back over `residual`, when one is given)
//   n   = v * (1 / sqrt(mean(v^2) + eps))         (fp32; IEEE division and square root)
//   y   = bf16(n * weight)                        (one rounding)
//   xq  = e4m3(clamp(y / max(scale, 1e-12), +-448))
//
// This is RMSNorm.rms_forward / add_rms_forward of the reference as it runs them (both are compiled, and the
// compiler keeps the whole expression in fp32: one rounding, on the product with the weight), followed by the
// activation quantiser of the W8A8 linear that consumes the result.  A row is handled by one CTA; the row's
// fp32 values stay in registers between the sum of squares and the scaling (hidden sizes up to 8192), so x is
// read once and only the e4m3 row (and/or the bf16 row, if asked for) is written: 2 (+2+2 with a residual)
// bytes read and 1 (+2) written per element instead of the 2+2 of the norm plus the 2+1 of a separate
// quantiser pass.  HBM-bound; decode-sized calls are launch-bound.
#include "common.cuh"
#include "kernels.h"

namespace fp8lin {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;          // 8-element vectors per thread: H <= 256 * 8 * 4 = 8192

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, __nv_bfloat16* __restrict__ residual, int64_t ld_res,
                     const __nv_bfloat16* __restrict__ weight, float eps, const float* __restrict__ input_scale,
                     unsigned char* __restrict__ xq, __nv_bfloat16* __restrict__ y, int64_t ldy, int H) {
    __shared__ float s_part[kNormThreads / 32];
    __shared__ float s_inv;
    pdl_launch_dependents();
    pdl_wait();                                    // x and the residual come from the kernels before
    const int64_t row = blockIdx.x;
    const int nvec = H >> 3;
    const __nv_bfloat16* xr = x + row * ldx;
    __nv_bfloat16* rr = residual ? residual + row * ld_res : nullptr;
    float v[kNormMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kNormMaxVec; ++j) {
        const int vec = threadIdx.x + j * kNormThreads;
        if (vec < nvec) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(xr + vec * 8));
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) { v[j][2 * e] = bf16_lo(aw[e]); v[j][2 * e + 1] = bf16_hi(aw[e]); }
            if (rr) {
                const uint4 b = *reinterpret_cast<const uint4*>(rr + vec * 8);
                const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
                uint4 o;
                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[j][2 * e] = __fadd_rn(v[j][2 * e], bf16_lo(bw[e]));
                    v[j][2 * e + 1] = __fadd_rn(v[j][2 * e + 1], bf16_hi(bw[e]));
                    ow[e] = pack_bf16x2(v[j][2 * e], v[j][2 * e + 1]);
                }
                *reinterpret_cast<uint4*>(rr + vec * 8) = o;          // the residual stream for the next layer
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(v[j][e], v[j][e], ss);
        }
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < kNormThreads / 32; ++i) t += s_part[i];
        const float var = __fdiv_rn(t, (float)H);
        s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    }
    __syncthreads();
    const float inv = s_inv;
    const bool quant = xq != nullptr;
    const ExactDiv div(quant ? fmaxf(__ldg(input_scale), 1e-12f) : 1.f);
#pragma unroll
    for (int j = 0; j < kNormMaxVec; ++j) {
        const int vec = threadIdx.x + j * kNormThreads;
        if (vec < nvec) {
            const uint4 w = __ldg(reinterpret_cast<const uint4*>(weight + vec * 8));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                ow[e] = pack_bf16x2(__fmul_rn(__fmul_rn(v[j][2 * e], inv), bf16_lo(ww[e])),
                                    __fmul_rn(__fmul_rn(v[j][2 * e + 1], inv), bf16_hi(ww[e])));
            if (y) *reinterpret_cast<uint4*>(y + row * ldy + vec * 8) = o;
            if (quant) *reinterpret_cast<uint2*>(xq + row * H + vec * 8) = quant8_e4m3(o, div);
        }
    }
}

cudaError_t launch_rmsnorm_quant(const __nv_bfloat16* x, int64_t ldx, __nv_bfloat16* residual, int64_t ld_res,
                                 const __nv_bfloat16* weight, float eps, const float* input_scale, unsigned char* xq,
                                 __nv_bfloat16* y, int64_t ldy, int64_t M, int64_t H, cudaStream_t stream) {
    if (M == 0) return cudaSuccess;
    if (H > kNormThreads * 8 * kNormMaxVec) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)M);
    cfg.blockDim = dim3(kNormThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = pdl_attribute(attr);
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, rmsnorm_quant_kernel, x, ldx, residual, ld_res, weight, eps, input_scale, xq, y, ldy, (int)H));
}

}  // namespace fp8lin
