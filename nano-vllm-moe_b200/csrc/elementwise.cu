// HBM-bound helpers: static activation quantiser and the one-off weight transpose.
#include "common.cuh"
#include "kernels.h"

namespace fp8lin {

// xq[m][k] = e4m3(clamp(x[m][k] / max(s, 1e-12), +-448)).  3 bytes of traffic per
// element (2 read + 1 written); each thread converts 16 elements per iteration
// (two 16-byte loads, one 16-byte store), grid-stride over [M][K/16].
__global__ void __launch_bounds__(256)
act_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const float* __restrict__ input_scale,
                 unsigned char* __restrict__ xq, int64_t M, int64_t K) {
    pdl_launch_dependents();       // the GEMM behind this pass may set up and prefetch its weights now
    pdl_wait();                    // x may come from the kernel before
    const ExactDiv s(fmaxf(__ldg(input_scale), 1e-12f));
    const int64_t vec_per_row = K / 16;
    const int64_t total = M * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec_per_row;
        const int64_t c = (i - r * vec_per_row) * 16;
        const uint4* src = reinterpret_cast<const uint4*>(x + r * ldx + c);
        const uint4 a = __ldg(src);
        const uint4 b = __ldg(src + 1);
        const uint2 qa = quant8_e4m3(a, s);
        const uint2 qb = quant8_e4m3(b, s);
        *reinterpret_cast<uint4*>(xq + r * K + c) = make_uint4(qa.x, qa.y, qb.x, qb.y);
    }
}

cudaError_t launch_act_quant(const __nv_bfloat16* x, int64_t ldx, const float* input_scale,
                             unsigned char* xq, int64_t M, int64_t K, cudaStream_t stream) {
    const int64_t total = M * (K / 16);
    if (total == 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = sm_count() * 16;
    if (blocks > cap) blocks = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = pdl_attribute(attr);
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, act_quant_kernel, x, ldx, input_scale, xq, M, K));
}

// y[m][n] = bf16( sum over slots r of slots[r][m][n] ), added in slot order in fp32: the reduction step
// of a row-parallel linear whose ranks have scattered their bf16 partial outputs into every rank's slots.
__global__ void __launch_bounds__(256)
sum_slots_kernel(const __nv_bfloat16* __restrict__ slots, int n_slots, int64_t slot_stride, __nv_bfloat16* __restrict__ y,
                 int64_t ldy, int64_t M, int64_t N, int64_t ld_slot) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t vec_per_row = N / 8;
    const int64_t total = M * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / vec_per_row;
        const int64_t c = (i - m * vec_per_row) * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < n_slots; ++r) {
            // peers wrote these lines: read them past L1
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(slots + r * slot_stride + m * ld_slot + c));
            acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
            acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(y + m * ldy + c) = o;
    }
}

cudaError_t launch_sum_slots(const __nv_bfloat16* slots, int n_slots, int64_t slot_stride, __nv_bfloat16* y, int64_t ldy,
                             int64_t M, int64_t N, int64_t ld_slot, cudaStream_t stream) {
    const int64_t total = M * (N / 8);
    if (total == 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    sum_slots_kernel<<<(unsigned)blocks, 256, 0, stream>>>(slots, n_slots, slot_stride, y, ldy, M, N, ld_slot);
    return counted(cudaGetLastError());
}

// The same sum, written to every destination: y_d[m][n] for d < dst.n.  The destinations are the output matrices of
// all ranks of a row-parallel linear (this rank's own among them), so the reduced band reaches its peers by plain
// 16-byte stores over NVLink while the slots are read from local memory.
__global__ void __launch_bounds__(256)
sum_slots_gather_kernel(const __nv_bfloat16* __restrict__ slots, int n_slots, int64_t slot_stride, int64_t ld_slot, SumDst dst,
                        int64_t ld_dst, int64_t M, int64_t N) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t vec_per_row = N / 8;
    const int64_t total = M * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / vec_per_row;
        const int64_t c = (i - m * vec_per_row) * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < n_slots; ++r) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(slots + r * slot_stride + m * ld_slot + c));
            acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
            acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
#pragma unroll
        for (int d = 0; d < 8; ++d)
            if (d < dst.n) *reinterpret_cast<uint4*>(dst.y[d] + m * ld_dst + c) = o;
    }
}

cudaError_t launch_sum_slots_gather(const __nv_bfloat16* slots, int n_slots, int64_t slot_stride, int64_t ld_slot, SumDst dst,
                                    int64_t ld_dst, int64_t M, int64_t N, cudaStream_t stream) {
    const int64_t total = M * (N / 8);
    if (total == 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    sum_slots_gather_kernel<<<(unsigned)blocks, 256, 0, stream>>>(slots, n_slots, slot_stride, ld_slot, dst, ld_dst, M, N);
    return counted(cudaGetLastError());
}

// x (bf16, row pitch ldx) -> f16 [M][K] contiguous, round to nearest: the "A" operand of the
// large-M W8A16 GEMM.  Eight elements per thread and iteration.
__global__ void __launch_bounds__(256)
x_to_f16_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, __half* __restrict__ x16, int64_t M, int64_t K) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t vec_per_row = K / 8;
    const int64_t total = M * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec_per_row;
        const int64_t c = (i - r * vec_per_row) * 8;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + r * ldx + c));
        *reinterpret_cast<uint4*>(x16 + r * K + c) = bf16x8_to_f16x8(v);
    }
}

cudaError_t launch_x_to_f16(const __nv_bfloat16* x, int64_t ldx, void* x16, int64_t M, int64_t K, cudaStream_t stream) {
    const int64_t total = M * (K / 8);
    if (total == 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = pdl_attribute(attr);
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, x_to_f16_kernel, x, ldx, (__half*)x16, M, K));
}

// Packed e4m3 tiles (128 channels x 128 K bytes, 16 KiB each) -> packed f16 tiles (128 channels x 64
// elements = 128 bytes per row, 16 KiB each): source tile t becomes destination tiles 2t and 2t+1, so a
// channel block keeps its tiles consecutive along K.  The conversion is exact (every e4m3 value is an
// f16 value); the per-channel scale stays in the GEMM's epilogue.  A thread reads 16 bytes and writes 32.
__global__ void __launch_bounds__(256)
dequant_tiles_f16_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst, int64_t src_bytes) {
    pdl_launch_dependents();
    pdl_wait();                    // the GEMM before this pass may still read the destination
    const int64_t total = src_bytes / 16;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t off = i * 16;
        const int64_t tile = off >> 14;
        const int within = (int)(off & 16383);
        const int r = within >> 7;
        const int c = (within & 127) >> 4;            // 16-byte piece of the 128-byte row
        const uint4 v = ld_stream16(src + off);
        uint4 lo, hi;
        lo.x = cvt_e4m3x2_to_f16x2((uint16_t)(v.x & 0xffffu)); lo.y = cvt_e4m3x2_to_f16x2((uint16_t)(v.x >> 16));
        lo.z = cvt_e4m3x2_to_f16x2((uint16_t)(v.y & 0xffffu)); lo.w = cvt_e4m3x2_to_f16x2((uint16_t)(v.y >> 16));
        hi.x = cvt_e4m3x2_to_f16x2((uint16_t)(v.z & 0xffffu)); hi.y = cvt_e4m3x2_to_f16x2((uint16_t)(v.z >> 16));
        hi.z = cvt_e4m3x2_to_f16x2((uint16_t)(v.w & 0xffffu)); hi.w = cvt_e4m3x2_to_f16x2((uint16_t)(v.w >> 16));
        uint4* out = reinterpret_cast<uint4*>(dst + ((2 * tile + (c >> 2)) << 14) + r * 128 + (c & 3) * 32);
        out[0] = lo;
        out[1] = hi;
    }
}

cudaError_t launch_dequant_tiles_f16(const unsigned char* src, void* dst, int64_t src_bytes, cudaStream_t stream) {
    const int64_t total = src_bytes / 16;
    if (total == 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = pdl_attribute(attr);
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, dequant_tiles_f16_kernel, src, (unsigned char*)dst, src_bytes));
}

// Small-batch half of the fused MLP: gu = bf16 [M][2I] as the gate_up GEMM wrote it with interleaved
// weights (columns [256t, 256t+128) = gate channels 128t.., [256t+128, 256t+256) = up channels 128t..);
// hq[m][i] = e4m3( bf16(silu(g) * u) / h_scale ), the pre-quantised input of the down projection.
__global__ void __launch_bounds__(256)
silu_mul_quant_interleaved_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ h_scale,
                                  unsigned char* __restrict__ hq, int64_t M, int64_t I) {
    pdl_launch_dependents();
    pdl_wait();
    const ExactDiv div_scale(fmaxf(__ldg(h_scale), 1e-12f));
    const int64_t vec_per_row = I / 8;
    const int64_t total = M * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec_per_row;
        const int64_t c = (i - r * vec_per_row) * 8;
        const int64_t gcol = (c >> 7) * 256 + (c & 127);
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gu + r * 2 * I + gcol));
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(gu + r * 2 * I + gcol + 128));
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint4 h;
        uint32_t* hw = reinterpret_cast<uint32_t*>(&h);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = bf16_lo(gw[j]), g1 = bf16_hi(gw[j]);
            const float s0 = g0 / (1.f + expf(-g0)), s1 = g1 / (1.f + expf(-g1));
            hw[j] = pack_bf16x2(s0 * bf16_lo(uw[j]), s1 * bf16_hi(uw[j]));
        }
        *reinterpret_cast<uint2*>(hq + r * I + c) = quant8_e4m3(h, div_scale);
    }
}

cudaError_t launch_silu_mul_quant_interleaved(const __nv_bfloat16* gu, const float* h_scale, unsigned char* hq, int64_t M,
                                              int64_t I, cudaStream_t stream) {
    const int64_t total = M * (I / 8);
    if (total == 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = pdl_attribute(attr);
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, silu_mul_quant_interleaved_kernel, gu, h_scale, hq, M, I));
}

// ---- exporter arithmetic ------------------------------------------------------------------------
// Per-output-channel weight quantisation of the checkpoint exporter: scale[n] = max(amax_k |w[n][k]|, 1e-8) / 448,
// q[n][k] = e4m3(clamp(w[n][k] / scale[n], +-448)), true division, round to nearest even.  One CTA per
// channel: a pass for the maximum (the row then sits in L2), a pass that quantises.  kF32: fp32 source.
template <bool kF32>
__global__ void __launch_bounds__(256)
quantize_weight_kernel(const void* __restrict__ w_, int64_t ldw, unsigned char* __restrict__ q, float* __restrict__ scale,
                       int64_t K) {
    __shared__ float s_red[8];
    const int64_t n = blockIdx.x;
    const float* wf = reinterpret_cast<const float*>(w_) + n * ldw;
    const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(w_) + n * ldw;
    // bf16 rows that allow it are read 16 bytes and written 8 bytes at a time
    const bool vec = !kF32 && K % 8 == 0 && ldw % 8 == 0 && (reinterpret_cast<uintptr_t>(w_) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    float amax = 0.f;
    if (vec) {
        for (int64_t k = 8 * (int64_t)threadIdx.x; k < K; k += 8 * 256) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(wb + k));
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf16_lo(v.x)), fabsf(bf16_hi(v.x))), fmaxf(fabsf(bf16_lo(v.y)), fabsf(bf16_hi(v.y)))));
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf16_lo(v.z)), fabsf(bf16_hi(v.z))), fmaxf(fabsf(bf16_lo(v.w)), fabsf(bf16_hi(v.w)))));
        }
    } else {
        for (int64_t k = threadIdx.x; k < K; k += 256)
            amax = fmaxf(amax, fabsf(kF32 ? wf[k] : __bfloat162float(wb[k])));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = s_red[0];
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_red[i]);
    const float s = __fdiv_rn(fmaxf(amax, 1e-8f), 448.f);
    if (threadIdx.x == 0) scale[n] = s;
    const ExactDiv d(s);
    unsigned char* out = q + n * K;
    if (vec) {
        for (int64_t k = 8 * (int64_t)threadIdx.x; k < K; k += 8 * 256)
            *reinterpret_cast<uint2*>(out + k) = quant8_e4m3(__ldg(reinterpret_cast<const uint4*>(wb + k)), d);
        return;
    }
    for (int64_t k = 2 * (int64_t)threadIdx.x; k < K; k += 512) {          // K is even: two codes per store
        const float a = kF32 ? wf[k] : __bfloat162float(wb[k]);
        const float b = kF32 ? wf[k + 1] : __bfloat162float(wb[k + 1]);
        *reinterpret_cast<uint16_t*>(out + k) = cvt_e4m3x2(d(a), d(b));
    }
}

cudaError_t launch_quantize_weight(const void* w, bool w_is_f32, int64_t ldw, unsigned char* q, float* scale, int64_t N,
                                   int64_t K, cudaStream_t stream) {
    if (N == 0 || K == 0) return cudaSuccess;
    if (w_is_f32) quantize_weight_kernel<true><<<(unsigned)N, 256, 0, stream>>>(w, ldw, q, scale, K);
    else quantize_weight_kernel<false><<<(unsigned)N, 256, 0, stream>>>(w, ldw, q, scale, K);
    return counted(cudaGetLastError());
}

// Running maximum of |x| for the static activation scale of the exporter's calibration:
// *amax = max(*amax, max |x[m][k]|).  Non-negative floats order like their bit patterns, so the
// update is an integer atomicMax.
__global__ void __launch_bounds__(256)
abs_max_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int64_t M, int64_t K, float* __restrict__ amax) {
    const int64_t vec_per_row = K / 8;
    const int64_t total = M * vec_per_row;
    float m = 0.f;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec_per_row;
        const int64_t c = (i - r * vec_per_row) * 8;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + r * ldx + c));
        m = fmaxf(m, fmaxf(fmaxf(fabsf(bf16_lo(v.x)), fabsf(bf16_hi(v.x))), fmaxf(fabsf(bf16_lo(v.y)), fabsf(bf16_hi(v.y)))));
        m = fmaxf(m, fmaxf(fmaxf(fabsf(bf16_lo(v.z)), fabsf(bf16_hi(v.z))), fmaxf(fabsf(bf16_lo(v.w)), fabsf(bf16_hi(v.w)))));
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
}

cudaError_t launch_abs_max(const __nv_bfloat16* x, int64_t ldx, int64_t M, int64_t K, float* amax, cudaStream_t stream) {
    const int64_t total = M * (K / 8);
    if (total == 0) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    abs_max_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, ldx, M, K, amax);
    return counted(cudaGetLastError());
}

// Pack e4m3 weight bytes into the tiled layout (see pack_offset).  One CTA fills one
// 128 x 128 tile through shared memory; `src_is_kn` selects the source orientation:
// [K][N] (the reference's runtime buffer) or [N][K] (the checkpoint's layout).
__global__ void __launch_bounds__(256)
pack_tiles_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst, int64_t K, int64_t N,
                  int src_is_kn) {
    __shared__ unsigned char tile[128][128 + 4];      // [n][k]
    const int64_t KB = pack_kblocks(K);
    const int64_t tn = blockIdx.x, kb = blockIdx.y;
    const int64_t n0 = tn * 128, k0 = kb * 128;
    if (src_is_kn) {
        // rows of the source are k, columns n: read along n (coalesced), store transposed
        for (int i = threadIdx.x; i < 128 * 128; i += 256) {
            const int kk = i >> 7, nn = i & 127;
            const int64_t k = k0 + kk, n = n0 + nn;
            tile[nn][kk] = (k < K && n < N) ? src[k * N + n] : 0;
        }
    } else {
        for (int i = threadIdx.x; i < 128 * 128; i += 256) {
            const int nn = i >> 7, kk = i & 127;
            const int64_t k = k0 + kk, n = n0 + nn;
            tile[nn][kk] = (k < K && n < N) ? src[n * K + k] : 0;
        }
    }
    __syncthreads();
    unsigned char* out = dst + (size_t)(tn * KB + kb) * kPackTileBytes;
    for (int i = threadIdx.x; i < 128 * 32; i += 256) {             // 4 bytes per thread, coalesced
        const int nn = i >> 5, k4 = (i & 31) * 4;
        const uint32_t v = (uint32_t)tile[nn][k4] | ((uint32_t)tile[nn][k4 + 1] << 8) |
                           ((uint32_t)tile[nn][k4 + 2] << 16) | ((uint32_t)tile[nn][k4 + 3] << 24);
        *reinterpret_cast<uint32_t*>(out + nn * 128 + k4) = v;
    }
}

cudaError_t launch_pack_tiles(const unsigned char* src, unsigned char* dst, int64_t K, int64_t N, bool src_is_kn,
                              cudaStream_t stream) {
    if (K == 0 || N == 0) return cudaSuccess;
    dim3 grid((unsigned)pack_ntiles(N), (unsigned)pack_kblocks(K));
    pack_tiles_kernel<<<grid, 256, 0, stream>>>(src, dst, K, N, src_is_kn ? 1 : 0);
    return counted(cudaGetLastError());
}

}  // namespace fp8lin
