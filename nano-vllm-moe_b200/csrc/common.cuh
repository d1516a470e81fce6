// Shared device helpers for the fp8lin kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fp8lin.h"

namespace fp8lin {

// ---- scratch header ---------------------------------------------------------
// The first FP8LIN_WS_HEADER_BYTES of the caller's scratch.  Everything in it
// is zero between calls: counters are reset by the CTA that consumes them.
constexpr int kWsStatusWords = 64;                                  // word 0 = device status
constexpr int kWsMaxCounters = FP8LIN_WS_HEADER_BYTES / 4 - kWsStatusWords;

struct WsView {
    int* status;          // device status word (0 = ok)
    int* counters;        // kWsMaxCounters split-K arrival counters
    unsigned char* body;  // shape-dependent area, 256-byte aligned
    size_t body_bytes;
};

__host__ __device__ inline WsView ws_view(void* ws, size_t bytes) {
    WsView v;
    v.status = reinterpret_cast<int*>(ws);
    v.counters = reinterpret_cast<int*>(ws) + kWsStatusWords;
    v.body = reinterpret_cast<unsigned char*>(ws) + FP8LIN_WS_HEADER_BYTES;
    v.body_bytes = bytes > FP8LIN_WS_HEADER_BYTES ? bytes - FP8LIN_WS_HEADER_BYTES : 0;
    return v;
}

// device status codes written by kernels that gave up a bounded wait
enum : int { kDevOk = 0, kDevTimeoutFull = 0x101, kDevTimeoutEmpty = 0x102, kDevTimeoutTmemFull = 0x103,
             kDevTimeoutTmemEmpty = 0x104, kDevTimeoutQuant = 0x105, kDevTimeoutPeer = 0x106 };

// ---- packed weight layout ----------------------------------------------------------
// Weights are stored as 128-channel x 128-byte tiles, each tile contiguous (16 KiB),
// tiles of one channel block consecutive along K:
//   byte(n, k) = ((n / 128) * KB + k / 128) * 16384 + (n % 128) * 128 + (k % 128),  KB = ceil(K / 128)
// N and K are zero-padded to multiples of 128.  A CTA that streams a channel block
// reads one long sequential range of HBM, and a tile is exactly one TMA box.
constexpr int kPackTile = 128;
constexpr int kPackTileBytes = kPackTile * kPackTile;
__host__ __device__ inline int64_t pack_kblocks(int64_t K) { return (K + kPackTile - 1) / kPackTile; }
__host__ __device__ inline int64_t pack_ntiles(int64_t N) { return (N + kPackTile - 1) / kPackTile; }
__host__ __device__ inline size_t pack_offset(int64_t n, int64_t k, int64_t KB) {
    return (size_t)((n >> 7) * KB + (k >> 7)) * kPackTileBytes + (size_t)(n & 127) * kPackTile + (size_t)(k & 127);
}

// ---- programmatic dependent launch ------------------------------------------------
// Every kernel lets the next kernel in the stream start launching early
// (pdl_launch_dependents) and, before it touches memory a predecessor may still be
// writing or reading (activations, outputs, scratch), waits for the predecessors to
// finish (pdl_wait).  Weights are never written by a kernel, so their first loads are
// issued before the wait.  Both are no-ops when the launch carries no such dependency.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- small numeric helpers ----------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

// Two floats -> two e4m3 bytes (lo in bits 0-7), RNE, saturating to +-448.
__device__ __forceinline__ uint16_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// Two e4m3 bytes -> packed f16x2 (exact).
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return r;
}

// Correctly rounded x / s in three instructions, given r = 1/s rounded to nearest
// (Markstein): q0 = x*r is within an ulp, the FMA residual e = x - q0*s is exact,
// and q0 + e*r rounds to the true quotient.  Overflowing or non-finite q0 is
// returned as is (the exact division overflows there too), and so is a zero q0
// (the correction would turn -0 into +0), so the saturating e4m3 conversion
// that follows sees the same value as after a true division.
struct ExactDiv {
    float s, r;
    __device__ __forceinline__ explicit ExactDiv(float scale) {
        s = scale;
        r = __fdiv_rn(1.0f, scale);
    }
    __device__ __forceinline__ float operator()(float x) const {
        const float q0 = x * r;
        const float e = fmaf(-q0, s, x);
        const float q1 = fmaf(e, r, q0);
        return (fabsf(q0) <= 3.0e38f && q0 != 0.f) ? q1 : q0;
    }
};

// Static activation quantiser for 8 bf16 values (one 16-byte word) -> 8 e4m3 bytes;
// the codes equal the reference's torch path (true division, RNE, clamp to +-448) bit for bit.
__device__ __forceinline__ uint2 quant8_e4m3(uint4 v, const ExactDiv& d) {
    uint2 r;
    uint32_t a = cvt_e4m3x2(d(bf16_lo(v.x)), d(bf16_hi(v.x)));
    uint32_t b = cvt_e4m3x2(d(bf16_lo(v.y)), d(bf16_hi(v.y)));
    uint32_t c = cvt_e4m3x2(d(bf16_lo(v.z)), d(bf16_hi(v.z)));
    uint32_t e = cvt_e4m3x2(d(bf16_lo(v.w)), d(bf16_hi(v.w)));
    r.x = a | (b << 16);
    r.y = c | (e << 16);
    return r;
}

// 8 bf16 -> 8 f16 (RNE; exact for every bf16 inside the f16 normal range).
__device__ __forceinline__ uint4 bf16x8_to_f16x8(uint4 v) {
    uint4 r;
    __half2 h;
    h = __floats2half2_rn(bf16_lo(v.x), bf16_hi(v.x)); r.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(bf16_lo(v.y), bf16_hi(v.y)); r.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(bf16_lo(v.z), bf16_hi(v.z)); r.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(bf16_lo(v.w), bf16_hi(v.w)); r.w = *reinterpret_cast<uint32_t*>(&h);
    return r;
}

// Streaming 16-byte load that does not pollute L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ uint4 ld_cached16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

}  // namespace fp8lin
