// PTX wrappers shared by the tcgen05 kernels: mbarriers with bounded waits, TMA
// loads/stores, TMEM allocation and loads, UMMA descriptors, cluster helpers.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace fp8lin {

constexpr long long kWaitCycles = 2000000000LL;   // about a second: then a wait gives up

// ---- PTX wrappers --------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// Bounded wait; false = gave up after `limit` clock cycles (status word written).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code,
                                          long long limit = kWaitCycles) {
    long long start = -1;
    for (uint32_t it = 0;; ++it) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 0x3ff) == 0x3ff) {
            const long long now = clock64();
            if (start < 0) start = now;
            else if (now - start > limit) { atomicExch(status, code); return false; }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// TMA store of one shared-memory box; elements outside the tensor are not written,
// which is what clips the M and N tails.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}

// Same, f16 operands from shared memory (K = 16 elements = 32 bytes per instruction).
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}

// ---- CTA pairs (cta_group::2): one MMA spans the tensor cores, shared memory and TMEM of two CTAs ----
// Every collective below is executed by the same warp of BOTH CTAs of the pair.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Issued by one thread of the leader CTA; `bar` is a shared::cluster address (own or the peer's barrier).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}
// TMA load into this CTA's shared memory whose completion is counted on a barrier that may live in the
// peer CTA (`bar` is a shared::cluster address); the data itself goes to one CTA only.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {     // bar: shared::cluster address
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 columns of fp32 from TMEM (lane i of the warp reads TMEM lane base+i); no wait.
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// cluster helpers (split-K)
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// 16 bytes into a CTA of the cluster (dst and bar are shared::cluster addresses of the same CTA); the store is
// asynchronous and counts its bytes on that CTA's barrier when it lands
__device__ __forceinline__ void st_async_v4(uint32_t dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(dst), "r"(a), "r"(b), "r"(c), "r"(d), "r"(bar) : "memory");
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffff) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                    // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}


// Instruction descriptor: D fp32, A/B formats (0 = e4m3 for kind::f8f6f4; 0 = f16, 1 = bf16 for
// kind::f16), both operands K-major, MMA shape M x N.
__host__ __device__ constexpr uint32_t make_idesc_mn(int m, int n, uint32_t a_fmt, uint32_t b_fmt) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (0u << 15) | (0u << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Opt a kernel in to `bytes` of dynamic shared memory once per device (function attributes are per device).
struct SmemOptIn {
    bool done[64] = {};
};
inline cudaError_t ensure_dynamic_smem(const void* kernel, int bytes, SmemOptIn& state) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && state.done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) state.done[dev] = true;
    return e;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn();     // defined in umma_gemm.cu
// How many clusters of `cluster` CTAs of this kernel can be resident at once (cached; when no
// device can be asked, the figure for 148 SMs in 8 GPCs with one CTA per SM).
int max_active_clusters(const void* kernel, int threads, size_t smem_bytes, int cluster);
// 2-D byte tensor [rows][cols] (cols contiguous), box = 128 bytes x box_rows, 128-byte swizzle.
bool encode_u8_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
// Output map: bf16 [rows][cols] with a row pitch in bytes, box = box_cols x 32 rows, swizzle span = the
// box's row length (128 or 64 bytes).
bool encode_out_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                   uint32_t box_cols);

// ---- activation quantisation inside the large-M GEMM ------------------------------------------------
// The GEMM kernels that take bf16 activations carry kQuantWarps extra warps.  Those warps turn rows
// [row_start, M) of x into e4m3 rows of the scratch matrix xq that the kernel's own TMA producer loads as
// the "A" operand, while the tensor cores work on rows quantised earlier (rows below row_start are
// quantised by a short pass in front of the kernel, so the first round of tiles does not wait).
//
// The work is handed out in units of kQuantRows rows through a ticket counter in global scratch: a warp
// takes the next ticket, converts its rows, and adds one to the "done" counter of the 128-row block the
// rows belong to.  A TMA producer that needs a row block waits (bounded) until that block's counter has
// reached its number of units.  Tickets are only ever taken by warps that are already running, and a warp
// holding a ticket waits for nothing, so the scheme makes progress however many of the grid's CTAs are
// resident at a time.  The last CTA to leave zeroes the counters again (scratch counters are zero between
// calls).  The quantiser warps stay at most `lead` row blocks ahead of the furthest row block any producer has
// started on (the "frontier"): running far ahead would stream all of x and xq through L2 while the GEMM's own
// tiles live there, which measurably slows the GEMM down.  The lead is large enough that a producer never needs
// a block beyond frontier + lead, so the throttle cannot stall the kernel (and a throttle wait that runs out
// simply proceeds).  Layout of ctrl: [0] next ticket, [1] CTAs that have left, [2] frontier, [3 + b] units done
// in row block b.
constexpr int kQuantWarps = 4;
constexpr int kQuantRows = 8;           // rows per unit; divides 128, so a unit lies inside one row block

struct QuantJob {
    const __nv_bfloat16* x;      // bf16 activations [M][ldx]; nullptr = nothing to do (xq arrives complete)
    unsigned char* xq;           // e4m3 [M][K]
    int* ctrl;
    int ldx;
    int row_start;               // multiple of 128
    int lead;                    // row blocks the quantiser may run ahead of the frontier
};
constexpr int kQuantCtrlWords = 3;

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// orders earlier generic-proxy accesses to global memory against later async-proxy (TMA) ones
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Units of the 128-row block `block` that the in-kernel quantiser produces.
__device__ __forceinline__ int quant_units_in_block(const QuantJob& j, int M, int block) {
    const int r0 = max(block * 128, j.row_start);
    const int r1 = min(block * 128 + 128, M);
    return r1 > r0 ? (r1 - r0 + kQuantRows - 1) / kQuantRows : 0;
}

// Producer side: wait until row block `block` of xq is complete.  false = gave up (status written).
__device__ __forceinline__ bool quant_wait_block(const QuantJob& j, int M, int block, int* status) {
    const int need = quant_units_in_block(j, M, block);
    if (need == 0) { atomicMax(j.ctrl + 2, block); return true; }
    atomicMax(j.ctrl + 2, block);          // the frontier moves before the wait: the quantiser may be throttled on it
    const int* flag = j.ctrl + kQuantCtrlWords + block;
    long long start = -1;
    for (uint32_t it = 0;; ++it) {
        if (ld_acquire_gpu(flag) >= need) break;
        if ((it & 0xff) == 0xff) {
            const long long now = clock64();
            if (start < 0) start = now;
            else if (now - start > kWaitCycles) { atomicExch(status, (int)kDevTimeoutQuant); return false; }
        }
        __nanosleep(64);
    }
    fence_proxy_async_all();       // the rows were written with ordinary stores; the TMA unit reads them next
    return true;
}

// Early, non-blocking look at a row block the producer will need one tile from now: true = already complete
// (completeness is monotonic, so the answer stays valid).  Issued a whole tile ahead, the global round trip of the
// flag load overlaps the tile's loads instead of stalling the producer at the tile boundary.  Also moves the frontier.
__device__ __forceinline__ bool quant_probe_block(const QuantJob& j, int M, int block) {
    atomicMax(j.ctrl + 2, block);
    const int need = quant_units_in_block(j, M, block);
    return need == 0 || ld_acquire_gpu(j.ctrl + kQuantCtrlWords + block) >= need;
}

// One quantiser warp: take units until none are left.
__device__ __forceinline__ void quant_worker(const QuantJob& j, const float* input_scale, int M, int K, int lane) {
    const ExactDiv div(fmaxf(__ldg(input_scale), 1e-12f));
    const int total_units = M > j.row_start ? (M - j.row_start + kQuantRows - 1) / kQuantRows : 0;
    const int vec_per_row = K >> 4;
    for (;;) {
        int u = 0;
        if (lane == 0) u = atomicAdd(j.ctrl, 1);
        u = __shfl_sync(0xffffffffu, u, 0);
        if (u >= total_units) break;
        const int row0 = j.row_start + u * kQuantRows;
        const int rows = min(kQuantRows, M - row0);
        if ((row0 >> 7) > ld_acquire_gpu(j.ctrl + 2) + j.lead) {          // too far ahead of the GEMM: hold back
            const long long t0 = clock64();
            while ((row0 >> 7) > ld_acquire_gpu(j.ctrl + 2) + j.lead && clock64() - t0 < kWaitCycles) __nanosleep(256);
        }
        // four rows per step: eight 16-byte loads in flight per lane.  The quantiser is latency-bound (a few
        // warps per SM), and it has to keep up with the rate at which the GEMM consumes rows.
        for (int r = 0; r < rows; r += 4) {
            const __nv_bfloat16* src[4];
            unsigned char* dst[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int rr = min(r + q, rows - 1);                   // a short tail re-reads the last row (not stored)
                src[q] = j.x + (size_t)(row0 + rr) * j.ldx;
                dst[q] = j.xq + (size_t)(row0 + rr) * K;
            }
            for (int v = lane; v < vec_per_row; v += 32) {
                uint4 a[4][2];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    a[q][0] = ld_stream16(src[q] + v * 16);
                    a[q][1] = ld_stream16(src[q] + v * 16 + 8);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (r + q < rows) {
                        const uint2 q0 = quant8_e4m3(a[q][0], div), q1 = quant8_e4m3(a[q][1], div);
                        *reinterpret_cast<uint4*>(dst[q] + v * 16) = make_uint4(q0.x, q0.y, q1.x, q1.y);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) {
            fence_proxy_async_all();
            __threadfence();
            atomicAdd(j.ctrl + kQuantCtrlWords + (row0 >> 7), 1);
        }
    }
}

// Every CTA calls this once all its warps are done with the counters (after its last __syncthreads):
// the last one to arrive zeroes them for the next call.
__device__ __forceinline__ void quant_ctrl_release(const QuantJob& j, int M) {
    __threadfence();
    const int left = atomicAdd(j.ctrl + 1, 1);
    if (left == (int)gridDim.x - 1) {
        const int blocks = (M + 127) >> 7;
        for (int b = 0; b < blocks; ++b) j.ctrl[kQuantCtrlWords + b] = 0;
        j.ctrl[0] = 0;
        j.ctrl[2] = 0;
        __threadfence();
        j.ctrl[1] = 0;
    }
}

// Destinations of a GEMM epilogue's TMA stores (all describe a bf16 [M][N] matrix of the same shape).
struct OutMaps {
    CUtensorMap m[8];
    int n;
    // 0: every output box is stored to all n destinations.  > 0 (a multiple of 32): destination d receives only the
    // rows [d * band_rows, (d + 1) * band_rows) of the result, at row (r - d * band_rows) of its matrix: the
    // reduce-scatter form of a row-parallel linear, where rank d sums the bands it receives.
    int band_rows;
};

// Store one staged 32-row box whose first row is `row0` of the result to its destination(s).
__device__ __forceinline__ void store_box(const OutMaps& outs, uint32_t box, int col0, int row0) {
    if (outs.band_rows > 0) {
        const int d = row0 / outs.band_rows;
        if (d < outs.n) tma_store_2d(&outs.m[d], box, col0, row0 - d * outs.band_rows);
        else asm volatile("cp.async.bulk.commit_group;" ::: "memory");      // keep the group count per box uniform
        return;
    }
    for (int d = 0; d < outs.n; ++d) tma_store_2d(&outs.m[d], box, col0, row0);
}

}  // namespace fp8lin
