// Large-M W8A8 linear on the 5th-generation tensor cores (sm_100a).
//
//   y[M,N] = bf16( (xq[M,K] . W[N,K]^T) * in_scale * w_scale[n] + bias[n] )
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: cp.async.bulk.tensor.2d loads of a 128 x 128-byte
//               xq tile and a BN x 128-byte weight tile per K block into a
//               multi-stage shared-memory ring (128-byte swizzle), signalled by
//               mbarrier complete_tx.  No cluster multicast anywhere.
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma
//               .cta_group::1.kind::f8f6f4 (M=128, N=BN, K=32) four times per K
//               block, accumulating in TMEM; tcgen05.commit releases the ring
//               slot and, after the last K block, publishes the accumulator.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp owns one
//               32-lane quarter of TMEM), apply in_scale * w_scale[n] + bias[n]
//               in fp32, round once to bf16 and store.  Two accumulator stages
//               in TMEM let the epilogue of tile i overlap the main loop of
//               tile i+1.
// Split-K (few output tiles, long K): every split writes its fp32 tile to
// scratch and the last CTA to arrive at the tile's counter sums the splits in
// order and runs the epilogue.
//
// Tensor-bound for M >= ~1024: 2*M*K*N flops per call; HBM-bound below that.
// Every wait is bounded: a barrier that does not flip within about a second
// records a status code in the caller's scratch header and the CTA unwinds
// (drains its ring, frees TMEM) instead of hanging the GPU.
#include "common.cuh"
#include "kernels.h"

namespace fp8lin {

constexpr int kBM = 128;
constexpr int kBK = 128;  // bytes == e4m3 elements per K block
constexpr long long kWaitCycles = 2000000000LL;

template <int BN>
struct UmmaCfg {
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBBytes = BN * kBK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int kTmemCols = 2 * BN;
    // epilogue staging: per epilogue warp two 32-row x 128-byte boxes (4 KiB each)
    static constexpr int kStagingBytes = 4 * 2 * 4096;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024;
};

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
// Bounded wait; false = gave up (status word written).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
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
            else if (now - start > kWaitCycles) { atomicExch(status, code); return false; }
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
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
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

// 32 lanes x 32 columns of fp32 from TMEM (lane i of the warp reads TMEM lane base+i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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

template <int BN>
__host__ __device__ constexpr uint32_t make_idesc() {
    return (1u << 4)                     // accumulator fp32
           | (0u << 7) | (0u << 10)      // A, B = e4m3
           | (0u << 15) | (0u << 16)     // A, B K-major
           | ((uint32_t)(BN >> 3) << 17) // N
           | ((uint32_t)(kBM >> 4) << 24);
}

struct UmmaSched {
    int m_tiles, n_tiles, splits, kblocks_total, kblocks_per_split, total_work;
};

// work item -> (tile_m, tile_n, split); 8 M-tiles share a weight column block
// before the next column block starts, so concurrently running CTAs reuse L2 lines.
__device__ __forceinline__ void decode_work(const UmmaSched& s, int w, int& tm, int& tn, int& split) {
    split = w % s.splits;
    const int tile = w / s.splits;
    constexpr int kGroupM = 8;
    const int per_group = kGroupM * s.n_tiles;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int gsize = min(s.m_tiles - first_m, kGroupM);
    const int r = tile - group * per_group;
    tm = first_m + r % gsize;
    tn = r / gsize;
}

template <int BN>
__global__ void __launch_bounds__(192, 1)
umma_w8a8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ CUtensorMap tmap_part,
                 UmmaArgs p, UmmaSched sched) {
    using Cfg = UmmaCfg<BN>;
    constexpr int S = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[S];
    __shared__ __align__(8) uint64_t bar_empty[S];
    __shared__ __align__(8) uint64_t bar_tfull[2];
    __shared__ __align__(8) uint64_t bar_tempty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
    __shared__ int s_last;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(smem_u32(&bar_full[i]), 1); mbar_init(smem_u32(&bar_empty[i]), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bar_tfull[i]), 1); mbar_init(smem_u32(&bar_tempty[i]), 4); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < sched.total_work && ok; w += gridDim.x) {
                int tm, tn, split;
                decode_work(sched, w, tm, tn, split);
                const int kb0 = split * sched.kblocks_per_split;
                const int kb1 = min(sched.kblocks_total, kb0 + sched.kblocks_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t full = smem_u32(&bar_full[st]);
                    mbar_expect_tx(full, Cfg::kStageBytes);
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    tma_load_2d(sa, &tmap_a, kb * kBK, tm * kBM, full);
                    tma_load_2d(sa + Cfg::kABytes, &tmap_b, kb * kBK, tn * BN, full);
                }
            }
            if (!ok) {
                // let copies that are still in flight land before the CTA exits
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000) {}
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc<BN>();
            uint32_t it = 0;
            int tl = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < sched.total_work && ok; w += gridDim.x, ++tl) {
                int tm, tn, split;
                decode_work(sched, w, tm, tn, split);
                const int kb0 = split * sched.kblocks_per_split;
                const int kb1 = min(sched.kblocks_total, kb0 + sched.kblocks_per_split);
                const int as = tl & 1;
                const uint32_t aph = (tl >> 1) & 1;
                if (s_abort || !mbar_wait(smem_u32(&bar_tempty[as]), aph ^ 1, p.status, kDevTimeoutTmemEmpty)) {
                    s_abort = 1; ok = false; break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_full[st]), ph, p.status, kDevTimeoutFull)) {
                        s_abort = 1; ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + Cfg::kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k) {
                        // advance 32 bytes along K inside the 128-byte swizzle span: +2 in 16-byte units
                        umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bar_empty[st]));
                }
                if (ok) umma_commit(smem_u32(&bar_tfull[as]));
            }
        }
    } else {
        // ================= epilogue (warps 2..5) =================
        // Each warp owns TMEM lanes [32q, 32q+32) = 32 rows of the tile.  A lane holds one
        // row; 32 columns at a time come out of TMEM, are scaled/biased/rounded and written
        // to a 32-row x 128-byte staging box in shared memory in the 128-byte-swizzle
        // pattern (16-byte chunk index XOR row&7, bank-conflict free), and lane 0 hands
        // the box to a TMA store.  Two boxes per warp alternate so the next 64 columns
        // are converted while the previous store drains.
        const int q = warp & 3;
        const int ew = warp - 2;                                   // 0..3: staging slot
        const float in_scale = fmaxf(__ldg(p.input_scale), 1e-12f);
        const uint32_t stage0 = smem_base + S * Cfg::kStageBytes + ew * 8192;
        const uint32_t row_off = lane * 128;
        const uint32_t sw = lane & 7;
        int tl = 0;
        uint32_t nstore = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < sched.total_work && ok; w += gridDim.x, ++tl) {
            int tm, tn, split;
            decode_work(sched, w, tm, tn, split);
            const int as = tl & 1;
            const uint32_t aph = (tl >> 1) & 1;
            // (no s_abort shortcut here: the four epilogue warps must take the same
            //  branch because they meet at a named barrier below)
            if (!mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull)) {
                s_abort = 1; ok = false; break;
            }
            tc_fence_after();
            const int row0 = tm * kBM + q * 32;                    // first row of this warp's box
            const int n0 = tn * BN;
            const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN;

            if (sched.splits == 1) {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int nc = n0 + c * 32;
                    if (nc >= p.N) break;                          // uniform: whole chunk is past N
                    const uint32_t box = stage0 + ((nstore & 1) * 4096);
                    if ((c & 1) == 0) {
                        // the store issued two boxes ago read this buffer: wait until it is done with it
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                    }
                    uint32_t v[32];
                    tmem_ld32(t_addr + c * 32, v);
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        const int n = min(nc + j, p.N - 8);        // clamp keeps the loads in bounds; TMA clips the store
                        const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.w_scale + n));
                        const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.w_scale + n + 4));
                        float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        if (p.bias) {
                            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + n));
                            b[0] = bf16_lo(bv.x); b[1] = bf16_hi(bv.x); b[2] = bf16_lo(bv.y); b[3] = bf16_hi(bv.y);
                            b[4] = bf16_lo(bv.z); b[5] = bf16_hi(bv.z); b[6] = bf16_lo(bv.w); b[7] = bf16_hi(bv.w);
                        }
                        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                        float o[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) o[e] = fmaf(__uint_as_float(v[j + e]) * in_scale, sc[e], b[e]);
                        const uint32_t chunk = (uint32_t)((c & 1) * 4 + (j >> 3));
                        const uint32_t dst = box + row_off + ((chunk ^ sw) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                                     "r"(pack_bf16x2(o[0], o[1])), "r"(pack_bf16x2(o[2], o[3])),
                                     "r"(pack_bf16x2(o[4], o[5])), "r"(pack_bf16x2(o[6], o[7])) : "memory");
                    }
                    if ((c & 1) == 1 || nc + 32 >= p.N) {
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) tma_store_2d(&tmap_y, box, n0 + (c & ~1) * 32, row0);
                        ++nstore;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
            } else {
                // split-K: park the fp32 tile in scratch ([split][m_tiles*128][N]); a box is 32 rows x 32 floats
                const int prow0 = (split * sched.m_tiles + tm) * kBM + q * 32;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int nc = n0 + c * 32;
                    if (nc >= p.N) break;
                    const uint32_t box = stage0 + ((nstore & 1) * 4096);
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    uint32_t v[32];
                    tmem_ld32(t_addr + c * 32, v);
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const uint32_t dst = box + row_off + ((((uint32_t)j >> 2) ^ sw) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[j]), "r"(v[j + 1]),
                                     "r"(v[j + 2]), "r"(v[j + 3]) : "memory");
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) tma_store_2d(&tmap_part, box, nc, prow0);
                    ++nstore;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&bar_tempty[as]));
                    tma_store_wait_all();          // this warp's partial rows are in global memory
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    int* counter = p.counters + (tm * sched.n_tiles + tn);
                    const int prev = atomicAdd(counter, 1);
                    s_last = (prev == sched.splits - 1);
                    if (s_last) *counter = 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool last = s_last != 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");  // s_last may be rewritten next tile
                if (last) {
                    __threadfence();
                    // coalesced reduction: the warp walks its 32 rows, lanes span the columns
                    const int ncols = min(BN, p.N - n0);
                    const size_t split_stride = (size_t)sched.m_tiles * kBM * p.N;
                    for (int r = 0; r < 32; ++r) {
                        const int row = tm * kBM + q * 32 + r;
                        if (row >= p.M) break;
                        const float* prow = p.partial + (size_t)row * p.N + n0;
                        __nv_bfloat16* yrow = p.y + (size_t)row * p.ldy + n0;
                        for (int cc = lane * 4; cc < ncols; cc += 128) {
                            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                            for (int sp = 0; sp < sched.splits; ++sp) {
                                const float4 u = __ldcg(reinterpret_cast<const float4*>(prow + sp * split_stride + cc));
                                a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
                            }
                            const float4 sc = __ldg(reinterpret_cast<const float4*>(p.w_scale + n0 + cc));
                            float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
                            if (p.bias) {
                                const uint2 bv = __ldg(reinterpret_cast<const uint2*>(p.bias + n0 + cc));
                                b0 = bf16_lo(bv.x); b1 = bf16_hi(bv.x); b2 = bf16_lo(bv.y); b3 = bf16_hi(bv.y);
                            }
                            uint2 out;
                            out.x = pack_bf16x2(fmaf(a.x * in_scale, sc.x, b0), fmaf(a.y * in_scale, sc.y, b1));
                            out.y = pack_bf16x2(fmaf(a.z * in_scale, sc.z, b2), fmaf(a.w * in_scale, sc.w, b3));
                            *reinterpret_cast<uint2*>(yrow + cc) = out;
                        }
                    }
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---- host side -------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
    return fn;
}

// 2-D byte tensor [rows][cols] (cols contiguous), box = 128 bytes x box_rows, 128-byte swizzle.
static bool encode_u8_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols};
    cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Output-side maps: 2-D tensor [rows][cols] with a row pitch in bytes, box = 128 bytes x 32 rows.
static bool encode_out_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, uint32_t elem_bytes,
                          uint64_t rows, uint64_t cols, uint64_t pitch_bytes) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {128u / elem_bytes, 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

UmmaPlan plan_umma(int64_t M, int64_t K, int64_t N, int force_bn, int force_splits) {
    UmmaPlan best{};
    const int kblocks = (int)((K + kBK - 1) / kBK);
    const int m_tiles = (int)((M + kBM - 1) / kBM);
    double best_cost = 1e30;
    const int bns[3] = {256, 128, 64};
    const double unit[3] = {1.0, 0.85, 0.6};  // relative time of one K block of a tile (smaller tiles use shared memory less well)
    for (int i = 0; i < 3; ++i) {
        const int bn = bns[i];
        if (force_bn > 0 && bn != force_bn) continue;
        const int n_tiles = (int)((N + bn - 1) / bn);
        const long tiles = (long)m_tiles * n_tiles;
        int splits = 1;
        if (force_splits > 0) splits = force_splits;
        else if (tiles < 148) {
            splits = (int)(148 / tiles);
            const int max_by_k = kblocks / 4 > 0 ? kblocks / 4 : 1;  // at least four K blocks per split
            if (splits > max_by_k) splits = max_by_k;
            if (splits > 16) splits = 16;
        }
        if (splits > kblocks) splits = kblocks;
        if (tiles > kWsMaxCounters) splits = 1;
        const int kps = (kblocks + splits - 1) / splits;
        splits = (kblocks + kps - 1) / kps;
        const long work = tiles * splits;
        const long waves = (work + 147) / 148;
        // main-loop time + fixed per-tile epilogue/prologue + split-K reduction traffic
        const double cost = waves * (kps * unit[i] + 3.0 * unit[i]) + (splits > 1 ? 0.5 * splits : 0.0);
        if (cost < best_cost) {
            best_cost = cost;
            best.bn = bn; best.splits = splits; best.kblocks_per_split = kps;
            best.m_tiles = m_tiles; best.n_tiles = n_tiles;
            best.grid = (int)(work < 148 ? work : 148);
            best.partial_bytes = splits > 1 ? (size_t)splits * m_tiles * kBM * N * sizeof(float) : 0;
        }
    }
    return best;
}

template <int BN>
static cudaError_t launch_bn(const UmmaPlan& pl, const UmmaArgs& a, const CUtensorMap& ta, const CUtensorMap& tb,
                             const CUtensorMap& ty, const CUtensorMap& tp, cudaStream_t stream) {
    using Cfg = UmmaCfg<BN>;
    auto kern = umma_w8a8_kernel<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    UmmaSched s;
    s.m_tiles = pl.m_tiles; s.n_tiles = pl.n_tiles; s.splits = pl.splits;
    s.kblocks_total = (a.K + kBK - 1) / kBK; s.kblocks_per_split = pl.kblocks_per_split;
    s.total_work = pl.m_tiles * pl.n_tiles * pl.splits;
    kern<<<pl.grid, 192, Cfg::kSmemBytes, stream>>>(ta, tb, ty, tp, a, s);
    return cudaGetLastError();
}

cudaError_t launch_umma_w8a8(const UmmaPlan& pl, const UmmaArgs& a, cudaStream_t stream, const char** why) {
    CUtensorMap ta, tb;
    if (!encode_u8_2d(&ta, a.xq, (uint64_t)a.M, (uint64_t)a.K, kBM) ||
        !encode_u8_2d(&tb, a.w, (uint64_t)a.N, (uint64_t)a.K, (uint32_t)pl.bn)) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    CUtensorMap ty, tp;
    if (!encode_out_2d(&ty, a.y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.M, (uint64_t)a.N,
                       (uint64_t)a.ldy * 2)) {
        if (why) *why = "cuTensorMapEncodeTiled failed for y";
        return cudaErrorInvalidValue;
    }
    tp = ty;
    if (pl.splits > 1 &&
        !encode_out_2d(&tp, a.partial, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                       (uint64_t)pl.splits * pl.m_tiles * kBM, (uint64_t)a.N, (uint64_t)a.N * 4)) {
        if (why) *why = "cuTensorMapEncodeTiled failed for the split-K scratch";
        return cudaErrorInvalidValue;
    }
    switch (pl.bn) {
        case 256: return launch_bn<256>(pl, a, ta, tb, ty, tp, stream);
        case 128: return launch_bn<128>(pl, a, ta, tb, ty, tp, stream);
        case 64: return launch_bn<64>(pl, a, ta, tb, ty, tp, stream);
    }
    if (why) *why = "unsupported tile width";
    return cudaErrorInvalidValue;
}

}  // namespace fp8lin
