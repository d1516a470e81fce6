// Decode-sized W8A16 linear (used for 33 <= M <= 64; works from M = 1) on tcgen05, operands swapped:
//
//   y^T[N, M] = f16(W_e4m3[N, K]) . f16(x[M, K])^T         fp32 accumulation in TMEM
//
// The e4m3 weight tile arrives by TMA exactly as in the W8A8 kernel, but kind::f16 needs 16-bit
// operands.  Instead of writing a widened copy back to shared memory (which would double the
// shared-memory traffic of a kernel that is supposed to be HBM-bound), converter warps widen the
// tile in registers (cvt.rn.f16x2.e4m3x2, exact) and put it into TENSOR MEMORY with tcgen05.st;
// the MMA then takes its "A" operand from TMEM and only the small activation tile from shared
// memory.  HBM-bound: K*N + 2*M*K + 2*M*N + 6*N bytes per call.
//
//   warp 0       TMA producer: per 128-element K block one packed 128 x 128-byte weight tile
//                (128-byte swizzle) and the raw bf16 activation block [M x 128].
//   warps 2..9   two converter teams of four warps (one warp per 32-lane quarter of TMEM), one ring
//                slot per team in turn: each lane widens one weight row (128 bytes -> 64 f16x2 words
//                -> tcgen05.st.32x32b.x64), the team also rewrites the activation block as f16 into
//                two K-major 128-byte-swizzled "B" tiles (64 elements each).
//   warp 1       MMA issuer: eight tcgen05.mma.cta_group::1.kind::f16 (M=128, N=MP, K=16) per K
//                block, A from TMEM, B from shared memory.
//   warps 10..13 epilogue: as in the W8A8 kernel, y[m][n] = bf16(acc * w_scale[n] + bias[n]).
//
// Persistent over the N/128 channel tiles or cluster split-K with the partial sums pushed to the
// CTA that finishes a band (st.async, no cluster barrier after set-up), bounded waits, programmatic
// dependent launch: all as in umma_swap.cu.
#include "umma_common.cuh"

namespace fp8lin {

constexpr int kS16ConvWarps = 8;           // two teams of four warps (12 and 16 warps measured no faster)
constexpr int kS16Teams = kS16ConvWarps / 4;
constexpr int kS16Threads = (2 + kS16ConvWarps + 4) * 32;
constexpr int kS16Tile = 128;
constexpr int kS16KB = 128;

template <int MP>
struct Swap16Cfg {
    static constexpr int kWBytes = kS16Tile * kS16KB;            // raw e4m3 weight tile
    static constexpr int kXfBytes = MP * kS16KB * 2;             // f16 activation tiles (two 64-element halves)
    static constexpr int kXrawBytes = MP * kS16KB * 2;           // raw bf16 activation block
    static constexpr int kStageBytes = kWBytes + kXfBytes + kXrawBytes;
    static constexpr int kStages = MP <= 16 ? 7 : (MP <= 32 ? 6 : 4);
    static constexpr int kRingBytes = kStages * kStageBytes;
    static constexpr int kSmemBytes = kRingBytes + 1024;
    static constexpr int kAccCols = 2 * MP < 32 ? 32 : 2 * MP;   // two accumulator stages
    static constexpr int kACols = 64;                            // one widened weight tile: 128 K / 2 per column
    static constexpr int kTmemCols = 512;
    static constexpr int kPartPitch = MP * 4 + 16;
    static_assert(kAccCols + kStages * kACols <= kTmemCols, "TMEM budget");
    static_assert(kStageBytes % 1024 == 0, "stage alignment");
    static_assert((kS16Tile + 8) * kPartPitch <= kRingBytes, "the received slices of a band must fit in the ring");
};

struct Swap16Sched {
    int n_tiles, splits, kblocks_total, kblocks_per_split;
};

__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}

// 64 consecutive 32-bit TMEM columns of this lane <- 64 registers
__device__ __forceinline__ void tmem_st64(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x64.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,"
        "%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,"
        "%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63,%64};"
        ::"r"(taddr),
          "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]),
          "r"(v[32]), "r"(v[33]), "r"(v[34]), "r"(v[35]), "r"(v[36]), "r"(v[37]), "r"(v[38]), "r"(v[39]),
          "r"(v[40]), "r"(v[41]), "r"(v[42]), "r"(v[43]), "r"(v[44]), "r"(v[45]), "r"(v[46]), "r"(v[47]),
          "r"(v[48]), "r"(v[49]), "r"(v[50]), "r"(v[51]), "r"(v[52]), "r"(v[53]), "r"(v[54]), "r"(v[55]),
          "r"(v[56]), "r"(v[57]), "r"(v[58]), "r"(v[59]), "r"(v[60]), "r"(v[61]), "r"(v[62]), "r"(v[63])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void s16_tmem_ld(uint32_t taddr, uint32_t* v) {
    if (N == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr) : "memory");
    } else {
#pragma unroll
        for (int c = 0; c < N; c += 32) tmem_ld32_nowait(taddr + c, v + c);
    }
}

template <int MP, bool kSplit>
__global__ void __launch_bounds__(kS16Threads, 1)
swap_w8a16_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                  UmmaArgs p, Swap16Sched sched) {
    using Cfg = Swap16Cfg<MP>;
    constexpr int S = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[S];     // TMA bytes landed (weights + raw x)
    __shared__ __align__(8) uint64_t bar_conv[S];     // operands converted (four warps of the owning team)
    __shared__ __align__(8) uint64_t bar_empty[S];    // MMAs that read the slot are done
    __shared__ __align__(8) uint64_t bar_tfull[2];
    __shared__ __align__(8) uint64_t bar_tempty[2];
    __shared__ __align__(8) uint64_t bar_ready;       // split-K: every CTA of the cluster is past its MMAs
    __shared__ __align__(8) uint64_t bar_recv;        // split-K: the partials of this CTA's band have landed
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int split_rank = kSplit ? (int)cluster_ctarank() : 0;
    const int first_tile = kSplit ? (int)(blockIdx.x / sched.splits) : (int)blockIdx.x;
    const int tile_step = kSplit ? sched.n_tiles : (int)gridDim.x;
    const int kb0 = split_rank * sched.kblocks_per_split;
    const int kb1 = kSplit ? min(sched.kblocks_total, kb0 + sched.kblocks_per_split) : sched.kblocks_total;
    const uint32_t x_bytes = (uint32_t)p.M * 256u;
    const int band = kSplit ? (kS16Tile + sched.splits - 1) / sched.splits : kS16Tile;
    const int band_rows = kSplit ? min(kS16Tile, (split_rank + 1) * band) - split_rank * band : 0;
    const int m_groups = (p.M + 3) >> 2;
    constexpr uint32_t kXfOff = Cfg::kWBytes;
    constexpr uint32_t kXrawOff = Cfg::kWBytes + Cfg::kXfBytes;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(smem_u32(&bar_full[i]), 1);
            mbar_init(smem_u32(&bar_conv[i]), 4);
            mbar_init(smem_u32(&bar_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bar_tfull[i]), 1); mbar_init(smem_u32(&bar_tempty[i]), 4); }
        s_abort = 0;
        if (kSplit) {
            mbar_init(smem_u32(&bar_ready), (uint32_t)sched.splits);
            mbar_init(smem_u32(&bar_recv), 1);
            mbar_expect_tx(smem_u32(&bar_recv), (uint32_t)(sched.splits * band_rows * m_groups * 16));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), Cfg::kTmemCols);
    // rows M..MP-1 of every f16 activation tile are zero for the whole kernel
    for (int i = threadIdx.x; i < S * (Cfg::kXfBytes / 16); i += kS16Threads) {
        const int st = i / (Cfg::kXfBytes / 16), r = i % (Cfg::kXfBytes / 16);
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(smem_base + st * Cfg::kStageBytes + kXfOff + r * 16), "r"(0u) : "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    const uint32_t tmem_a0 = tmem_base + Cfg::kAccCols;            // first widened-weight buffer
    pdl_launch_dependents();
    if (kSplit) cluster_arrive();                            // (waited for before the first remote access)
    // scale and bias of the first channel this thread finishes, fetched long before they are needed
    float ws0 = 0.f, bs0 = 0.f;
    if constexpr (kSplit) {
        if (band_rows > 0 && (int)threadIdx.x < band_rows * m_groups) {
            const int n0 = first_tile * kS16Tile + split_rank * band + (int)threadIdx.x % band_rows;
            if (n0 < p.N) {
                ws0 = __ldg(p.w_scale + n0);
                if (p.bias) bs0 = __bfloat162float(p.bias[n0]);
            }
        }
    }

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
            uint32_t it = 0;
            bool ok = true;
            const int first_kb = min(kb1 - kb0, S);
            if (first_tile < sched.n_tiles) {
                for (int i = 0; i < first_kb; ++i) {           // weights do not depend on the predecessor
                    const uint32_t full = smem_u32(&bar_full[i]);
                    mbar_expect_tx(full, Cfg::kWBytes + x_bytes);
                    tma_load_2d(smem_base + i * Cfg::kStageBytes, &tmap_w, 0,
                                (first_tile * sched.kblocks_total + kb0 + i) * kS16Tile, full);
                }
                pdl_wait();
                for (int i = 0; i < first_kb; ++i)
                    tma_load_2d(smem_base + i * Cfg::kStageBytes + kXrawOff, &tmap_x, (kb0 + i) * kS16KB, 0,
                                smem_u32(&bar_full[i]));
            }
            for (int t = first_tile; t < sched.n_tiles && ok; t += tile_step) {
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    if (it < (uint32_t)first_kb) continue;
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t full = smem_u32(&bar_full[st]);
                    mbar_expect_tx(full, Cfg::kWBytes + x_bytes);
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    tma_load_2d(sa, &tmap_w, 0, (t * sched.kblocks_total + kb) * kS16Tile, full);
                    tma_load_2d(sa + kXrawOff, &tmap_x, kb * kS16KB, 0, full);
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000) {}
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_mn(kS16Tile, MP, 0, 0);      // A, B = f16
            uint32_t it = 0;
            int tl = 0;
            bool ok = true;
            for (int t = first_tile; t < sched.n_tiles && ok; t += tile_step, ++tl) {
                const int as = tl & 1;
                const uint32_t aph = (tl >> 1) & 1;
                if (s_abort || !mbar_wait(smem_u32(&bar_tempty[as]), aph ^ 1, p.status, kDevTimeoutTmemEmpty)) {
                    s_abort = 1; ok = false; break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * MP;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_conv[st]), ph, p.status, kDevTimeoutFull)) {
                        s_abort = 1; ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t xf = smem_base + st * Cfg::kStageBytes + kXfOff;
                    const uint32_t a_t = tmem_a0 + st * Cfg::kACols;
#pragma unroll
                    for (int k = 0; k < kS16KB / 16; ++k) {
                        // K = 16 f16 per MMA: 8 TMEM columns of A; 32 bytes inside the 128-byte swizzle
                        // span of the B half-tile (four steps per half)
                        const uint64_t db = make_smem_desc(xf + (k >> 2) * (MP * 128)) + 2 * (k & 3);
                        umma_f16_ts(d_tmem, a_t + k * 8, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bar_empty[st]));
                }
                if (ok) umma_commit(smem_u32(&bar_tfull[as]));
            }
        }
    } else if (warp < 2 + kS16ConvWarps) {
        // ================= converters (warps 2..9) =================
        const int team = (warp - 2) >> 2;                 // a ring slot always belongs to the same team
        const int q = warp & 3;                           // TMEM lane quarter this warp may write
        const int tt = ((warp - 2) & 3) * 32 + lane;      // 0..127 inside the team
        const int row = q * 32 + lane;                    // weight row (channel) of this lane
        const uint32_t wsw = (uint32_t)(row & 7);
        const int x_items = p.M * 16;                     // (row, 8-element chunk) pairs of the real rows
        uint32_t it = 0;
        bool ok = true;
        for (int t = first_tile; t < sched.n_tiles && ok; t += tile_step) {
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int st = it % S;
                if (st % kS16Teams != team) continue;
                const uint32_t ph = (it / S) & 1;
                if (!mbar_wait(smem_u32(&bar_full[st]), ph, p.status, kDevTimeoutFull)) { s_abort = 1; ok = false; break; }
                const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                // ---- weights: one 128-byte row per lane -> 64 f16x2 words -> TMEM
                uint32_t v[64];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint4 w;
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                                 : "r"(sa + row * 128 + (((uint32_t)c ^ wsw) << 4)));
                    v[8 * c + 0] = cvt_e4m3x2_to_f16x2((uint16_t)(w.x & 0xffff)); v[8 * c + 1] = cvt_e4m3x2_to_f16x2((uint16_t)(w.x >> 16));
                    v[8 * c + 2] = cvt_e4m3x2_to_f16x2((uint16_t)(w.y & 0xffff)); v[8 * c + 3] = cvt_e4m3x2_to_f16x2((uint16_t)(w.y >> 16));
                    v[8 * c + 4] = cvt_e4m3x2_to_f16x2((uint16_t)(w.z & 0xffff)); v[8 * c + 5] = cvt_e4m3x2_to_f16x2((uint16_t)(w.z >> 16));
                    v[8 * c + 6] = cvt_e4m3x2_to_f16x2((uint16_t)(w.w & 0xffff)); v[8 * c + 7] = cvt_e4m3x2_to_f16x2((uint16_t)(w.w >> 16));
                }
                __syncwarp();
                tmem_st64(tmem_a0 + st * Cfg::kACols + ((uint32_t)(q * 32) << 16), v);
                // ---- activations: bf16 -> f16 into the two swizzled half-tiles
                const uint32_t xf = sa + kXfOff, xr = sa + kXrawOff;
                for (int i = tt; i < x_items; i += 128) {
                    const int m = i >> 4, c16 = i & 15;
                    uint4 a;
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w)
                                 : "r"(xr + m * 256 + c16 * 16));
                    const uint4 h = bf16x8_to_f16x8(a);
                    const uint32_t dst = xf + (c16 >> 3) * (MP * 128) + m * 128 + ((((uint32_t)c16 & 7) ^ (uint32_t)(m & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(h.x), "r"(h.y), "r"(h.z), "r"(h.w) : "memory");
                }
                fence_async_smem();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_conv[st]));
            }
        }
    } else {
        // ================= epilogue (warps 10..13) =================
        pdl_wait();
        const int q = warp & 3;
        int tl = 0;
        bool ok = true;
        for (int t = first_tile; t < sched.n_tiles && ok; t += tile_step, ++tl) {
            const int as = tl & 1;
            const uint32_t aph = (tl >> 1) & 1;
            const int n = t * kS16Tile + q * 32 + lane;
            float ws = 0.f, bs = 0.f;
            if (!kSplit && n < p.N) {
                ws = __ldg(p.w_scale + n);
                if (p.bias) bs = __bfloat162float(p.bias[n]);
            }
            if (!mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull)) { s_abort = 1; ok = false; break; }
            tc_fence_after();
            uint32_t v[MP];
            __syncwarp();
            s16_tmem_ld<MP>(tmem_base + ((uint32_t)(q * 32) << 16) + as * MP, v);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
            if (!kSplit) {
                if (n < p.N) {
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < p.M) p.y[(size_t)m * p.ldy + n] = __float2bfloat16_rn(fmaf(__uint_as_float(v[m]), ws, bs));
                }
            } else {
                // this CTA's ring is free: tell every peer, wait for all of them, push each channel's sums to its owner
                cluster_wait();
                if (q == 0 && lane < sched.splits) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_ready), (uint32_t)lane));
                if (!mbar_wait(smem_u32(&bar_ready), 0, p.status, kDevTimeoutPeer)) { s_abort = 1; ok = false; break; }
                const int c = q * 32 + lane;
                const uint32_t owner = (uint32_t)(c / band);
                const uint32_t dst = map_to_cta(smem_base + (uint32_t)(split_rank * band + (c - (int)owner * band)) * Cfg::kPartPitch, owner);
                const uint32_t rbar = map_to_cta(smem_u32(&bar_recv), owner);
#pragma unroll
                for (int m = 0; m < MP; m += 4)
                    if (m < p.M) st_async_v4(dst + m * 4, v[m], v[m + 1], v[m + 2], v[m + 3], rbar);
            }
        }
    }

    if constexpr (kSplit) {
        // ---- this CTA finishes its band: slices added in rank order, scaled, stored ----
        __syncwarp();
        if (warp < 2 + kS16ConvWarps) cluster_wait();        // (the epilogue warps did before their first remote access)
        if (warp == 1) {                                     // the accumulator has been read by the four epilogue warps
            mbar_wait(smem_u32(&bar_tempty[0]), 0, p.status, kDevTimeoutTmemEmpty);
            __syncwarp();
            tc_fence_after();
            tmem_dealloc(tmem_base, Cfg::kTmemCols);
        }
        pdl_wait();
        if ((int)threadIdx.x >= band_rows * m_groups) return;
        if (s_abort || !mbar_wait(smem_u32(&bar_recv), 0, p.status, kDevTimeoutPeer)) return;
        const uint32_t slice = (uint32_t)band * Cfg::kPartPitch;
        for (int i = threadIdx.x; i < band_rows * m_groups; i += kS16Threads) {
            const int rl = i % band_rows;
            const int mg = (i / band_rows) * 4;
            const int n = first_tile * kS16Tile + split_rank * band + rl;
            if (n >= p.N) continue;
            const uint32_t local = smem_base + (uint32_t)rl * Cfg::kPartPitch + (uint32_t)mg * 4;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) {
                if (sl < sched.splits) {
                    const float4 u = ld_shared_f4(local + (uint32_t)sl * slice);
                    a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
                }
            }
            const bool first = i == (int)threadIdx.x;
            const float ws = first ? ws0 : __ldg(p.w_scale + n);
            const float bs = first ? bs0 : (p.bias ? __bfloat162float(p.bias[n]) : 0.f);
            const float o[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (mg + j < p.M) p.y[(size_t)(mg + j) * p.ldy + n] = __float2bfloat16_rn(fmaf(o[j], ws, bs));
        }
        return;
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
static bool encode_x_bf16_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                               uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)kS16KB, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int MP>
static int swap16_max_clusters(int cluster) {
    return max_active_clusters((const void*)swap_w8a16_kernel<MP, true>, kS16Threads, Swap16Cfg<MP>::kSmemBytes, cluster);
}

SwapPlan plan_swap_w8a16(int64_t M, int64_t K, int64_t N, int force_splits) {
    SwapPlan pl{};
    pl.preq = 0;
    pl.mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    pl.n_tiles = (int)((N + kS16Tile - 1) / kS16Tile);
    const int kblocks = (int)((K + kS16KB - 1) / kS16KB);
    int best_s = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= 8; ++s) {
        if (force_splits > 0 && s != (force_splits > 8 ? 8 : force_splits)) continue;
        if (s > kblocks) break;
        if (force_splits <= 0 && s > 1 && kblocks / s < 4) break;
        const int kps = (kblocks + s - 1) / s;
        if ((kblocks + kps - 1) / kps != s) continue;
        int slots = sm_count();
        if (s > 1) slots = pl.mp == 16 ? swap16_max_clusters<16>(s) : (pl.mp == 32 ? swap16_max_clusters<32>(s) : swap16_max_clusters<64>(s));
        if (slots < 1) slots = 1;
        // microseconds per wave of clusters, as in plan_swap; a CTA alone is bound by the widening of its weight
        // tiles (0.52 us per 16 KB block), and waves do not overlap
        const int ctas = pl.n_tiles * s;
        const int resident = ctas < slots * s ? ctas : slots * s;
        const double shared = 16384.0 * resident / 6.5e6;
        const double t_block = shared > 0.52 ? shared : 0.52;
        const int waves = (pl.n_tiles + slots - 1) / slots;
        const double fixed = 3.5 + (s > 1 ? 0.5 + (0.1 + 0.006 * (double)M) * s : 0.0);
        const double cost = waves * (kps * t_block + fixed);
        if (cost < best_cost) { best_cost = cost; best_s = s; }
    }
    pl.splits = best_s;
    pl.kblocks_per_split = (kblocks + best_s - 1) / best_s;
    pl.grid = pl.splits > 1 ? pl.n_tiles * pl.splits : (pl.n_tiles < sm_count() ? pl.n_tiles : sm_count());
    return pl;
}

template <int MP, bool kSplit>
static cudaError_t launch_swap16(const SwapPlan& pl, const UmmaArgs& a, const CUtensorMap& tw, const CUtensorMap& tx,
                                 cudaStream_t stream) {
    using Cfg = Swap16Cfg<MP>;
    auto kern = swap_w8a16_kernel<MP, kSplit>;
    static SmemOptIn opted;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, Cfg::kSmemBytes, opted);
        if (e != cudaSuccess) return e;
    }
    Swap16Sched s;
    s.n_tiles = pl.n_tiles; s.splits = pl.splits;
    s.kblocks_total = (a.K + kS16KB - 1) / kS16KB; s.kblocks_per_split = pl.kblocks_per_split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.grid);
    cfg.blockDim = dim3(kS16Threads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = pdl_attribute(attr);
    if (kSplit) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)pl.splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return counted(cudaLaunchKernelEx(&cfg, kern, tw, tx, a, s));
}

cudaError_t launch_swap_w8a16(const SwapPlan& pl, const UmmaArgs& a, const void* x, int64_t ldx, cudaStream_t stream,
                              const char** why) {
    CUtensorMap tw, tx;
    if (!encode_u8_2d(&tw, a.w, (uint64_t)(pack_ntiles(a.N) * pack_kblocks(a.K) * 128), 128, kS16Tile) ||
        !encode_x_bf16_rows(&tx, x, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)ldx * 2, (uint32_t)a.M)) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    const bool split = pl.splits > 1;
    switch (pl.mp) {
        case 16: return split ? launch_swap16<16, true>(pl, a, tw, tx, stream) : launch_swap16<16, false>(pl, a, tw, tx, stream);
        case 32: return split ? launch_swap16<32, true>(pl, a, tw, tx, stream) : launch_swap16<32, false>(pl, a, tw, tx, stream);
        case 64: return split ? launch_swap16<64, true>(pl, a, tw, tx, stream) : launch_swap16<64, false>(pl, a, tw, tx, stream);
    }
    if (why) *why = "unsupported token-tile width";
    return cudaErrorInvalidValue;
}

}  // namespace fp8lin
