// Decode-sized W8A8 linear (M <= 64) on tcgen05 with the operands swapped:
//
//   y^T[N, M] = W[N, K] . xq[M, K]^T        (weights are the 128-row MMA "A" operand,
//                                            the few tokens are the MMA "N" dimension)
//
// HBM-bound: the kernel exists to keep as many weight bytes in flight per SM as
// shared memory allows.  Algorithmic bytes per call: K*N + 2*M*K + 2*M*N + 6*N.
//
//   warp 0       TMA producer.  Per 128-byte K block: one 128 x 128-byte weight
//                tile (128-byte swizzle) and the raw bf16 activation block
//                [MP x 128] into a ring of 5..9 stages (144..80 KB of weights in
//                flight per SM).
//   warps 2..9   activation converters in teams of 1, 2, 4 or 8 warps (one lane per 16 elements
//                of the real rows, so a block is converted in one step: the first block's
//                conversion is on the critical path of every call), one ring slot per
//                team (several K blocks are converted concurrently): quantise the M real rows of
//                the raw block to e4m3 with the static scale (exact division)
//                and write them into the K-major, 128-byte-swizzled MMA "B"
//                tile (rows M..MP-1 stay zero); fence.proxy.async; arrive.
//   warp 1       MMA issuer: tcgen05.mma.cta_group::1.kind::f8f6f4, M=128, N=MP,
//                K=32, four per K block, fp32 accumulators in TMEM (2 stages).
//   warps 10..13 epilogue: tcgen05.ld one output channel per lane, MP tokens per
//                lane; y[m][n] = bf16(acc*in_scale*w_scale[n] + bias[n]); the 32
//                lanes of a warp write 32 consecutive channels of one token.
//
// Launch shapes: persistent over the N/128 channel tiles, or, when there are too
// few tiles to occupy 148 SMs, cluster split-K: the CTAs of a cluster (2..8)
// take K slices of one tile and each finishes a band of channels.  A CTA whose
// MMAs are done tells every peer that its ring is free (remote mbarrier arrive);
// the epilogue lanes then push their fp32 partials of band r straight into CTA r's
// ring with st.async, which counts the bytes on CTA r's barrier; CTA r adds the
// slices in rank order (deterministic), writes y and leaves -- no cluster-wide
// barrier after set-up, no remote loads.  All mbarrier waits are bounded.
#include "umma_common.cuh"

namespace fp8lin {

constexpr int kConvWarps = 8;
constexpr int kSwapThreads = (2 + kConvWarps + 4) * 32;
constexpr int kTileN = 128;   // output channels per tile = MMA M
constexpr int kKB = 128;      // K elements per block

// kPreQ: the activations were quantised by a pass before the kernel and arrive as ready MMA "B"
// tiles by TMA; no raw block, no converter work, so more ring slots fit (used for 33..64 rows,
// where the raw block would leave only five slots).
// kGateUp (16-row tiles, pre-quantised rows): the weights are a gate_up projection with its 128-channel tile rows
// alternating gate / up.  Clusters of two CTAs take tile PAIRS: CTA 0 the gate tile, CTA 1 the up tile.  The up CTA's
// epilogue sends its bf16 results to the gate CTA (st.async into a 4 KB buffer behind the ring, counted on a barrier
// of the gate CTA, one barrier per epilogue warp), and the gate CTA writes e4m3 h = silu(gate) * up for the down
// projection instead of y.  Still two CTAs per SM: the ring is one slot shorter to make room for the buffer.
template <int MP, bool kPreQ = false, bool kGateUp = false>
struct SwapCfg {
    static constexpr int kWBytes = kTileN * kKB;                 // 16 KB e4m3 weight tile
    static constexpr int kXqBytes = MP * kKB;                    // quantised activation tile (MMA B)
    static constexpr int kXrawBytes = kPreQ ? 0 : MP * kKB * 2;  // raw bf16 activation block
    static constexpr int kStageBytes = kWBytes + kXqBytes + kXrawBytes;
    // M <= 16: two CTAs share an SM (5 stages each, 160 KB of weights in flight per SM), so the
    // CTAs of the next kernel can start on an SM while this kernel's other CTA is still draining
    static constexpr int kCtasPerSm = MP <= 16 ? 2 : 1;
    static constexpr int kStages = kGateUp ? 5 : (kPreQ ? (MP <= 16 ? 6 : 9) : (MP <= 16 ? 5 : (MP <= 32 ? 7 : 5)));
    static constexpr int kRecvBytes = kGateUp ? kTileN * MP * 2 : 0;   // bf16 [channel][row] from the up CTA
    static_assert(!kGateUp || (kPreQ && MP == 16), "the gate_up form exists for 16-row tiles of pre-quantised rows");
    static constexpr int kRingBytes = kStages * kStageBytes;
    static constexpr int kSmemBytes = kRingBytes + 1024 + kRecvBytes;
    static constexpr int kTmemCols = 2 * MP < 32 ? 32 : 2 * MP;
    static constexpr int kPartPitch = MP * 4 + 16;               // row pitch of the received fp32 partial sums (split-K)
    static_assert(kStageBytes % 1024 == 0, "stages must keep 1024-byte alignment for the swizzle");
    static_assert((kTileN + 8) * kPartPitch <= kRingBytes, "the received slices of a band must fit in the ring");
};

struct SwapSched {
    int n_tiles, splits, kblocks_total, kblocks_per_split;
};

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* v);
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t* v) { tmem_ld32_nowait(taddr, v); }
template <>
__device__ __forceinline__ void tmem_ld_cols<64>(uint32_t taddr, uint32_t* v) {
    tmem_ld32_nowait(taddr, v);
    tmem_ld32_nowait(taddr + 32, v + 32);
}

// converter warps that share one K block: one lane per (row, 16-element chunk) of the M real rows
__host__ __device__ inline int conv_team(int m) { return m <= 4 ? 1 : (m <= 8 ? 2 : (m <= 16 ? 4 : 8)); }

template <int MP, bool kSplit, bool kPreQ = false, bool kGateUp = false>
__global__ void __launch_bounds__(kSwapThreads, SwapCfg<MP, kPreQ, kGateUp>::kCtasPerSm)
swap_w8a8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 UmmaArgs p, SwapSched sched) {
    static_assert(!(kGateUp && kSplit), "tile pairs are not split along K");
    __shared__ __align__(8) uint64_t bar_up[4];       // gate CTA: the up values of epilogue warp q's channels have landed
    __shared__ __align__(8) uint64_t bar_free[4];     // up CTA: the gate CTA has read warp q's values (buffer reusable)
    using Cfg = SwapCfg<MP, kPreQ, kGateUp>;
    // bytes of activations one K block brings in: M real rows, raw bf16 or ready e4m3
    const uint32_t x_bytes = (uint32_t)p.M * (kPreQ ? 128u : 256u);
    constexpr uint32_t kXDst = Cfg::kWBytes + (kPreQ ? 0 : Cfg::kXqBytes);   // where the TMA puts them
    constexpr int S = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[S];     // TMA bytes landed (weights + raw x)
    __shared__ __align__(8) uint64_t bar_xq[S];       // quantised x tile written (one converter warp)
    __shared__ __align__(8) uint64_t bar_empty[S];    // MMAs that read the stage are done
    __shared__ __align__(8) uint64_t bar_tfull[2];
    __shared__ __align__(8) uint64_t bar_tempty[2];
    __shared__ __align__(8) uint64_t bar_ready;       // split-K: every CTA of the cluster is past its MMAs (its ring may be written)
    __shared__ __align__(8) uint64_t bar_recv;        // split-K: the partials of this CTA's band have landed
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int split_rank = kSplit ? (int)cluster_ctarank() : 0;
    const int pair_rank = kGateUp ? (int)cluster_ctarank() : 0;                  // gate_up form: 0 = gate tile, 1 = up tile
    const int first_tile = kSplit ? (int)(blockIdx.x / sched.splits) : (kGateUp ? (int)(blockIdx.x & ~1u) + pair_rank : (int)blockIdx.x);
    const int tile_step = kSplit ? sched.n_tiles : (int)gridDim.x;
    // the tl-th tile of this CTA: every gridDim.x-th tile (gate_up form: this CTA's half of every (gridDim.x / 2)-th pair)
    auto tile_of = [&](int tl) -> int { return first_tile + tl * tile_step; };
    const uint32_t recv_bytes_warp = 32u * (uint32_t)((p.M + 7) >> 3) * 16u;      // what one up warp sends per pair
    const int kb0 = split_rank * sched.kblocks_per_split;
    const int kb1 = kSplit ? min(sched.kblocks_total, kb0 + sched.kblocks_per_split) : sched.kblocks_total;
    // split-K: CTA r of the cluster finishes channels [r * band, r * band + band_rows) of the tile; a slice's partials
    // of one channel are MP floats kPartPitch bytes apart, the slices of a band follow each other in the owner's ring
    const int band = kSplit ? (kTileN + sched.splits - 1) / sched.splits : kTileN;
    const int band_rows = kSplit ? min(kTileN, (split_rank + 1) * band) - split_rank * band : 0;
    const int m_groups = (p.M + 3) >> 2;                          // rows travel in groups of four

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(smem_u32(&bar_full[i]), 1);
            mbar_init(smem_u32(&bar_xq[i]), conv_team(p.M));
            mbar_init(smem_u32(&bar_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bar_tfull[i]), 1); mbar_init(smem_u32(&bar_tempty[i]), 4); }
        s_abort = 0;
        if (kGateUp) {
            for (int i = 0; i < 4; ++i) {
                mbar_init(smem_u32(&bar_up[i]), 1);
                mbar_init(smem_u32(&bar_free[i]), 1);
                if (pair_rank == 0) mbar_expect_tx(smem_u32(&bar_up[i]), recv_bytes_warp);
            }
        }
        if (kSplit) {
            mbar_init(smem_u32(&bar_ready), (uint32_t)sched.splits);
            mbar_init(smem_u32(&bar_recv), 1);
            mbar_expect_tx(smem_u32(&bar_recv), (uint32_t)(sched.splits * band_rows * m_groups * 16));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), Cfg::kTmemCols);
    // rows M..MP-1 of every quantised-activation tile are zero for the whole kernel
    for (int i = threadIdx.x; i < S * MP * 8; i += kSwapThreads) {
        const int st = i / (MP * 8), r = i % (MP * 8);
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(smem_base + st * Cfg::kStageBytes + Cfg::kWBytes + r * 16), "r"(0u) : "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    pdl_launch_dependents();
    if (kSplit || kGateUp) cluster_arrive();                 // (waited for before the first remote access: the peers' barriers exist)
    // scale and bias of the first channel this thread finishes, fetched long before they are needed
    float ws0 = 0.f, bs0 = 0.f, in_scale0 = 0.f;
    if constexpr (kSplit) {
        in_scale0 = fmaxf(__ldg(p.input_scale), 1e-12f);
        if (band_rows > 0 && (int)threadIdx.x < band_rows * m_groups) {
            const int n0 = first_tile * kTileN + split_rank * band + (int)threadIdx.x % band_rows;
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
            // First pass over the ring: the weight tiles go out at once; the activation blocks
            // follow when the predecessor kernel (which may be producing x) has finished.
            const int first_kb = min(kb1 - kb0, S);
            if (first_tile < sched.n_tiles) {
                for (int i = 0; i < first_kb; ++i) {
                    const uint32_t full = smem_u32(&bar_full[i]);
                    mbar_expect_tx(full, Cfg::kWBytes + x_bytes);   // the x box holds the M real rows only
                    tma_load_2d(smem_base + i * Cfg::kStageBytes, &tmap_w, 0,
                                (first_tile * sched.kblocks_total + kb0 + i) * kTileN, full);   // one packed tile
                }
                pdl_wait();
                for (int i = 0; i < first_kb; ++i)
                    tma_load_2d(smem_base + i * Cfg::kStageBytes + kXDst, &tmap_x,
                                (kb0 + i) * kKB, 0, smem_u32(&bar_full[i]));
            }
            for (int tl = 0; ok; ++tl) {
                const int t = tile_of(tl);
                if (t >= sched.n_tiles) break;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    if (it < (uint32_t)first_kb) continue;                       // issued above
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t full = smem_u32(&bar_full[st]);
                    mbar_expect_tx(full, Cfg::kWBytes + x_bytes);
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    tma_load_2d(sa, &tmap_w, 0, (t * sched.kblocks_total + kb) * kTileN, full);
                    tma_load_2d(sa + kXDst, &tmap_x, kb * kKB, 0, full);
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
            constexpr uint32_t idesc = make_idesc_mn(kTileN, MP, 0, 0);
            uint32_t it = 0;
            bool ok = true;
            for (int tl = 0; ok; ++tl) {
                if (tile_of(tl) >= sched.n_tiles) break;
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
                    if (s_abort || !mbar_wait(smem_u32(&bar_full[st]), ph, p.status, kDevTimeoutFull) ||
                        (!kPreQ && !mbar_wait(smem_u32(&bar_xq[st]), ph, p.status, kDevTimeoutFull))) {
                        s_abort = 1; ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + Cfg::kWBytes);
#pragma unroll
                    for (int k = 0; k < kKB / 32; ++k)
                        umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&bar_empty[st]));
                }
                if (ok) umma_commit(smem_u32(&bar_tfull[as]));
            }
        }
    } else if (warp < 2 + kConvWarps) {
        // ================= activation converters (warps 2..9); idle when the rows come pre-quantised ====
        if (!kPreQ) {
        const int team_sz = conv_team(p.M);
        const int kTeams = kConvWarps / team_sz;
        const int team = (warp - 2) / team_sz;               // a ring slot always belongs to the same team
        const int member = (warp - 2) % team_sz;
        const ExactDiv div_scale(fmaxf(__ldg(p.input_scale), 1e-12f));
        const int items = p.M * 8;                          // (row, 16-element chunk) pairs of the real rows
        uint32_t it = 0;
        bool ok = true;
        for (int tl = 0; ok; ++tl) {
            if (tile_of(tl) >= sched.n_tiles) break;
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                // a ring slot always belongs to the same warp, so every warp sees the phases of
                // the barriers it waits on in order (a parity wait may only look one phase ahead)
                const int st = it % S;
                if (st % kTeams != team) continue;
                const uint32_t ph = (it / S) & 1;
                if (s_abort || !mbar_wait(smem_u32(&bar_full[st]), ph, p.status, kDevTimeoutFull)) { s_abort = 1; ok = false; break; }
                const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                const uint32_t xq = sa + Cfg::kWBytes;
                const uint32_t xr = xq + Cfg::kXqBytes;
                for (int i = member * 32 + lane; i < items; i += 32 * team_sz) {
                    const int m = i >> 3, c = i & 7;
                    uint4 a, b;
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w)
                                 : "r"(xr + m * 256 + c * 32));
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
                                 : "r"(xr + m * 256 + c * 32 + 16));
                    const uint2 qa = quant8_e4m3(a, div_scale);
                    const uint2 qb = quant8_e4m3(b, div_scale);
                    const uint32_t dst = xq + m * 128 + (((uint32_t)c ^ (uint32_t)(m & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(qa.x), "r"(qa.y), "r"(qb.x), "r"(qb.y)
                                 : "memory");
                }
                fence_async_smem();                          // generic-proxy writes -> visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_xq[st]));
            }
        }
        }
    } else {
        // ================= epilogue (warps 10..13) =================
        pdl_wait();                                          // y may still be read by the predecessor
        const int q = warp & 3;
        const float in_scale = fmaxf(__ldg(p.input_scale), 1e-12f);
        bool ok = true;
        if constexpr (kGateUp) {
            // ---- pairs of tiles: h = silu(gate) * up, quantised for the down projection ----
            const ExactDiv div_h(fmaxf(__ldg(p.h_scale), 1e-12f));
            const int inter = p.N >> 1;
            const int groups = (p.M + 7) >> 3;                                     // rows travel in groups of eight bf16
            const uint32_t recv = smem_base + Cfg::kRingBytes + (uint32_t)(q * 32 + lane) * (MP * 2);
            cluster_wait();
            for (int tl = 0; ok; ++tl) {
                const int t = tile_of(tl);
                if (t >= sched.n_tiles) break;
                const bool more = tile_of(tl + 1) < sched.n_tiles;
                const int as = tl & 1;
                const uint32_t aph = (tl >> 1) & 1;
                const int n = t * kTileN + q * 32 + lane;                           // (N is a multiple of 256: in range)
                const float ws = __ldg(p.w_scale + n);
                const float bs = p.bias ? __bfloat162float(p.bias[n]) : 0.f;
                uint32_t v[MP];
                if (!mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull)) { s_abort = 1; ok = false; break; }
                tc_fence_after();
                __syncwarp();
                tmem_ld_cols<MP>(tmem_base + ((uint32_t)(q * 32) << 16) + as * MP, v);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
                // this tile's values rounded to bf16, as the two-step form stores them
                uint32_t r[MP / 2];
#pragma unroll
                for (int m = 0; m < MP; m += 2)
                    r[m >> 1] = pack_bf16x2(fmaf(__uint_as_float(v[m]) * in_scale, ws, bs), fmaf(__uint_as_float(v[m + 1]) * in_scale, ws, bs));
                if (pair_rank == 1) {
                    // up tile: hand the values to the gate CTA (after it has read the previous pair's)
                    if (tl > 0 && !mbar_wait(smem_u32(&bar_free[q]), (uint32_t)((tl - 1) & 1), p.status, kDevTimeoutPeer)) { s_abort = 1; ok = false; break; }
                    const uint32_t dst = map_to_cta(recv, 0);
                    const uint32_t rbar = map_to_cta(smem_u32(&bar_up[q]), 0);
#pragma unroll
                    for (int gI = 0; gI < MP / 8; ++gI)
                        if (gI < groups) st_async_v4(dst + gI * 16, r[4 * gI], r[4 * gI + 1], r[4 * gI + 2], r[4 * gI + 3], rbar);
                } else {
                    if (!mbar_wait(smem_u32(&bar_up[q]), (uint32_t)(tl & 1), p.status, kDevTimeoutPeer)) { s_abort = 1; ok = false; break; }
                    uint32_t u[MP / 2];
#pragma unroll
                    for (int gI = 0; gI < MP / 8; ++gI) {
                        if (gI < groups)
                            asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(u[4 * gI]), "=r"(u[4 * gI + 1]), "=r"(u[4 * gI + 2]), "=r"(u[4 * gI + 3])
                                         : "r"(recv + gI * 16));
                        else u[4 * gI] = u[4 * gI + 1] = u[4 * gI + 2] = u[4 * gI + 3] = 0u;
                    }
                    __syncwarp();
                    if (more && lane == 0) {                                        // (no signal after the last pair: the up CTA may be gone)
                        mbar_expect_tx(smem_u32(&bar_up[q]), recv_bytes_warp);
                        mbar_arrive_cluster(map_to_cta(smem_u32(&bar_free[q]), 1));
                    }
                    // the values and roundings of the two-step form: bf16(silu(g) * u) from bf16 g and u, then the quantiser
                    unsigned char* hcol = p.hq + (size_t)(t >> 1) * kTileN + q * 32 + lane;
#pragma unroll
                    for (int gI = 0; gI < MP / 8; ++gI) {
                        if (gI >= groups) break;
                        uint4 hv;
                        uint32_t* hw = reinterpret_cast<uint32_t*>(&hv);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t gp = r[4 * gI + j], up = u[4 * gI + j];
                            const float g0 = bf16_lo(gp), g1 = bf16_hi(gp);
                            const float s0 = g0 / (1.f + expf(-g0)), s1 = g1 / (1.f + expf(-g1));
                            hw[j] = pack_bf16x2(s0 * bf16_lo(up), s1 * bf16_hi(up));
                        }
                        const uint2 qd = quant8_e4m3(hv, div_h);
#pragma unroll
                        for (int rr = 0; rr < 8; ++rr)
                            if (gI * 8 + rr < p.M) hcol[(size_t)(gI * 8 + rr) * inter] = (unsigned char)(((rr < 4 ? qd.x : qd.y) >> (8 * (rr & 3))) & 0xffu);
                    }
                }
            }
        } else
        for (int tl = 0; ok; ++tl) {
            const int t = tile_of(tl);
            if (t >= sched.n_tiles) break;
            const int as = tl & 1;
            const uint32_t aph = (tl >> 1) & 1;
            const int n = t * kTileN + q * 32 + lane;
            float ws = 0.f, bs = 0.f;
            if (!kSplit && n < p.N) {
                ws = __ldg(p.w_scale + n);
                if (p.bias) bs = __bfloat162float(p.bias[n]);
            }
            if (!mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull)) { s_abort = 1; ok = false; break; }
            tc_fence_after();
            uint32_t v[MP];
            __syncwarp();
            tmem_ld_cols<MP>(tmem_base + ((uint32_t)(q * 32) << 16) + as * MP, v);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
            if (!kSplit) {
                if (n < p.N) {
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < p.M) p.y[(size_t)m * p.ldy + n] = __float2bfloat16_rn(fmaf(__uint_as_float(v[m]) * in_scale, ws, bs));
                }
            } else {
                // (one tile per cluster)  Tell every peer that this CTA's ring is free, wait until all of them are,
                // then send each channel's partial sums to the CTA that finishes it.
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
        if (warp < 2 + kConvWarps) cluster_wait();           // (the epilogue warps did before their first remote access)
        if (warp == 1) {                                     // the accumulator has been read by the four epilogue warps
            mbar_wait(smem_u32(&bar_tempty[0]), 0, p.status, kDevTimeoutTmemEmpty);
            __syncwarp();
            tc_fence_after();
            tmem_dealloc(tmem_base, Cfg::kTmemCols);
        }
        pdl_wait();
        if ((int)threadIdx.x >= band_rows * m_groups) return;
        if (s_abort || !mbar_wait(smem_u32(&bar_recv), 0, p.status, kDevTimeoutPeer)) return;
        const float in_scale = in_scale0;
        const uint32_t slice = (uint32_t)band * Cfg::kPartPitch;
        // consecutive threads take consecutive channels, so the stores of one token coalesce
        for (int i = threadIdx.x; i < band_rows * m_groups; i += kSwapThreads) {
            const int rl = i % band_rows;
            const int mg = (i / band_rows) * 4;
            const int n = first_tile * kTileN + split_rank * band + rl;
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
                if (mg + j < p.M) p.y[(size_t)(mg + j) * p.ldy + n] = __float2bfloat16_rn(fmaf(o[j] * in_scale, ws, bs));
        }
        return;
    }

    if constexpr (kGateUp) {
        __syncwarp();
        if (warp < 2 + kConvWarps) cluster_wait();           // (the epilogue warps did before their first remote access)
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

// raw bf16 activations [M][ldx]: box = 128 elements x box_rows, no swizzle; rows past M read as zero
static bool encode_x_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                          uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)kKB, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int MP, bool kPreQ>
static int swap_max_clusters(int cluster) {
    using Cfg = SwapCfg<MP, kPreQ>;
    const void* kern = (const void*)swap_w8a8_kernel<MP, true, kPreQ>;
    return max_active_clusters(kern, kSwapThreads, Cfg::kSmemBytes, cluster);
}

SwapPlan plan_swap(int64_t M, int64_t K, int64_t N, int force_splits, bool preq) {
    SwapPlan pl{};
    pl.preq = preq ? 1 : 0;
    pl.mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    pl.n_tiles = (int)((N + kTileN - 1) / kTileN);
    const int kblocks = (int)((K + kKB - 1) / kKB);
    int best_s = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= 8; ++s) {
        if (force_splits > 0 && s != (force_splits > 8 ? 8 : force_splits)) continue;
        if (s > kblocks) break;
        // at least four K blocks per slice -- two when every cluster is resident at one CTA per SM (a 4 MB layer such as
        // 2048 -> 2048 at one row: 4.4 us with 8 slices of 2 blocks against 5.8 us with 4 slices of 4)
        const int min_blocks = (pl.n_tiles * s <= sm_count()) ? 2 : 4;
        if (force_splits <= 0 && s > 1 && kblocks / s < min_blocks) break;
        const int kps = (kblocks + s - 1) / s;
        if ((kblocks + kps - 1) / kps != s) continue;                        // would leave an empty slice
        int slots = sm_count() * (pl.mp == 16 ? 2 : 1);
        if (s > 1) {
            if (preq) slots = pl.mp == 16 ? swap_max_clusters<16, true>(s) : (pl.mp == 32 ? swap_max_clusters<32, true>(s) : swap_max_clusters<64, true>(s));
            else slots = pl.mp == 16 ? swap_max_clusters<16, false>(s) : (pl.mp == 32 ? swap_max_clusters<32, false>(s) : swap_max_clusters<64, false>(s));
        }
        // The occupancy query answers as if one CTA had an SM to itself (74 clusters of two, 15 of eight) whatever the
        // kernel's shared memory; two CTAs of the 16-row kernel do share an SM (86 clusters of two run as one wave:
        // 7.9 us against 10.9 us unsplit on 2048 -> 11008), so for that kernel the figure is doubled.
        if (s > 1 && pl.mp == 16) slots *= 2;
        if (slots < 1) slots = 1;
        // Time of one wave of clusters, in microseconds: the K blocks of a slice at the rate the resident CTAs share
        // the HBM stream (a CTA alone is bound by its ring and the MMA issue rate: 0.32 us per 16 KB block, more with
        // wider token tiles), plus what every wave pays once -- ramp, the hand-over of the partial sums (grows with
        // rows x slices), drain.  A wave does not overlap the next: 86 tiles x 3 slices of 64-row tiles in two waves
        // took 19.3 us where one wave of unsplit tiles takes 11.0.  Fitted to a sweep of all slice counts over
        // 3584 -> 4608 / 3584 / 9472 / 18944, 2048 -> 11008 / 5632, 4736 / 11008 / 18944 -> 2048 or 3584 at 1, 16, 64 rows.
        const int ctas = pl.n_tiles * s;
        const int resident = ctas < slots * s ? ctas : slots * s;
        // (rows converted inside the kernel add to a lone CTA's block time: 0.45 us at 16 rows)
        const double alone = (pl.mp == 16 ? 0.32 : (pl.mp == 32 ? 0.36 : 0.40)) + (preq ? 0.0 : 0.008 * (double)(M < 16 ? M : 16));
        const double shared = 16384.0 * resident / 6.5e6;
        const double t_block = shared > alone ? shared : alone;
        const int waves = (pl.n_tiles + slots - 1) / slots;
        const double fixed = 3.5 + (s > 1 ? 0.5 + (0.1 + 0.006 * (double)M) * s : 0.0);
        const double cost = waves * (kps * t_block + fixed);
        if (cost < best_cost) { best_cost = cost; best_s = s; }
    }
    // Long K over few channel tiles (18944 -> 3584: 28 tiles x 148 K blocks), two CTAs per SM: measured
    // 20.0 / 19.1 / 18.3 us with 6 / 7 / 8 slices although fewer 8-CTA clusters are resident at once --
    // shorter slices ramp and drain faster than the wave model above credits.  Take the most slices
    // that still leave 16 K blocks each.
    if (force_splits <= 0 && pl.mp == 16 && kblocks >= 64 && pl.n_tiles * 8 <= 2 * sm_count()) {
        for (int s = 8; s > best_s; --s) {
            const int kps = (kblocks + s - 1) / s;
            if (kps >= 16 && (kblocks + kps - 1) / kps == s) { best_s = s; break; }
        }
    }
    pl.splits = best_s;
    pl.kblocks_per_split = (kblocks + best_s - 1) / best_s;
    const int resident = sm_count() * (pl.mp == 16 ? 2 : 1);
    pl.grid = pl.splits > 1 ? pl.n_tiles * pl.splits : (pl.n_tiles < resident ? pl.n_tiles : resident);
    return pl;
}

template <int MP, bool kSplit, bool kPreQ>
static cudaError_t launch_swap(const SwapPlan& pl, const UmmaArgs& a, const CUtensorMap& tw, const CUtensorMap& tx,
                               cudaStream_t stream) {
    using Cfg = SwapCfg<MP, kPreQ>;
    auto kern = swap_w8a8_kernel<MP, kSplit, kPreQ>;
    static SmemOptIn opted;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, Cfg::kSmemBytes, opted);
        if (e != cudaSuccess) return e;
    }
    SwapSched s;
    s.n_tiles = pl.n_tiles; s.splits = pl.splits;
    s.kblocks_total = (a.K + kKB - 1) / kKB; s.kblocks_per_split = pl.kblocks_per_split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.grid);
    cfg.blockDim = dim3(kSwapThreads);
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

cudaError_t launch_swap_gate_up(const UmmaArgs& a, cudaStream_t stream, const char** why) {
    using Cfg = SwapCfg<16, true, true>;
    if (a.M < 1 || a.M > 16 || a.N % 256 != 0 || !a.hq || !a.h_scale || !a.xq) {
        if (why) *why = "the gate_up form takes 1..16 pre-quantised rows and an even number of 128-channel tiles";
        return cudaErrorInvalidValue;
    }
    CUtensorMap tw, tx;
    bool ok = encode_u8_2d(&tw, a.w, (uint64_t)(pack_ntiles(a.N) * pack_kblocks(a.K) * 128), 128, kTileN);
    ok = ok && encode_u8_2d(&tx, a.xq, (uint64_t)a.M, (uint64_t)a.K, (uint32_t)a.M);
    if (!ok) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    auto kern = swap_w8a8_kernel<16, false, true, true>;
    static SmemOptIn opted;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, Cfg::kSmemBytes, opted);
        if (e != cudaSuccess) return e;
    }
    SwapSched s;
    s.n_tiles = (int)pack_ntiles(a.N); s.splits = 1;
    s.kblocks_total = (a.K + kKB - 1) / kKB; s.kblocks_per_split = s.kblocks_total;
    const int pairs = s.n_tiles / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * (pairs < sm_count() ? pairs : sm_count())));     // two CTAs per SM, one pair per cluster
    cfg.blockDim = dim3(kSwapThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = pdl_attribute(attr);
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return counted(cudaLaunchKernelEx(&cfg, kern, tw, tx, a, s));
}

cudaError_t launch_swap_w8a8(const SwapPlan& pl, const UmmaArgs& a, const void* x, int64_t ldx, cudaStream_t stream,
                             const char** why) {
    CUtensorMap tw, tx;
    bool ok = encode_u8_2d(&tw, a.w, (uint64_t)(pack_ntiles(a.N) * pack_kblocks(a.K) * 128), 128, kTileN);
    if (pl.preq) ok = ok && encode_u8_2d(&tx, a.xq, (uint64_t)a.M, (uint64_t)a.K, (uint32_t)a.M);      // ready e4m3 rows
    else ok = ok && encode_x_bf16(&tx, x, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)ldx * 2, (uint32_t)a.M);
    if (!ok) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    const bool split = pl.splits > 1;
#define FP8LIN_SWAP_CASE(MP_)                                                                                   \
    if (pl.mp == MP_) {                                                                                         \
        if (pl.preq) return split ? launch_swap<MP_, true, true>(pl, a, tw, tx, stream) : launch_swap<MP_, false, true>(pl, a, tw, tx, stream); \
        return split ? launch_swap<MP_, true, false>(pl, a, tw, tx, stream) : launch_swap<MP_, false, false>(pl, a, tw, tx, stream);            \
    }
    FP8LIN_SWAP_CASE(16)
    FP8LIN_SWAP_CASE(32)
    FP8LIN_SWAP_CASE(64)
#undef FP8LIN_SWAP_CASE
    if (why) *why = "unsupported token-tile width";
    return cudaErrorInvalidValue;
}

}  // namespace fp8lin
