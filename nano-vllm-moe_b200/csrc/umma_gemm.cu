// Large- and mid-M W8A8 linear on the 5th-generation tensor cores (sm_100a).
//
//   y[M,N] = bf16( (xq[M,K] . W[N,K]^T) * in_scale * w_scale[n] + bias[n] )
//
// Warp-specialised kernel, one CTA per SM, 10 warps:
//   warp 0      TMA producer: cp.async.bulk.tensor.2d loads of a 128 x 128-byte
//               xq tile and a BN x 128-byte weight tile per K block into a
//               multi-stage shared-memory ring (128-byte swizzle), signalled by
//               mbarrier complete_tx; every CTA issues its own loads.
//   warp 1      MMA issuer: one lane issues tcgen05.mma.cta_group::1
//               .kind::f8f6f4 (M=128, N=BN, K=32) four times per K block,
//               accumulating in TMEM; tcgen05.commit releases the ring slot
//               and, after the last K block, publishes the accumulator.
//   warps 2..9  epilogue: two warps per 32-lane quarter of TMEM, each taking
//               half of the tile's columns: tcgen05.ld 64 columns, one FMA per
//               element with in_scale*w_scale[n] and bias[n] staged in shared
//               memory, one rounding to bf16, swizzled staging box, TMA store
//               (which clips the M and N tails).
//
// Two launch shapes:
//  * persistent (kSplit = false): grid = min(tiles, SMs); two accumulator
//    stages in TMEM let the epilogue of tile i overlap the main loop of tile
//    i+1.  Tensor-bound: 2*M*K*N flops per call.
//  * cluster split-K (kSplit = true): for shapes with few output tiles and a
//    long K, the CTAs of a thread-block cluster (2..8) each run one K slice of
//    the same tile, park their fp32 accumulators in their own shared memory and,
//    after a cluster barrier, every CTA sums one band of rows across the
//    cluster's shared memories (ld.shared::cluster, fixed order, deterministic),
//    applies the epilogue and stores.  No global scratch, no counters.
//    HBM/L2-bound: K*N + M*K + 2*M*N bytes per call.
//
// Every mbarrier wait is bounded: a barrier that does not flip within about a
// second records a status code in the caller's scratch header and the CTA
// unwinds (drains its ring, frees TMEM) instead of hanging the GPU.
#include <stdio.h>
#include <stdlib.h>

#include "umma_common.cuh"

namespace fp8lin {

constexpr int kBM = 128;
constexpr int kBK = 128;  // bytes == e4m3 elements per K block
constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + kEpiWarps) * 32;

template <int BN>
struct UmmaCfg {
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBBytes = BN * kBK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 5 : 8);   // ring + staging + statics <= 227 KB
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kRingBytes = kStages * kStageBytes;
    // columns per TMEM read / staging box of an epilogue warp: 64 bf16 = one full 128-byte line per
    // row (32-column boxes wrote every line in two halves, and DRAM write traffic was 2.8x the output)
    static constexpr int kPiece = BN / 2 < 64 ? BN / 2 : 64;
    static constexpr int kBoxBytes = 32 * kPiece * 2;
    // One 32-row staging box per epilogue warp; the 256-wide tile has one per warp PAIR (the two warps that
    // own the same 32 rows fill the two 32-column halves of a 64-column box).  With a box per warp the CTA
    // came within 400 bytes of the SM's shared memory, no CTA of the preceding kernel could stay resident
    // beside it, and the overlap of programmatic dependent launch was lost (measured 2-8 % per call).
    static constexpr bool kPairBox = BN == 256;
    static constexpr int kStagingBytes = (kPairBox ? kEpiWarps / 2 : kEpiWarps) * kBoxBytes;
    static constexpr int kSmemBytes = kRingBytes + kStagingBytes + 1024;
    // split-K: fp32 tile parked over the (then idle) ring; 16 bytes of padding per row
    // spread consecutive rows over the banks
    static constexpr int kPartPitch = BN * 4 + 16;
    static_assert(kBM * kPartPitch <= kRingBytes, "parked tile must fit in the ring");
};

template <int BN>
__host__ __device__ constexpr uint32_t make_idesc() {
    return (1u << 4)                     // accumulator fp32
           | (0u << 7) | (0u << 10)      // A, B = e4m3 (kind::f8f6f4) or f16 (kind::f16): code 0 in both
           | (0u << 15) | (0u << 16)     // A, B K-major
           | ((uint32_t)(BN >> 3) << 17) // N
           | ((uint32_t)(kBM >> 4) << 24);
}

struct UmmaSched {
    int m_tiles, n_tiles, splits, kblocks_total, kblocks_per_split;
    int tile_base, total_work;      // this launch covers work items [tile_base, total_work)
    // Work items below narrow_from are whole tiles (item index = tile index).  From narrow_from on
    // (256-wide persistent launches only) two consecutive items are the 128-column halves of one tile,
    // so that a last round of r <= 74 tiles keeps 2r SMs busy for half as long.
    int narrow_from;
};

// tile index -> (tile_m, tile_n); 8 M-tiles share a weight column block before the next
// column block starts, so concurrently running CTAs reuse L2 lines.
__device__ __forceinline__ void decode_tile(const UmmaSched& s, int tile, int& tm, int& tn) {
    constexpr int kGroupM = 8;
    const int per_group = kGroupM * s.n_tiles;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int gsize = min(s.m_tiles - first_m, kGroupM);
    const int r = tile - group * per_group;
    tm = first_m + r % gsize;
    tn = r / gsize;
}

struct WorkItem {
    int tm;      // tile row
    int n0;      // first output channel
    int bn;      // channels of this item (BN, or 128 for a half tile)
};

template <int BN, bool kNarrow>
__device__ __forceinline__ WorkItem decode_work(const UmmaSched& s, int w) {
    WorkItem it;
    int tile = w, part = 0;
    it.bn = BN;
    if (kNarrow && w >= s.narrow_from) {
        const int u = w - s.narrow_from;
        tile = s.narrow_from + (u >> 1);
        part = u & 1;
        it.bn = 128;
    }
    int tn;
    decode_tile(s, tile, it.tm, tn);
    it.n0 = tn * BN + part * 128;
    return it;
}

// kF16 = false: e4m3 x e4m3 (W8A8; A = quantised activations, B = packed weights).
// kF16 = true:  f16 x f16 (large-M W8A16; A = activations converted to f16, B = weight tiles widened to
// f16 by dequant_tiles_f16_kernel into scratch).  A K block is 128 bytes of a row in both cases.
// kNarrow (256-wide persistent launches only): the launch ends with half-width work items.
// kFuseQ (persistent e4m3 launches only): kQuantWarps more warps quantise the bf16 activations into xq while
// the GEMM runs (umma_common.cuh); the producer waits for a row block of xq before it loads from it.
template <int BN, bool kSplit, bool kF16 = false, bool kNarrow = false, bool kFuseQ = false>
__global__ void __launch_bounds__(kThreads + (kFuseQ ? kQuantWarps * 32 : 0), 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ OutMaps outs, UmmaArgs p, UmmaSched sched) {
    using Cfg = UmmaCfg<BN>;
    constexpr int S = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[S];
    __shared__ __align__(8) uint64_t bar_empty[S];
    __shared__ __align__(8) uint64_t bar_tfull[2];
    __shared__ __align__(8) uint64_t bar_tempty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
    // in_scale * w_scale[n] and bias[n] of the tile whose epilogue runs (single copy, bias kept as
    // bf16: the 256-wide tile needs the shared memory for its 4 KB staging boxes); the next tile's
    // values wait in registers
    __shared__ __align__(16) float s_scale[BN];
    __shared__ __align__(16) __nv_bfloat16 s_bias[BN];

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // In split mode a cluster shares one tile: tile = cluster id, K slice = rank in the cluster.
    const int split_rank = kSplit ? (int)cluster_ctarank() : 0;
    const int first_work = sched.tile_base + (kSplit ? (int)(blockIdx.x / sched.splits) : (int)blockIdx.x);
    const int work_step = kSplit ? sched.total_work : (int)gridDim.x;      // split mode: exactly one tile

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(smem_u32(&bar_full[i]), 1); mbar_init(smem_u32(&bar_empty[i]), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bar_tfull[i]), 1); mbar_init(smem_u32(&bar_tempty[i]), kEpiWarps); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    pdl_launch_dependents();
    static_assert(!kFuseQ || (!kSplit && !kF16), "in-kernel quantisation: persistent e4m3 launches only");
    QuantJob qjob;
    qjob.x = p.x; qjob.xq = const_cast<unsigned char*>(p.xq); qjob.ctrl = p.q_ctrl; qjob.ldx = p.ldx; qjob.row_start = p.q_row_start; qjob.lead = p.q_lead;

    if (kFuseQ && warp >= 2 + kEpiWarps) {
        // ================= activation quantiser (warps 10..13) =================
        pdl_wait();                    // x comes from the kernel before; xq may still be read by it
        quant_worker(qjob, p.input_scale, p.M, p.K, lane);
    } else if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            uint32_t it = 0;
            bool ok = true;
            bool waited = false;      // weight tiles of the first ring pass go out before the predecessor is done
            bool next_ready = false;  // (kFuseQ) the next tile's rows of xq were complete when last looked at
            if (kF16) pdl_wait();     // ... unless the predecessor is the pass that writes the f16 weight tiles
            for (int w = first_work; w < sched.total_work && ok; w += work_step) {
                const WorkItem wk = decode_work<BN, kNarrow>(sched, w);
                const int tm = wk.tm;
                const int nsub = kNarrow ? (wk.bn >> 7) : (BN + 127) / 128;  // 128-row weight boxes per K block
                const uint32_t stage_tx = kNarrow ? (uint32_t)(Cfg::kABytes + wk.bn * kBK) : (uint32_t)Cfg::kStageBytes;
                const int kb0 = split_rank * sched.kblocks_per_split;
                const int kb1 = kSplit ? min(sched.kblocks_total, kb0 + sched.kblocks_per_split) : sched.kblocks_total;
                if (!waited) {
                    const int first_kb = min(kb1 - kb0, S);
                    for (int i = 0; i < first_kb; ++i) {
                        const uint32_t full = smem_u32(&bar_full[i]);
                        mbar_expect_tx(full, stage_tx);
#pragma unroll
                        for (int sub = 0; sub < nsub; ++sub) {
                            const int n_sub = wk.n0 + sub * 128;
                            const int wrow = ((n_sub >> 7) * sched.kblocks_total + kb0 + i) * 128 + (n_sub & 127);
                            tma_load_2d(smem_base + i * Cfg::kStageBytes + Cfg::kABytes + sub * 128 * kBK, &tmap_b, 0, wrow, full);
                        }
                    }
                    pdl_wait();       // the quantised activations are written by the kernel before this one
                    if (kFuseQ && !quant_wait_block(qjob, p.M, tm, p.status)) { s_abort = 1; ok = false; break; }
                    if (kFuseQ && w + work_step < sched.total_work)
                        next_ready = quant_probe_block(qjob, p.M, decode_work<BN, kNarrow>(sched, w + work_step).tm);
                    for (int i = 0; i < first_kb; ++i)
                        tma_load_2d(smem_base + i * Cfg::kStageBytes, &tmap_a, (kb0 + i) * kBK, tm * kBM, smem_u32(&bar_full[i]));
                    waited = true;
                    it = (uint32_t)first_kb;
                    if (kb0 + first_kb >= kb1) continue;
                } else if (kFuseQ) {
                    if (next_ready) fence_proxy_async_all();
                    else if (s_abort || !quant_wait_block(qjob, p.M, tm, p.status)) { s_abort = 1; ok = false; break; }
                    next_ready = w + work_step < sched.total_work &&
                                 quant_probe_block(qjob, p.M, decode_work<BN, kNarrow>(sched, w + work_step).tm);
                }
                for (int kb = kb0 + (w == first_work ? min(kb1 - kb0, S) : 0); kb < kb1; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t full = smem_u32(&bar_full[st]);
                    mbar_expect_tx(full, stage_tx);
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    tma_load_2d(sa, &tmap_a, kb * kBK, tm * kBM, full);
                    // packed weights: the tile of channel block cb and K block kb is rows
                    // [(cb*KB + kb)*128, +128) of a [tiles*128][128-byte] matrix
#pragma unroll
                    for (int sub = 0; sub < nsub; ++sub) {
                        const int n_sub = wk.n0 + sub * 128;
                        const int wrow = ((n_sub >> 7) * sched.kblocks_total + kb) * 128 + (n_sub & 127);
                        tma_load_2d(sa + Cfg::kABytes + sub * 128 * kBK, &tmap_b, 0, wrow, full);
                    }
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
            constexpr uint32_t idesc_full = make_idesc<BN>();
            uint32_t it = 0;
            int tl = 0;
            bool ok = true;
            for (int w = first_work; w < sched.total_work && ok; w += work_step, ++tl) {
                const int kb0 = split_rank * sched.kblocks_per_split;
                const int kb1 = kSplit ? min(sched.kblocks_total, kb0 + sched.kblocks_per_split) : sched.kblocks_total;
                const int as = tl & 1;
                const uint32_t aph = (tl >> 1) & 1;
                // a half tile is the same instruction with N = 128
                const uint32_t idesc = (kNarrow && w >= sched.narrow_from)
                                           ? ((idesc_full & ~(0x3fu << 17)) | ((128u >> 3) << 17)) : idesc_full;
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
                        if (kF16) umma_f16_ss(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                        else umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bar_empty[st]));
                }
                if (ok) umma_commit(smem_u32(&bar_tfull[as]));
            }
        }
    } else {
        // ================= epilogue (warps 2..9) =================
        // Warp (q, h): TMEM lanes [32q, 32q+32) = 32 rows of the tile, column half h.
        pdl_wait();                                            // y may still be in use by the predecessor
        const int ew = warp - 2;
        const int q = warp & 3;
        const int h = ew >> 2;
        const int et = threadIdx.x - 64;                            // 0..255 among the epilogue threads
        constexpr int kPiece = Cfg::kPiece;
        const float in_scale = p.input_scale ? fmaxf(__ldg(p.input_scale), 1e-12f) : 1.f;   // W8A16: weights' scale only
        const uint32_t box = smem_base + Cfg::kRingBytes + ew * Cfg::kBoxBytes;
        const uint32_t row_off = lane * (kPiece * 2);
        const uint32_t sw = kPiece == 64 ? (lane & 7) : ((lane >> 1) & 3);   // 128-byte / 64-byte swizzle
        int tl = 0;
        bool ok = true;
        static_assert(BN <= kEpiWarps * 32, "one column per epilogue thread");
        float next_scale = 0.f;
        __nv_bfloat16 next_bias = __float2bfloat16(0.f);
        auto fetch_columns = [&](int work) {            // thread et holds column et of that tile
            const WorkItem f = decode_work<BN, kNarrow>(sched, work);
            const int n = f.n0 + et;
            const bool in = et < f.bn && n < p.N;
            next_scale = in ? in_scale * __ldg(p.w_scale + n) : 0.f;
            next_bias = (in && p.bias) ? p.bias[n] : __float2bfloat16(0.f);
        };
        if (first_work < sched.total_work) fetch_columns(first_work);
        for (int w = first_work; w < sched.total_work && ok; w += work_step, ++tl) {
            const WorkItem wk = decode_work<BN, kNarrow>(sched, w);
            const int tm = wk.tm;
            const int as = tl & 1;
            const uint32_t aph = (tl >> 1) & 1;
            const int n0 = wk.n0;
            const int half_cols = kNarrow ? (wk.bn >> 1) : BN / 2;   // columns of this warp's half of the item
            // every epilogue warp is done with the previous tile's multipliers before they are replaced
            if (tl > 0) asm volatile("bar.sync 1, 256;" ::: "memory");
            if (et < BN) { s_scale[et] = next_scale; s_bias[et] = next_bias; }
            // the loads for the tile after this one land while this tile's epilogue runs
            if (w + work_step < sched.total_work) fetch_columns(w + work_step);
            if (kSplit) {
                // one tile per CTA: nothing after this loop meets at a named barrier, so each warp may give
                // up on its own, and the barrier stays off the path between the last MMA and the reduction
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (!mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull)) {
                    s_abort = 1; ok = false; break;
                }
            } else {
                const bool arrived = mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull);
                // One barrier makes the multipliers visible and takes the vote: if the wait ran out in any
                // warp, every epilogue warp leaves here together (they meet at named barriers again on the
                // next tile, so they must agree).
                uint32_t any_failed;
                asm volatile(
                    "{\n .reg .pred pin, pout;\n setp.ne.b32 pin, %1, 0;\n"
                    " barrier.cta.red.or.pred pout, 1, 256, pin;\n selp.u32 %0, 1, 0, pout;\n}"
                    : "=r"(any_failed) : "r"(arrived ? 0u : 1u) : "memory");
                if (any_failed) { s_abort = 1; ok = false; break; }
            }
            tc_fence_after();
            const int row0 = tm * kBM + q * 32;
            if (Cfg::kPairBox && !kSplit) {
                // Piece = 64 columns of the item; warp h converts columns [32h, 32h + 32) of it into its half
                // of the pair's box, warp 0 of the pair issues the store.
                const int bn_cur = kNarrow ? wk.bn : BN;
                const uint32_t pbox = smem_base + Cfg::kRingBytes + q * Cfg::kBoxBytes;
                const uint32_t t_pair = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN + h * 32;
#pragma unroll 1
                for (int col = 0; col < bn_cur; col += 64) {
                    if (n0 + col >= p.N) break;                      // same for both warps of the pair
                    uint32_t v[32];
                    __syncwarp();
                    tmem_ld32_nowait(t_pair + col, v);
                    tmem_ld_wait();
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 sc = *reinterpret_cast<const float4*>(&s_scale[col + h * 32 + j]);
                        const uint2 bb = *reinterpret_cast<const uint2*>(&s_bias[col + h * 32 + j]);     // four bf16
                        o[j / 2] = pack_bf16x2(fmaf(__uint_as_float(v[j]), sc.x, __uint_as_float(bb.x << 16)),
                                               fmaf(__uint_as_float(v[j + 1]), sc.y, __uint_as_float(bb.x & 0xffff0000u)));
                        o[j / 2 + 1] = pack_bf16x2(fmaf(__uint_as_float(v[j + 2]), sc.z, __uint_as_float(bb.y << 16)),
                                                   fmaf(__uint_as_float(v[j + 3]), sc.w, __uint_as_float(bb.y & 0xffff0000u)));
                    }
                    // the pair's previous store must have finished reading the box
                    if (h == 0 && lane == 0) tma_store_wait_read();
                    asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t dst = pbox + lane * 128 + (((uint32_t)(h * 4 + j) ^ (uint32_t)(lane & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[4 * j]), "r"(o[4 * j + 1]),
                                     "r"(o[4 * j + 2]), "r"(o[4 * j + 3]) : "memory");
                    }
                    fence_async_smem();
                    asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
                    if (h == 0 && lane == 0) {
                        // one store per destination: the local output, or (row-parallel scatter) this
                        // rank's slot in every rank's buffer, peers reached over NVLink
                        store_box(outs, pbox, n0 + col, row0);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
                continue;
            }
            const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN + h * half_cols;

#pragma unroll 1
            for (int c0 = 0; c0 < half_cols; c0 += kPiece) {
                const int col = h * half_cols + c0;                      // first column of this piece inside the tile
                if (n0 + col >= p.N) break;                          // uniform: the rest is past N
                if (kSplit) {
                    // park the raw fp32 accumulators in this CTA's shared memory (over the idle ring); this
                    // is on the critical path of a one-tile CTA, so all TMEM loads of the piece go out together
                    uint32_t v[kPiece];
                    __syncwarp();
                    tmem_ld32_nowait(t_addr + c0, v);
                    if (kPiece == 64) tmem_ld32_nowait(t_addr + c0 + 32, v + 32);
                    tmem_ld_wait();
                    const uint32_t dst0 = smem_base + (uint32_t)(q * 32 + lane) * Cfg::kPartPitch + (uint32_t)col * 4;
#pragma unroll
                    for (int j = 0; j < kPiece; j += 4) {
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst0 + j * 4), "r"(v[j]), "r"(v[j + 1]),
                                     "r"(v[j + 2]), "r"(v[j + 3]) : "memory");
                    }
                    continue;
                }
                // A piece (one staging box, one TMA store) is converted 32 columns at a time: registers
                // for 32 accumulators only, and the store still writes whole 128-byte lines.
#pragma unroll
                for (int sp = 0; sp < kPiece / 32; ++sp) {
                    uint32_t v[32];
                    __syncwarp();
                    tmem_ld32_nowait(t_addr + c0 + sp * 32, v);
                    tmem_ld_wait();
                    {
                        uint32_t o[16];
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 sc = *reinterpret_cast<const float4*>(&s_scale[col + sp * 32 + j]);
                            const uint2 bb = *reinterpret_cast<const uint2*>(&s_bias[col + sp * 32 + j]);     // four bf16
                            o[j / 2] = pack_bf16x2(fmaf(__uint_as_float(v[j]), sc.x, __uint_as_float(bb.x << 16)),
                                                   fmaf(__uint_as_float(v[j + 1]), sc.y, __uint_as_float(bb.x & 0xffff0000u)));
                            o[j / 2 + 1] = pack_bf16x2(fmaf(__uint_as_float(v[j + 2]), sc.z, __uint_as_float(bb.y << 16)),
                                                       fmaf(__uint_as_float(v[j + 3]), sc.w, __uint_as_float(bb.y & 0xffff0000u)));
                        }
                        if (sp == 0) {
                            // the previous store out of this box must have finished reading it
                            if (lane == 0) tma_store_wait_read();
                            __syncwarp();
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t dst = box + row_off + (((uint32_t)(sp * 4 + j) ^ sw) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[4 * j]), "r"(o[4 * j + 1]),
                                         "r"(o[4 * j + 2]), "r"(o[4 * j + 3]) : "memory");
                        }
                    }
                }
                if (!kSplit) {
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        // one store per destination: the local output, or (row-parallel scatter) this
                        // rank's slot in every rank's buffer, peers reached over NVLink
                        store_box(outs, box, n0 + col, row0);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
        }
        if (!kSplit && lane == 0) tma_store_wait_all();
    }

    if (kSplit) {
        // ---- cluster reduction: CTA r sums rows [r*band, (r+1)*band) of the tile over all K slices ----
        __syncwarp();
        pdl_wait();
        cluster_sync_all();                                   // every CTA's parked tile is visible
        int tm, tn;
        decode_tile(sched, first_work, tm, tn);
        const int n0 = tn * BN;
        const int band = (kBM + sched.splits - 1) / sched.splits;
        const int r_beg = split_rank * band;
        const int r_end = min(kBM, r_beg + band);
        constexpr int kVecPerRow = BN / 4;
        const int total = (r_end - r_beg) * kVecPerRow;
        const bool healthy = (s_abort == 0);
        for (int i = threadIdx.x; i < total && healthy; i += kThreads) {
            const int r = r_beg + i / kVecPerRow;
            const int c = (i % kVecPerRow) * 4;
            const int row = tm * kBM + r;
            const int n = n0 + c;
            if (row >= p.M || n >= p.N) continue;
            const uint32_t local = smem_base + (uint32_t)r * Cfg::kPartPitch + (uint32_t)c * 4;
            // all slices' loads go out before the first add: remote shared memory is a long trip
            float4 u[8];
#pragma unroll
            for (int s = 0; s < 8; ++s)
                u[s] = s < sched.splits ? ld_cluster_f4(map_to_cta(local, (uint32_t)s)) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < 8; ++s) { a.x += u[s].x; a.y += u[s].y; a.z += u[s].z; a.w += u[s].w; }
            const float4 sc = *reinterpret_cast<const float4*>(&s_scale[c]);
            const uint2 bb = *reinterpret_cast<const uint2*>(&s_bias[c]);
            uint2 out;
            out.x = pack_bf16x2(fmaf(a.x, sc.x, __uint_as_float(bb.x << 16)), fmaf(a.y, sc.y, __uint_as_float(bb.x & 0xffff0000u)));
            out.y = pack_bf16x2(fmaf(a.z, sc.z, __uint_as_float(bb.y << 16)), fmaf(a.w, sc.w, __uint_as_float(bb.y & 0xffff0000u)));
            *reinterpret_cast<uint2*>(p.y + (size_t)row * p.ldy + n) = out;
        }
        cluster_sync_all();                                   // nobody exits while a peer still reads its tile
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
    if (kFuseQ && threadIdx.x == 0) quant_ctrl_release(qjob, p.M);
}

// ---- the give-up path of a bounded wait, exercised on its own ----------------------------------
// One CTA initialises an mbarrier that nothing ever arrives on and waits for it with the routine every
// tcgen05 kernel here uses, but with a limit of `limit_cycles` instead of about a second.  The wait runs
// out, records kDevTimeoutFull in the status word and the kernel returns normally: the context stays
// usable and the host sees the code through fp8lin_read_status.  Nothing faults, traps or spins on.
__global__ void __launch_bounds__(32)
wait_timeout_probe_kernel(int* status, long long limit_cycles, int* gave_up) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool arrived = mbar_wait(smem_u32(&bar), 0, status, kDevTimeoutFull, limit_cycles);
        if (gave_up) *gave_up = arrived ? 0 : 1;
    }
}

cudaError_t launch_wait_timeout_probe(int* status, long long limit_cycles, int* gave_up, cudaStream_t stream) {
    wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(status, limit_cycles, gave_up);
    return counted(cudaGetLastError());
}

// ---- host side -------------------------------------------------------------------
int max_active_clusters(const void* kernel, int threads, size_t smem_bytes, int cluster) {
    static const int fallback[9] = {148, 148, 74, 45, 33, 26, 22, 15, 15};     // what a B200 answers
    if (cluster < 1 || cluster > 8) return 0;
    (void)threads;
    struct Entry { const void* k; int c; int n; };
    static Entry cache[64];
    static int used = 0;
    for (int i = 0; i < used; ++i)
        if (cache[i].k == kernel && cache[i].c == cluster) return cache[i].n;
    int n = fallback[cluster];
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(cluster * 64));
        cfg.blockDim = dim3((unsigned)threads);
        cfg.dynamicSmemBytes = smem_bytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)cluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int q = 0;
        cudaError_t qe = cudaOccupancyMaxActiveClusters(&q, kernel, &cfg);
        if (qe == cudaSuccess && q > 0) n = q;
        else cudaGetLastError();
        if (getenv("FP8LIN_DEBUG"))
            fprintf(stderr, "[fp8lin] max active clusters: size %d smem %zu threads %d -> %d (%s)\n", cluster, smem_bytes,
                    threads, q, cudaGetErrorString(qe));
    } else {
        cudaGetLastError();
        return n;            // no device: do not cache, a later call may have one
    }
    if (used < 64) cache[used++] = Entry{kernel, cluster, n};
    return n;
}

EncodeTiledFn get_encode_fn() {
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
bool encode_u8_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
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

// Output map: bf16 [rows][cols] with a row pitch in bytes, box = box_cols x 32 rows,
// swizzle span = the box's row length (128 or 64 bytes).
bool encode_out_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                   uint32_t box_cols) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    box_cols * 2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

UmmaPlan plan_umma(int64_t M, int64_t K, int64_t N, int force_bn, int force_splits) {
    UmmaPlan best{};
    const int kblocks = (int)((K + kBK - 1) / kBK);
    const int m_tiles = (int)((M + kBM - 1) / kBM);
    double best_cost = 1e30;
    const int bns[3] = {256, 128, 64};
    const double unit[3] = {1.0, 0.8, 0.6};  // relative time of one K block of a tile (smaller tiles use shared memory less well)
    for (int i = 0; i < 3; ++i) {
        const int bn = bns[i];
        if (force_bn > 0 && bn != force_bn) continue;
        const int n_tiles = (int)((N + bn - 1) / bn);
        const long tiles = (long)m_tiles * n_tiles;
        int splits = 1;
        if (force_splits > 0) splits = force_splits;
        else if (tiles <= (sm_count() / 2)) {
            splits = (int)(sm_count() / tiles);
            const int max_by_k = kblocks / 4 > 0 ? kblocks / 4 : 1;  // at least four K blocks per slice
            if (splits > max_by_k) splits = max_by_k;
        }
        if (splits > 8) splits = 8;                                   // portable cluster size
        if (splits > kblocks) splits = kblocks;
        if (splits < 1) splits = 1;
        int kps = (kblocks + splits - 1) / splits;
        splits = (kblocks + kps - 1) / kps;                           // no empty K slice
        const long work = tiles * splits;
        long waves = (work + (sm_count() - 1)) / sm_count();
        if (splits > 1) {
            const void* kern = bn == 256 ? (const void*)umma_gemm_kernel<256, true>
                             : bn == 128 ? (const void*)umma_gemm_kernel<128, true> : (const void*)umma_gemm_kernel<64, true>;
            const size_t smem = bn == 256 ? UmmaCfg<256>::kSmemBytes : bn == 128 ? UmmaCfg<128>::kSmemBytes : UmmaCfg<64>::kSmemBytes;
            int slots = max_active_clusters(kern, kThreads, smem, splits);
            if (slots < 1) slots = 1;
            waves = (tiles + slots - 1) / slots;
        }
        double rounds = (double)waves;
        if (splits == 1 && force_splits <= 0 && kblocks >= 64 && tiles > sm_count() && tiles % sm_count() != 0 && tiles % sm_count() <= (sm_count() / 2))
            rounds = (double)(tiles / sm_count()) + 0.4;      // the last partial round goes to the split-K tail launch
        else if (bn == 256 && splits == 1 && force_splits <= 0 && tiles > sm_count() && tiles % sm_count() != 0 && tiles % sm_count() <= (sm_count() / 2))
            rounds = (double)(tiles / sm_count()) + 0.62;     // ... or runs as half-width work items
        // main loop + fixed per-tile prologue/epilogue; split-K pays one cluster reduction
        const double cost = rounds * (kps * unit[i] + 3.0 * unit[i]) + (splits > 1 ? 2.0 : 0.0);
        if (cost < best_cost) {
            best_cost = cost;
            best.bn = bn; best.splits = splits; best.kblocks_per_split = kps;
            best.m_tiles = m_tiles; best.n_tiles = n_tiles;
            best.grid = splits > 1 ? (int)work : (int)(work < sm_count() ? work : sm_count());
            best.partial_bytes = 0;
        }
    }
    // Wave quantisation: a persistent launch over q*148 + r tiles runs q + 1 rounds even when r is
    // small.  Then the last r tiles go to a second, cluster split-K launch (r * s CTAs <= 148) that
    // finishes them in about 1/s of a round.
    best.tail_tiles = 0; best.tail_splits = 1; best.tail_kps = 0; best.narrow_tiles = 0;
    const long tiles = (long)best.m_tiles * best.n_tiles;
    if (force_splits <= 0 && best.splits == 1 && tiles > sm_count() && kblocks >= 64) {   // a round must outlast a launch
        const int r = (int)(tiles % sm_count());
        if (r > 0 && r <= (sm_count() / 2)) {
            int s = sm_count() / r;
            if (s > 8) s = 8;
            while (s > 1 && kblocks / s < 2) --s;
            if (s > 1) {
                const void* kern = best.bn == 256 ? (const void*)umma_gemm_kernel<256, true>
                                 : best.bn == 128 ? (const void*)umma_gemm_kernel<128, true> : (const void*)umma_gemm_kernel<64, true>;
                const size_t smem = best.bn == 256 ? UmmaCfg<256>::kSmemBytes : best.bn == 128 ? UmmaCfg<128>::kSmemBytes : UmmaCfg<64>::kSmemBytes;
                while (s > 1 && max_active_clusters(kern, kThreads, smem, s) < r) --s;
            }
            if (s > 1) {
                const int kps = (kblocks + s - 1) / s;
                best.tail_tiles = r; best.tail_kps = kps; best.tail_splits = (kblocks + kps - 1) / kps;
            }
        }
    }
    // Short K: a second launch costs more than it saves; the last r <= 74 tiles of a 256-wide plan are
    // instead cut into 2r half-width work items of the same persistent launch.
    if (force_splits <= 0 && best.bn == 256 && best.splits == 1 && best.tail_tiles == 0 && tiles > sm_count()) {
        const int r = (int)(tiles % sm_count());
        if (r > 0 && r <= (sm_count() / 2)) best.narrow_tiles = r;
    }
    return best;
}

template <int BN, bool kSplit, bool kF16, bool kNarrow = false, bool kFuseQ = false>
static cudaError_t launch_bn(const UmmaPlan& pl, const UmmaArgs& a, const CUtensorMap& ta, const CUtensorMap& tb,
                             const OutMaps& ty, cudaStream_t stream, int tile_base, int tile_end, int splits, int kps,
                             int grid, int narrow_tiles) {
    using Cfg = UmmaCfg<BN>;
    static_assert(!kNarrow || (BN == 256 && !kSplit), "half-width items exist in the 256-wide persistent kernel only");
    auto kern = umma_gemm_kernel<BN, kSplit, kF16, kNarrow, kFuseQ>;
    static SmemOptIn opted;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, Cfg::kSmemBytes, opted);
        if (e != cudaSuccess) return e;
    }
    UmmaSched s;
    s.m_tiles = pl.m_tiles; s.n_tiles = pl.n_tiles; s.splits = splits;
    // f16: every packed e4m3 tile became two f16 tiles, so the K-block count is even; a last block
    // past the end of x reads zeros from the tensor map's out-of-bounds fill
    s.kblocks_total = kF16 ? 2 * (int)pack_kblocks(a.K) : (a.K + kBK - 1) / kBK; s.kblocks_per_split = kps;
    s.tile_base = tile_base; s.total_work = tile_end + narrow_tiles;      // r tiles become 2r items
    s.narrow_from = tile_end - narrow_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads + (kFuseQ ? kQuantWarps * 32 : 0));
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = pdl_attribute(attr);
    if (kSplit) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return counted(cudaLaunchKernelEx(&cfg, kern, ta, tb, ty, a, s));
}

static cudaError_t launch_umma(bool f16, const UmmaPlan& pl, const UmmaArgs& a, cudaStream_t stream, const char** why,
                               int n_dst, void* const* dst_ptrs, int64_t ld_dst, int64_t band_rows = 0) {
    CUtensorMap ta, tb;
    OutMaps ty;
    ty.band_rows = (int)band_rows;
    const uint32_t piece = pl.bn / 2 < 64 ? pl.bn / 2 : 64;      // UmmaCfg<BN>::kPiece
    const uint64_t esz = f16 ? 2 : 1;                            // the operand matrices are described in bytes
    bool ok = encode_u8_2d(&ta, a.xq, (uint64_t)a.M, (uint64_t)a.K * esz, kBM) &&
              encode_u8_2d(&tb, a.w, (uint64_t)(pack_ntiles(a.N) * pack_kblocks(a.K) * esz * 128), 128,
                           (uint32_t)(pl.bn < 128 ? pl.bn : 128));
    if (n_dst <= 0) {
        ty.n = 1;
        ok = ok && encode_out_2d(&ty.m[0], a.y, (uint64_t)a.M, (uint64_t)a.N, (uint64_t)a.ldy * 2, piece);
    } else {
        if (n_dst > 8 || pl.splits > 1) {
            if (why) *why = "scatter epilogue needs 1..8 destinations and a non-split plan";
            return cudaErrorInvalidValue;
        }
        ty.n = n_dst;
        for (int d = 0; d < n_dst && ok; ++d) {
            int64_t rows = a.M;
            if (band_rows > 0) {          // destination d holds one band of rows (at least one row: a map cannot be empty)
                rows = a.M - d * band_rows;
                rows = rows > band_rows ? band_rows : (rows < 1 ? 1 : rows);
            }
            ok = encode_out_2d(&ty.m[d], dst_ptrs[d], (uint64_t)rows, (uint64_t)a.N, (uint64_t)ld_dst * 2, piece);
        }
    }
    if (!ok) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    const int tiles = pl.m_tiles * pl.n_tiles;
    const int main_tiles = tiles - pl.tail_tiles;
    auto go = [&](bool split, int base, int end, int splits, int kps, int grid, int narrow = 0) -> cudaError_t {
#define FP8LIN_GO(BN_, SPLIT_, F16_) launch_bn<BN_, SPLIT_, F16_>(pl, a, ta, tb, ty, stream, base, end, splits, kps, grid, narrow)
#define FP8LIN_GO_BN(BN_) (f16 ? (split ? FP8LIN_GO(BN_, true, true) : FP8LIN_GO(BN_, false, true)) \
                               : (split ? FP8LIN_GO(BN_, true, false) : FP8LIN_GO(BN_, false, false)))
        if (narrow > 0) {     // (only set for 256-wide non-split plans)
            if (!f16 && a.x) return launch_bn<256, false, false, true, true>(pl, a, ta, tb, ty, stream, base, end, splits, kps, grid, narrow);
            return f16 ? launch_bn<256, false, true, true>(pl, a, ta, tb, ty, stream, base, end, splits, kps, grid, narrow)
                       : launch_bn<256, false, false, true>(pl, a, ta, tb, ty, stream, base, end, splits, kps, grid, narrow);
        }
        if (!f16 && !split && a.x) {     // activations quantised inside the persistent launch
            switch (pl.bn) {
                case 256: return launch_bn<256, false, false, false, true>(pl, a, ta, tb, ty, stream, base, end, splits, kps, grid, narrow);
                case 128: return launch_bn<128, false, false, false, true>(pl, a, ta, tb, ty, stream, base, end, splits, kps, grid, narrow);
                case 64: return launch_bn<64, false, false, false, true>(pl, a, ta, tb, ty, stream, base, end, splits, kps, grid, narrow);
            }
        }
        switch (pl.bn) {
            case 256: return FP8LIN_GO_BN(256);
            case 128: return FP8LIN_GO_BN(128);
            case 64: return FP8LIN_GO_BN(64);
        }
#undef FP8LIN_GO_BN
#undef FP8LIN_GO
        if (why) *why = "unsupported tile width";
        return cudaErrorInvalidValue;
    };
    if (pl.splits > 1) return go(true, 0, tiles, pl.splits, pl.kblocks_per_split, pl.grid);
    const int narrow = pl.bn == 256 && pl.tail_tiles == 0 ? pl.narrow_tiles : 0;
    const int main_work = main_tiles + narrow;
    cudaError_t e = go(false, 0, main_tiles, 1, pl.kblocks_per_split, main_work < sm_count() ? main_work : sm_count(), narrow);
    if (e != cudaSuccess || pl.tail_tiles == 0) return e;
    return go(true, main_tiles, tiles, pl.tail_splits, pl.tail_kps, pl.tail_tiles * pl.tail_splits);
}

cudaError_t launch_umma_w8a8(const UmmaPlan& pl, const UmmaArgs& a, cudaStream_t stream, const char** why,
                             int n_dst, void* const* dst_ptrs, int64_t ld_dst, int64_t band_rows) {
    return launch_umma(false, pl, a, stream, why, n_dst, dst_ptrs, ld_dst, band_rows);
}

cudaError_t launch_umma_f16(const UmmaPlan& pl, const UmmaArgs& a, cudaStream_t stream, const char** why) {
    return launch_umma(true, pl, a, stream, why, 0, nullptr, 0);
}

}  // namespace fp8lin
