// Large-M GEMM on CTA pairs (tcgen05 cta_group::2): y = (A . B^T) * scale[n] + bias[n], bf16 out.
//
// Two CTAs of a cluster compute one 256 x 256 output tile.  CTA r of the pair holds rows
// [128r, 128r + 128) of the A tile and channels [128r, 128r + 128) of the B tile in its shared memory,
// and the 128 x 256 accumulator of ITS rows in its tensor memory; one thread of the leader CTA (rank 0)
// issues a single MMA per 32 bytes of K that reads both CTAs' shared memory and writes both CTAs'
// tensor memory.  Against two independent 128 x 256 tiles this halves the B bytes every CTA loads and
// feeds to its tensor core per MMA (32 KB instead of 48 KB of shared memory written, and as much read,
// per K block), which is what bounds the one-CTA kernel (umma_gemm.cu) on large shapes.
//
// Barriers (per CTA unless noted):
//   full[s]   (used in the leader only)  both CTAs' TMA loads complete their bytes on the LEADER's
//             barrier; the leader's producer thread arms it with the byte count of both.
//   empty[s]  the MMA thread commits to the barrier of the same name in both CTAs (two commits), so each
//             producer refills its own stage.
//   tfull[a]  likewise committed to both CTAs after the last K block: the epilogue warps of each CTA
//             read their own tensor memory.
//   tempty[a] (leader only) the eight epilogue warps of both CTAs arrive on the leader's barrier (the
//             peer's with a cluster-scope remote arrive).
// No load in this file is a cluster broadcast: every TMA load lands in exactly one CTA.
// Every wait is bounded (about a second); a CTA that gives up still joins the cluster barrier at the
// end, so its partner is never left waiting for it.
#include "umma_common.cuh"

namespace fp8lin {

namespace {

constexpr int kBM = 128;            // rows per CTA (256 per pair)
constexpr int kBN = 256;
constexpr int kBK = 128;            // bytes of K per block
constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + kEpiWarps) * 32;
constexpr int kABytes = kBM * kBK;            // 16 KB: this CTA's rows of A
constexpr int kBBytes = (kBN / 2) * kBK;      // 16 KB: this CTA's half of the channels
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStages = 6;
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kBoxBytes = 32 * 64 * 2;        // staging box: 32 rows x 64 bf16
constexpr int kStagingBytes = (kEpiWarps / 2) * kBoxBytes;
constexpr int kSmemBytes = kRingBytes + kStagingBytes + 1024;
constexpr int kTmemCols = 2 * kBN;

struct PairSched {
    int mp_tiles;        // 256-row tile rows
    int n_tiles;         // 256-channel tile columns
    int kblocks;
    int total;           // mp_tiles * n_tiles
};

// tile index -> (pair row, tile column); eight tile rows share a weight column block before the next
// column block starts, so that concurrently running pairs reuse L2 lines.
__device__ __forceinline__ void decode_pair_tile(const PairSched& s, int tile, int& tmp, int& tn) {
    constexpr int kGroupM = 8;
    const int per_group = kGroupM * s.n_tiles;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int gsize = min(s.mp_tiles - first_m, kGroupM);
    const int r = tile - group * per_group;
    tmp = first_m + r % gsize;
    tn = r / gsize;
}

// kMlp: the weight is a gate_up projection packed with its 128-channel tile rows interleaved (gate tile t,
// up tile t, gate tile t+1, ...; scale and bias permuted alike), so the 256 columns of a tile are 128 gate
// channels followed by the 128 up channels of the same indices.  The epilogue then produces what the down
// projection consumes instead of the bf16 tile: h = bf16(silu(g) * u) from g, u rounded to bf16 (the values
// the unfused path materialises), quantised to e4m3 with the down projection's static scale `h_scale`;
// 128 bytes per row and tile go to the e4m3 matrix [M][N/2] described by outs.m[0].
// kFuseQ (e4m3 operands only): kQuantWarps more warps per CTA quantise the bf16 activations into xq while the
// GEMM runs (umma_common.cuh); each CTA's producer waits for its own 128-row block of xq before loading it.
// kS: ring slots in use (kStages; fewer only for pipeline-depth studies).
template <bool kF16, bool kMlp, bool kFuseQ = false, int kS = kStages>
__global__ void __launch_bounds__(kThreads + (kFuseQ ? kQuantWarps * 32 : 0), 1)
umma_pair_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ OutMaps outs, UmmaArgs p, PairSched sched, const float* h_scale) {
    constexpr int S = kS;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[S];
    __shared__ __align__(8) uint64_t bar_empty[S];
    __shared__ __align__(8) uint64_t bar_tfull[2];
    __shared__ __align__(8) uint64_t bar_tempty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
    __shared__ __align__(16) float s_scale[kBN];
    __shared__ __align__(16) __nv_bfloat16 s_bias[kBN];

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;
    const int first_tile = (int)(blockIdx.x >> 1);
    const int tile_step = (int)(gridDim.x >> 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(smem_u32(&bar_full[i]), 1); mbar_init(smem_u32(&bar_empty[i]), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bar_tfull[i]), 1); mbar_init(smem_u32(&bar_tempty[i]), 2 * kEpiWarps); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(&s_tmem_base), kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // the partner's barriers exist before anything is signalled on them
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    pdl_launch_dependents();
    static_assert(!kFuseQ || !kF16, "in-kernel quantisation: e4m3 operands only");
    QuantJob qjob;
    qjob.x = p.x; qjob.xq = const_cast<unsigned char*>(p.xq); qjob.ctrl = p.q_ctrl; qjob.ldx = p.ldx; qjob.row_start = p.q_row_start; qjob.lead = p.q_lead;

    if (kFuseQ && warp >= 2 + kEpiWarps) {
        // ================= activation quantiser (warps 10..13 of both CTAs) =================
        pdl_wait();
        quant_worker(qjob, p.input_scale, p.M, p.K, lane);
    } else if (warp == 0) {
        // ================= TMA producer (both CTAs) =================
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
            pdl_wait();            // the activations (and, for f16, the weight tiles) come from the kernel before
            uint32_t it = 0;
            bool ok = true;
            bool next_ready = false;     // (kFuseQ) the next tile's rows of xq were complete when last looked at
            for (int t = first_tile; t < sched.total && ok; t += tile_step) {
                int tmp, tn;
                decode_pair_tile(sched, t, tmp, tn);
                const int row0 = (2 * tmp + (int)rank) * kBM;
                const int n_sub = tn * kBN + (int)rank * 128;             // this CTA's 128 channels
                if (kFuseQ) {
                    if (next_ready) fence_proxy_async_all();
                    else if (s_abort || !quant_wait_block(qjob, p.M, 2 * tmp + (int)rank, p.status)) { s_abort = 1; ok = false; break; }
                    next_ready = false;
                    if (t + tile_step < sched.total) {
                        int ntmp, ntn;
                        decode_pair_tile(sched, t + tile_step, ntmp, ntn);
                        next_ready = quant_probe_block(qjob, p.M, 2 * ntmp + (int)rank);
                    }
                }
                for (int kb = 0; kb < sched.kblocks; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t full_local = smem_u32(&bar_full[st]);
                    if (leader) mbar_expect_tx(full_local, 2 * kStageBytes);
                    const uint32_t full = leader ? full_local : map_to_cta(full_local, 0);
                    const uint32_t sa = smem_base + st * kStageBytes;
                    tma_load_2d_pair(sa, &tmap_a, kb * kBK, row0, full);
                    // packed weights: the tile of channel block cb and K block kb is rows
                    // [(cb*KB + kb)*128, +128) of a [tiles*128][128-byte] matrix
                    const int wrow = ((n_sub >> 7) * sched.kblocks + kb) * 128;
                    tma_load_2d_pair(sa + kABytes, &tmap_b, 0, wrow, full);
                }
            }
            if (!ok) {
                const long long t0 = clock64();      // let copies that are still in flight land
                while (clock64() - t0 < 2000000) {}
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer (leader CTA only) =================
        if (leader && lane == 0) {
            constexpr uint32_t idesc = make_idesc_mn(2 * kBM, kBN, 0, 0);
            const uint32_t peer = 1;
            uint32_t it = 0;
            int tl = 0;
            bool ok = true;
            for (int t = first_tile; t < sched.total && ok; t += tile_step, ++tl) {
                const int as = tl & 1;
                const uint32_t aph = (tl >> 1) & 1;
                if (s_abort || !mbar_wait(smem_u32(&bar_tempty[as]), aph ^ 1, p.status, kDevTimeoutTmemEmpty)) {
                    s_abort = 1; ok = false; break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * kBN;
                for (int kb = 0; kb < sched.kblocks; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_full[st]), ph, p.status, kDevTimeoutFull)) {
                        s_abort = 1; ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + st * kStageBytes;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k) {
                        if (kF16) umma_f16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        else umma_f8_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    const uint32_t e = smem_u32(&bar_empty[st]);
                    umma_commit_pair(e);                        // this CTA's stage is free again ...
                    umma_commit_pair(map_to_cta(e, peer));      // ... and so is the partner's
                }
                if (ok) {
                    const uint32_t f = smem_u32(&bar_tfull[as]);
                    umma_commit_pair(f);
                    umma_commit_pair(map_to_cta(f, peer));
                }
            }
        }
    } else {
        // ================= epilogue (warps 2..9 of both CTAs) =================
        // Warp (q, h): TMEM lanes [32q, 32q+32) = 32 rows of this CTA's half of the tile; of every 64
        // columns warp h converts [32h, 32h + 32) into its half of the pair's staging box.
        pdl_wait();                                            // y may still be in use by the predecessor
        const int ew = warp - 2;
        const int q = warp & 3;
        const int h = ew >> 2;
        const int et = threadIdx.x - 64;                            // 0..255 among the epilogue threads
        const float in_scale = p.input_scale ? fmaxf(__ldg(p.input_scale), 1e-12f) : 1.f;
        const uint32_t pbox = smem_base + kRingBytes + q * kBoxBytes;
        int tl = 0;
        bool ok = true;
        float next_scale = 0.f;
        __nv_bfloat16 next_bias = __float2bfloat16(0.f);
        auto fetch_columns = [&](int tile) {                        // thread et holds column et of that tile
            int ftmp, ftn;
            decode_pair_tile(sched, tile, ftmp, ftn);
            const int n = ftn * kBN + et;
            const bool in = n < p.N;
            next_scale = in ? in_scale * __ldg(p.w_scale + n) : 0.f;
            next_bias = (in && p.bias) ? p.bias[n] : __float2bfloat16(0.f);
        };
        if (first_tile < sched.total) fetch_columns(first_tile);
        for (int t = first_tile; t < sched.total && ok; t += tile_step, ++tl) {
            int tmp, tn;
            decode_pair_tile(sched, t, tmp, tn);
            const int as = tl & 1;
            const uint32_t aph = (tl >> 1) & 1;
            const int n0 = tn * kBN;
            if (tl > 0) asm volatile("bar.sync 1, 256;" ::: "memory");
            s_scale[et] = next_scale;
            s_bias[et] = next_bias;
            if (t + tile_step < sched.total) fetch_columns(t + tile_step);
            const bool arrived = mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull);
            // one barrier publishes the multipliers and takes the vote: the eight warps leave together
            uint32_t any_failed;
            asm volatile(
                "{\n .reg .pred pin, pout;\n setp.ne.b32 pin, %1, 0;\n"
                " barrier.cta.red.or.pred pout, 1, 256, pin;\n selp.u32 %0, 1, 0, pout;\n}"
                : "=r"(any_failed) : "r"(arrived ? 0u : 1u) : "memory");
            if (any_failed) { s_abort = 1; ok = false; break; }
            tc_fence_after();
            const int row0 = (2 * tmp + (int)rank) * kBM + q * 32;
            if (kMlp) {
                // warp h owns output bytes [64h, 64h + 64) of the tile's 128: two steps of 32 columns, each from
                // 32 gate accumulators (columns c..) and the 32 up accumulators 128 columns further on
                const ExactDiv div_h(fmaxf(__ldg(h_scale), 1e-12f));
                const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * kBN;
                if (n0 < p.N) {
#pragma unroll 1
                    for (int sp = 0; sp < 2; ++sp) {
                        const int c = 64 * h + 32 * sp;
                        uint32_t g[32], u[32];
                        __syncwarp();
                        tmem_ld32_nowait(t_row + c, g);
                        tmem_ld32_nowait(t_row + 128 + c, u);
                        tmem_ld_wait();
                        uint32_t hw[16];
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const float2 sg = *reinterpret_cast<const float2*>(&s_scale[c + j]);
                            const float2 su = *reinterpret_cast<const float2*>(&s_scale[128 + c + j]);
                            const uint32_t bg = *reinterpret_cast<const uint32_t*>(&s_bias[c + j]);
                            const uint32_t bu = *reinterpret_cast<const uint32_t*>(&s_bias[128 + c + j]);
                            // gate and up as the bf16 values a separate gate_up GEMM would have stored
                            const uint32_t gp = pack_bf16x2(fmaf(__uint_as_float(g[j]), sg.x, bf16_lo(bg)),
                                                            fmaf(__uint_as_float(g[j + 1]), sg.y, bf16_hi(bg)));
                            const uint32_t up = pack_bf16x2(fmaf(__uint_as_float(u[j]), su.x, bf16_lo(bu)),
                                                            fmaf(__uint_as_float(u[j + 1]), su.y, bf16_hi(bu)));
                            const float g0 = bf16_lo(gp), g1 = bf16_hi(gp);
                            const float s0 = g0 / (1.f + expf(-g0)), s1 = g1 / (1.f + expf(-g1));
                            hw[j / 2] = pack_bf16x2(s0 * bf16_lo(up), s1 * bf16_hi(up));
                        }
                        uint2 qv[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            qv[j] = quant8_e4m3(make_uint4(hw[4 * j], hw[4 * j + 1], hw[4 * j + 2], hw[4 * j + 3]), div_h);
                        if (sp == 0) {
                            if (h == 0 && lane == 0) tma_store_wait_read();      // the previous store has read the box
                            asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
                        }
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint32_t chunk = (uint32_t)(4 * h + 2 * sp + j);
                            const uint32_t dst = pbox + lane * 128 + ((chunk ^ (uint32_t)(lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(qv[2 * j].x), "r"(qv[2 * j].y),
                                         "r"(qv[2 * j + 1].x), "r"(qv[2 * j + 1].y) : "memory");
                        }
                    }
                    fence_async_smem();
                    asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
                    if (h == 0 && lane == 0) tma_store_2d(&outs.m[0], pbox, n0 >> 1, row0);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    const uint32_t te = smem_u32(&bar_tempty[as]);
                    if (leader) mbar_arrive(te);
                    else mbar_arrive_cluster(map_to_cta(te, 0));
                }
                continue;
            }
            const uint32_t t_pair = tmem_base + ((uint32_t)(q * 32) << 16) + as * kBN + h * 32;
#pragma unroll 1
            for (int col = 0; col < kBN; col += 64) {
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
                if (h == 0 && lane == 0) tma_store_wait_read();      // the previous store has read the box
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
                    store_box(outs, pbox, n0 + col, row0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                const uint32_t te = smem_u32(&bar_tempty[as]);
                if (leader) mbar_arrive(te);
                else mbar_arrive_cluster(map_to_cta(te, 0));
            }
        }
        if (lane == 0) tma_store_wait_all();
    }

    // nobody leaves while its partner may still signal its barriers or the leader's MMAs may still
    // read its shared memory and write its tensor memory
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
    if (kFuseQ && threadIdx.x == 0) quant_ctrl_release(qjob, p.M);
}

int g_pair_stages = kStages;       // tuning knob "pair_stages" (studies only)

template <bool kF16, bool kMlp, bool kFuseQ = false, int kS = kStages>
cudaError_t launch_pair(const UmmaArgs& a, const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& ty,
                        cudaStream_t stream, const char** why, const float* h_scale = nullptr) {
    auto kern = umma_pair_gemm_kernel<kF16, kMlp, kFuseQ, kS>;
    constexpr int kBlock = kThreads + (kFuseQ ? kQuantWarps * 32 : 0);
    static SmemOptIn opted;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, kSmemBytes, opted);
        if (e != cudaSuccess) return e;
    }
    PairSched s;
    s.mp_tiles = (a.M + 2 * kBM - 1) / (2 * kBM);
    s.n_tiles = (a.N + kBN - 1) / kBN;
    s.kblocks = kF16 ? 2 * (int)pack_kblocks(a.K) : (a.K + kBK - 1) / kBK;
    s.total = s.mp_tiles * s.n_tiles;
    int pairs = max_active_clusters((const void*)kern, kBlock, kSmemBytes, 2);
    if (pairs < 1) {
        if (why) *why = "no CTA pair fits on this device";
        return cudaErrorInvalidConfiguration;
    }
    if (pairs > s.total) pairs = s.total;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kBlock);
    cfg.dynamicSmemBytes = kSmemBytes;
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
    return counted(cudaLaunchKernelEx(&cfg, kern, ta, tb, ty, a, s, h_scale));
}

}  // namespace

void set_pair_stages(int n) { g_pair_stages = (n == 4 || n == 5) ? n : kStages; }

cudaError_t launch_umma_pair(bool f16, const UmmaArgs& a, cudaStream_t stream, const char** why, int n_dst,
                             void* const* dst_ptrs, int64_t ld_dst, int64_t band_rows) {
    CUtensorMap ta, tb;
    OutMaps ty;
    ty.band_rows = (int)band_rows;
    const uint64_t esz = f16 ? 2 : 1;                            // the operand matrices are described in bytes
    bool ok = encode_u8_2d(&ta, a.xq, (uint64_t)a.M, (uint64_t)a.K * esz, kBM) &&
              encode_u8_2d(&tb, a.w, (uint64_t)(pack_ntiles(a.N) * pack_kblocks(a.K) * esz * 128), 128, 128);
    if (n_dst <= 0) {
        ty.n = 1;
        ok = ok && encode_out_2d(&ty.m[0], a.y, (uint64_t)a.M, (uint64_t)a.N, (uint64_t)a.ldy * 2, 64);
    } else {
        if (n_dst > 8) {
            if (why) *why = "scatter epilogue takes 1..8 destinations";
            return cudaErrorInvalidValue;
        }
        ty.n = n_dst;
        for (int d = 0; d < n_dst && ok; ++d) {
            int64_t rows = a.M;
            if (band_rows > 0) {
                rows = a.M - d * band_rows;
                rows = rows > band_rows ? band_rows : (rows < 1 ? 1 : rows);
            }
            ok = encode_out_2d(&ty.m[d], dst_ptrs[d], (uint64_t)rows, (uint64_t)a.N, (uint64_t)ld_dst * 2, 64);
        }
    }
    if (!ok) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    if (!f16 && a.x) return launch_pair<false, false, true>(a, ta, tb, ty, stream, why);
    if (!f16 && g_pair_stages == 5) return launch_pair<false, false, false, 5>(a, ta, tb, ty, stream, why);
    if (!f16 && g_pair_stages == 4) return launch_pair<false, false, false, 4>(a, ta, tb, ty, stream, why);
    return f16 ? launch_pair<true, false>(a, ta, tb, ty, stream, why) : launch_pair<false, false>(a, ta, tb, ty, stream, why);
}

// gate_up GEMM with the SiLU-multiply-quantise epilogue: a.w = interleaved gate/up tiles, a.N = 2 * I (a multiple
// of 256), a.w_scale / a.bias permuted like the tiles; hq = e4m3 [M][I] (row pitch I), h_scale = the down
// projection's activation scale.  a.y is unused.
cudaError_t launch_umma_pair_mlp(const UmmaArgs& a, unsigned char* hq, const float* h_scale, cudaStream_t stream,
                                 const char** why) {
    if (a.N % 256 != 0) {
        if (why) *why = "the intermediate size must be a multiple of 128";
        return cudaErrorInvalidValue;
    }
    CUtensorMap ta, tb;
    OutMaps ty;
    ty.n = 1;
    ty.band_rows = 0;
    const bool ok = encode_u8_2d(&ta, a.xq, (uint64_t)a.M, (uint64_t)a.K, kBM) &&
                    encode_u8_2d(&tb, a.w, (uint64_t)(pack_ntiles(a.N) * pack_kblocks(a.K) * 128), 128, 128) &&
                    encode_u8_2d(&ty.m[0], hq, (uint64_t)a.M, (uint64_t)(a.N / 2), 32);
    if (!ok) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    if (a.x) return launch_pair<false, true, true>(a, ta, tb, ty, stream, why, h_scale);
    return launch_pair<false, true>(a, ta, tb, ty, stream, why, h_scale);
}

}  // namespace fp8lin
