// Grouped W8A8 GEMM for the MoE expert FFN on tcgen05 (operands swapped, as in umma_swap.cu):
// for every chunk of up to MP routed rows that share an expert e and every 128-channel tile t
//
//     D[128 channels, MP rows] = W_e[tile t, K] . xq[rows, K]^T
//
// The expert's weight tile is the 128-row MMA "A" operand (TMA, packed layout, one 16 KiB box
// per K block); the routed rows are the MMA "N" dimension.  Work items (chunk, tile) come from
// the chunk list moe_align_kernel leaves in device memory, so no host synchronisation is needed;
// the grid is persistent (one CTA per SM) and every CTA strides over the items.
//
// Source of the rows (template flag kGather):
//   true   decode-sized batches of the gate_up projection: the rows are gathered from the bf16
//          token matrix through the sorted row index and quantised on the fly (static scale,
//          exact division) by converter warps straight into the swizzled MMA "B" tile.
//   false  the rows are already e4m3 and contiguous in sorted order (down projection always;
//          gate_up after moe_gather_quant_kernel for prefill-sized batches): one TMA box.
// Epilogue (run-time flag `scatter`):
//   0      gu[sorted position][channel] = bf16(acc * in_scale * w_scale[e][channel])
//   1      out[routed row][channel] = bf16(acc * in_scale * w_scale[e][channel] * topk_w[routed row])
//
// kFused (prefill-sized gate_up only, rows already e4m3): a work item covers the gate tile t AND the up tile t of the
// expert (two weight boxes per K block against one box of rows, two accumulators), and the epilogue writes what the down
// projection reads instead of the bf16 gate_up rows: hq[sorted position][channel] = e4m3(h / h_scale) with
// h = bf16(bf16(silu(g)) * u) from g, u rounded to bf16 -- the values and roundings of the unfused path (the eager
// two-rounding SiluAndMul of the reference's experts).  Half the row bytes per MAC through L2 -> SM, and the bf16 gate_up
// tensor (rows x 2I x 2 bytes each way) and the separate activation pass disappear.
//
// Weight-bandwidth-bound for small batches (each expert's weights are read once per chunk),
// tensor-bound for prefill-sized batches.  All mbarrier waits are bounded.
#include "umma_common.cuh"

namespace fp8lin {

constexpr int kGrpConvWarps = 8;
constexpr int kGrpThreads = (2 + kGrpConvWarps + 4) * 32;
constexpr int kGrpTile = 128;
constexpr int kGrpKB = 128;

template <int MP, bool kFused = false>
struct GroupedCfg {
    static constexpr int kWBytes = kGrpTile * kGrpKB;
    static constexpr int kWTiles = kFused ? 2 : 1;                 // weight boxes per K block (gate and up)
    static constexpr int kXqBytes = MP * kGrpKB;
    static constexpr int kStageBytes = kWTiles * kWBytes + kXqBytes;
    static constexpr int kStagesRaw = (225 * 1024) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
    static constexpr int kAccCols = kWTiles * MP;                  // TMEM columns of one accumulator stage
    static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
    static constexpr int kTeam = MP <= 16 ? 1 : (MP <= 32 ? 2 : 4);
    static constexpr int kPiece = MP < 32 ? MP : 32;            // accumulator columns per TMEM read
    static_assert(kStageBytes % 1024 == 0, "stage alignment");
};

template <int MP, bool kGather, bool kFused = false>
__global__ void __launch_bounds__(kGrpThreads, 1)
grouped_w8a8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_xq, GroupedArgs p) {
    static_assert(!kFused || !kGather, "the fused activation epilogue takes pre-quantised rows");
    using Cfg = GroupedCfg<MP, kFused>;
    constexpr int S = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[S];
    __shared__ __align__(8) uint64_t bar_xq[S];
    __shared__ __align__(8) uint64_t bar_empty[S];
    __shared__ __align__(8) uint64_t bar_tfull[2];
    __shared__ __align__(8) uint64_t bar_tempty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(smem_u32(&bar_full[i]), 1);
            mbar_init(smem_u32(&bar_xq[i]), Cfg::kTeam);
            mbar_init(smem_u32(&bar_empty[i]), 1);
        }
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
    pdl_launch_dependents();
    pdl_wait();                                   // the chunk list, the rows and the outputs all come from predecessors

    const int n_chunks = p.meta[0];
    const int total = n_chunks * p.n_tiles;       // item w = chunk * n_tiles + tile
    const int KB = p.kblocks;

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            if (!kGather) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_xq) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                const int4 ch = p.chunks[w / p.n_tiles];
                const int t = w % p.n_tiles;
                const int wrow0 = (ch.x * p.w_tiles + t) * KB;        // packed tile index of (expert, tile, kb = 0)
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t full = smem_u32(&bar_full[st]);
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    mbar_expect_tx(full, kGather ? Cfg::kWBytes : Cfg::kWTiles * Cfg::kWBytes + Cfg::kXqBytes);
                    tma_load_2d(sa, &tmap_w, 0, (wrow0 + kb) * kGrpTile, full);
                    // fused: the up tile of the same channels sits up_tile_offset tile rows further on in the expert's weight
                    if (kFused) tma_load_2d(sa + Cfg::kWBytes, &tmap_w, 0, (wrow0 + p.up_tile_offset * KB + kb) * kGrpTile, full);
                    if (!kGather) tma_load_2d(sa + Cfg::kWTiles * Cfg::kWBytes, &tmap_xq, kb * kGrpKB, ch.y, full);
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
            constexpr uint32_t idesc = make_idesc_mn(kGrpTile, MP, 0, 0);
            uint32_t it = 0;
            int tl = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++tl) {
                const int as = tl & 1;
                const uint32_t aph = (tl >> 1) & 1;
                if (s_abort || !mbar_wait(smem_u32(&bar_tempty[as]), aph ^ 1, p.status, kDevTimeoutTmemEmpty)) {
                    s_abort = 1; ok = false; break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * Cfg::kAccCols;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_full[st]), ph, p.status, kDevTimeoutFull) ||
                        (kGather && !mbar_wait(smem_u32(&bar_xq[st]), ph, p.status, kDevTimeoutFull))) {
                        s_abort = 1; ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + st * Cfg::kStageBytes;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + Cfg::kWTiles * Cfg::kWBytes);
#pragma unroll
                    for (int k = 0; k < kGrpKB / 32; ++k) {
                        umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        if (kFused)        // the up tile against the same rows, into the second half of the accumulator stage
                            umma_f8(d_tmem + MP, make_smem_desc(sa + Cfg::kWBytes) + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bar_empty[st]));
                }
                if (ok) umma_commit(smem_u32(&bar_tfull[as]));
            }
        }
    } else if (warp < 2 + kGrpConvWarps) {
        // ================= row gather + quantise (gate_up flavour only) =================
        if (kGather) {
            constexpr int kTeams = kGrpConvWarps / Cfg::kTeam;
            const int team = (warp - 2) / Cfg::kTeam;       // a ring slot always belongs to the same team
            const int member = (warp - 2) % Cfg::kTeam;
            const ExactDiv div_scale(fmaxf(__ldg(p.input_scale), 1e-12f));
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                const int4 ch = p.chunks[w / p.n_tiles];
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int st = it % S;
                    if (st % kTeams != team) continue;
                    const uint32_t ph = (it / S) & 1;
                    // the slot's previous MMAs must be done before its "B" tile is overwritten
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t xq = smem_base + st * Cfg::kStageBytes + Cfg::kWBytes;
                    for (int i = member * 32 + lane; i < MP * 8; i += 32 * Cfg::kTeam) {
                        const int r = i >> 3, c = i & 7;
                        const int k = kb * kGrpKB + c * 16;
                        uint2 qa = make_uint2(0u, 0u), qb = make_uint2(0u, 0u);
                        if (r < ch.z && k < p.K) {
                            const int src_row = __ldg(p.sorted_rows + ch.y + r) / p.x_div;
                            const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)src_row * p.ldx + k);
                            qa = quant8_e4m3(__ldg(src), div_scale);
                            qb = quant8_e4m3(__ldg(src + 1), div_scale);
                        }
                        const uint32_t dst = xq + r * 128 + (((uint32_t)c ^ (uint32_t)(r & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(qa.x), "r"(qa.y), "r"(qb.x),
                                     "r"(qb.y) : "memory");
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_xq[st]));
                }
            }
        }
    } else {
        // ================= epilogue (warps 10..13) =================
        const int q = warp & 3;
        const float in_scale = fmaxf(__ldg(p.input_scale), 1e-12f);
        int tl = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++tl) {
            const int4 ch = p.chunks[w / p.n_tiles];
            const int t = w % p.n_tiles;
            const int as = tl & 1;
            const uint32_t aph = (tl >> 1) & 1;
            const int n = t * kGrpTile + q * 32 + lane;                         // output channel of this lane
            const float ws = (!kFused && n < p.N) ? in_scale * __ldg(p.w_scale + (size_t)ch.x * p.N + n) : 0.f;
            // routed-row index and routing weight of the chunk's rows, one row per lane and piece;
            // the inner loop gets them by shuffle instead of two dependent global loads per row
            int my_routed[(MP + 31) / 32];
            float my_w[(MP + 31) / 32];
#pragma unroll
            for (int i = 0; i < (MP + 31) / 32; ++i) {
                const int r = i * 32 + lane;
                my_routed[i] = 0; my_w[i] = 0.f;
                if (p.scatter && r < ch.z) {
                    my_routed[i] = __ldg(p.sorted_rows + ch.y + r);
                    my_w[i] = __ldg(p.topk_w + my_routed[i]);
                }
            }
            if (!mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull)) { s_abort = 1; ok = false; break; }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + as * Cfg::kAccCols;
            if (kFused) {
                // lane = gate channel n of the expert; its up channel is n + N.  One e4m3 byte per row and lane.
                const float wu = n < p.N ? in_scale * __ldg(p.w_scale + (size_t)ch.x * 2 * p.N + p.N + n) : 0.f;
                const float wg = n < p.N ? in_scale * __ldg(p.w_scale + (size_t)ch.x * 2 * p.N + n) : 0.f;
                const ExactDiv div_h(fmaxf(__ldg(p.h_scale), 1e-12f));
#pragma unroll 1
                for (int c0 = 0; c0 < MP; c0 += 32) {
                    if (c0 >= ch.z) break;
                    uint32_t g[32], u[32];
                    __syncwarp();
                    tmem_ld32_nowait(t_addr + c0, g);
                    tmem_ld32_nowait(t_addr + MP + c0, u);
                    tmem_ld_wait();
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (c0 + j < ch.z) {
                                const uint32_t gu = pack_bf16x2(__uint_as_float(g[j]) * wg, __uint_as_float(u[j]) * wu);   // as the bf16 gate_up row
                                const float gv = bf16_lo(gu);
                                const uint32_t sv = pack_bf16x2(gv / (1.f + expf(-gv)), 0.f);                              // bf16(silu(g))
                                const uint32_t hv = pack_bf16x2(bf16_lo(sv) * bf16_hi(gu), 0.f);                           // bf16(. * u)
                                p.hq[(size_t)(ch.y + c0 + j) * p.N + n] = (unsigned char)(cvt_e4m3x2(div_h(bf16_lo(hv)), 0.f) & 0xffu);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < MP; c0 += Cfg::kPiece) {
                if (c0 >= ch.z) break;                                           // uniform: no rows left in this chunk
                uint32_t v[Cfg::kPiece];
                __syncwarp();
                if (Cfg::kPiece == 32) tmem_ld32_nowait(t_addr + c0, v);
                else {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                        : "r"(t_addr + c0) : "memory");
                }
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < Cfg::kPiece; ++j) {
                    const int r = c0 + j;                                       // uniform across the warp
                    const int routed = __shfl_sync(0xffffffffu, my_routed[(c0 + j) / 32], (c0 + j) & 31);
                    const float rw = __shfl_sync(0xffffffffu, my_w[(c0 + j) / 32], (c0 + j) & 31);
                    if (r < ch.z && n < p.N) {
                        const float acc = __uint_as_float(v[j]) * ws;
                        if (!p.scatter) p.out[(size_t)(ch.y + r) * p.ld_out + n] = __float2bfloat16_rn(acc);
                        else p.out[(size_t)routed * p.ld_out + n] = __float2bfloat16_rn(acc * rw);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[as]));
        }
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
template <int MP, bool kGather, bool kFused = false>
static cudaError_t launch_grouped(const GroupedArgs& a, const CUtensorMap& tw, const CUtensorMap& tx, cudaStream_t stream) {
    using Cfg = GroupedCfg<MP, kFused>;
    auto kern = grouped_w8a8_kernel<MP, kGather, kFused>;
    static SmemOptIn opted;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, Cfg::kSmemBytes, opted);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(kGrpThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = pdl_attribute(attr);
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, kern, tw, tx, a));
}

int grouped_chunk_rows(int64_t rows, int num_experts) {
    const int64_t avg = num_experts > 0 ? (rows + num_experts - 1) / num_experts : rows;
    return avg <= 16 ? 16 : (avg <= 32 ? 32 : (avg <= 64 ? 64 : 128));
}

cudaError_t launch_grouped_w8a8(bool gather, int mp, GroupedArgs a, const void* w_packed, int num_experts,
                                const void* xq_sorted, int64_t xq_rows, cudaStream_t stream, const char** why) {
    CUtensorMap tw, tx;
    const bool fused = a.hq != nullptr;           // a.N = I gate channels; the expert's weight holds 2 I channels
    a.n_tiles = (int)pack_ntiles(a.N);
    a.w_tiles = fused ? 2 * a.n_tiles : a.n_tiles;
    a.up_tile_offset = fused ? a.n_tiles : 0;
    a.kblocks = (int)pack_kblocks(a.K);
    if (fused && (gather || a.N % kGrpTile != 0 || mp < 32 || mp > 128)) {
        if (why) *why = "the fused activation epilogue needs pre-quantised rows and an intermediate size that is a multiple of 128";
        return cudaErrorInvalidValue;
    }
    if (!encode_u8_2d(&tw, w_packed, (uint64_t)num_experts * a.w_tiles * a.kblocks * 128, 128, kGrpTile)) {
        if (why) *why = "cuTensorMapEncodeTiled failed for the expert weights";
        return cudaErrorInvalidValue;
    }
    tx = tw;
    if (!gather && !encode_u8_2d(&tx, xq_sorted, (uint64_t)xq_rows, (uint64_t)a.K, (uint32_t)mp)) {
        if (why) *why = "cuTensorMapEncodeTiled failed for the quantised rows";
        return cudaErrorInvalidValue;
    }
#define FP8LIN_GROUPED_CASE(MP_) \
    if (mp == MP_) return fused ? launch_grouped<MP_, false, true>(a, tw, tx, stream) \
                                : (gather ? launch_grouped<MP_, true>(a, tw, tx, stream) : launch_grouped<MP_, false>(a, tw, tx, stream));
    FP8LIN_GROUPED_CASE(16)
    FP8LIN_GROUPED_CASE(32)
    FP8LIN_GROUPED_CASE(64)
    FP8LIN_GROUPED_CASE(128)
#undef FP8LIN_GROUPED_CASE
    if (why) *why = "unsupported chunk size";
    return cudaErrorInvalidValue;
}

}  // namespace fp8lin
