// Grouped W8A8 GEMM for prefill-sized MoE batches, with the routed rows as the MMA's M dimension.
//
// The decode-oriented grouped kernel (umma_grouped.cu) makes the expert's 128 weight channels the MMA M and the
// few rows the MMA N.  With 128-row chunks that orientation moves 32 KB through L2 -> SM per 128 x 128 x 128 MACs
// and ends in an epilogue whose lanes are channels: every row costs a 64-byte store per warp.  Here a work item is
//
//     D[128 rows, 256 channels] = xq[chunk rows, K] . W_e[256 channels, K]^T
//
// (48 KB per 128 x 256 x 128 MACs), the accumulator's TMEM lanes are rows, and an epilogue thread owns one routed
// row: it reads that row's index and routing weight once and writes 32 consecutive channels (64 bytes) at a time.
//
//   kFusedAct = true   gate_up: the item's 256 channels are gate tile t and up tile t of the expert (two weight boxes
//                      from two places of the packed weight, no re-packing); the epilogue writes
//                      hq[sorted position][128 t + c] = e4m3( bf16(bf16(silu(g)) * u) / h_scale ), g and u rounded to
//                      bf16 first -- the same values and roundings as the separate activation pass.
//   kFusedAct = false  down: out[routed row][n] = bf16( acc * in_scale * w_scale[e][n] * topk_w[routed row] ).
//
// Chunks are the 128-row chunks of moe_align_kernel's list; rows of a chunk's 128-row box beyond its own rows belong
// to the next chunk (or lie past the end and read as zeros): they are multiplied but never stored.  Persistent, one CTA
// per SM, TMA producer / MMA issuer / 8 epilogue warps, two accumulator stages in TMEM; every mbarrier wait is bounded.
#include "umma_common.cuh"

namespace fp8lin {

namespace {

constexpr int kRowsM = 128;
constexpr int kColsN = 256;
constexpr int kKB = 128;
constexpr int kEpiWarpsR = 8;
constexpr int kThreadsR = (2 + kEpiWarpsR) * 32;
constexpr int kABytesR = kRowsM * kKB;
constexpr int kBBytesR = kColsN * kKB;
constexpr int kStageBytesR = kABytesR + kBBytesR;
constexpr int kStagesR = 4;
constexpr int kSmemBytesR = kStagesR * kStageBytesR + 1024;
constexpr int kTmemColsR = 2 * kColsN;

template <bool kFusedAct>
__global__ void __launch_bounds__(kThreadsR, 1)
grouped_rows_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_xq, GroupedArgs p) {
    constexpr int S = kStagesR;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[S];
    __shared__ __align__(8) uint64_t bar_empty[S];
    __shared__ __align__(8) uint64_t bar_tfull[2];
    __shared__ __align__(8) uint64_t bar_tempty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile int s_abort;
    __shared__ __align__(16) float s_scale[kColsN];

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(smem_u32(&bar_full[i]), 1); mbar_init(smem_u32(&bar_empty[i]), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&bar_tfull[i]), 1); mbar_init(smem_u32(&bar_tempty[i]), kEpiWarpsR); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), kTmemColsR);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    pdl_launch_dependents();
    pdl_wait();                                   // the chunk list, the rows and the outputs all come from predecessors

    const int n_chunks = p.meta[0];
    const int n_items = p.n_tiles;                // channel items per chunk (set by the launcher)
    const int total = n_chunks * n_items;         // item w = chunk * n_items + t
    const int KB = p.kblocks;
    // 128-channel weight boxes of item t: fused = gate tile t and up tile t; plain = tiles 2t and 2t + 1 (the second may not exist)
    auto sub_tile = [&](int t, int s) { return kFusedAct ? (s == 0 ? t : p.up_tile_offset + t) : 2 * t + s; };
    auto n_sub = [&](int t) { return (kFusedAct || 2 * t + 1 < p.w_tiles) ? 2 : 1; };

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_xq) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                const int4 ch = p.chunks[w / n_items];
                const int t = w % n_items;
                const int ns = n_sub(t);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1, p.status, kDevTimeoutEmpty)) {
                        s_abort = 1; ok = false; break;
                    }
                    const uint32_t full = smem_u32(&bar_full[st]);
                    const uint32_t sa = smem_base + st * kStageBytesR;
                    mbar_expect_tx(full, (uint32_t)(kABytesR + ns * kRowsM * kKB));
                    tma_load_2d(sa, &tmap_xq, kb * kKB, ch.y, full);
                    for (int s = 0; s < ns; ++s)
                        tma_load_2d(sa + kABytesR + s * 128 * kKB, &tmap_w, 0, ((ch.x * p.w_tiles + sub_tile(t, s)) * KB + kb) * 128, full);
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
            uint32_t it = 0;
            int tl = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++tl) {
                const int t = w % n_items;
                const uint32_t idesc = make_idesc_mn(kRowsM, n_sub(t) * 128, 0, 0);
                const int as = tl & 1;
                const uint32_t aph = (tl >> 1) & 1;
                if (s_abort || !mbar_wait(smem_u32(&bar_tempty[as]), aph ^ 1, p.status, kDevTimeoutTmemEmpty)) {
                    s_abort = 1; ok = false; break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * kColsN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int st = it % S;
                    const uint32_t ph = (it / S) & 1;
                    if (s_abort || !mbar_wait(smem_u32(&bar_full[st]), ph, p.status, kDevTimeoutFull)) {
                        s_abort = 1; ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + st * kStageBytesR;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + kABytesR);
#pragma unroll
                    for (int k = 0; k < kKB / 32; ++k) umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&bar_empty[st]));
                }
                if (ok) umma_commit(smem_u32(&bar_tfull[as]));
            }
        }
    } else {
        // ================= epilogue (warps 2..9): a thread owns one row of the chunk =================
        const int ew = warp - 2;
        const int q = warp & 3;                   // TMEM lane quarter = rows [32q, 32q + 32) of the item
        const int h = ew >> 2;                    // column half of the item
        const int et = threadIdx.x - 64;          // 0..255 among the epilogue threads: stages column et's multiplier
        const float in_scale = fmaxf(__ldg(p.input_scale), 1e-12f);
        const ExactDiv div_h(kFusedAct ? fmaxf(__ldg(p.h_scale), 1e-12f) : 1.f);
        int tl = 0;
        bool ok = true;
        auto column_scale = [&](int work) -> float {
            const int4 c = p.chunks[work / n_items];
            const int t = work % n_items;
            if (kFusedAct) {                      // columns [0,128) gate channels 128 t + c, [128,256) the up channels of the same c
                const int ch_idx = t * 128 + (et & 127);
                return ch_idx < p.N ? in_scale * __ldg(p.w_scale + (size_t)c.x * 2 * p.N + (et >> 7) * p.N + ch_idx) : 0.f;
            }
            const int n = t * kColsN + et;
            return n < p.N ? in_scale * __ldg(p.w_scale + (size_t)c.x * p.N + n) : 0.f;
        };
        float next_scale = blockIdx.x < total ? column_scale(blockIdx.x) : 0.f;
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++tl) {
            const int4 ch = p.chunks[w / n_items];
            const int t = w % n_items;
            const int as = tl & 1;
            const uint32_t aph = (tl >> 1) & 1;
            if (tl > 0) asm volatile("bar.sync 1, 256;" ::: "memory");        // everybody is done with the previous multipliers
            s_scale[et] = next_scale;
            if (w + (int)gridDim.x < total) next_scale = column_scale(w + gridDim.x);
            const int r = q * 32 + lane;                                      // this thread's row of the chunk
            const bool live = r < ch.z;
            int routed = 0;
            float rw = 0.f;
            if (!kFusedAct && live) {
                routed = __ldg(p.sorted_rows + ch.y + r);
                rw = __ldg(p.topk_w + routed);
            }
            const bool arrived = mbar_wait(smem_u32(&bar_tfull[as]), aph, p.status, kDevTimeoutTmemFull);
            uint32_t any_failed;                                              // publishes the multipliers and takes the vote
            asm volatile(
                "{\n .reg .pred pin, pout;\n setp.ne.b32 pin, %1, 0;\n"
                " barrier.cta.red.or.pred pout, 1, 256, pin;\n selp.u32 %0, 1, 0, pout;\n}"
                : "=r"(any_failed) : "r"(arrived ? 0u : 1u) : "memory");
            if (any_failed) { s_abort = 1; ok = false; break; }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * kColsN;
            if (kFusedAct) {
                // warp h: gate columns [64h, 64h + 64) and the up columns 128 further on -> 64 bytes of the row's hq
                unsigned char* dst = p.hq + (size_t)(ch.y + r) * p.N + t * 128 + h * 64;
#pragma unroll 1
                for (int sp = 0; sp < 2; ++sp) {
                    const int c = h * 64 + sp * 32;
                    uint32_t g[32], u[32];
                    __syncwarp();
                    tmem_ld32_nowait(t_row + c, g);
                    tmem_ld32_nowait(t_row + 128 + c, u);
                    tmem_ld_wait();
                    uint32_t out[8];
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        uint32_t word = 0;
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            const uint32_t gu = pack_bf16x2(__uint_as_float(g[j + b]) * s_scale[c + j + b],
                                                            __uint_as_float(u[j + b]) * s_scale[128 + c + j + b]);   // as the bf16 gate_up row
                            const float gv = bf16_lo(gu);
                            const uint32_t sv = pack_bf16x2(gv / (1.f + expf(-gv)), 0.f);                          // bf16(silu(g))
                            const uint32_t hv = pack_bf16x2(bf16_lo(sv) * bf16_hi(gu), 0.f);                       // bf16(. * u)
                            word |= (uint32_t)(cvt_e4m3x2(div_h(bf16_lo(hv)), 0.f) & 0xffu) << (8 * b);
                        }
                        out[j / 4] = word;
                    }
                    if (live) {
                        uint4* d4 = reinterpret_cast<uint4*>(dst + sp * 32);
                        d4[0] = make_uint4(out[0], out[1], out[2], out[3]);
                        d4[1] = make_uint4(out[4], out[5], out[6], out[7]);
                    }
                }
            } else {
                __nv_bfloat16* dst = p.out + (size_t)routed * p.ld_out + t * kColsN + h * 128;
                const int n_left = p.N - (t * kColsN + h * 128);              // channels of this half that exist
#pragma unroll 1
                for (int sp = 0; sp < 4; ++sp) {
                    const int c = h * 128 + sp * 32;
                    if (sp * 32 >= n_left) break;                             // uniform
                    uint32_t v[32];
                    __syncwarp();
                    tmem_ld32_nowait(t_row + c, v);
                    tmem_ld_wait();
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        o[j / 2] = pack_bf16x2(__uint_as_float(v[j]) * s_scale[c + j] * rw, __uint_as_float(v[j + 1]) * s_scale[c + j + 1] * rw);
                    if (live) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (sp * 32 + j * 8 < n_left)                     // N is a multiple of 8: whole 16-byte pieces
                                reinterpret_cast<uint4*>(dst + sp * 32)[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
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
        tmem_dealloc(tmem_base, kTmemColsR);
    }
}

template <bool kFusedAct>
cudaError_t launch_rows(const GroupedArgs& a, const CUtensorMap& tw, const CUtensorMap& tx, cudaStream_t stream) {
    auto kern = grouped_rows_kernel<kFusedAct>;
    static SmemOptIn opted;
    {
        cudaError_t e = ensure_dynamic_smem((const void*)kern, kSmemBytesR, opted);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(kThreadsR);
    cfg.dynamicSmemBytes = kSmemBytesR;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = pdl_attribute(attr);
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, kern, tw, tx, a));
}

}  // namespace

// a.N: output channels of the projection (down) or the intermediate size I (fused gate_up: the expert's weight holds 2 I
// channels); a.hq / a.h_scale set = the fused gate_up flavour.  The chunk list must have been made with 128-row chunks.
cudaError_t launch_grouped_rows_w8a8(GroupedArgs a, const void* w_packed, int num_experts, const void* xq_sorted,
                                     int64_t xq_rows, cudaStream_t stream, const char** why) {
    const bool fused = a.hq != nullptr;
    if ((fused && a.N % 128 != 0) || (!fused && (a.N % 8 != 0 || a.ld_out % 8 != 0))) {
        if (why) *why = "row-major grouped GEMM: the intermediate size must be a multiple of 128 / the output width a multiple of 8";
        return cudaErrorInvalidValue;
    }
    a.kblocks = (int)pack_kblocks(a.K);
    if (fused) {
        a.n_tiles = a.N / 128;                    // items per chunk: one per gate tile
        a.w_tiles = 2 * a.n_tiles;
        a.up_tile_offset = a.n_tiles;
    } else {
        a.w_tiles = (int)pack_ntiles(a.N);
        a.n_tiles = (a.w_tiles + 1) / 2;          // items per chunk: 256 channels each
        a.up_tile_offset = 0;
    }
    CUtensorMap tw, tx;
    if (!encode_u8_2d(&tw, w_packed, (uint64_t)num_experts * a.w_tiles * a.kblocks * 128, 128, 128) ||
        !encode_u8_2d(&tx, xq_sorted, (uint64_t)xq_rows, (uint64_t)a.K, kRowsM)) {
        if (why) *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    return fused ? launch_rows<true>(a, tw, tx, stream) : launch_rows<false>(a, tw, tx, stream);
}

}  // namespace fp8lin
