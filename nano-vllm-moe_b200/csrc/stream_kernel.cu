// Weight-streaming FP8 linear for decode-sized M (M <= 64 per pass).
//
// out^T[N, M] = W[N, K] . x^T[K, M]: the weight matrix is the 16-row MMA "A"
// operand and is streamed from HBM exactly once with 128-bit loads straight
// into tensor-core fragments; the (small) activation panel is converted once
// per CTA into shared memory.  HBM-bound: algorithmic bytes per call are
// K*N (weights) + 2*M*K (x) + 2*M*N (y) + 4*N (scale) + 2*N (bias).
//
//  * W8A8: activations are quantised to e4m3 on the fly (static per-tensor
//    scale, true division) and multiplied with the raw e4m3 weight bytes by
//    mma.sync.m16n8k32.e4m3.e4m3.f32.
//  * W8A16: weight bytes are widened in registers with cvt.f16x2.e4m3x2 (exact)
//    and multiplied with f16 activations by mma.sync.m16n8k16.f16.f32.
//
// A warp owns 16 output channels.  Each lane loads 16 consecutive K bytes of
// rows g and g+8; because a dot product does not care about the order of K,
// the lane's 16 bytes are fed to the MMA as the K positions its fragment
// expects, and the activation fragment is read with the same permutation.
//
// K is cut into chunks of kChunk = 256; the CTA double-buffers the converted
// activation chunk in shared memory and keeps the next chunk's weight loads
// in flight in registers while it multiplies the current one.  When N gives
// too few CTAs to fill 148 SMs, K is also split across CTAs (grid.y); each
// split writes fp32 partials to scratch and the last CTA to arrive sums them
// in split order (deterministic) and runs the fused epilogue.  Up to 16 rows
// and eight splits the splits of a channel tile are launched as a cluster
// instead and push their accumulators into split 0's shared memory
// (st.async counted on split 0's mbarrier); split 0 adds them in split order --
// the same sums, without the scratch round trip and the counter.
#include "umma_common.cuh"

namespace fp8lin {

constexpr int kChunk = 256;  // K elements per pipeline step

template <int SCHEME>
struct XTraits;
template <>
struct XTraits<FP8LIN_W8A8_STATIC> {
    static constexpr int kElemBytes = 1;
    static constexpr int kRowBytes = kChunk + 64;       // stride = 64 mod 128 -> conflict-free 16 B reads
};
template <>
struct XTraits<FP8LIN_W8A16> {
    static constexpr int kElemBytes = 2;
    static constexpr int kRowBytes = kChunk * 2 + 16;   // stride = 16 mod 128 -> conflict-free 16 B reads
};

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Number of 16-byte global loads each thread issues to stage one x chunk.
template <int MT, int NWARPS>
struct XStage {
    static constexpr int kRows = MT * 8;
    static constexpr int kVecPerRow = kChunk / 8;                 // 8 bf16 per 16-byte load
    static constexpr int kVecs = kRows * kVecPerRow;
    static constexpr int kThreads = NWARPS * 32;
    static constexpr int kPerThread = (kVecs + kThreads - 1) / kThreads;
};

template <int SCHEME, int MT, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32, (MT >= 4 ? 2 : 4))
stream_linear_kernel(StreamArgs p) {
    using XT = XTraits<SCHEME>;
    using XS = XStage<MT, NWARPS>;
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int kBufBytes = MT * 8 * XT::kRowBytes;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int mz = blockIdx.z;                       // pass over M (64 rows each) when M > 64
    const int m_base = mz * (MT * 8);
    const int m_valid = min(p.M - m_base, MT * 8);   // rows of x that exist in this pass
    const __nv_bfloat16* x = p.x + (size_t)m_base * p.ldx;

    const int n_tile = blockIdx.x;
    const int n_warp0 = n_tile * (NWARPS * 16) + warp * 16;
    const int split = blockIdx.y;
    const int k_beg = split * p.k_per_split;
    const int k_end = min(p.K, k_beg + p.k_per_split);
    const int n_chunks = (k_end - k_beg + kChunk - 1) / kChunk;

    // rows of W this lane streams (clamped: out-of-range rows are computed but never stored)
    const int row_a = min(n_warp0 + g, p.N - 1);
    const int row_b = min(n_warp0 + g + 8, p.N - 1);
    // packed layout: tile (row / 128, k / 128) is 16 KiB contiguous, row r of a tile at r * 128
    const int KB = (p.K + 127) >> 7;
    const unsigned char* wa = p.w + ((size_t)(row_a >> 7) * KB) * kPackTileBytes + (row_a & 127) * 128;
    const unsigned char* wb = p.w + ((size_t)(row_b >> 7) * KB) * kPackTileBytes + (row_b & 127) * 128;
    auto tile_off = [](int k) { return (size_t)(k >> 7) * kPackTileBytes + (k & 127); };

    // cluster form of split-K: split 0 will receive the other splits' accumulators
    __shared__ __align__(8) uint64_t bar_recv;
    const bool push = p.cluster_push != 0;
    uint32_t crank = 0;
    if (push) {
        crank = cluster_ctarank();
        if (threadIdx.x == 0) {
            mbar_init(smem_u32(&bar_recv), 1);
            if (crank == 0) mbar_expect_tx(smem_u32(&bar_recv), (uint32_t)((gridDim.y - 1) * NWARPS * 32 * MT * 16));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
        cluster_arrive();                              // (waited for before the first remote access)
    }

    float in_scale = 1.f;
    if (SCHEME == FP8LIN_W8A8_STATIC) in_scale = fmaxf(__ldg(p.input_scale), 1e-12f);
    const ExactDiv div_scale(in_scale);

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

    // x staging registers; wide-M variants stage a chunk in two halves to stay under 128 registers
    constexpr int kParts = XS::kPerThread > 4 ? 2 : 1;
    constexpr int kPerPart = (XS::kPerThread + kParts - 1) / kParts;
    uint4 xr[kPerPart];
    auto load_x = [&](int chunk, int part) {
        const int k0 = k_beg + chunk * kChunk;
#pragma unroll
        for (int i = 0; i < kPerPart; ++i) {
            const int v = threadIdx.x + (part * kPerPart + i) * XS::kThreads;
            const int r = v / XS::kVecPerRow;
            const int k = k0 + (v % XS::kVecPerRow) * 8;
            xr[i] = make_uint4(0, 0, 0, 0);
            if (v < XS::kVecs && r < m_valid && k < k_end) xr[i] = ld_cached16(x + (size_t)r * p.ldx + k);
        }
    };
    auto store_x = [&](int buf, int part) {
        unsigned char* base = smem + buf * kBufBytes;
#pragma unroll
        for (int i = 0; i < kPerPart; ++i) {
            const int v = threadIdx.x + (part * kPerPart + i) * XS::kThreads;
            if (v >= XS::kVecs) continue;
            const int r = v / XS::kVecPerRow;
            const int c = (v % XS::kVecPerRow) * 8;
            if (SCHEME == FP8LIN_W8A8_STATIC) {
                // rows beyond M (and K tails) were loaded as zeros: nothing to convert
                const bool zero = (xr[i].x | xr[i].y | xr[i].z | xr[i].w) == 0u;
                *reinterpret_cast<uint2*>(base + r * XT::kRowBytes + c) =
                    zero ? make_uint2(0u, 0u) : quant8_e4m3(xr[i], div_scale);
            } else {
                *reinterpret_cast<uint4*>(base + r * XT::kRowBytes + c * 2) = bf16x8_to_f16x8(xr[i]);
            }
        }
    };

    // weight registers: a ring of 4 k-steps of 64 (rows g and g+8).  A slot is
    // refilled with the next chunk's bytes as soon as its MMAs are issued, so
    // about one chunk (4 KB per warp) is always in flight.
    uint4 wr[8];
    auto load_w_step = [&](int chunk, int s) {
        const int k = k_beg + chunk * kChunk + s * 64 + t * 16;
        if (k < k_end) {
            wr[2 * s] = ld_stream16(wa + tile_off(k));
            wr[2 * s + 1] = ld_stream16(wb + tile_off(k));
        } else {
            wr[2 * s] = make_uint4(0, 0, 0, 0);
            wr[2 * s + 1] = make_uint4(0, 0, 0, 0);
        }
    };

#pragma unroll
    for (int s = 0; s < 4; ++s) load_w_step(0, s);       // weights first: they do not depend on the predecessor
    pdl_launch_dependents();
    pdl_wait();                                           // x, y and the split-K scratch may belong to the predecessor
#pragma unroll
    for (int part = 0; part < kParts; ++part) { load_x(0, part); store_x(0, part); }
    __syncthreads();

    for (int c = 0; c < n_chunks; ++c) {
        const bool more = (c + 1 < n_chunks);
        if (more) load_x(c + 1, 0);
        const unsigned char* xb = smem + (c & 1) * kBufBytes;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint4 A = wr[2 * s];      // row g
            const uint4 B = wr[2 * s + 1];  // row g + 8
            if (SCHEME == FP8LIN_W8A8_STATIC) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint4 X = *reinterpret_cast<const uint4*>(xb + (mt * 8 + g) * XT::kRowBytes + s * 64 + t * 16);
                    mma_e4m3(acc[mt], A.x, B.x, A.y, B.y, X.x, X.y);
                    mma_e4m3(acc[mt], A.z, B.z, A.w, B.w, X.z, X.w);
                }
            } else {
                uint32_t fa[8], fb[8];
                fa[0] = cvt_e4m3x2_to_f16x2((uint16_t)(A.x & 0xffff)); fa[1] = cvt_e4m3x2_to_f16x2((uint16_t)(A.x >> 16));
                fa[2] = cvt_e4m3x2_to_f16x2((uint16_t)(A.y & 0xffff)); fa[3] = cvt_e4m3x2_to_f16x2((uint16_t)(A.y >> 16));
                fa[4] = cvt_e4m3x2_to_f16x2((uint16_t)(A.z & 0xffff)); fa[5] = cvt_e4m3x2_to_f16x2((uint16_t)(A.z >> 16));
                fa[6] = cvt_e4m3x2_to_f16x2((uint16_t)(A.w & 0xffff)); fa[7] = cvt_e4m3x2_to_f16x2((uint16_t)(A.w >> 16));
                fb[0] = cvt_e4m3x2_to_f16x2((uint16_t)(B.x & 0xffff)); fb[1] = cvt_e4m3x2_to_f16x2((uint16_t)(B.x >> 16));
                fb[2] = cvt_e4m3x2_to_f16x2((uint16_t)(B.y & 0xffff)); fb[3] = cvt_e4m3x2_to_f16x2((uint16_t)(B.y >> 16));
                fb[4] = cvt_e4m3x2_to_f16x2((uint16_t)(B.z & 0xffff)); fb[5] = cvt_e4m3x2_to_f16x2((uint16_t)(B.z >> 16));
                fb[6] = cvt_e4m3x2_to_f16x2((uint16_t)(B.w & 0xffff)); fb[7] = cvt_e4m3x2_to_f16x2((uint16_t)(B.w >> 16));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const unsigned char* xp = xb + (mt * 8 + g) * XT::kRowBytes + (s * 64 + t * 16) * 2;
                    const uint4 X0 = *reinterpret_cast<const uint4*>(xp);
                    const uint4 X1 = *reinterpret_cast<const uint4*>(xp + 16);
                    mma_f16(acc[mt], fa[0], fb[0], fa[1], fb[1], X0.x, X0.y);
                    mma_f16(acc[mt], fa[2], fb[2], fa[3], fb[3], X0.z, X0.w);
                    mma_f16(acc[mt], fa[4], fb[4], fa[5], fb[5], X1.x, X1.y);
                    mma_f16(acc[mt], fa[6], fb[6], fa[7], fb[7], X1.z, X1.w);
                }
            }
            if (more) {
                load_w_step(c + 1, s);
                if (kParts == 2 && s == 1) { store_x((c + 1) & 1, 0); load_x(c + 1, 1); }
            }
        }
        if (more) store_x((c + 1) & 1, kParts - 1);
        __syncthreads();
    }

    // ---- epilogue ------------------------------------------------------------
    // acc[mt][0..3] = (n=g, m=2t), (n=g, m=2t+1), (n=g+8, m=2t), (n=g+8, m=2t+1)
    const int n_a = n_warp0 + g;
    const int n_b = n_warp0 + g + 8;
    const int n_splits = gridDim.y;

    if (n_splits > 1 && push) {
        cluster_wait();
        const uint32_t recv = smem_u32(smem) + 2 * kBufBytes;           // behind the x double buffer: [split - 1][thread][MT][4]
        if (crank != 0) {
            const uint32_t dst = map_to_cta(recv + ((crank - 1) * (NWARPS * 32) + threadIdx.x) * (MT * 16), 0);
            const uint32_t rbar = map_to_cta(smem_u32(&bar_recv), 0);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                st_async_v4(dst + mt * 16, __float_as_uint(acc[mt][0]), __float_as_uint(acc[mt][1]), __float_as_uint(acc[mt][2]),
                            __float_as_uint(acc[mt][3]), rbar);
            return;
        }
        if (!mbar_wait(smem_u32(&bar_recv), 0, p.status, kDevTimeoutPeer)) return;
        for (int s = 1; s < n_splits; ++s) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const float4 v = ld_shared_f4(recv + ((s - 1) * (NWARPS * 32) + threadIdx.x) * (MT * 16) + mt * 16);
                acc[mt][0] += v.x; acc[mt][1] += v.y; acc[mt][2] += v.z; acc[mt][3] += v.w;
            }
        }
    } else if (n_splits > 1) {
        // partial[split][mz][n][MT*8] fp32
        constexpr int MP = MT * 8;
        float* part = p.partial + ((size_t)(split * gridDim.z + mz) * p.N) * MP;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int m = mt * 8 + 2 * t;
            if (n_a < p.N) __stcg(reinterpret_cast<float2*>(part + (size_t)n_a * MP + m), make_float2(acc[mt][0], acc[mt][1]));
            if (n_b < p.N) __stcg(reinterpret_cast<float2*>(part + (size_t)n_b * MP + m), make_float2(acc[mt][2], acc[mt][3]));
        }
        __threadfence();
        __syncthreads();
        __shared__ int s_last;
        int* counter = p.counters + mz * gridDim.x + n_tile;
        if (threadIdx.x == 0) {
            const int prev = atomicAdd(counter, 1);
            s_last = (prev == n_splits - 1);
            if (s_last) *counter = 0;  // leave the scratch header zeroed for the next call
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f; }
        for (int s = 0; s < n_splits; ++s) {
            const float* ps = p.partial + ((size_t)(s * gridDim.z + mz) * p.N) * MP;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int m = mt * 8 + 2 * t;
                if (n_a < p.N) {
                    const float2 v = __ldcg(reinterpret_cast<const float2*>(ps + (size_t)n_a * MP + m));
                    acc[mt][0] += v.x; acc[mt][1] += v.y;
                }
                if (n_b < p.N) {
                    const float2 v = __ldcg(reinterpret_cast<const float2*>(ps + (size_t)n_b * MP + m));
                    acc[mt][2] += v.x; acc[mt][3] += v.y;
                }
            }
        }
    }

    __nv_bfloat16* y = p.y + (size_t)m_base * p.ldy;
    float sa = 0.f, sb = 0.f, ba = 0.f, bb = 0.f;
    if (n_a < p.N) { sa = __ldg(p.w_scale + n_a); if (p.bias) ba = __bfloat162float(p.bias[n_a]); }
    if (n_b < p.N) { sb = __ldg(p.w_scale + n_b); if (p.bias) bb = __bfloat162float(p.bias[n_b]); }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + 2 * t;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (m + j >= m_valid) continue;
            float va = acc[mt][j], vb = acc[mt][2 + j];
            if (SCHEME == FP8LIN_W8A8_STATIC) { va *= in_scale; vb *= in_scale; }
            if (n_a < p.N) y[(size_t)(m + j) * p.ldy + n_a] = __float2bfloat16_rn(fmaf(va, sa, ba));
            if (n_b < p.N) y[(size_t)(m + j) * p.ldy + n_b] = __float2bfloat16_rn(fmaf(vb, sb, bb));
        }
    }
}

template <int SCHEME, int MT, int NWARPS>
static cudaError_t launch_one(const StreamArgs& a, dim3 grid, cudaStream_t stream) {
    const int smem = 2 * MT * 8 * XTraits<SCHEME>::kRowBytes + (a.cluster_push ? ((int)grid.y - 1) * NWARPS * 32 * MT * 16 : 0);
    auto kern = stream_linear_kernel<SCHEME, MT, NWARPS>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NWARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = pdl_attribute(attr);
    if (a.cluster_push) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = grid.y;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.numAttrs = na;
    cfg.attrs = attr;
    return counted(cudaLaunchKernelEx(&cfg, kern, a));
}

static int g_stream_push = 1;
void set_stream_push(int on) { g_stream_push = on; }

StreamPlan plan_stream(int scheme, int64_t M, int64_t K, int64_t N, int force_splits) {
    StreamPlan pl;
    const int mpass = (int)(M < 64 ? M : 64);
    pl.mt = mpass <= 8 ? 1 : mpass <= 16 ? 2 : mpass <= 32 ? 4 : 8;
    pl.nwarps = pl.mt >= 4 ? 8 : 4;
    pl.m_passes = (int)((M + pl.mt * 8 - 1) / (pl.mt * 8));
    const int bn = pl.nwarps * 16;
    pl.n_tiles = (int)((N + bn - 1) / bn);
    const int chunks = (int)((K + kChunk - 1) / kChunk);
    // aim for about four resident CTAs per SM (two for the wide-M variants)
    const int target = sm_count() * (pl.mt >= 4 ? 2 : 4);
    const int tiles = pl.n_tiles * pl.m_passes;
    int splits = force_splits > 0 ? force_splits : (target + tiles / 2) / tiles;
    if (splits < 1) splits = 1;
    // keep at least two chunks per split so the register prefetch has something to overlap
    const int max_splits = chunks >= 2 ? chunks / 2 : 1;
    if (force_splits <= 0 && splits > max_splits) splits = max_splits;
    // up to 16 rows the splits of a tile run as a cluster (at most eight CTAs) that hands its partial sums over in shared
    // memory: eight such slices beat eleven through global scratch (18944 -> 3584 at one row: 15.8 us against 17.8)
    if (force_splits <= 0 && pl.mt <= 2 && splits > 8) splits = 8;
    if (splits > chunks) splits = chunks;
    const int chunks_per_split = (chunks + splits - 1) / splits;
    pl.k_per_split = chunks_per_split * kChunk;
    pl.splits = (chunks + chunks_per_split - 1) / chunks_per_split;
    if ((size_t)tiles > (size_t)kWsMaxCounters) pl.splits = 1, pl.k_per_split = chunks * kChunk;
    pl.partial_bytes = pl.splits > 1 ? (size_t)pl.splits * pl.m_passes * N * (pl.mt * 8) * sizeof(float) : 0;
    (void)scheme;
    return pl;
}

cudaError_t launch_stream(int scheme, const StreamPlan& pl, StreamArgs a, cudaStream_t stream) {
    a.k_per_split = pl.k_per_split;
    a.cluster_push = (g_stream_push && a.status && pl.splits > 1 && pl.splits <= 8 && pl.mt <= 2) ? 1 : 0;
    dim3 grid(pl.n_tiles, pl.splits, pl.m_passes);
#define FP8LIN_STREAM_CASE(S, MT_, NW_) \
    if (scheme == S && pl.mt == MT_) return launch_one<S, MT_, NW_>(a, grid, stream);
    FP8LIN_STREAM_CASE(FP8LIN_W8A8_STATIC, 1, 4)
    FP8LIN_STREAM_CASE(FP8LIN_W8A8_STATIC, 2, 4)
    FP8LIN_STREAM_CASE(FP8LIN_W8A8_STATIC, 4, 8)
    FP8LIN_STREAM_CASE(FP8LIN_W8A8_STATIC, 8, 8)
    FP8LIN_STREAM_CASE(FP8LIN_W8A16, 1, 4)
    FP8LIN_STREAM_CASE(FP8LIN_W8A16, 2, 4)
    FP8LIN_STREAM_CASE(FP8LIN_W8A16, 4, 8)
    FP8LIN_STREAM_CASE(FP8LIN_W8A16, 8, 8)
#undef FP8LIN_STREAM_CASE
    return cudaErrorInvalidValue;
}

}  // namespace fp8lin
