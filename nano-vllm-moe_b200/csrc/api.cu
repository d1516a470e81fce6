// extern "C" surface of libfp8lin.so (declared in include/fp8lin.h).
#include <stdarg.h>
#include <atomic>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"

using namespace fp8lin;

namespace {

thread_local char g_err[256] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

struct Tuning {
    int stream_splits = -1;   // force split-K factor of the streaming kernel
    int stream_max_m = -1;    // largest M routed to the streaming kernel (W8A8)
    int umma_bn = -1;         // force tile width of the tcgen05 kernel
    int umma_splits = -1;     // force split-K factor of the tcgen05 kernel
    int swap_splits = -1;     // force split-K factor of the swapped-operand decode kernel
    int swap_enable = -1;     // 0 routes decode-sized W8A8 to the mma.sync streaming kernel instead
    int swap_min_m = -1;      // smallest M routed to the swapped-operand kernel
    int swap_preq_min_m = -1; // smallest M for which that kernel takes pre-quantised activations
    int w8a16_swap_enable = -1; // 0 keeps W8A16 on the mma.sync streaming kernel for every M
    int w8a16_swap_min_m = -1;
    int w8a16_umma_min_m = -1;  // smallest M for the dequantise-to-f16 + tcgen05 GEMM route (0 = never)
    int w8a16_chunk_mb = -1;    // size of the f16 weight chunk that route keeps in L2
    int umma_pair = -1;         // 1 = large-M GEMMs on CTA pairs (256 x 256 tiles), 0 = never
    int fuse_quant = -1;        // large-M W8A8: <= 0 (default) = quantise x in a separate pass; 1 = the pass takes the rows
                                // of the first round of tiles, the GEMM's own quantiser warps the rest; n > 1 = the pass
                                // takes the first n rows (rounded up to 128)
    int moe_rows_major = -1;    // 0 = prefill-sized expert batches stay on the channel-major grouped kernel
    int mlp_decode_fused = -1;  // 1 = the fused MLP on up to 16 pre-quantised rows computes silu * up in the gate_up kernel (study knob)
    int moe_fused = -1;         // 0 = the expert FFN keeps its separate silu-multiply-quantise pass for every batch size
    int quant_lead = -1;        // row blocks the in-kernel quantiser may run ahead (default: from the tile schedule)
} g_tune;

constexpr int kDefaultStreamMaxM = 64;

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_arch() {
    static int cached = -1;
    if (cached >= 0) return cached;
    int dev = 0;
    cudaDeviceProp prop;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return cached = 0;
    return cached = (prop.major == 10) ? 1 : 0;
}

int validate_common(const void* x, int64_t ldx, const void* w, const float* w_scale, const void* bias, void* y,
                    int64_t ldy, int64_t M, int64_t K, int64_t N) {
    if (M < 0 || K <= 0 || N <= 0) return fail(FP8LIN_ERR_SHAPE, "bad shape M=%lld K=%lld N=%lld", (long long)M, (long long)K, (long long)N);
    if (M > (1ll << 30) || K > (1ll << 30) || N > (1ll << 30)) return fail(FP8LIN_ERR_SHAPE, "dimension too large");
    if (K % 16 != 0) return fail(FP8LIN_ERR_SHAPE, "K=%lld must be a multiple of 16", (long long)K);
    if (M == 0) return FP8LIN_OK;
    if (!x || !w || !w_scale || !y) return fail(FP8LIN_ERR_NULL, "x, w_nk, w_scale and y must not be NULL");
    if (ldx < K || ldy < N) return fail(FP8LIN_ERR_SHAPE, "ldx=%lld < K or ldy=%lld < N", (long long)ldx, (long long)ldy);
    if (ldx % 8 != 0) return fail(FP8LIN_ERR_ALIGN, "ldx=%lld must be a multiple of 8 elements", (long long)ldx);
    if (!aligned16(x) || !aligned16(w) || !aligned16(w_scale) || (bias && !aligned16(bias)))
        return fail(FP8LIN_ERR_ALIGN, "x, w_nk, w_scale and bias must be 16-byte aligned");
    if (!check_arch()) return fail(FP8LIN_ERR_ARCH, "fp8lin kernels are built for sm_100a only");
    return FP8LIN_OK;
}

bool w8a16_swap_eligible(int64_t M, int64_t N) {
    // measured (us, mma.sync kernel / tcgen05 kernel): at 32 rows 3584 -> 4608 11.4 / 10.4, 3584 -> 3584 11.4 / 9.1,
    // 18944 -> 3584 29.8 / 23.5, 3584 -> 37888 34.1 / 34.4; at 16 rows 9.5 / 9.7, 9.4 / 8.5, 21.6 / 22.7, 26.8 / 33.6;
    // at 64 rows on 3584 -> 37888 67 / 38.  So: from 17 rows, from 33 when there is a channel tile for every SM.
    const int wide = (N + 127) / 128 >= fp8lin::sm_count();
    const int min_m = g_tune.w8a16_swap_min_m >= 0 ? g_tune.w8a16_swap_min_m : (wide ? 33 : 17);
    return g_tune.w8a16_swap_enable != 0 && M >= min_m && M <= 64;
}

// Large-M W8A16: channel chunks of the weights are widened to f16 into scratch (small enough to stay
// in L2) and multiplied by the tcgen05 f16 GEMM; below this many rows the 64-row passes of the
// mma.sync kernel are cheaper than the per-chunk launches.
bool w8a16_umma_eligible(int64_t M, int64_t K, int64_t N, int64_t ldy, const void* y) {
    // measured on 3584 -> 37888: 128 rows 237 vs 132 us (passes win), 256 rows 270 vs 261 us (equal;
    // 32 vs 38 us on 3584 -> 4608), 1024 rows 319 vs 1032 us, 4096 rows 0.90 vs 4.1 ms
    const int min_m = g_tune.w8a16_umma_min_m >= 0 ? g_tune.w8a16_umma_min_m : 256;
    return min_m > 0 && M >= min_m && K % 8 == 0 && N % 8 == 0 && ldy % 8 == 0 && aligned16(y);
}

struct F16Chunks {
    int64_t chunk_tiles;     // 128-channel tile rows per chunk (even: a chunk is a multiple of 256 channels)
    int64_t n_chunks;
    size_t x16_bytes, w16_bytes;
};

F16Chunks plan_f16_chunks(int64_t M, int64_t K, int64_t N) {
    F16Chunks c;
    const int64_t ntiles = fp8lin::pack_ntiles(N);
    const size_t tile_row_bytes = (size_t)fp8lin::pack_kblocks(K) * 2 * fp8lin::kPackTileBytes;   // f16 bytes of 128 channels
    const size_t budget = (size_t)(g_tune.w8a16_chunk_mb > 0 ? g_tune.w8a16_chunk_mb : 64) << 20;
    // Chunks are counted in 256-channel column blocks (the GEMM's widest tile).  Every chunk is its own
    // GEMM launch of m_tiles x blocks tiles over 148 SMs, so the chunk size decides how many rounds of
    // tiles the whole call takes: try every size that fits the budget and keep the cheapest, a round
    // costing one tile's main loop and a chunk a fixed launch/ramp overhead.
    const int64_t nblocks = (ntiles + 1) / 2;
    int64_t max_blocks = (int64_t)(budget / (2 * tile_row_bytes));
    if (max_blocks < 1) max_blocks = 1;
    if (max_blocks > nblocks) max_blocks = nblocks;
    const int64_t m_tiles = (M + 127) / 128;
    const double t_tile = (double)fp8lin::pack_kblocks(K) * 2 * 0.115;     // us per 128x256 tile (64-element K blocks)
    auto rounds_of = [&](int64_t blocks) -> double {
        const int64_t tiles = m_tiles * blocks;
        if (tiles > (sm_count() / 2)) return (double)((tiles + (sm_count() - 1)) / sm_count());
        int64_t splits = sm_count() / tiles;                                       // few tiles: cluster split-K
        if (splits > 8) splits = 8;
        return 1.0 / (double)splits + 0.15;
    };
    double best_cost = 1e30;
    int64_t best_blocks = max_blocks;
    for (int64_t b = max_blocks; b >= 1 && b * 4 >= max_blocks; --b) {
        const int64_t full = nblocks / b, rest = nblocks - full * b;
        const double cost = (double)full * (rounds_of(b) * t_tile + 8.0) + (rest ? rounds_of(rest) * t_tile + 8.0 : 0.0);
        if (cost < best_cost - 1e-9) { best_cost = cost; best_blocks = b; }
    }
    const int64_t per = 2 * best_blocks;
    c.chunk_tiles = per;
    c.n_chunks = (ntiles + per - 1) / per;
    c.x16_bytes = align_up((size_t)M * K * 2, 256);
    c.w16_bytes = (size_t)per * tile_row_bytes;
    return c;
}

// CTA-pair GEMM (256 x 256 tiles over two SMs) instead of the one-CTA kernel.
// Measured (W8A8, same bits as the one-CTA kernel): 4096 x 3584 -> 37888 449 vs 470 us, 16384 rows 1911 vs
// 1980 us; but 4096 x 18944 -> 3584 (224 pair tiles = 3.03 rounds of 74 pairs) 294 vs 260 us and
// 1024 x 2048 -> 11008 28.7 vs 26.1 us.  So: only when there are at least four rounds of pair tiles and the
// last round is nearly full, and no worse filled than the one-CTA kernel's.
bool pair_eligible(int64_t M, int64_t N) {
    if (g_tune.umma_pair >= 0) return g_tune.umma_pair != 0 && M > 64;
    const int64_t nt = (N + 255) / 256;
    const int64_t pt = ((M + 255) / 256) * nt;
    const int64_t tiles = ((M + 127) / 128) * nt;
    if (pt < 4 * (sm_count() / 2)) return false;
    const double pair_fill = (double)pt / (double)(((pt + (sm_count() / 2 - 1)) / (sm_count() / 2)) * (sm_count() / 2));
    const double one_fill = (double)tiles / (double)(((tiles + (sm_count() - 1)) / sm_count()) * sm_count());
    return pair_fill >= 0.95 && pair_fill >= one_fill - 1e-9;
}

bool swap_eligible(int64_t M, int64_t K, int64_t N) {
    const int max_m = g_tune.stream_max_m >= 0 ? g_tune.stream_max_m : kDefaultStreamMaxM;
    // The tcgen05 kernel from the first row on, except on layers of up to ~17 MB with a short K (qkv, o_proj), where up to
    // 8 rows the mma.sync streaming kernel -- many small CTAs, its split-K slices handing their sums over inside a
    // cluster -- starts and drains faster.  Measured at one row / eight rows, us, tcgen05 against streaming kernel:
    // 3584 -> 4608 6.8 / 7.1 against 6.0 / 6.5, 3584 -> 3584 5.8 / 6.3 against 5.1 / 5.5, 4736 -> 3584 6.9 against 6.5
    // (four rows), 2048 -> 2048 4.1 against 4.0; but 2048 -> 11008 7.2 / 7.4 against 9.1 / 9.7, 11008 -> 2048 8.3 against
    // 9.6, 18944 -> 3584 14.9 / 15.2 against 16.6 / 19.0, 3584 -> 37888 21.7 against 24.0.
    int min_m = g_tune.swap_min_m >= 0 ? g_tune.swap_min_m : 1;
    if (g_tune.swap_min_m < 0 && K <= 8192 && N <= 4736) min_m = 9;
    return g_tune.swap_enable != 0 && M >= min_m && M <= 64 && M <= max_m;
}

// from this many rows on the swapped-operand kernel takes pre-quantised rows (one extra small
// pass, but nine ring slots instead of five or seven; measured faster from 17 rows up)
bool swap_prequant(int64_t M) {
    const int min_m = g_tune.swap_preq_min_m >= 0 ? g_tune.swap_preq_min_m : 17;
    return M >= min_m;
}

// Large-M W8A8 with the activation quantiser inside the GEMM: a short pass quantises the rows that the first
// round of tiles reads (tiles are walked in groups of eight tile rows), the kernel's quantiser warps do the
// rest while the tensor cores run.  Returns the number of rows for the pass; M = everything (no fusion).
int64_t prequant_rows(int64_t M, int64_t n_tiles, int tile_rows, int first_round_tiles) {
    // Off unless asked for.  Measured on a B200 (same process, alternating windows, 7B layer shapes at 4096 / 8192 /
    // 16384 rows): with the quantiser inside the GEMM qkv 77 / 141 / 274 us against 74 / 142 / 277 us with the
    // separate pass, o_proj 68 / 124 / 235 against 65 / 122 / 232, gate_up 511 / 1017 / 2045 against 513 / 1021 /
    // 2040, down 328 / 607 / 1180 against 296 / 579 / 1150.  These GEMMs run at the board's power limit (SM clock
    // 1.25-1.5 GHz of 1.965): hiding the pass does not remove its energy, the clock drops by what the extra warps
    // draw, and the pass alone runs at a power the GEMM never sees.
    if (g_tune.fuse_quant <= 0 || 3 + (M + 127) / 128 > kWsMaxCounters) return M;
    if (g_tune.fuse_quant > 1) {                      // forced split (tests): this many rows, rounded up to a row block
        const int64_t forced = ((int64_t)g_tune.fuse_quant + 127) / 128 * 128;
        return forced >= M ? M : forced;
    }
    const int64_t m_tiles = (M + tile_rows - 1) / tile_rows;
    const int64_t total = m_tiles * n_tiles;
    const int64_t first = total < first_round_tiles ? total : first_round_tiles;
    const int64_t groups = (first + 8 * n_tiles - 1) / (8 * n_tiles);
    const int64_t rows = groups * 8 * tile_rows;
    return rows >= M ? M : rows;
}

// Quantise rows [0, pre) in a pass of their own and hand the rest to the GEMM's quantiser warps.
// n_tiles, tile_rows, round_tiles: the GEMM's column tiles, rows per tile (128, or 256 on CTA pairs) and tiles in flight.
int start_quant(const void* x, int64_t ldx, const float* input_scale, unsigned char* xq, int64_t M, int64_t K, int64_t pre,
                const WsView& ws, UmmaArgs& a, cudaStream_t st, int64_t n_tiles, int tile_rows, int round_tiles) {
    cudaError_t e = launch_act_quant((const __nv_bfloat16*)x, ldx, input_scale, xq, pre, K, st);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "activation quantiser launch: %s", cudaGetErrorString(e));
    if (pre < M) {
        a.x = (const __nv_bfloat16*)x; a.ldx = (int)ldx; a.q_row_start = (int)pre; a.q_ctrl = ws.counters;
        // a CTA's next tile lies one round ahead: that many groups of eight tile rows, plus the group in progress
        // and one more so that the next blocks are ready when the tiles get there
        const int64_t groups_per_round = (round_tiles + 8 * n_tiles - 1) / (8 * n_tiles);
        a.q_lead = (int)((groups_per_round + 2) * 8 * (tile_rows / 128));
        if (g_tune.quant_lead >= 0) a.q_lead = g_tune.quant_lead;
    }
    return FP8LIN_OK;
}

bool umma_eligible(int64_t M, int64_t N, int64_t ldy, const void* y) {
    const int max_m = g_tune.stream_max_m >= 0 ? g_tune.stream_max_m : kDefaultStreamMaxM;
    return M > max_m && N % 8 == 0 && ldy % 8 == 0 && aligned16(y);
}

}  // namespace

namespace fp8lin {
static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
bool device_is_sm100() { return check_arch() != 0; }
int sm_count() {
    static int cached = 0;
    if (cached > 0) return cached;
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
        return cached = n;
    cudaGetLastError();
    return 148;              // no device to ask (host-side planning only): not cached, a later call may have one
}
static int g_pdl = 1;
void set_pdl_enabled(int on) { g_pdl = on; }
int pdl_attribute(cudaLaunchAttribute* attr) {
    if (!g_pdl) return 0;
    attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr->val.programmaticStreamSerializationAllowed = 1;
    return 1;
}
int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
}  // namespace fp8lin

extern "C" {

int fp8lin_version(void) { return FP8LIN_VERSION; }
unsigned long long fp8lin_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* fp8lin_last_error(void) { return g_err; }

size_t fp8lin_packed_bytes(int64_t K, int64_t N) {
    return (K > 0 && N > 0) ? (size_t)pack_ntiles(N) * (size_t)pack_kblocks(K) * kPackTileBytes : 0;
}

static int pack_common(const void* src, void* dst, int64_t K, int64_t N, bool src_is_kn, void* stream) {
    if (K <= 0 || N <= 0) return fail(FP8LIN_ERR_SHAPE, "bad shape K=%lld N=%lld", (long long)K, (long long)N);
    if (K % 16 != 0) return fail(FP8LIN_ERR_SHAPE, "K=%lld must be a multiple of 16", (long long)K);
    if (!src || !dst) return fail(FP8LIN_ERR_NULL, "source and destination must not be NULL");
    if (!aligned16(dst)) return fail(FP8LIN_ERR_ALIGN, "w_packed must be 16-byte aligned");
    cudaError_t e = launch_pack_tiles((const unsigned char*)src, (unsigned char*)dst, K, N, src_is_kn, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "prepack launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_prepack_weight(const void* qweight_kn, void* w_packed, int64_t K, int64_t N, void* stream) {
    return pack_common(qweight_kn, w_packed, K, N, true, stream);
}

int fp8lin_pack_weight_nk(const void* qweight_nk, void* w_packed, int64_t K, int64_t N, void* stream) {
    return pack_common(qweight_nk, w_packed, K, N, false, stream);
}

size_t fp8lin_workspace_bytes(int scheme, int64_t M, int64_t K, int64_t N) {
    if (M <= 0 || K <= 0 || N <= 0) return FP8LIN_WS_HEADER_BYTES;
    size_t body = 0;
    // streaming route (any M for W8A16; M <= 64 or odd shapes for W8A8)
    StreamPlan sp = plan_stream(scheme, M, K, N, g_tune.stream_splits);
    body = sp.partial_bytes;
    if (scheme == FP8LIN_W8A8_STATIC) {
        UmmaPlan up = plan_umma(M, K, N, g_tune.umma_bn, g_tune.umma_splits);
        size_t u = align_up((size_t)M * K, 256) + up.partial_bytes;
        if (u > body) body = u;
    } else if (w8a16_umma_eligible(M, K, N, 8, nullptr)) {
        F16Chunks c = plan_f16_chunks(M, K, N);
        if (c.x16_bytes + c.w16_bytes > body) body = c.x16_bytes + c.w16_bytes;
    }
    return FP8LIN_WS_HEADER_BYTES + align_up(body, 256);
}

static int run_stream(int scheme, const void* x, int64_t ldx, const void* w, const float* w_scale,
                      const float* input_scale, const void* bias, void* y, int64_t ldy, int64_t M, int64_t K,
                      int64_t N, void* workspace, size_t ws_bytes, cudaStream_t stream) {
    StreamPlan pl = plan_stream(scheme, M, K, N, g_tune.stream_splits);
    WsView ws = ws_view(workspace, ws_bytes);
    if (pl.splits > 1) {
        if (!workspace || ws.body_bytes < pl.partial_bytes)
            return fail(FP8LIN_ERR_WORKSPACE, "workspace too small: need %zu bytes", FP8LIN_WS_HEADER_BYTES + pl.partial_bytes);
    }
    StreamArgs a;
    a.x = (const __nv_bfloat16*)x; a.w = (const unsigned char*)w; a.w_scale = w_scale; a.input_scale = input_scale;
    a.bias = (const __nv_bfloat16*)bias; a.y = (__nv_bfloat16*)y;
    a.partial = workspace ? (float*)ws.body : nullptr; a.counters = workspace ? ws.counters : nullptr;
    a.status = workspace ? ws.status : nullptr;
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.ldx = (int)ldx; a.ldy = (int)ldy; a.k_per_split = pl.k_per_split;
    cudaError_t e = launch_stream(scheme, pl, a, stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "stream kernel launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_w8a16(const void* x, int64_t ldx, const void* w_nk, const float* w_scale, const void* bias, void* y,
                 int64_t ldy, int64_t M, int64_t K, int64_t N, void* workspace, size_t workspace_bytes,
                 void* stream) {
    int rc = validate_common(x, ldx, w_nk, w_scale, bias, y, ldy, M, K, N);
    if (rc != FP8LIN_OK || M == 0) return rc;
    if (w8a16_swap_eligible(M, N) && workspace) {
        SwapPlan sp = plan_swap_w8a16(M, K, N, g_tune.swap_splits);
        UmmaArgs a;
        a.xq = nullptr; a.w = (const unsigned char*)w_nk; a.w_scale = w_scale; a.input_scale = nullptr;
        a.bias = (const __nv_bfloat16*)bias; a.y = (__nv_bfloat16*)y; a.partial = nullptr; a.counters = nullptr;
        a.status = ws_view(workspace, workspace_bytes).status; a.M = (int)M; a.K = (int)K; a.N = (int)N; a.ldy = (int)ldy;
        const char* why = nullptr;
        cudaError_t e = launch_swap_w8a16(sp, a, x, ldx, (cudaStream_t)stream, &why);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "tcgen05 W8A16 decode kernel launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
        return FP8LIN_OK;
    }
    if (w8a16_umma_eligible(M, K, N, ldy, y)) {
        cudaStream_t st = (cudaStream_t)stream;
        const F16Chunks c = plan_f16_chunks(M, K, N);
        WsView ws = ws_view(workspace, workspace_bytes);
        if (!workspace || ws.body_bytes < c.x16_bytes + c.w16_bytes)
            return fail(FP8LIN_ERR_WORKSPACE, "workspace too small: need %zu bytes",
                        (size_t)FP8LIN_WS_HEADER_BYTES + c.x16_bytes + c.w16_bytes);
        unsigned char* x16 = ws.body;
        unsigned char* w16 = ws.body + c.x16_bytes;
        cudaError_t e = launch_x_to_f16((const __nv_bfloat16*)x, ldx, x16, M, K, st);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "f16 activation pass launch: %s", cudaGetErrorString(e));
        const int64_t kb = pack_kblocks(K);
        for (int64_t ci = 0; ci < c.n_chunks; ++ci) {
            const int64_t t0 = ci * c.chunk_tiles;
            const int64_t n0 = t0 * kPackTile;
            const int64_t nc = (N - n0) < c.chunk_tiles * kPackTile ? (N - n0) : c.chunk_tiles * kPackTile;
            const int64_t tiles = pack_ntiles(nc);
            e = launch_dequant_tiles_f16((const unsigned char*)w_nk + (size_t)t0 * kb * kPackTileBytes, w16,
                                         tiles * kb * kPackTileBytes, st);
            if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "f16 weight pass launch: %s", cudaGetErrorString(e));
            UmmaPlan pl = plan_umma(M, 2 * kb * kPackTile, nc, g_tune.umma_bn, g_tune.umma_splits);
            UmmaArgs a;
            a.xq = x16; a.w = w16; a.w_scale = w_scale + n0; a.input_scale = nullptr;
            a.bias = bias ? (const __nv_bfloat16*)bias + n0 : nullptr; a.y = (__nv_bfloat16*)y + n0;
            a.partial = nullptr; a.counters = ws.counters; a.status = ws.status;
            a.M = (int)M; a.K = (int)K; a.N = (int)nc; a.ldy = (int)ldy;
            const char* why = nullptr;
            e = pair_eligible(M, nc) ? launch_umma_pair(true, a, st, &why) : launch_umma_f16(pl, a, st, &why);
            if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "tcgen05 f16 GEMM launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
        }
        return FP8LIN_OK;
    }
    return run_stream(FP8LIN_W8A16, x, ldx, w_nk, w_scale, nullptr, bias, y, ldy, M, K, N, workspace,
                      workspace_bytes, (cudaStream_t)stream);
}

int fp8lin_w8a8(const void* x, int64_t ldx, const void* w_nk, const float* w_scale, const float* input_scale,
                const void* bias, void* y, int64_t ldy, int64_t M, int64_t K, int64_t N, void* workspace,
                size_t workspace_bytes, void* stream) {
    int rc = validate_common(x, ldx, w_nk, w_scale, bias, y, ldy, M, K, N);
    if (rc != FP8LIN_OK || M == 0) return rc;
    if (!input_scale) return fail(FP8LIN_ERR_NULL, "input_scale must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    if (swap_eligible(M, K, N)) {
        const bool preq = swap_prequant(M);
        SwapPlan sp = plan_swap(M, K, N, g_tune.swap_splits, preq);
        WsView wsv = ws_view(workspace, workspace_bytes);
        if (!workspace) return fail(FP8LIN_ERR_WORKSPACE, "workspace (at least the %d-byte header) is required", FP8LIN_WS_HEADER_BYTES);
        UmmaArgs a;
        a.xq = nullptr;
        if (preq) {
            if (wsv.body_bytes < align_up((size_t)M * K, 256))
                return fail(FP8LIN_ERR_WORKSPACE, "workspace too small: need %zu bytes", FP8LIN_WS_HEADER_BYTES + align_up((size_t)M * K, 256));
            cudaError_t qe = launch_act_quant((const __nv_bfloat16*)x, ldx, input_scale, wsv.body, M, K, st);
            if (qe != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "activation quantiser launch: %s", cudaGetErrorString(qe));
            a.xq = wsv.body;
        } a.w = (const unsigned char*)w_nk; a.w_scale = w_scale; a.input_scale = input_scale;
        a.bias = (const __nv_bfloat16*)bias; a.y = (__nv_bfloat16*)y; a.partial = nullptr; a.counters = nullptr;
        a.status = wsv.status; a.M = (int)M; a.K = (int)K; a.N = (int)N; a.ldy = (int)ldy;
        const char* why = nullptr;
        cudaError_t e = launch_swap_w8a8(sp, a, x, ldx, st, &why);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "tcgen05 decode kernel launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
        return FP8LIN_OK;
    }
    if (!umma_eligible(M, N, ldy, y))
        return run_stream(FP8LIN_W8A8_STATIC, x, ldx, w_nk, w_scale, input_scale, bias, y, ldy, M, K, N, workspace,
                          workspace_bytes, st);

    UmmaPlan pl = plan_umma(M, K, N, g_tune.umma_bn, g_tune.umma_splits);
    WsView ws = ws_view(workspace, workspace_bytes);
    const size_t xq_bytes = align_up((size_t)M * K, 256);
    if (!workspace || ws.body_bytes < xq_bytes + pl.partial_bytes)
        return fail(FP8LIN_ERR_WORKSPACE, "workspace too small: need %zu bytes",
                    FP8LIN_WS_HEADER_BYTES + xq_bytes + pl.partial_bytes);
    unsigned char* xq = ws.body;
    UmmaArgs a;
    a.xq = xq; a.w = (const unsigned char*)w_nk; a.w_scale = w_scale; a.input_scale = input_scale;
    a.bias = (const __nv_bfloat16*)bias; a.y = (__nv_bfloat16*)y;
    a.partial = (float*)(ws.body + xq_bytes); a.counters = ws.counters; a.status = ws.status;
    a.M = (int)M; a.K = (int)K; a.N = (int)N; a.ldy = (int)ldy;
    const bool pair = pair_eligible(M, N);
    const int64_t pre = pair ? prequant_rows(M, (N + 255) / 256, 256, sm_count() / 2)
                             : (pl.splits > 1 ? M : prequant_rows(M, pl.n_tiles, 128, sm_count()));
    rc = pair ? start_quant(x, ldx, input_scale, xq, M, K, pre, ws, a, st, (N + 255) / 256, 256, sm_count() / 2)
              : start_quant(x, ldx, input_scale, xq, M, K, pre, ws, a, st, pl.n_tiles, 128, sm_count());
    if (rc != FP8LIN_OK) return rc;
    const char* why = nullptr;
    cudaError_t e = pair ? launch_umma_pair(false, a, st, &why) : launch_umma_w8a8(pl, a, st, &why);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "tcgen05 GEMM launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
    return FP8LIN_OK;
}

static int w8a8_to_destinations(const void* x, int64_t ldx, const void* w_nk, const float* w_scale, const float* input_scale,
                                const void* bias, int n_dst, void* const* dst_ptrs, int64_t ld_dst, int64_t band_rows, int64_t M,
                                int64_t K, int64_t N, void* workspace, size_t workspace_bytes, void* stream) {
    if (n_dst < 1 || n_dst > 8 || !dst_ptrs) return fail(FP8LIN_ERR_ARG, "n_dst must be 1..8 and dst_ptrs non-NULL");
    for (int d = 0; d < n_dst; ++d)
        if (!dst_ptrs[d] || !aligned16(dst_ptrs[d])) return fail(FP8LIN_ERR_ALIGN, "destination %d is NULL or not 16-byte aligned", d);
    int rc = validate_common(x, ldx, w_nk, w_scale, bias, dst_ptrs[0], ld_dst, M, K, N);
    if (rc != FP8LIN_OK || M == 0) return rc;
    if (!input_scale) return fail(FP8LIN_ERR_NULL, "input_scale must not be NULL");
    if (N % 8 != 0 || ld_dst % 8 != 0) return fail(FP8LIN_ERR_SHAPE, "N and ld_dst must be multiples of 8");
    if (band_rows != 0 && (band_rows < 32 || band_rows % 32 != 0 || band_rows * n_dst < M))
        return fail(FP8LIN_ERR_SHAPE, "band_rows=%lld must be a multiple of 32 with band_rows * n_dst >= M", (long long)band_rows);
    cudaStream_t st = (cudaStream_t)stream;
    UmmaPlan pl = plan_umma(M, K, N, g_tune.umma_bn, 1);      // the multi-destination epilogue exists in the non-split kernels only
    pl.tail_tiles = 0;
    WsView ws = ws_view(workspace, workspace_bytes);
    const size_t xq_bytes = align_up((size_t)M * K, 256);
    if (!workspace || ws.body_bytes < xq_bytes)
        return fail(FP8LIN_ERR_WORKSPACE, "workspace too small: need %zu bytes", FP8LIN_WS_HEADER_BYTES + xq_bytes);
    UmmaArgs a;
    a.xq = ws.body; a.w = (const unsigned char*)w_nk; a.w_scale = w_scale; a.input_scale = input_scale;
    a.bias = (const __nv_bfloat16*)bias; a.y = (__nv_bfloat16*)dst_ptrs[0]; a.partial = nullptr; a.counters = ws.counters;
    a.status = ws.status; a.M = (int)M; a.K = (int)K; a.N = (int)N; a.ldy = (int)ld_dst;
    const bool pair = pair_eligible(M, N);
    rc = pair ? start_quant(x, ldx, input_scale, ws.body, M, K, prequant_rows(M, (N + 255) / 256, 256, sm_count() / 2), ws, a, st,
                            (N + 255) / 256, 256, sm_count() / 2)
              : start_quant(x, ldx, input_scale, ws.body, M, K, prequant_rows(M, pl.n_tiles, 128, sm_count()), ws, a, st, pl.n_tiles, 128,
                            sm_count());
    if (rc != FP8LIN_OK) return rc;
    const char* why = nullptr;
    cudaError_t e = pair ? launch_umma_pair(false, a, st, &why, n_dst, dst_ptrs, ld_dst, band_rows)
                         : launch_umma_w8a8(pl, a, st, &why, n_dst, dst_ptrs, ld_dst, band_rows);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "tcgen05 GEMM launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
    return FP8LIN_OK;
}

int fp8lin_w8a8_scatter(const void* x, int64_t ldx, const void* w_nk, const float* w_scale, const float* input_scale,
                        const void* bias, int n_dst, void* const* dst_ptrs, int64_t ld_dst, int64_t M, int64_t K, int64_t N,
                        void* workspace, size_t workspace_bytes, void* stream) {
    return w8a8_to_destinations(x, ldx, w_nk, w_scale, input_scale, bias, n_dst, dst_ptrs, ld_dst, 0, M, K, N, workspace,
                                workspace_bytes, stream);
}

int fp8lin_w8a8_reduce_scatter(const void* x, int64_t ldx, const void* w_nk, const float* w_scale, const float* input_scale,
                               const void* bias, int n_dst, void* const* dst_ptrs, int64_t ld_dst, int64_t band_rows, int64_t M,
                               int64_t K, int64_t N, void* workspace, size_t workspace_bytes, void* stream) {
    if (band_rows <= 0) return fail(FP8LIN_ERR_SHAPE, "band_rows must be positive");
    return w8a8_to_destinations(x, ldx, w_nk, w_scale, input_scale, bias, n_dst, dst_ptrs, ld_dst, band_rows, M, K, N, workspace,
                                workspace_bytes, stream);
}

// ---- fused MLP: y = down( silu(gate(x)) * up(x) ), both projections W8A8-static -----------------------
namespace {

struct MlpLayout {
    size_t inner;       // scratch of the gate_up linear itself (quantised x, split-K partials)
    size_t gu_off, hq_off, total;
};

MlpLayout mlp_layout(int64_t M, int64_t H, int64_t I) {
    MlpLayout l;
    size_t inner = fp8lin_workspace_bytes(FP8LIN_W8A8_STATIC, M, H, 2 * I) - FP8LIN_WS_HEADER_BYTES;
    const size_t xq = align_up((size_t)M * H, 256);
    if (xq > inner) inner = xq;
    l.inner = align_up(inner, 256);
    l.gu_off = l.inner;
    const size_t gu = M <= kDefaultStreamMaxM ? align_up((size_t)M * 2 * I * 2, 256) : 0;   // bf16 gate_up result, small batches only
    l.hq_off = l.gu_off + gu;
    l.total = l.hq_off + align_up((size_t)M * I, 256);
    return l;
}

// W8A8 linear whose activations are already e4m3 (row pitch K): the second half of the fused MLP.
int run_w8a8_prequantised(const unsigned char* xq, const void* w, const float* w_scale, const float* input_scale,
                          const void* bias, void* y, int64_t ldy, int64_t M, int64_t K, int64_t N, const WsView& ws,
                          cudaStream_t st) {
    UmmaArgs a;
    a.xq = xq; a.w = (const unsigned char*)w; a.w_scale = w_scale; a.input_scale = input_scale;
    a.bias = (const __nv_bfloat16*)bias; a.y = (__nv_bfloat16*)y; a.partial = nullptr; a.counters = ws.counters;
    a.status = ws.status; a.M = (int)M; a.K = (int)K; a.N = (int)N; a.ldy = (int)ldy;
    const char* why = nullptr;
    cudaError_t e;
    if (M <= 64) {
        SwapPlan sp = plan_swap(M, K, N, g_tune.swap_splits, true);
        e = launch_swap_w8a8(sp, a, nullptr, 0, st, &why);
    } else if (pair_eligible(M, N)) {
        e = launch_umma_pair(false, a, st, &why);
    } else {
        UmmaPlan pl = plan_umma(M, K, N, g_tune.umma_bn, g_tune.umma_splits);
        e = launch_umma_w8a8(pl, a, st, &why);
    }
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "down projection launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
    return FP8LIN_OK;
}

}  // namespace

size_t fp8lin_mlp_workspace_bytes(int64_t M, int64_t H, int64_t I, int64_t N) {
    (void)N;
    if (M <= 0 || H <= 0 || I <= 0) return FP8LIN_WS_HEADER_BYTES;
    return FP8LIN_WS_HEADER_BYTES + mlp_layout(M, H, I).total;
}

static int mlp_w8a8_impl(const void* x, int64_t ldx, bool x_is_e4m3, const void* w_gate_up, const float* gate_up_scale,
                         const float* gate_up_input_scale, const void* gate_up_bias, const void* w_down,
                         const float* down_scale, const float* down_input_scale, const void* down_bias, void* y, int64_t ldy,
                         int64_t M, int64_t H, int64_t I, int64_t N, void* workspace, size_t workspace_bytes, void* stream) {
    if (I <= 0 || I % 128 != 0) return fail(FP8LIN_ERR_SHAPE, "the intermediate size must be a positive multiple of 128 (got %lld)", (long long)I);
    int rc = validate_common(x, ldx, w_gate_up, gate_up_scale, gate_up_bias, y, 2 * I, M, H, 2 * I);   // (its output is internal)
    if (rc != FP8LIN_OK) return rc;
    rc = validate_common(x, I, w_down, down_scale, down_bias, y, ldy, M, I, N);      // (the down input is internal, pitch I)
    if (rc != FP8LIN_OK || M == 0) return rc;
    if (!gate_up_input_scale || !down_input_scale) return fail(FP8LIN_ERR_NULL, "both input scales are required");
    if (N % 8 != 0 || ldy % 8 != 0) return fail(FP8LIN_ERR_SHAPE, "N and ldy must be multiples of 8");
    const MlpLayout l = mlp_layout(M, H, I);
    WsView ws = ws_view(workspace, workspace_bytes);
    if (!workspace || ws.body_bytes < l.total)
        return fail(FP8LIN_ERR_WORKSPACE, "workspace too small: need %zu bytes", (size_t)FP8LIN_WS_HEADER_BYTES + l.total);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char* hq = ws.body + l.hq_off;
    if (x_is_e4m3 && M <= 16 && g_tune.mlp_decode_fused > 0) {
        // Opt-in: up to 16 pre-quantised rows, clusters of two CTAs of the decode kernel take (gate, up) tile pairs, the
        // up CTA hands its values to the gate CTA, which writes e4m3 h itself (one launch fewer, no bf16 gate_up round
        // trip, same bits).  Off by default, it buys nothing: 55.9 us per 7B decoder layer at one row against 55.5 us
        // with the separate 3 us activation pass (58.7 against 58.3 at 16 rows; 28 layers under one CUDA graph) -- the
        // hand-over buffer costs the ring its sixth slot and the hand-over sits on the kernel's tail.  A first form
        // (both tiles in one CTA with a 12-slot ring, one CTA per SM) was slower still: 58.6 us.
        UmmaArgs a;
        a.xq = (const unsigned char*)x; a.w = (const unsigned char*)w_gate_up; a.w_scale = gate_up_scale; a.input_scale = gate_up_input_scale;
        a.bias = (const __nv_bfloat16*)gate_up_bias; a.y = nullptr; a.partial = nullptr; a.counters = nullptr;
        a.status = ws.status; a.M = (int)M; a.K = (int)H; a.N = (int)(2 * I); a.ldy = 0;
        a.hq = hq; a.h_scale = down_input_scale;
        const char* why = nullptr;
        cudaError_t e = launch_swap_gate_up(a, st, &why);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "decode gate_up launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
    } else if (M <= kDefaultStreamMaxM) {
        // small batches: gate_up through the decode kernels into a bf16 buffer, one pass for silu * up + quantise
        __nv_bfloat16* gu = (__nv_bfloat16*)(ws.body + l.gu_off);
        if (x_is_e4m3) {
            WsView inner = ws_view(workspace, FP8LIN_WS_HEADER_BYTES + l.inner);
            rc = run_w8a8_prequantised((const unsigned char*)x, w_gate_up, gate_up_scale, gate_up_input_scale, gate_up_bias, gu, 2 * I,
                                       M, H, 2 * I, inner, st);
        } else {
            rc = fp8lin_w8a8(x, ldx, w_gate_up, gate_up_scale, gate_up_input_scale, gate_up_bias, gu, 2 * I, M, H, 2 * I, workspace,
                             FP8LIN_WS_HEADER_BYTES + l.inner, stream);
        }
        if (rc != FP8LIN_OK) return rc;
        cudaError_t e = launch_silu_mul_quant_interleaved(gu, down_input_scale, hq, M, I, st);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "silu-multiply pass launch: %s", cudaGetErrorString(e));
    } else {
        unsigned char* xq = x_is_e4m3 ? (unsigned char*)const_cast<void*>(x) : ws.body;
        UmmaArgs a;
        a.xq = xq; a.w = (const unsigned char*)w_gate_up; a.w_scale = gate_up_scale; a.input_scale = gate_up_input_scale;
        a.bias = (const __nv_bfloat16*)gate_up_bias; a.y = nullptr; a.partial = nullptr; a.counters = ws.counters;
        a.status = ws.status; a.M = (int)M; a.K = (int)H; a.N = (int)(2 * I); a.ldy = 0;
        if (!x_is_e4m3) {
            rc = start_quant(x, ldx, gate_up_input_scale, xq, M, H, prequant_rows(M, (2 * I + 255) / 256, 256, sm_count() / 2), ws, a, st,
                             (2 * I + 255) / 256, 256, sm_count() / 2);
            if (rc != FP8LIN_OK) return rc;
        }
        const char* why = nullptr;
        cudaError_t e = launch_umma_pair_mlp(a, hq, down_input_scale, st, &why);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "fused gate_up launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
    }
    return run_w8a8_prequantised(hq, w_down, down_scale, down_input_scale, down_bias, y, ldy, M, I, N, ws, st);
}

int fp8lin_w8a8_preq(const void* xq, const void* w_nk, const float* w_scale, const float* input_scale, const void* bias,
                     void* y, int64_t ldy, int64_t M, int64_t K, int64_t N, void* workspace, size_t workspace_bytes,
                     void* stream) {
    int rc = validate_common(xq, K, w_nk, w_scale, bias, y, ldy, M, K, N);      // (xq rows are K bytes apart)
    if (rc != FP8LIN_OK || M == 0) return rc;
    if (!input_scale) return fail(FP8LIN_ERR_NULL, "input_scale must not be NULL");
    if (N % 8 != 0 || ldy % 8 != 0 || !aligned16(y)) return fail(FP8LIN_ERR_ALIGN, "N and ldy must be multiples of 8 and y 16-byte aligned");
    if (!workspace || workspace_bytes < FP8LIN_WS_HEADER_BYTES)
        return fail(FP8LIN_ERR_WORKSPACE, "workspace (at least the %d-byte header) is required", FP8LIN_WS_HEADER_BYTES);
    return run_w8a8_prequantised((const unsigned char*)xq, w_nk, w_scale, input_scale, bias, y, ldy, M, K, N,
                                 ws_view(workspace, workspace_bytes), (cudaStream_t)stream);
}

int fp8lin_rmsnorm_quant(const void* x, int64_t ldx, void* residual, int64_t ld_res, const void* weight, float eps,
                         const float* input_scale, void* xq, void* y, int64_t ldy, int64_t M, int64_t H, void* stream) {
    if (M < 0 || H <= 0 || H % 8 != 0 || H > 8192)
        return fail(FP8LIN_ERR_SHAPE, "bad shape M=%lld H=%lld (H a multiple of 8, at most 8192)", (long long)M, (long long)H);
    if (M == 0) return FP8LIN_OK;
    if (!x || !weight || (!xq && !y)) return fail(FP8LIN_ERR_NULL, "x, weight and at least one of xq / y must not be NULL");
    if (xq && !input_scale) return fail(FP8LIN_ERR_NULL, "input_scale is required when xq is asked for");
    if (ldx < H || (residual && ld_res < H) || (y && ldy < H)) return fail(FP8LIN_ERR_SHAPE, "a row stride is smaller than H");
    if (ldx % 8 != 0 || (residual && ld_res % 8 != 0) || (y && ldy % 8 != 0))
        return fail(FP8LIN_ERR_ALIGN, "row strides must be multiples of 8 elements");
    if (!aligned16(x) || !aligned16(weight) || (residual && !aligned16(residual)) || (y && !aligned16(y)) ||
        (xq && (reinterpret_cast<uintptr_t>(xq) & 7) != 0))
        return fail(FP8LIN_ERR_ALIGN, "x, residual, weight and y must be 16-byte aligned, xq 8-byte aligned");
    if (!(eps >= 0.f)) return fail(FP8LIN_ERR_ARG, "eps must not be negative");
    if (!check_arch()) return fail(FP8LIN_ERR_ARCH, "fp8lin kernels are built for sm_100a only");
    cudaError_t e = launch_rmsnorm_quant((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)residual, ld_res, (const __nv_bfloat16*)weight,
                                         eps, input_scale, (unsigned char*)xq, (__nv_bfloat16*)y, ldy, M, H, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "RMSNorm launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_mlp_w8a8(const void* x, int64_t ldx, const void* w_gate_up, const float* gate_up_scale,
                    const float* gate_up_input_scale, const void* gate_up_bias, const void* w_down,
                    const float* down_scale, const float* down_input_scale, const void* down_bias, void* y, int64_t ldy,
                    int64_t M, int64_t H, int64_t I, int64_t N, void* workspace, size_t workspace_bytes, void* stream) {
    return mlp_w8a8_impl(x, ldx, false, w_gate_up, gate_up_scale, gate_up_input_scale, gate_up_bias, w_down, down_scale,
                         down_input_scale, down_bias, y, ldy, M, H, I, N, workspace, workspace_bytes, stream);
}

int fp8lin_mlp_w8a8_preq(const void* xq, const void* w_gate_up, const float* gate_up_scale,
                         const float* gate_up_input_scale, const void* gate_up_bias, const void* w_down,
                         const float* down_scale, const float* down_input_scale, const void* down_bias, void* y, int64_t ldy,
                         int64_t M, int64_t H, int64_t I, int64_t N, void* workspace, size_t workspace_bytes, void* stream) {
    return mlp_w8a8_impl(xq, (H + 7) / 8 * 8, true, w_gate_up, gate_up_scale, gate_up_input_scale, gate_up_bias, w_down, down_scale,
                         down_input_scale, down_bias, y, ldy, M, H, I, N, workspace, workspace_bytes, stream);
}

int fp8lin_sum_slots(const void* slots, int n_slots, int64_t slot_stride, int64_t ld_slot, void* y, int64_t ldy,
                     int64_t M, int64_t N, void* stream) {
    if (n_slots < 1 || M < 0 || N <= 0 || N % 8 != 0 || ld_slot % 8 != 0 || ldy % 8 != 0 || slot_stride % 8 != 0)
        return fail(FP8LIN_ERR_SHAPE, "bad shape: N, ld_slot, ldy and slot_stride must be multiples of 8");
    if (M == 0) return FP8LIN_OK;
    if (!slots || !y) return fail(FP8LIN_ERR_NULL, "slots and y must not be NULL");
    if (!aligned16(slots) || !aligned16(y)) return fail(FP8LIN_ERR_ALIGN, "slots and y must be 16-byte aligned");
    cudaError_t e = launch_sum_slots((const __nv_bfloat16*)slots, n_slots, slot_stride, (__nv_bfloat16*)y, ldy, M, N, ld_slot,
                                     (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "slot sum launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_sum_slots_gather(const void* slots, int n_slots, int64_t slot_stride, int64_t ld_slot, int n_dst, void* const* dst_ptrs,
                            int64_t ld_dst, int64_t dst_row, int64_t M, int64_t N, void* stream) {
    if (n_slots < 1 || M < 0 || N <= 0 || N % 8 != 0 || ld_slot % 8 != 0 || ld_dst % 8 != 0 || slot_stride % 8 != 0 || dst_row < 0)
        return fail(FP8LIN_ERR_SHAPE, "bad shape: N, ld_slot, ld_dst and slot_stride must be multiples of 8");
    if (n_dst < 1 || n_dst > 8 || !dst_ptrs) return fail(FP8LIN_ERR_ARG, "n_dst must be 1..8 and dst_ptrs non-NULL");
    if (M == 0) return FP8LIN_OK;
    if (!slots || !aligned16(slots)) return fail(FP8LIN_ERR_ALIGN, "slots must be non-NULL and 16-byte aligned");
    SumDst dst;
    dst.n = n_dst;
    for (int d = 0; d < n_dst; ++d) {
        if (!dst_ptrs[d] || !aligned16(dst_ptrs[d])) return fail(FP8LIN_ERR_ALIGN, "destination %d is NULL or not 16-byte aligned", d);
        dst.y[d] = (__nv_bfloat16*)dst_ptrs[d] + dst_row * ld_dst;
    }
    cudaError_t e = launch_sum_slots_gather((const __nv_bfloat16*)slots, n_slots, slot_stride, ld_slot, dst, ld_dst, M, N,
                                            (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "slot sum launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_quantize_weight(const void* w, int w_is_f32, int64_t ldw, void* qweight_nk, float* weight_scale, int64_t N,
                           int64_t K, void* stream) {
    if (N < 0 || K <= 0 || K % 2 != 0 || ldw < K) return fail(FP8LIN_ERR_SHAPE, "bad shape N=%lld K=%lld ldw=%lld (K must be even)", (long long)N, (long long)K, (long long)ldw);
    if (N == 0) return FP8LIN_OK;
    if (!w || !qweight_nk || !weight_scale) return fail(FP8LIN_ERR_NULL, "w, qweight_nk and weight_scale must not be NULL");
    if ((reinterpret_cast<uintptr_t>(qweight_nk) & 1) != 0) return fail(FP8LIN_ERR_ALIGN, "qweight_nk must be 2-byte aligned");
    if (!check_arch()) return fail(FP8LIN_ERR_ARCH, "fp8lin kernels are built for sm_100a only");
    cudaError_t e = launch_quantize_weight(w, w_is_f32 != 0, ldw, (unsigned char*)qweight_nk, weight_scale, N, K, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "weight quantiser launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_abs_max(const void* x, int64_t ldx, int64_t M, int64_t K, float* amax, void* stream) {
    if (M < 0 || K <= 0 || K % 8 != 0 || ldx < K || ldx % 8 != 0) return fail(FP8LIN_ERR_SHAPE, "bad shape M=%lld K=%lld ldx=%lld (multiples of 8)", (long long)M, (long long)K, (long long)ldx);
    if (M == 0) return FP8LIN_OK;
    if (!x || !amax) return fail(FP8LIN_ERR_NULL, "x and amax must not be NULL");
    if (!aligned16(x)) return fail(FP8LIN_ERR_ALIGN, "x must be 16-byte aligned");
    if (!check_arch()) return fail(FP8LIN_ERR_ARCH, "fp8lin kernels are built for sm_100a only");
    cudaError_t e = launch_abs_max((const __nv_bfloat16*)x, ldx, M, K, amax, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "abs-max launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_quantize_activation(const void* x, int64_t ldx, const float* input_scale, void* xq, int64_t M, int64_t K,
                               void* stream) {
    if (M < 0 || K <= 0 || K % 16 != 0) return fail(FP8LIN_ERR_SHAPE, "bad shape M=%lld K=%lld", (long long)M, (long long)K);
    if (M == 0) return FP8LIN_OK;
    if (!x || !input_scale || !xq) return fail(FP8LIN_ERR_NULL, "x, input_scale and xq must not be NULL");
    if (ldx < K || ldx % 8 != 0 || !aligned16(x) || !aligned16(xq)) return fail(FP8LIN_ERR_ALIGN, "x/xq alignment or ldx");
    cudaError_t e = launch_act_quant((const __nv_bfloat16*)x, ldx, input_scale, (unsigned char*)xq, M, K, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "activation quantiser launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

const char* fp8lin_variant_name(int scheme, int64_t M, int64_t K, int64_t N) {
    static thread_local char buf[64];
    if (M <= 0 || K <= 0 || N <= 0) return "none";
    const int max_m = g_tune.stream_max_m >= 0 ? g_tune.stream_max_m : kDefaultStreamMaxM;
    if (scheme == FP8LIN_W8A8_STATIC && M > max_m && N % 8 == 0 && pair_eligible(M, N)) return "umma_pair_w8a8_256x256";
    if (scheme == FP8LIN_W8A8_STATIC && M > max_m && N % 8 == 0) {
        UmmaPlan pl = plan_umma(M, K, N, g_tune.umma_bn, g_tune.umma_splits);
        if (pl.tail_tiles) snprintf(buf, sizeof(buf), "umma_w8a8_128x%d_s1+tail%dx%d", pl.bn, pl.tail_tiles, pl.tail_splits);
        else if (pl.narrow_tiles) snprintf(buf, sizeof(buf), "umma_w8a8_128x%d_s1+half%d", pl.bn, pl.narrow_tiles);
        else snprintf(buf, sizeof(buf), "umma_w8a8_128x%d_s%d", pl.bn, pl.splits);
        return buf;
    }
    if (scheme == FP8LIN_W8A8_STATIC && swap_eligible(M, K, N)) {
        SwapPlan pl = plan_swap(M, K, N, g_tune.swap_splits, swap_prequant(M));
        snprintf(buf, sizeof(buf), "umma_swap_w8a8_m%d_s%d%s", pl.mp, pl.splits, pl.preq ? "_preq" : "");
        return buf;
    }
    if (scheme == FP8LIN_W8A16 && w8a16_umma_eligible(M, K, N, 8, nullptr)) {
        const F16Chunks c = plan_f16_chunks(M, K, N);
        const int64_t full = c.chunk_tiles * kPackTile < N ? c.chunk_tiles * kPackTile : N;
        UmmaPlan pl = plan_umma(M, 2 * pack_kblocks(K) * kPackTile, full, g_tune.umma_bn, g_tune.umma_splits);
        snprintf(buf, sizeof(buf), "umma_w8a16_f16_128x%d_s%d_c%d", pl.bn, pl.splits, (int)c.n_chunks);
        return buf;
    }
    if (scheme == FP8LIN_W8A16 && w8a16_swap_eligible(M, N)) {
        SwapPlan pl = plan_swap_w8a16(M, K, N, g_tune.swap_splits);
        snprintf(buf, sizeof(buf), "umma_swap_w8a16_m%d_s%d", pl.mp, pl.splits);
        return buf;
    }
    StreamPlan sp = plan_stream(scheme, M, K, N, g_tune.stream_splits);
    snprintf(buf, sizeof(buf), "stream_mma_%s_m%d_s%d", scheme == FP8LIN_W8A16 ? "w8a16" : "w8a8", sp.mt * 8, sp.splits);
    return buf;
}

int fp8lin_set_tuning(const char* knob, int value) {
    if (!knob) return fail(FP8LIN_ERR_NULL, "knob is NULL");
    if (!strcmp(knob, "stream_splits")) g_tune.stream_splits = value;
    else if (!strcmp(knob, "stream_max_m")) g_tune.stream_max_m = value;
    else if (!strcmp(knob, "umma_bn")) g_tune.umma_bn = value;
    else if (!strcmp(knob, "umma_splits")) g_tune.umma_splits = value;
    else if (!strcmp(knob, "swap_splits")) g_tune.swap_splits = value;
    else if (!strcmp(knob, "swap_enable")) g_tune.swap_enable = value;
    else if (!strcmp(knob, "swap_min_m")) g_tune.swap_min_m = value;
    else if (!strcmp(knob, "swap_preq_min_m")) g_tune.swap_preq_min_m = value;
    else if (!strcmp(knob, "w8a16_swap_enable")) g_tune.w8a16_swap_enable = value;
    else if (!strcmp(knob, "w8a16_swap_min_m")) g_tune.w8a16_swap_min_m = value;
    else if (!strcmp(knob, "w8a16_umma_min_m")) g_tune.w8a16_umma_min_m = value;
    else if (!strcmp(knob, "w8a16_chunk_mb")) g_tune.w8a16_chunk_mb = value;
    else if (!strcmp(knob, "umma_pair")) g_tune.umma_pair = value;
    else if (!strcmp(knob, "fuse_quant")) g_tune.fuse_quant = value;
    else if (!strcmp(knob, "quant_lead")) g_tune.quant_lead = value;
    else if (!strcmp(knob, "stream_push")) set_stream_push(value != 0);
    else if (!strcmp(knob, "mlp_decode_fused")) g_tune.mlp_decode_fused = value;
    else if (!strcmp(knob, "moe_fused")) g_tune.moe_fused = value;
    else if (!strcmp(knob, "moe_rows_major")) g_tune.moe_rows_major = value;
    else if (!strcmp(knob, "pair_stages")) set_pair_stages(value);
    else if (!strcmp(knob, "pdl")) set_pdl_enabled(value != 0);
    else return fail(FP8LIN_ERR_ARG, "unknown tuning knob '%s'", knob);
    return FP8LIN_OK;
}

// ---- MoE -------------------------------------------------------------------------------------
namespace {
// from this many routed rows on, the rows are gathered and quantised once by a separate pass
// instead of inside the gate_up GEMM (where every channel tile would redo it)
constexpr int64_t kMoePrequantRows = 512;
struct MoeWs {
    size_t off_offsets, off_sorted, off_chunks, off_meta, off_gu, off_hq, off_xq, total;
};
MoeWs moe_ws_layout(int64_t rows, int E, int64_t H, int64_t I) {
    MoeWs w;
    size_t o = FP8LIN_WS_HEADER_BYTES;
    auto take = [&](size_t bytes) { size_t at = o; o = align_up(o + bytes, 256); return at; };
    w.off_offsets = take((size_t)(E + 1) * 4);
    w.off_sorted = take((size_t)(rows > 0 ? rows : 1) * 4);
    w.off_chunks = take((size_t)(E + rows / 16 + 2) * 16);
    w.off_meta = take(16);
    w.off_gu = take((size_t)rows * 2 * I * 2);
    w.off_hq = take((size_t)rows * I);
    w.off_xq = take(rows >= kMoePrequantRows ? (size_t)rows * H : 0);
    w.total = o;
    return w;
}
}  // namespace

int fp8lin_moe_route(const void* logits, int logits_dtype, int64_t ld, int64_t T, int E, int top_k, int renormalize,
                     float* topk_w, int32_t* topk_ids, void* stream) {
    if (T < 0 || E <= 0 || E > 1024 || top_k <= 0 || top_k > 32 || top_k > E || ld < E)
        return fail(FP8LIN_ERR_SHAPE, "bad router shape T=%lld E=%d top_k=%d ld=%lld (E <= 1024, top_k <= 32)",
                    (long long)T, E, top_k, (long long)ld);
    if (logits_dtype != 0 && logits_dtype != 1) return fail(FP8LIN_ERR_ARG, "logits_dtype must be 0 (f32) or 1 (bf16)");
    if (T == 0) return FP8LIN_OK;
    if (!logits || !topk_w || !topk_ids) return fail(FP8LIN_ERR_NULL, "logits, topk_w and topk_ids must not be NULL");
    cudaError_t e = launch_moe_route(logits, logits_dtype, ld, (int)T, E, top_k, renormalize, topk_w, topk_ids, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "router launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_moe_align(const int32_t* ids, int64_t rows, int E, int chunk_rows, int32_t* expert_offsets, int32_t* sorted_rows,
                     int32_t* chunks, int32_t* meta, void* stream) {
    if (rows < 0 || rows > (1ll << 24) || E <= 0 || E > 3071)
        return fail(FP8LIN_ERR_SHAPE, "bad grouping shape rows=%lld E=%d (E <= 3071)", (long long)rows, E);
    if (chunk_rows != 16 && chunk_rows != 32 && chunk_rows != 64 && chunk_rows != 128)
        return fail(FP8LIN_ERR_ARG, "chunk_rows must be 16, 32, 64 or 128");
    if (!ids || !expert_offsets || !sorted_rows || !chunks || !meta) return fail(FP8LIN_ERR_NULL, "a required pointer is NULL");
    if (!aligned16(chunks)) return fail(FP8LIN_ERR_ALIGN, "chunks must be 16-byte aligned");
    cudaError_t e = launch_moe_align(ids, (int)rows, E, chunk_rows, expert_offsets, sorted_rows, (int4*)chunks, meta,
                                     (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "row grouping launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

size_t fp8lin_moe_workspace_bytes(int64_t rows, int E, int64_t H, int64_t I) {
    if (rows < 0 || E <= 0 || H <= 0 || I <= 0) return FP8LIN_WS_HEADER_BYTES;
    return moe_ws_layout(rows, E, H, I).total;
}

int fp8lin_moe_experts_w8a8(const void* x, int64_t ldx, int x_div, const int32_t* ids, const float* topk_w, int64_t rows,
                            const void* w13_packed, const float* w13_scale, const float* w13_input_scale,
                            const void* w2_packed, const float* w2_scale, const float* w2_input_scale,
                            int E, int64_t H, int64_t I, void* out_routed, int64_t ld_out,
                            void* workspace, size_t workspace_bytes, void* stream) {
    // E <= 3071: the row-grouping kernel keeps 4E + 2 counters in 48 KB of shared memory
    if (rows < 0 || E <= 0 || E > 3071 || H <= 0 || I <= 0 || H % 16 != 0 || I % 16 != 0 || x_div <= 0)
        return fail(FP8LIN_ERR_SHAPE, "bad MoE shape rows=%lld E=%d H=%lld I=%lld (E <= 3071; H, I multiples of 16)", (long long)rows, E,
                    (long long)H, (long long)I);
    if (rows == 0) return FP8LIN_OK;
    if (rows > (1ll << 24)) return fail(FP8LIN_ERR_SHAPE, "too many routed rows");
    if (!x || !ids || !topk_w || !w13_packed || !w13_scale || !w13_input_scale || !w2_packed || !w2_scale ||
        !w2_input_scale || !out_routed)
        return fail(FP8LIN_ERR_NULL, "a required MoE pointer is NULL");
    if (ldx < H || ldx % 8 != 0 || ld_out < H || !aligned16(x) || !aligned16(w13_packed) || !aligned16(w2_packed))
        return fail(FP8LIN_ERR_ALIGN, "x / packed weights must be 16-byte aligned, ldx a multiple of 8, ldx and ld_out >= H");
    if (!check_arch()) return fail(FP8LIN_ERR_ARCH, "fp8lin kernels are built for sm_100a only");
    const MoeWs L = moe_ws_layout(rows, E, H, I);
    if (!workspace || workspace_bytes < L.total)
        return fail(FP8LIN_ERR_WORKSPACE, "workspace too small: need %zu bytes", L.total);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char* ws = (unsigned char*)workspace;
    int* offsets = (int*)(ws + L.off_offsets);
    int* sorted = (int*)(ws + L.off_sorted);
    int4* chunks = (int4*)(ws + L.off_chunks);
    int* meta = (int*)(ws + L.off_meta);
    __nv_bfloat16* gu = (__nv_bfloat16*)(ws + L.off_gu);
    unsigned char* hq = ws + L.off_hq;
    const int mp = grouped_chunk_rows(rows, E);
    cudaError_t e = launch_moe_align(ids, (int)rows, E, mp, offsets, sorted, chunks, meta, st);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "row grouping launch: %s", cudaGetErrorString(e));
    const char* why = nullptr;
    GroupedArgs a;
    a.x = (const __nv_bfloat16*)x; a.sorted_rows = sorted; a.chunks = chunks; a.meta = meta; a.w_scale = w13_scale;
    a.input_scale = w13_input_scale; a.topk_w = topk_w; a.out = gu; a.status = (int*)workspace;
    a.ldx = (int)ldx; a.x_div = x_div; a.ld_out = (int)(2 * I); a.N = (int)(2 * I); a.K = (int)H; a.n_tiles = 0; a.kblocks = 0;
    a.scatter = 0;
    // Prefill-sized batches whose experts fill 128-row chunks: both projections run with the rows as the MMA M dimension
    // (umma_grouped_rows.cu).  Measured on 4096 tokens (60 experts, top-4, H 2048, I 1408) against the channel-major kernel.
    const bool rows_major = rows >= kMoePrequantRows && mp == 128 && g_tune.moe_rows_major != 0;
    // prefill-sized batches with whole 128-channel tiles: the gate_up GEMM's epilogue applies the activation and writes hq
    // (from 32-row chunks on: the epilogue reads the two accumulators 32 rows at a time)
    const bool fused_act = rows >= kMoePrequantRows && I % 128 == 0 && mp >= 32 && g_tune.moe_fused != 0;
    if (rows >= kMoePrequantRows) {
        unsigned char* xq = ws + L.off_xq;
        e = launch_moe_gather_quant((const __nv_bfloat16*)x, ldx, x_div, sorted, meta, w13_input_scale, xq, (int)rows, (int)H, st);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "row gather launch: %s", cudaGetErrorString(e));
        if (fused_act) {
            GroupedArgs f = a;
            f.N = (int)I; f.hq = hq; f.h_scale = w2_input_scale; f.out = nullptr;
            e = rows_major ? launch_grouped_rows_w8a8(f, w13_packed, E, xq, rows, st, &why)
                           : launch_grouped_w8a8(false, mp, f, w13_packed, E, xq, rows, st, &why);
        } else {
            e = launch_grouped_w8a8(false, mp, a, w13_packed, E, xq, rows, st, &why);
        }
    } else {
        e = launch_grouped_w8a8(true, mp, a, w13_packed, E, nullptr, 0, st, &why);
    }
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "gate_up grouped GEMM launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
    if (!fused_act) {
        e = launch_silu_mul_quant(gu, w2_input_scale, hq, meta, (int)rows, (int)I, st);
        if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "activation launch: %s", cudaGetErrorString(e));
    }
    a.w_scale = w2_scale; a.input_scale = w2_input_scale; a.out = (__nv_bfloat16*)out_routed; a.ld_out = (int)ld_out;
    a.N = (int)H; a.K = (int)I; a.scatter = 1;
    if (rows_major && H % 8 == 0 && ld_out % 8 == 0 && aligned16(out_routed))
        e = launch_grouped_rows_w8a8(a, w2_packed, E, hq, rows, st, &why);
    else
        e = launch_grouped_w8a8(false, mp, a, w2_packed, E, hq, rows, st, &why);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "down grouped GEMM launch: %s (%s)", cudaGetErrorString(e), why ? why : "");
    return FP8LIN_OK;
}

int fp8lin_moe_combine(const void* routed, void* y, int64_t T, int top_k, int64_t H, void* stream) {
    if (T < 0 || top_k <= 0 || H <= 0 || H % 8 != 0) return fail(FP8LIN_ERR_SHAPE, "bad combine shape");
    if (T == 0) return FP8LIN_OK;
    if (!routed || !y) return fail(FP8LIN_ERR_NULL, "routed and y must not be NULL");
    if (!aligned16(routed) || !aligned16(y)) return fail(FP8LIN_ERR_ALIGN, "routed and y must be 16-byte aligned");
    cudaError_t e = launch_moe_combine((const __nv_bfloat16*)routed, (__nv_bfloat16*)y, (int)T, top_k, (int)H, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "combine launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_debug_wait_timeout(void* workspace, int64_t limit_us, void* stream) {
    if (!workspace) return fail(FP8LIN_ERR_NULL, "workspace must not be NULL");
    if (limit_us < 1 || limit_us > 100000) return fail(FP8LIN_ERR_ARG, "limit_us must be 1..100000");
    if (!check_arch()) return fail(FP8LIN_ERR_ARCH, "fp8lin kernels are built for sm_100a only");
    // clock64 ticks at the SM clock: at most ~2 GHz, so 2000 cycles per microsecond is an upper bound
    cudaError_t e = launch_wait_timeout_probe((int*)workspace, (long long)limit_us * 2000, nullptr, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "probe launch: %s", cudaGetErrorString(e));
    return FP8LIN_OK;
}

int fp8lin_read_status(void* workspace, void* stream, int* status_out) {
    if (!workspace || !status_out) return fail(FP8LIN_ERR_NULL, "workspace and status_out must not be NULL");
    cudaStream_t st = (cudaStream_t)stream;
    int v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(FP8LIN_ERR_LAUNCH, "status read: %s", cudaGetErrorString(e));
    *status_out = v;
    if (v != 0) {
        cudaMemsetAsync(workspace, 0, sizeof(int), st);
        cudaStreamSynchronize(st);
        return fail(FP8LIN_ERR_DEVICE, "a kernel gave up a bounded wait (device status 0x%x)", v);
    }
    return FP8LIN_OK;
}

}  // extern "C"
