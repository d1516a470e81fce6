// Internal launch interfaces between the C-ABI layer (api.cu) and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fp8lin {

// Record a printf-style message for fp8lin_last_error() and return `code` (defined in api.cu).
int set_error(int code, const char* fmt, ...);

// Fills the attribute that makes a launch a programmatic dependent of the previous kernel in
// its stream; returns the number of attributes written (0 when disabled by the tuning knob).
// Streaming multiprocessors of the current device (cached per process; 148, a B200's, when no device can be
// asked).  Grid sizes and the tile-round arithmetic of the launch plans are derived from it.
int sm_count();
// Whether the current device is an sm_100 part (cached per process; defined in api.cu).
bool device_is_sm100();
int pdl_attribute(cudaLaunchAttribute* attr);
void set_pdl_enabled(int on);

// Every kernel launch the library makes passes its result through counted(): successful launches
// are tallied for fp8lin_launch_count() (defined in api.cu).
void note_launch();
inline cudaError_t counted(cudaError_t e) {
    if (e == cudaSuccess) note_launch();
    return e;
}

// ---- weight-streaming kernel (stream_kernel.cu) ------------------------------
struct StreamArgs {
    const __nv_bfloat16* x;      // [M][ldx]
    const unsigned char* w;      // packed e4m3 tiles (pack_offset)
    const float* w_scale;        // [N]
    const float* input_scale;    // 1 float (W8A8) or nullptr
    const __nv_bfloat16* bias;   // [N] or nullptr
    __nv_bfloat16* y;            // [M][ldy]
    float* partial;              // split-K scratch
    int* counters;               // split-K arrival counters (zero between calls)
    int M, K, N;
    int ldx, ldy;
    int k_per_split;
    // Split-K of up to eight slices and at most 16 rows, when a status word is given: the slices of a channel tile form
    // a cluster and push their partial sums into slice 0's shared memory (no scratch, no counters, no second
    // global round trip); set by launch_stream.
    int* status = nullptr;
    int cluster_push = 0;
};

struct StreamPlan {
    int mt;            // 8-row groups of x per pass: 1, 2, 4 or 8
    int nwarps;        // warps per CTA (16 output channels each)
    int m_passes;      // ceil(M / (mt*8))
    int n_tiles;
    int splits;
    int k_per_split;
    size_t partial_bytes;
};

StreamPlan plan_stream(int scheme, int64_t M, int64_t K, int64_t N, int force_splits);
void set_stream_push(int on);      // study knob: 0 = split-K of the streaming kernel always through global scratch
cudaError_t launch_stream(int scheme, const StreamPlan& plan, StreamArgs args, cudaStream_t stream);

// ---- elementwise helpers (elementwise.cu) ------------------------------------
cudaError_t launch_act_quant(const __nv_bfloat16* x, int64_t ldx, const float* input_scale,
                             unsigned char* xq, int64_t M, int64_t K, cudaStream_t stream);
cudaError_t launch_quantize_weight(const void* w, bool w_is_f32, int64_t ldw, unsigned char* q, float* scale, int64_t N,
                                   int64_t K, cudaStream_t stream);
cudaError_t launch_abs_max(const __nv_bfloat16* x, int64_t ldx, int64_t M, int64_t K, float* amax, cudaStream_t stream);
cudaError_t launch_pack_tiles(const unsigned char* src, unsigned char* dst, int64_t K, int64_t N, bool src_is_kn,
                              cudaStream_t stream);

// RMSNorm (+ residual add) fused with the static activation quantiser (rmsnorm_quant.cu).  residual (in/out), xq and y
// may each be nullptr; H <= 8192, a multiple of 8.
cudaError_t launch_rmsnorm_quant(const __nv_bfloat16* x, int64_t ldx, __nv_bfloat16* residual, int64_t ld_res,
                                 const __nv_bfloat16* weight, float eps, const float* input_scale, unsigned char* xq,
                                 __nv_bfloat16* y, int64_t ldy, int64_t M, int64_t H, cudaStream_t stream);

// ---- tcgen05 GEMM (umma_gemm.cu) ---------------------------------------------
struct UmmaArgs {
    const unsigned char* xq;     // [M][K] e4m3, contiguous (produced by launch_act_quant)
    const unsigned char* w;      // packed e4m3 tiles (pack_offset)
    const float* w_scale;
    const float* input_scale;
    const __nv_bfloat16* bias;
    __nv_bfloat16* y;
    float* partial;              // split-K scratch (fp32 [splits][M][N])
    int* counters;
    int* status;                 // device status word
    int M, K, N;
    int ldy;
    // Activation quantisation inside the kernel (large-M W8A8, e4m3 operands only): when x is not NULL the
    // kernel's quantiser warps write rows [q_row_start, M) of xq from x while the GEMM runs; rows below
    // q_row_start (a multiple of 128) must already be in xq.  q_ctrl: 3 + ceil(M / 128) zeroed ints of scratch.
    // q_lead: 128-row blocks the quantiser may run ahead of the tiles in progress (at least the blocks that two
    // consecutive rounds of tiles span, so that no tile ever waits for a throttled quantiser).
    const __nv_bfloat16* x = nullptr;
    int ldx = 0;
    int q_row_start = 0;
    int q_lead = 0;
    int* q_ctrl = nullptr;
    // decode gate_up form of the swapped-operand kernel: e4m3 h = silu(gate) * up, [M][N / 2], written instead of y
    unsigned char* hq = nullptr;
    const float* h_scale = nullptr;
};

struct UmmaPlan {
    int bn;            // tile N: 64, 128 or 256
    int splits;        // split-K factor
    int kblocks_per_split;
    int m_tiles, n_tiles;
    int grid;          // persistent CTAs
    int tail_tiles;    // last tiles finished by a second, cluster split-K launch (0 = none)
    int tail_splits, tail_kps;
    int narrow_tiles;  // last tiles of a 256-wide persistent launch run as two 128-column halves each (0 = none)
    size_t partial_bytes;
};

UmmaPlan plan_umma(int64_t M, int64_t K, int64_t N, int force_bn, int force_splits);
// Returns cudaSuccess or an error; `why` (optional) receives a static description.
// n_dst == 0: the result goes to args.y.  n_dst >= 1 (non-split plans only): the epilogue stores every
// output box to each of dst_ptrs[0..n_dst) (bf16 [M][ld_dst] matrices; may be peer-GPU memory).
// band_rows > 0 (a multiple of 32): destination d receives only rows [d * band_rows, (d + 1) * band_rows) of the result,
// stored from its row 0 on (dst_ptrs[d] is a bf16 [band_rows][ld_dst] matrix).
cudaError_t launch_umma_w8a8(const UmmaPlan& plan, const UmmaArgs& args, cudaStream_t stream, const char** why,
                             int n_dst = 0, void* const* dst_ptrs = nullptr, int64_t ld_dst = 0, int64_t band_rows = 0);
// Large-M W8A16: the same GEMM on f16 operands.  args.xq = activations as f16 [M][K] (launch_x_to_f16),
// args.w = f16 weight tiles of the channels [0, N) (launch_dequant_tiles_f16), args.input_scale = nullptr.
cudaError_t launch_umma_f16(const UmmaPlan& plan, const UmmaArgs& args, cudaStream_t stream, const char** why);
cudaError_t launch_x_to_f16(const __nv_bfloat16* x, int64_t ldx, void* x16, int64_t M, int64_t K, cudaStream_t stream);
cudaError_t launch_dequant_tiles_f16(const unsigned char* src, void* dst, int64_t src_bytes, cudaStream_t stream);
// The same GEMM on CTA pairs (umma_pair_gemm.cu): 256 x 256 tiles, one MMA across two CTAs.  f16 selects the
// operand type as above; destinations as launch_umma_w8a8.
void set_pair_stages(int n);        // 4 or 5 ring slots instead of 6 in the e4m3 pair kernel (pipeline-depth studies)
cudaError_t launch_umma_pair(bool f16, const UmmaArgs& args, cudaStream_t stream, const char** why, int n_dst = 0,
                             void* const* dst_ptrs = nullptr, int64_t ld_dst = 0, int64_t band_rows = 0);
// Fused MLP pieces: gate_up GEMM whose epilogue writes e4m3 h = silu(g) * u for the down projection
// (umma_pair_gemm.cu), and the separate pass that does the same from a bf16 gate_up result (small batches).
cudaError_t launch_umma_pair_mlp(const UmmaArgs& args, unsigned char* hq, const float* h_scale, cudaStream_t stream,
                                 const char** why);
cudaError_t launch_silu_mul_quant_interleaved(const __nv_bfloat16* gu, const float* h_scale, unsigned char* hq, int64_t M,
                                              int64_t I, cudaStream_t stream);
cudaError_t launch_sum_slots(const __nv_bfloat16* slots, int n_slots, int64_t slot_stride, __nv_bfloat16* y, int64_t ldy,
                             int64_t M, int64_t N, int64_t ld_slot, cudaStream_t stream);

// A one-CTA launch whose only mbarrier is never arrived on: the bounded wait gives up after
// `limit_cycles`, writes kDevTimeoutFull to *status (and 1 to *gave_up if given) and returns.
cudaError_t launch_wait_timeout_probe(int* status, long long limit_cycles, int* gave_up, cudaStream_t stream);

// The same sum written to several destinations (this rank's band of a row-parallel result stored into every rank's
// output matrix by plain stores; peers over NVLink).
struct SumDst {
    __nv_bfloat16* y[8];
    int n;
};
cudaError_t launch_sum_slots_gather(const __nv_bfloat16* slots, int n_slots, int64_t slot_stride, int64_t ld_slot, SumDst dst,
                                    int64_t ld_dst, int64_t M, int64_t N, cudaStream_t stream);

// ---- swapped-operand tcgen05 kernel for M <= 64 (umma_swap.cu) -------------------
struct SwapPlan {
    int mp;            // token tile (MMA N): 16, 32 or 64
    int n_tiles;       // 128-channel tiles
    int splits;        // cluster split-K factor (1 = persistent over tiles)
    int kblocks_per_split;
    int grid;
    int preq;          // 1 = activations pre-quantised by act_quant (a.xq), 0 = quantised in the kernel from x
};

SwapPlan plan_swap(int64_t M, int64_t K, int64_t N, int force_splits, bool preq);
// `a.partial`, `a.counters` are unused (split-K is reduced through cluster shared memory); `a.xq`
// only when plan.preq.
// Up to 16 pre-quantised rows (a.xq) through a gate_up projection with interleaved tile rows: writes a.hq (see UmmaArgs).
cudaError_t launch_swap_gate_up(const UmmaArgs& a, cudaStream_t stream, const char** why);
cudaError_t launch_swap_w8a8(const SwapPlan& plan, const UmmaArgs& a, const void* x, int64_t ldx,
                             cudaStream_t stream, const char** why);

// ---- MoE expert FFN (moe_kernels.cu, umma_grouped.cu) ------------------------------
cudaError_t launch_moe_route(const void* logits, int logits_bf16, int64_t ld, int T, int E, int top_k, int renormalize,
                             float* out_w, int* out_ids, cudaStream_t stream);
cudaError_t launch_moe_align(const int* ids, int rows, int E, int chunk_rows, int* expert_offsets, int* sorted_rows,
                             int4* chunks, int* meta, cudaStream_t stream);
cudaError_t launch_moe_gather_quant(const __nv_bfloat16* x, int64_t ldx, int x_div, const int* sorted_rows, const int* meta,
                                    const float* input_scale, unsigned char* xq, int max_rows, int H, cudaStream_t stream);
cudaError_t launch_silu_mul_quant(const __nv_bfloat16* gu, const float* input_scale, unsigned char* hq, const int* meta,
                                  int max_rows, int I, cudaStream_t stream);
cudaError_t launch_moe_combine(const __nv_bfloat16* routed, __nv_bfloat16* y, int T, int top_k, int H, cudaStream_t stream);

struct GroupedArgs {
    const __nv_bfloat16* x;      // gather flavour: token matrix [x_rows][ldx]
    const int* sorted_rows;      // routed-row index per sorted position
    const int4* chunks;          // {expert, first sorted position, rows, 0}
    const int* meta;             // meta[0] = number of chunks
    const float* w_scale;        // [E][N]
    const float* input_scale;    // one float
    const float* topk_w;         // [routed rows] (down flavour)
    __nv_bfloat16* out;          // gate_up: [sorted rows][ld_out]; down: [routed rows][ld_out]
    int scatter;                 // 1 = down flavour: multiply by topk_w and scatter to routed-row order
    int* status;
    int ldx, x_div, ld_out;
    int N, K, n_tiles, kblocks;
    // fused gate_up + activation (launch_grouped_w8a8 with hq set): N = I gate channels, w_scale = [E][2 I], the epilogue
    // writes hq[sorted position][I] = e4m3(bf16(bf16(silu(g)) * u) / *h_scale) instead of `out`
    unsigned char* hq = nullptr;
    const float* h_scale = nullptr;
    int w_tiles = 0;             // 128-channel tile rows per expert in the packed weight (set by the launcher)
    int up_tile_offset = 0;      // tile rows from a gate tile to the up tile of the same channels (set by the launcher)
};
int grouped_chunk_rows(int64_t rows, int num_experts);
// Prefill-sized batches (umma_grouped_rows.cu): the routed rows are the MMA M dimension, 128 rows x 256 channels per work
// item, one epilogue thread per row.  args.hq set = gate_up with the activation fused (args.N = I); else the down projection
// (scatter to routed rows, times the routing weight).  Needs the chunk list made with 128-row chunks and rows already e4m3.
cudaError_t launch_grouped_rows_w8a8(GroupedArgs args, const void* w_packed, int num_experts, const void* xq_sorted,
                                     int64_t xq_rows, cudaStream_t stream, const char** why);
cudaError_t launch_grouped_w8a8(bool gather, int mp, GroupedArgs a, const void* w_packed, int num_experts,
                                const void* xq_sorted, int64_t xq_rows, cudaStream_t stream, const char** why);

// ---- swapped-operand tcgen05 kernel for W8A16, 9 <= M <= 64 (umma_swap_w8a16.cu) ----
SwapPlan plan_swap_w8a16(int64_t M, int64_t K, int64_t N, int force_splits);
cudaError_t launch_swap_w8a16(const SwapPlan& plan, const UmmaArgs& a, const void* x, int64_t ldx,
                              cudaStream_t stream, const char** why);

}  // namespace fp8lin
