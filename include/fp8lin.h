/*
 * fp8lin — C ABI of the B200 (sm_100a) FP8 quantized-linear engine.
 *
 * Drop-in for the kernel launchers behind nano-vllm-moe's FP8 linear backend
 * (nanovllm/quantization/fp8.py, Fp8LinearMethod.apply).  Every pointer is a
 * CUDA device pointer unless stated otherwise; `stream` is a cudaStream_t
 * passed as void*.  All calls are asynchronous on `stream`, allocate nothing
 * on the device and never synchronise the host (except fp8lin_read_status);
 * the linears that take a caller-owned workspace are safe to capture in a CUDA
 * graph.  The library owns no tensor: every buffer, including scratch, belongs
 * to the caller (the one exception, fp8lin_linear_static_scratch, says so).
 *
 * Number formats
 *   activations x, bias, outputs y : bfloat16, row-major, row strides ldx/ldy in ELEMENTS
 *   weights                        : e4m3 (torch.float8_e4m3fn) bytes
 *   scales                         : float32
 *
 * Weight layouts
 *   "kn"     : [K][N], N contiguous — the layout of the reference's `qweight`
 *              buffer (fp8.py:80-83) after its loaders ran.
 *   "nk"     : [N][K], K contiguous — the checkpoint's own layout (quantize.py:56).
 *   "packed" : what every kernel here reads.  128-channel x 128-byte tiles, each
 *              tile contiguous (16 KiB), the tiles of one channel block consecutive
 *              along K; N and K zero-padded to multiples of 128:
 *                byte(n,k) = ((n/128)*ceil(K/128) + k/128)*16384 + (n%128)*128 + k%128
 *              A CTA streaming a channel block reads one sequential range of HBM and a
 *              tile is exactly one TMA box.  Produce it once per layer with
 *              fp8lin_prepack_weight (from "kn") or fp8lin_pack_weight_nk (from "nk").
 *              In the prototypes below `w_nk` names this packed buffer.
 *
 * Return value: 0 on success, otherwise one of the FP8LIN_ERR_* codes;
 * fp8lin_last_error() returns a thread-local description of the last failure.
 */
#ifndef FP8LIN_H
#define FP8LIN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FP8LIN_VERSION 1

enum {
    FP8LIN_OK = 0,
    FP8LIN_ERR_NULL = 1,       /* a required pointer is NULL */
    FP8LIN_ERR_SHAPE = 2,      /* M/K/N/ld out of range or K not a multiple of 16 */
    FP8LIN_ERR_ALIGN = 3,      /* pointer or stride not 16-byte aligned */
    FP8LIN_ERR_WORKSPACE = 4,  /* workspace missing or smaller than fp8lin_workspace_bytes */
    FP8LIN_ERR_ARCH = 5,       /* device is not sm_100 */
    FP8LIN_ERR_LAUNCH = 6,     /* CUDA reported a launch/driver error */
    FP8LIN_ERR_DEVICE = 7,     /* a kernel recorded a bounded-wait timeout (fp8lin_read_status) */
    FP8LIN_ERR_ARG = 8         /* unknown enum value / unsupported combination */
};

/* scheme ids; names follow the reference's `quantization_type` (fp8.py:20). */
enum { FP8LIN_W8A16 = 0, FP8LIN_W8A8_STATIC = 1 };

int fp8lin_version(void);
const char* fp8lin_last_error(void);
/* Number of kernel launches this library has made in this process (all devices, all streams).
 * A measurement aid with no counterpart in the reference: difference it around a call (or around
 * the capture of a CUDA graph) to know how many kernels that call enqueues. */
unsigned long long fp8lin_launch_count(void);

/* ---- weight prepack -------------------------------------------------------
 * Replaces the derived copies the reference builds in
 * Fp8LinearMethod.process_weights_after_loading (fp8.py:106-111).
 * qweight_kn: u8 [K][N] (or qweight_nk: u8 [N][K])  ->  packed tiles, fp8lin_packed_bytes(K,N)
 * bytes, 16-byte aligned.  K % 16 == 0. */
size_t fp8lin_packed_bytes(int64_t K, int64_t N);
int fp8lin_prepack_weight(const void* qweight_kn, void* w_packed, int64_t K, int64_t N, void* stream);
int fp8lin_pack_weight_nk(const void* qweight_nk, void* w_packed, int64_t K, int64_t N, void* stream);

/* ---- scratch --------------------------------------------------------------
 * Bytes of caller-owned scratch a linear call of this shape needs (split-K
 * partial sums, quantised activations, tile counters; W8A16 from 256 rows: the
 * activations as f16 plus one chunk, at most 64 MiB, of weights widened to f16).
 * Scratch must be
 * 256-byte aligned, ZERO-FILLED ONCE after allocation (the first
 * FP8LIN_WS_HEADER_BYTES hold counters that every kernel leaves at zero), and
 * must not be shared by calls that can run concurrently (one per stream). */
#define FP8LIN_WS_HEADER_BYTES 65536
size_t fp8lin_workspace_bytes(int scheme, int64_t M, int64_t K, int64_t N);

/* ---- the linears ----------------------------------------------------------
 * y[M,N] = bf16( (x . W^T) * w_scale[n] + bias[n] )
 * Replaces launch_w8a16_gemm (nanovllm/quantization/kernels/fp8.py:79-109) and
 * w8a16_cuda_forward (nanovllm/quantization/csrc/w8a16_ext.cpp:3-11).
 * bias may be NULL.  From 256 rows on (and for 33..64 rows) the call needs the
 * workspace that fp8lin_workspace_bytes(FP8LIN_W8A16, M, K, N) reports; below
 * that only when the shape is split along K. */
int fp8lin_w8a16(const void* x, int64_t ldx, const void* w_nk, const float* w_scale,
                 const void* bias, void* y, int64_t ldy,
                 int64_t M, int64_t K, int64_t N,
                 void* workspace, size_t workspace_bytes, void* stream);

/* xq = e4m3(clamp(x / max(*input_scale,1e-12), +-448));
 * y[M,N] = bf16( (xq . W^T) * max(*input_scale,1e-12) * w_scale[n] + bias[n] )
 * Replaces launch_w8a8_cuda_ptx_jit (nanovllm/quantization/w8a8_jit.py:521-542),
 * launch_w8a8_cutlass_gemm (nanovllm/quantization/cuda_ext.py:84-106 ->
 * csrc/w8a8_cutlass_kernel.cu:460-497) and launch_scaled_mm_w8a8
 * (kernels/fp8.py:376-396).  w_scale is per output channel ([N]); pass a
 * broadcast copy for a per-tensor scale.  input_scale points to ONE float on
 * the device. */
int fp8lin_w8a8(const void* x, int64_t ldx, const void* w_nk, const float* w_scale,
                const float* input_scale, const void* bias, void* y, int64_t ldy,
                int64_t M, int64_t K, int64_t N,
                void* workspace, size_t workspace_bytes, void* stream);

/* The same linear for activations that are ALREADY e4m3 (xq: u8 [M][K], rows K bytes apart, quantised with
 * *input_scale by fp8lin_rmsnorm_quant, fp8lin_quantize_activation or a producer of the caller's): no quantiser pass,
 * every M takes a tcgen05 kernel.  The reference has no such entry (its quantiser is always inside the linear call,
 * kernels/fp8.py:263-268 / csrc/w8a8_cutlass_kernel.cu:406-430); it is the second half of the RMSNorm fusion below.
 * workspace: at least FP8LIN_WS_HEADER_BYTES. */
int fp8lin_w8a8_preq(const void* xq, const void* w_nk, const float* w_scale, const float* input_scale,
                     const void* bias, void* y, int64_t ldy, int64_t M, int64_t K, int64_t N,
                     void* workspace, size_t workspace_bytes, void* stream);

/* RMSNorm fused with the static activation quantiser: the producer of a W8A8 linear's input.  Replaces
 * RMSNorm.rms_forward / add_rms_forward (nanovllm/layers/layernorm.py:17-41) followed by the quantiser of the linear
 * that consumes the result (kernels/fp8.py:250-252).
 *   v = x [+ residual] in fp32;  residual <- bf16(v) (in place, when residual is not NULL);
 *   y = bf16( v * (1 / sqrt(mean(v^2) + eps)) * weight )   -- one rounding: the arithmetic of the reference's compiled
 *                                                              methods, which keep the whole expression in fp32;
 *   xq = e4m3(clamp(y / max(*input_scale, 1e-12), +-448)).
 * x: bf16 [M][ldx]; residual: bf16 [M][ld_res] or NULL; weight: bf16 [H]; xq: u8 [M][H] (rows H bytes apart) or NULL;
 * y: bf16 [M][ldy] or NULL (for consumers that need the bf16 tensor, e.g. a W8A16 linear); at least one of xq / y.
 * H a multiple of 8, at most 8192.  One CTA per row; x is read once. */
int fp8lin_rmsnorm_quant(const void* x, int64_t ldx, void* residual, int64_t ld_res, const void* weight, float eps,
                         const float* input_scale, void* xq, void* y, int64_t ldy, int64_t M, int64_t H, void* stream);

/* Row-parallel W8A8 linear with the reduction folded into the GEMM's stores (no counterpart in
 * the reference, which calls dist.all_reduce after the GEMM, nanovllm/layers/linear.py:258-262).
 * fp8lin_w8a8_scatter computes this rank's bf16 partial output and its epilogue TMA-stores every
 * output box to each of dst_ptrs[0..n_dst) -- HOST array of device pointers to bf16 [M][ld_dst]
 * matrices, typically this rank's slot in every rank's peer-mapped buffer (NVLink stores, no
 * load from peer memory).  After a cross-rank barrier, fp8lin_sum_slots adds the n_slots partial
 * outputs of a local buffer (slot r at slots + r*slot_stride elements) in slot order in fp32 and
 * rounds once to bf16 -- the same sum the all-reduce produces, with a fixed order. */
int fp8lin_w8a8_scatter(const void* x, int64_t ldx, const void* w_nk, const float* w_scale,
                        const float* input_scale, const void* bias, int n_dst, void* const* dst_ptrs,
                        int64_t ld_dst, int64_t M, int64_t K, int64_t N,
                        void* workspace, size_t workspace_bytes, void* stream);
int fp8lin_sum_slots(const void* slots, int n_slots, int64_t slot_stride, int64_t ld_slot, void* y,
                     int64_t ldy, int64_t M, int64_t N, void* stream);
/* The same reduction in reduce-scatter / all-gather form, for more than two ranks (the store-to-everyone form above
 * sends (ranks - 1) x the payload per rank; this one 2 x (ranks - 1) / ranks).  fp8lin_w8a8_reduce_scatter computes
 * this rank's partial output and stores the rows of band d = [d * band_rows, (d + 1) * band_rows) ONLY to
 * dst_ptrs[d] (bf16 [band_rows][ld_dst]: this rank's slot in rank d's buffer), from that matrix's row 0 on;
 * band_rows a multiple of 32 with band_rows * n_dst >= M.  After a cross-rank barrier every rank owns all ranks'
 * partials of its band; fp8lin_sum_slots_gather adds them (fp32, slot order, one rounding) and stores the reduced
 * band at rows [dst_row, dst_row + M) of EVERY matrix in dst_ptrs (HOST array of n_dst device pointers to the ranks'
 * bf16 [..][ld_dst] outputs; plain 16-byte stores, peers over NVLink).  A second barrier, and every rank holds the
 * whole reduced result -- or skip the gather and keep the result sharded by rows. */
int fp8lin_w8a8_reduce_scatter(const void* x, int64_t ldx, const void* w_nk, const float* w_scale,
                               const float* input_scale, const void* bias, int n_dst, void* const* dst_ptrs,
                               int64_t ld_dst, int64_t band_rows, int64_t M, int64_t K, int64_t N,
                               void* workspace, size_t workspace_bytes, void* stream);
int fp8lin_sum_slots_gather(const void* slots, int n_slots, int64_t slot_stride, int64_t ld_slot, int n_dst,
                            void* const* dst_ptrs, int64_t ld_dst, int64_t dst_row, int64_t M, int64_t N, void* stream);

/* Decode-sized linear (M <= 64, either scheme) that needs no workspace from the
 * caller and allocates nothing.  It has no counterpart in the reference; it
 * exists for callers that cannot allocate: a server whose KV-cache pool has
 * taken all free HBM, or a latency-critical loop that must not risk the stall
 * an allocation can cause.  Its split-K scratch is a fixed 16 MiB (+64 KiB
 * header) array inside the library image, one copy per GPU.  CUDA loads that
 * part of the image lazily: a GPU sets its copy aside at the first call of this
 * function on that GPU and holds it until the process exits.  Make that first
 * call (any small shape) early on every GPU -- before the process gives the
 * remaining HBM to a pool, else the call fails with FP8LIN_ERR_WORKSPACE -- and
 * outside any stream capture: it looks up the array's device address with
 * cudaGetSymbolAddress.  Shapes whose split-K partial sums exceed 16 MiB, or
 * M > 64, are refused with FP8LIN_ERR_WORKSPACE.  All calls on a GPU share the
 * array: calls that may overlap in time (different streams or threads) race on
 * it and must be serialised by the caller.  input_scale is ignored for
 * FP8LIN_W8A16. */
int fp8lin_linear_static_scratch(int scheme, const void* x, int64_t ldx, const void* w_nk,
                                 const float* w_scale, const float* input_scale, const void* bias,
                                 void* y, int64_t ldy, int64_t M, int64_t K, int64_t N, void* stream);

/* Stand-alone activation quantiser; replaces quantize_activation_kernel
 * (csrc/w8a8_cutlass_kernel.cu:406-430) / act_quant_fp8_kernel (kernels/fp8.py:232-249).
 * xq: u8 [M][K] contiguous. */
int fp8lin_quantize_activation(const void* x, int64_t ldx, const float* input_scale,
                               void* xq, int64_t M, int64_t K, void* stream);

/* ---- MoE expert FFN --------------------------------------------------------------
 * The routed expert FFN of nanovllm/executor/moe on FP8 operands, as a grouped GEMM
 * through the same tcgen05 kernels.  Expert weights are packed per expert with
 * fp8lin_pack_weight_nk and concatenated: w13_packed = E x packed(K=H, N=2I) with rows
 * [0,I) = gate, [I,2I) = up (the reference's w13 stacking, blocks/base.py:58-63),
 * w2_packed = E x packed(K=I, N=H).  Scales: w13_scale f32 [E][2I], w2_scale f32 [E][H],
 * one static activation scale per projection.
 *
 * From 512 routed rows on the rows are gathered and quantised once, the gate_up grouped GEMM applies silu(g) * u and
 * the down projection's quantiser in its epilogue (I a multiple of 128), and with more than 64 rows per expert on
 * average both grouped GEMMs run with the routed rows as the MMA M dimension (128 x 256 work items).
 * fp8lin_moe_route replaces SoftmaxTopKRouter.select_experts (executor/moe/router.py:24-34):
 * fp32 softmax over E logits (logits_dtype 0 = f32, 1 = bf16), top-k, optional
 * renormalisation; topk_w f32 [T][k], topk_ids i32 [T][k]. */
int fp8lin_moe_route(const void* logits, int logits_dtype, int64_t ld, int64_t T, int E, int top_k,
                     int renormalize, float* topk_w, int32_t* topk_ids, void* stream);

/* Grouping of routed rows by expert, the first step of fp8lin_moe_experts_w8a8, also callable on its
 * own; replaces moe_align_block_size (nanovllm/utils/moe.py:4-52).  ids: int32 [rows] expert id per
 * routed row (ids outside [0, E) are dropped: another expert-parallel rank owns them).  Outputs, all
 * device memory: expert_offsets int32 [E + 1] (first sorted position of every expert), sorted_rows
 * int32 [rows] (routed-row index at each sorted position; rows of one expert are adjacent, their
 * order inside an expert is unspecified), chunks int32 [(E + rows/16 + 2)][4] = {expert, first sorted
 * position, rows in the chunk, 0} with at most chunk_rows (16, 32, 64 or 128) rows each, meta int32 [2] =
 * {number of chunks, number of kept rows}.  E <= 3071.  Unlike the reference's block list the chunks
 * are not padded: a short chunk simply says how many rows it has. */
int fp8lin_moe_align(const int32_t* ids, int64_t rows, int E, int chunk_rows, int32_t* expert_offsets,
                     int32_t* sorted_rows, int32_t* chunks, int32_t* meta, void* stream);

/* Scratch for fp8lin_moe_experts_w8a8 (zero-filled once, like the linear workspace). */
size_t fp8lin_moe_workspace_bytes(int64_t rows, int E, int64_t H, int64_t I);

/* Replaces MoEExpertsKernel.apply (experts/eager_experts.py:9-35, experts/optimized.py:142-270)
 * for `rows` routed rows: ids[r] is the LOCAL expert of routed row r (rows whose id is outside
 * [0,E) are skipped and their output row is left untouched), topk_w[r] its routing weight, and
 * the row's activations are x[r / x_div] (x_div = top_k when x holds one row per token, as
 * NoEPPrepareFinalize.prepare expands it, no_ep.py:27; x_div = 1 when x already holds one row per
 * routed row, as after the expert-parallel dispatch, torch_alltoall.py:49).
 *   gu = bf16(W8A8(x_r, W13[e]));  h = bf16(silu(gate) * up);
 *   out_routed[r] = bf16( W8A8(h, W2[e]) * topk_w[r] )            bf16 [rows][ld_out]
 * Groups rows by expert on the device (no host synchronisation). */
int fp8lin_moe_experts_w8a8(const void* x, int64_t ldx, int x_div, const int32_t* ids, const float* topk_w,
                            int64_t rows, const void* w13_packed, const float* w13_scale,
                            const float* w13_input_scale, const void* w2_packed, const float* w2_scale,
                            const float* w2_input_scale, int E, int64_t H, int64_t I, void* out_routed,
                            int64_t ld_out, void* workspace, size_t workspace_bytes, void* stream);

/* y[t] = bf16( sum_j routed[t*top_k + j] ) in slot order; replaces the .view(T,k,H).sum(1) of
 * NoEPPrepareFinalize.finalize (no_ep.py:45) / TorchAllToAllPrepareFinalize.finalize (:90). */
int fp8lin_moe_combine(const void* routed, void* y, int64_t T, int top_k, int64_t H, void* stream);

/* ---- exporter arithmetic -----------------------------------------------------------------
 * fp8lin_quantize_weight replaces quantize_fp8_per_output_channel of the checkpoint exporter
 * (scripts/quantization/quantize.py:51-55): w [N][K] (bf16, or fp32 when w_is_f32; row pitch ldw
 * elements) -> qweight_nk u8 [N][K] e4m3 codes and weight_scale[n] = max(amax_k |w|, 1e-8) / 448;
 * codes = RNE(clamp(w / scale, +-448)) with a true division, so they equal the exporter's bit for
 * bit.  K even.
 * fp8lin_abs_max folds max |x| of a bf16 activation batch into *amax (one float on the device,
 * start it at 0): the per-linear maximum the exporter's calibration hooks track
 * (scripts/quantization/quantize.py:154-164 and :200-203); input_scale = max(amax, 1e-8) / 448. */
int fp8lin_quantize_weight(const void* w, int w_is_f32, int64_t ldw, void* qweight_nk, float* weight_scale, int64_t N,
                           int64_t K, void* stream);
int fp8lin_abs_max(const void* x, int64_t ldx, int64_t M, int64_t K, float* amax, void* stream);

/* ---- fused MLP (W8A8-static) ----------------------------------------------------
 * y[M,N] = down( silu(gate(x)) * up(x) ): replaces the three steps of the reference's MLP block,
 * gate_up_proj -> SiluAndMul -> down_proj (nanovllm/models/qwen2.py:110-114,
 * nanovllm/layers/activation.py:11-14), with the two linears on FP8 weights.  The bf16 gate_up
 * result is never written for M > 64: the gate_up GEMM's epilogue computes h = bf16(silu(g) * u)
 * from g, u rounded to bf16 and quantises it with the down projection's activation scale; the down
 * GEMM reads those e4m3 rows directly.  Same roundings as the three separate steps.
 *   w_gate_up      packed tiles of the merged [2I][H] weight with the 128-channel tile rows
 *                  INTERLEAVED: gate rows 0..127, up rows 0..127, gate rows 128..255, ...
 *                  (a permutation of the 16 KiB x ceil(H/128) tile rows of fp8lin_pack_weight_nk's
 *                  output); gate_up_scale / gate_up_bias [2I] permuted the same way
 *   w_down         packed tiles of the [N][I] down weight; I % 128 == 0
 * Scratch: fp8lin_mlp_workspace_bytes(M, H, I, N), rules as for the linears. */
size_t fp8lin_mlp_workspace_bytes(int64_t M, int64_t H, int64_t I, int64_t N);
int fp8lin_mlp_w8a8(const void* x, int64_t ldx, const void* w_gate_up, const float* gate_up_scale,
                    const float* gate_up_input_scale, const void* gate_up_bias, const void* w_down,
                    const float* down_scale, const float* down_input_scale, const void* down_bias, void* y, int64_t ldy,
                    int64_t M, int64_t H, int64_t I, int64_t N, void* workspace, size_t workspace_bytes, void* stream);
/* The same block for activations that are already e4m3 (xq: u8 [M][H], rows H bytes apart, quantised with
 * *gate_up_input_scale -- e.g. by fp8lin_rmsnorm_quant, the post-attention norm of the reference's decoder layer,
 * nanovllm/models/qwen2.py:155-160): no quantiser pass in front of the gate_up GEMM.  Same scratch. */
int fp8lin_mlp_w8a8_preq(const void* xq, const void* w_gate_up, const float* gate_up_scale,
                         const float* gate_up_input_scale, const void* gate_up_bias, const void* w_down,
                         const float* down_scale, const float* down_input_scale, const void* down_bias, void* y, int64_t ldy,
                         int64_t M, int64_t H, int64_t I, int64_t N, void* workspace, size_t workspace_bytes, void* stream);

/* Which kernel variant a shape is routed to ("stream_mma_w8a8_m16", "umma_w8a8_128x256", ...),
 * for labelling bench rows and ncu captures.  Host-only, returns a static string. */
const char* fp8lin_variant_name(int scheme, int64_t M, int64_t K, int64_t N);

/* Bench/ncu studies only: force a tuning knob (value < 0 restores the default).  Not thread safe.
 * Knobs: "stream_splits", "stream_max_m", "umma_bn", "umma_splits", "umma_pair" (CTA-pair GEMM on/off),
 * "swap_splits", "swap_enable", "swap_min_m", "swap_preq_min_m", "w8a16_swap_enable", "w8a16_swap_min_m", "fuse_quant" (1 = large-M W8A8 quantises most rows with warps of the GEMM
 * itself instead of a pass in front of it; n > 1 = the pass takes the first n rows), "quant_lead",
 * "w8a16_umma_min_m" (rows from which W8A16 takes the f16 GEMM route; 0 = never), "w8a16_chunk_mb", "pdl",
 * "stream_push" (0 = split-K of the mma.sync streaming kernel always through global scratch instead of a cluster),
 * "mlp_decode_fused" (1 = the fused MLP on up to 16 pre-quantised rows computes silu * up inside the gate_up kernel),
 * "moe_fused" (0 = the expert FFN keeps a separate activation pass), "moe_rows_major" (0 = prefill-sized expert
 * batches stay on the channel-major grouped kernel), "pair_stages" (4 or 5 ring slots in the CTA-pair GEMM). */
int fp8lin_set_tuning(const char* knob, int value);

/* Blocking: copies the device status word out of `workspace` (after syncing
 * `stream`) and clears it.  0 = no kernel gave up a bounded wait.  Otherwise the code of the wait
 * that ran out (about a second): 0x101 operand tile never landed, 0x102 ring slot never freed, 0x103 /
 * 0x104 accumulator never filled / never drained, 0x105 in-kernel activation quantiser, 0x106 a peer
 * CTA of the cluster (split-K hand-over) never answered. */
int fp8lin_read_status(void* workspace, void* stream, int* status_out);

/* Exercises the give-up path of the kernels' bounded waits without a fault (no counterpart in the
 * reference, whose kernels have no such waits): launches one CTA that waits, with the same routine the
 * tcgen05 kernels use but a limit of about `limit_us` microseconds (1..100000), on a barrier nothing
 * arrives on.  The wait runs out, the kernel writes its code to the status word at the start of
 * `workspace` and returns normally; the next fp8lin_read_status reports FP8LIN_ERR_DEVICE and clears it. */
int fp8lin_debug_wait_timeout(void* workspace, int64_t limit_us, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FP8LIN_H */
