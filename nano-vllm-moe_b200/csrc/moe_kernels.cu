// Small kernels around the MoE expert FFN: router, row grouping, activation, combine.
#include "common.cuh"
#include "kernels.h"

namespace fp8lin {

// ---- router ---------------------------------------------------------------------------
// One warp per token: fp32 softmax over the E router logits, then top-k by k rounds of a
// warp arg-max (ties go to the lower expert index), optional renormalisation of the k
// weights.  Same algebra as softmax(dtype=float32) -> topk -> (w / sum w).
// kMaxPerLane: experts per lane (E <= 32 * kMaxPerLane); small expert counts get a short unrolled loop.
template <typename LogitT, int kMaxPerLane>
__global__ void __launch_bounds__(256)
moe_route_kernel(const LogitT* __restrict__ logits, int64_t ld, int T, int E, int top_k, int renormalize,
                 float* __restrict__ out_w, int* __restrict__ out_ids) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= T) return;
    float v[kMaxPerLane];
    const LogitT* row = logits + (size_t)token * ld;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? (float)row[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? expf(v[i] - mx) : 0.f;
        sum += v[i];
    }
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) v[i] = (lane + 32 * i) < E ? v[i] / sum : -1.f;

    float picked_w = 0.f;     // lane j keeps the j-th pick
    int picked_id = 0;
    float wsum = 0.f;
    for (int j = 0; j < top_k; ++j) {
        float best = -2.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            const int e = lane + 32 * i;
            if (v[i] > best) { best = v[i]; best_e = e; }     // ascending e per lane keeps the lowest index on ties
        }
        for (int o = 16; o; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (lane == j) { picked_w = best; picked_id = best_e; }
        wsum += best;
        if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;     // remove it from the next round
    }
    if (lane < top_k) {
        out_w[(size_t)token * top_k + lane] = renormalize ? picked_w / wsum : picked_w;
        out_ids[(size_t)token * top_k + lane] = picked_id;
    }
}

cudaError_t launch_moe_route(const void* logits, int logits_bf16, int64_t ld, int T, int E, int top_k, int renormalize,
                             float* out_w, int* out_ids, cudaStream_t stream) {
    if (T == 0) return cudaSuccess;
    const int warps = 8;
    dim3 grid((unsigned)((T + warps - 1) / warps));
#define FP8LIN_ROUTE(PER_)                                                                                                \
    do {                                                                                                                  \
        if (logits_bf16)                                                                                                  \
            moe_route_kernel<__nv_bfloat16, PER_><<<grid, warps * 32, 0, stream>>>((const __nv_bfloat16*)logits, ld, T, E, \
                                                                                   top_k, renormalize, out_w, out_ids);   \
        else                                                                                                              \
            moe_route_kernel<float, PER_><<<grid, warps * 32, 0, stream>>>((const float*)logits, ld, T, E, top_k,         \
                                                                           renormalize, out_w, out_ids);                  \
    } while (0)
    if (E <= 64) FP8LIN_ROUTE(2);
    else if (E <= 256) FP8LIN_ROUTE(8);
    else FP8LIN_ROUTE(32);
#undef FP8LIN_ROUTE
    return counted(cudaGetLastError());
}

// ---- grouping of routed rows by expert ------------------------------------------------------
// One CTA.  counts -> exclusive scan -> scatter.  Also writes the chunk list the grouped GEMM
// walks: every expert's rows are cut into chunks of `chunk_rows`.
//   sorted_rows[pos]     routed-row index at sorted position pos (rows of one expert are adjacent)
//   expert_offsets[e]    first sorted position of expert e (E+1 entries)
//   chunks[c]            {expert, first sorted position, rows in chunk, 0}
//   meta[0] = number of chunks, meta[1] = number of rows that had a valid local expert id
// Rows whose id is outside [0, E) are dropped (they belong to another expert-parallel rank).
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int rows, int E, int chunk_rows, int* __restrict__ expert_offsets,
                 int* __restrict__ sorted_rows, int4* __restrict__ chunks, int* __restrict__ meta) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int sh[];
    int* count = sh;            // [E]
    int* start = sh + E;        // [E + 1]
    int* fill = sh + 2 * E + 1; // [E]
    int* cstart = sh + 3 * E + 1;  // [E + 1] chunk prefix
    for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const int e = ids[r];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, cacc = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = acc; cstart[e] = cacc;
            acc += count[e];
            cacc += (count[e] + chunk_rows - 1) / chunk_rows;
        }
        start[E] = acc; cstart[E] = cacc;
        meta[0] = cacc; meta[1] = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_offsets[e] = start[e];
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const int e = ids[r];
        if (e >= 0 && e < E) sorted_rows[start[e] + atomicAdd(&fill[e], 1)] = r;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = count[e];
        for (int c = 0, pos = 0; pos < n; ++c, pos += chunk_rows)
            chunks[cstart[e] + c] = make_int4(e, start[e] + pos, min(chunk_rows, n - pos), 0);
    }
}

cudaError_t launch_moe_align(const int* ids, int rows, int E, int chunk_rows, int* expert_offsets, int* sorted_rows,
                             int4* chunks, int* meta, cudaStream_t stream) {
    const size_t smem = (size_t)(4 * E + 2) * sizeof(int);
    moe_align_kernel<<<1, 1024, smem, stream>>>(ids, rows, E, chunk_rows, expert_offsets, sorted_rows, chunks, meta);
    return counted(cudaGetLastError());
}

// (Within an expert the rows land in the arrival order of the atomics.  Every routed row is an
// independent column of the grouped GEMM, so the order does not change a single output bit.)

// ---- gather + quantise the routed rows once (prefill-sized batches) --------------------------
// xq[pos][:] = e4m3(x[sorted_rows[pos] / x_div][:] / scale) for every sorted position; the grouped
// GEMM then takes its "B" tiles by TMA instead of re-quantising the rows for every channel tile.
__global__ void __launch_bounds__(256)
moe_gather_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int x_div, const int* __restrict__ sorted_rows,
                        const int* __restrict__ meta, const float* __restrict__ input_scale,
                        unsigned char* __restrict__ xq, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int rows = meta[1];
    const ExactDiv div_scale(fmaxf(__ldg(input_scale), 1e-12f));
    const int vec_per_row = H / 16;
    const int64_t total = (int64_t)rows * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pos = i / vec_per_row;
        const int c = (int)(i - pos * vec_per_row) * 16;
        const int src_row = __ldg(sorted_rows + pos) / x_div;
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)src_row * ldx + c);
        const uint2 qa = quant8_e4m3(__ldg(src), div_scale);
        const uint2 qb = quant8_e4m3(__ldg(src + 1), div_scale);
        *reinterpret_cast<uint4*>(xq + pos * H + c) = make_uint4(qa.x, qa.y, qb.x, qb.y);
    }
}

cudaError_t launch_moe_gather_quant(const __nv_bfloat16* x, int64_t ldx, int x_div, const int* sorted_rows, const int* meta,
                                    const float* input_scale, unsigned char* xq, int max_rows, int H, cudaStream_t stream) {
    int64_t blocks = ((int64_t)max_rows * (H / 16) + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    if (blocks < 1) blocks = 1;
    moe_gather_quant_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, ldx, x_div, sorted_rows, meta, input_scale, xq, H);
    return counted(cudaGetLastError());
}

// ---- h = silu(gate) * up, quantised for the down projection ----------------------------------
// gu: bf16 [rows][2I] (gate | up), hq: e4m3 [rows][I].  The reference's experts evaluate
// F.silu(gate) * up as two eager bf16 ops (experts/eager_experts.py:33): silu(gate) is rounded to
// bf16, the product is rounded to bf16 again; that tensor is then divided by the static scale.
__global__ void __launch_bounds__(256)
silu_mul_quant_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ input_scale,
                      unsigned char* __restrict__ hq, const int* __restrict__ meta, int I) {
    pdl_launch_dependents();
    pdl_wait();
    const int rows = meta[1];
    const ExactDiv div_scale(fmaxf(__ldg(input_scale), 1e-12f));
    const int vec_per_row = I / 8;
    const int64_t total = (int64_t)rows * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec_per_row;
        const int c = (int)(i - r * vec_per_row) * 8;
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gu + r * 2 * I + c));
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c));
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint4 h;
        uint32_t* hw = reinterpret_cast<uint32_t*>(&h);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = bf16_lo(gw[j]), g1 = bf16_hi(gw[j]);
            const uint32_t sp = pack_bf16x2(g0 / (1.f + expf(-g0)), g1 / (1.f + expf(-g1)));
            hw[j] = pack_bf16x2(bf16_lo(sp) * bf16_lo(uw[j]), bf16_hi(sp) * bf16_hi(uw[j]));
        }
        *reinterpret_cast<uint2*>(hq + r * I + c) = quant8_e4m3(h, div_scale);
    }
}

cudaError_t launch_silu_mul_quant(const __nv_bfloat16* gu, const float* input_scale, unsigned char* hq, const int* meta,
                                  int max_rows, int I, cudaStream_t stream) {
    int64_t blocks = ((int64_t)max_rows * (I / 8) + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    if (blocks < 1) blocks = 1;
    silu_mul_quant_kernel<<<(unsigned)blocks, 256, 0, stream>>>(gu, input_scale, hq, meta, I);
    return counted(cudaGetLastError());
}

// ---- combine: y[t] = bf16( sum over the k routed rows of token t ) ---------------------------
// routed: bf16 [T*k][H] in routed-row order (slot j of token t at row t*k + j), summed in slot order.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ routed, __nv_bfloat16* __restrict__ y, int T, int top_k, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int vec_per_row = H / 8;
    const int64_t total = (int64_t)T * vec_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / vec_per_row;
        const int c = (int)(i - t * vec_per_row) * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < top_k; ++j) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(routed + ((size_t)t * top_k + j) * H + c));
            acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
            acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(y + t * H + c) = o;
    }
}

cudaError_t launch_moe_combine(const __nv_bfloat16* routed, __nv_bfloat16* y, int T, int top_k, int H,
                               cudaStream_t stream) {
    if (T == 0) return cudaSuccess;
    int64_t blocks = ((int64_t)T * (H / 8) + 255) / 256;
    if (blocks > sm_count() * 8) blocks = sm_count() * 8;
    moe_combine_kernel<<<(unsigned)blocks, 256, 0, stream>>>(routed, y, T, top_k, H);
    return counted(cudaGetLastError());
}

}  // namespace fp8lin
