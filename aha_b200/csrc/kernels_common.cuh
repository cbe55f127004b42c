// kernels_common.cuh -- elementwise / normalisation / gather kernels shared by text, vision and audio paths.
// All activations are fp32; linear weights are fp16 (lossless for the fp16 checkpoints) and every
// product is formed in fp32 -- the same arithmetic as the reference's Candle F32 CPU path.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace aha {

// Embedding::forward (row gather), fp16 table -> fp32 rows.  /root/reference/src/models/qwen3/model.rs:191-193
static __global__ void embed_gather_kernel(const uint32_t* __restrict__ ids, const __half* __restrict__ table,
                                    float* __restrict__ out, int S, int H, int V) {
    const int s = blockIdx.x;
    uint32_t id = ids[s];
    if (id >= (uint32_t)V) id = V - 1;  // host validates; keep the kernel memory-safe regardless
    const __half* row = table + (size_t)id * H;
    for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
        float2 v = __half22float2(*reinterpret_cast<const __half2*>(row + i));
        *reinterpret_cast<float2*>(out + (size_t)s * H + i) = v;
    }
}

// candle_nn RmsNorm over the last dim: x / sqrt(mean(x^2) + eps) * w.  One block per row.
static __global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                               float* __restrict__ out, int H) {
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)blockIdx.x * H + i] = xr[i] * inv * w[i];
}

// x = hi + lo with both halves fp16 (|lo| <= 2^-11 |hi|): the operand format of the tensor-core GEMMs (gemm_tc.cuh).  Producers that feed
// a GEMM write the two halves directly instead of an fp32 tensor that a separate pass would have to read back and split.
__device__ __forceinline__ void split_half(float x, __half& h, __half& l) {
    h = __float2half_rn(x);
    l = __float2half_rn(x - __half2float(h));
}
// rmsnorm_kernel with the split output: out_hi / out_lo [rows, H] fp16
static __global__ void rmsnorm_split_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, __half* __restrict__ out_hi,
                                     __half* __restrict__ out_lo, int H) {
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        __half h, l;
        split_half(xr[i] * inv * w[i], h, l);
        out_hi[(size_t)blockIdx.x * H + i] = h;
        out_lo[(size_t)blockIdx.x * H + i] = l;
    }
}
// layernorm_kernel with the split output
static __global__ void layernorm_split_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                       __half* __restrict__ out_hi, __half* __restrict__ out_lo, int H) {
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += xr[i];
    const float mean = block_sum(s, red) / (float)H;
    float v = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float d = xr[i] - mean; v = fmaf(d, d, v); }
    const float inv = 1.0f / sqrtf(block_sum(v, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        __half h, l;
        split_half((xr[i] - mean) * inv * w[i] + b[i], h, l);
        out_hi[(size_t)blockIdx.x * H + i] = h;
        out_lo[(size_t)blockIdx.x * H + i] = l;
    }
}

// candle_nn LayerNorm (remove_mean, affine): (x-mean)/sqrt(var+eps)*w+b.  One block per row of length H.
static __global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                 const float* __restrict__ b, float eps, float* __restrict__ out, int H) {
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += xr[i];
    const float mean = block_sum(s, red) / (float)H;
    float v = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float d = xr[i] - mean; v = fmaf(d, d, v); }
    const float inv = 1.0f / sqrtf(block_sum(v, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t)blockIdx.x * H + i] = (xr[i] - mean) * inv * w[i] + b[i];
}

// out[idx[r], :] = src[r, :]   (masked_scatter_dim0, /root/reference/src/utils/tensor_utils.rs:294-321)
// add != 0: out[idx[r], :] += src[r, :]   (mask_index_add, tensor_utils.rs:466-470)
static __global__ void scatter_rows_kernel(const int* __restrict__ idx, const float* __restrict__ src,
                                    float* __restrict__ out, int H, int add) {
    const int r = blockIdx.x;
    float* o = out + (size_t)idx[r] * H;
    const float* s = src + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = add ? (o[i] + s[i]) : s[i];
}

// l2_normalize (/root/reference/src/models/common/modules.rs:1287-1294): x / sqrt(sum(x^2) + 1e-6), one row per block.
static __global__ void l2_normalize_kernel(const float* __restrict__ x, float* __restrict__ out, int H) {
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss + 1e-6f);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)blockIdx.x * H + i] = xr[i] * inv;
}

static __global__ void add_inplace_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += y[i];
}

// Two-stage argmax, "first maximal index" like candle's Sampling::ArgMax.
// Stage 1 is fused into the lm_head GEMV epilogue where possible; this standalone version covers logits[V].
static __global__ void argmax_partial_kernel(const float* __restrict__ logits, int V, float* __restrict__ pmax,
                                      int* __restrict__ pidx) {
    __shared__ float smax[32];
    __shared__ int sidx[32];
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
        float v = logits[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { smax[wid] = best; sidx[wid] = bi; }
    __syncthreads();
    if (wid == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? smax[lane] : -INFINITY;
        bi = lane < nw ? sidx[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { pmax[blockIdx.x] = best; pidx[blockIdx.x] = bi; }
    }
}

// Stage 2: reduce the per-block candidates, publish the token, and advance the device-side decode state:
// state[0] = next token, state[1] = position of the next token (ctx so far), history[state[2]++] = token.
struct DecodeState {
    uint32_t token;      // input token of the next step
    int32_t pos;         // seqlen_offset of the next step (= tokens already cached)
    int32_t rope_delta;  // Qwen3-VL rope_deltas (0 for text / ASR)
    int32_t n_hist;      // tokens written to history
    uint32_t n_draws;    // random draws the request's sampler has consumed (index into its ChaCha12 stream)
    uint32_t pad_[3];
};
static __global__ void argmax_final_kernel(const float* __restrict__ pmax, const int* __restrict__ pidx, int n,
                                    uint32_t* __restrict__ argmax_out, DecodeState* __restrict__ st,
                                    uint32_t* __restrict__ history, int hist_cap, int advance) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += 32) {
        float v = pmax[i];
        int id = pidx[i];
        if (v > best || (v == best && id < bi)) { best = v; bi = id; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) {
        if (bi == 0x7fffffff) bi = 0;   // every candidate NaN: publish a valid id
        if (argmax_out) *argmax_out = (uint32_t)bi;
        if (advance && st) {
            st->token = (uint32_t)bi;
            st->pos += 1;
            if (history && st->n_hist < hist_cap) history[st->n_hist] = (uint32_t)bi;
            st->n_hist += 1;
        }
    }
}


// ---- kernels of the ragged (varlen) path -------------------------------------------------------------------------------------------
// Row gather from an embedding table stored as fp32 or bf16 (both widen exactly to the fp32 residual stream), times `scale`.  pos_table
// ([max_pos, H] fp32): row tok_pos[s] of a learned position table is added (unscaled).  copy: the rows are stored there as well.
template <typename WT>
static __global__ void embed_gather_any_kernel(const uint32_t* __restrict__ ids, const WT* __restrict__ table, float* __restrict__ out, int H, int V, float scale = 1.f,
                                               const float* __restrict__ pos_table = nullptr, const int* __restrict__ tok_pos = nullptr, int max_pos = 0,
                                               float* __restrict__ copy = nullptr) {
    const int s = blockIdx.x;
    uint32_t id = ids[s];
    if (id >= (uint32_t)V) id = V - 1;  // the host validates; keep the kernel memory-safe regardless
    const WT* row = table + (size_t)id * H;
    const float* prow = pos_table ? pos_table + (size_t)min(max(tok_pos[s], 0), max_pos - 1) * H : nullptr;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = (float)row[i] * scale;
        if (prow) v += prow[i];
        out[(size_t)s * H + i] = v;
        if (copy) copy[(size_t)s * H + i] = v;
    }
}

// Post-norm residual step with a scalar gain: x[row] += g * y[row] / sqrt(mean(y[row]^2) + eps).  The gain is ONE number (read from
// device memory); the norm sits on the sublayer's output, the residual sum stays fp32.  One block per row.
static __global__ void scalar_rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gain, float eps, int H) {
    __shared__ float red[32];
    const float* yr = y + (size_t)blockIdx.x * H;
    float* xr = x + (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = yr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float sc = gain[0] / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) xr[i] = fmaf(yr[i], sc, xr[i]);
}

// out[r] = g * x[rows[r]] / sqrt(mean(x[rows[r]]^2) + eps): the final norm of the rows whose logits are wanted, gathered on the way.
static __global__ void scalar_rmsnorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ gain, float eps,
                                                  float* __restrict__ out, int H) {
    __shared__ float red[32];
    const float* xr = x + (size_t)rows[blockIdx.x] * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float sc = gain[0] / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)blockIdx.x * H + i] = xr[i] * sc;
}

// Tokens that never left the device: packed token t of a ragged step is the last sampled token of slot fb_slot[t] (>= 0), else the id the host sent.
static __global__ void feedback_tokens_kernel(uint32_t* __restrict__ tokens, const int* __restrict__ fb_slot, const DecodeState* __restrict__ states, int T) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T && fb_slot[t] >= 0) tokens[t] = states[fb_slot[t]].token;
}

}  // namespace aha
