// gemm_any.cuh -- C[M,N] = epilogue(A[M,K] (fp32) x W[N,K]^T + bias) on the CUDA cores for ANY M, N, K and for weights stored as
// fp32 or bf16.  Every product and every sum is fp32 (a bf16 weight widens exactly), so with fp32 weights this is the "true
// 32-bit" path of a model, and with bf16 weights it is the exact twin of the tensor-core path.  Two kernels:
//   gemm_any_kernel     64 x 64 tiles, bounds-checked on every side (sizes come from a checkpoint's config, nothing is assumed)
//   gemm_rows_kernel    M <= 8 rows (decode steps): a block owns 8 columns, its warps split K, activations in registers
//   gemm_skinny_kernel  M <= 8 rows that cannot be read 16 bytes at a time, or one or two rows of a short K: a warp streams two weight rows
// Each accumulates a given output element in an order that depends only on (K, kernel), never on the other rows' values.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace aha {

// SWIGLU: rows of W alternate gate / up; C[m][n / 2] = silu(gate) * up (N even); RELU2: max(v, 0)^2; CLAMP_GLU: rows alternate as for SWIGLU,
// the unit is clamp_glu_f(gate, up, act_a = limit, act_b = slope) (it runs the SWIGLU kernels with GemmAnyArgs::glu set)
enum AnyEpi { AEPI_STORE = 0, AEPI_XIELU = 1, AEPI_SWIGLU = 2, AEPI_RELU2 = 3, AEPI_CLAMP_GLU = 4 };

struct GemmAnyArgs {
    const float* A; int lda;
    const void* W;            // [N, K] row-major, float or __nv_bfloat16
    const float* bias;        // [N] or nullptr
    float* C; int ldc;
    int M, N, K;
    float act_a, act_b;       // AEPI_XIELU: alpha_p, alpha_n; AEPI_CLAMP_GLU: limit, slope
    int glu = 0;              // which gated unit the gate / up epilogue forms: 0 silu(gate) * up, 1 the clamped one (set by gemm_any)
    // Batches (grid z).  Batch b reads A + ai * a_bs and W + wi * w_bs (bias + wi * N) and writes C + b * c_bs, ai = a_index ? a_index[b] : b,
    // wi = w_index ? w_index[b] : b (both device arrays): per-head products (a_bs = the head's column offset), one expert's matrix per row, ...
    int batch = 1;
    size_t a_bs = 0, w_bs = 0, c_bs = 0;
    const int* a_index = nullptr;
    const int* w_index = nullptr;
    // ... or wi looked up on the way: wi = w_table[w_keys[b / w_div] * w_table_ld + b % w_div] (the choice b % w_div of the row whose key -- a
    // token id -- is w_keys[b / w_div], in a table of choices per key): a routed product needs no routing launch of its own
    const int* w_keys = nullptr;
    const int* w_table = nullptr;
    int w_table_ld = 0, w_div = 1;
    // row_offsets (device, [batch + 1]): batch b owns rows [ro[b], ro[b + 1]) of A and C, M is an upper bound of a batch's rows (tile kernel only)
    const int* row_offsets = nullptr;
    const int* a_gather = nullptr;   // (tile kernel only) row m of A is row a_gather[m] of the buffer: a gather folded into the load
};

// the block's batch: advances A, C, bias (and the returned W) and, with row offsets, narrows M
template <typename WT>
__device__ __forceinline__ const WT* any_batch_setup(GemmAnyArgs& g) {
    const WT* W = reinterpret_cast<const WT*>(g.W);
    const int b = blockIdx.z;
    const int wi = g.w_index ? g.w_index[b] : (g.w_keys ? g.w_table[(size_t)g.w_keys[b / g.w_div] * g.w_table_ld + b % g.w_div] : b);
    W += (size_t)wi * g.w_bs;
    if (g.bias) g.bias += (size_t)wi * (g.w_bs ? g.N : 0);
    g.A += (size_t)(g.a_index ? g.a_index[b] : b) * g.a_bs;
    g.C += (size_t)b * g.c_bs;
    if (g.row_offsets) {
        const int r0 = g.row_offsets[b];
        g.M = g.row_offsets[b + 1] - r0;
        if (g.a_gather) g.a_gather += r0; else g.A += (size_t)r0 * g.lda;
        g.C += (size_t)r0 * g.ldc;
    }
    return W;
}

__device__ __forceinline__ float wt_to_f(float v) { return v; }
__device__ __forceinline__ float wt_to_f(__nv_bfloat16 v) { return __bfloat162float(v); }

template <int EPI>
__device__ __forceinline__ float any_epilogue(const GemmAnyArgs& g, float v, int n) {
    if (g.bias) v += g.bias[n];
    if (EPI == AEPI_XIELU) v = xielu_f(v, g.act_a, g.act_b);
    if (EPI == AEPI_RELU2) v = relu2_f(v);
    return v;
}

__device__ __forceinline__ float any_swiglu(const GemmAnyArgs& g, float gate, float up, int n) {
    if (g.bias) { gate += g.bias[n]; up += g.bias[n + 1]; }
    return g.glu ? clamp_glu_f(gate, up, g.act_a, g.act_b) : silu_f(gate) * up;
}

template <typename WT, int EPI>
static __global__ void __launch_bounds__(256) gemm_any_kernel(GemmAnyArgs g) {
    constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Bs[BK][BN + PAD];
    const WT* __restrict__ W = any_batch_setup<WT>(g);
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    if (m0 >= g.M) return;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int m = m0 + lr, n = n0 + lr;
    const float* arow = g.A + (size_t)((g.a_gather && m < g.M) ? g.a_gather[m] : m) * g.lda;
    for (int k0 = 0; k0 < g.K; k0 += BK) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = k0 + lk + i;
            a[i] = (m < g.M && kk < g.K) ? arow[kk] : 0.f;
            b[i] = (n < g.N && kk < g.K) ? wt_to_f(W[(size_t)n * g.K + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) { As[lk + i][lr] = a[i]; Bs[lk + i][lr] = b[i]; }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int mm = m0 + ty * 4 + i;
        if (mm >= g.M) continue;
        if (EPI == AEPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int nn = n0 + tx * 4 + j;
                if (nn + 1 < g.N) g.C[(size_t)mm * g.ldc + nn / 2] = any_swiglu(g, acc[i][j], acc[i][j + 1], nn);
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nn = n0 + tx * 4 + j;
            if (nn < g.N) g.C[(size_t)mm * g.ldc + nn] = any_epilogue<EPI>(g, acc[i][j], nn);
        }
    }
}

// eight consecutive weights of a row as floats: one 16-byte streaming load for bf16, two for fp32
__device__ __forceinline__ void load_w8(const __nv_bfloat16* p, float (&w)[8]) {
    const uint4 u = ldg_stream(p);
    const uint32_t v[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { w[2 * i] = __uint_as_float(v[i] << 16); w[2 * i + 1] = __uint_as_float(v[i] & 0xffff0000u); }
}
__device__ __forceinline__ void load_w8(const float* p, float (&w)[8]) {
    const uint4 u0 = ldg_stream(p), u1 = ldg_stream(p + 4);
    w[0] = __uint_as_float(u0.x); w[1] = __uint_as_float(u0.y); w[2] = __uint_as_float(u0.z); w[3] = __uint_as_float(u0.w);
    w[4] = __uint_as_float(u1.x); w[5] = __uint_as_float(u1.y); w[6] = __uint_as_float(u1.z); w[7] = __uint_as_float(u1.w);
}

// M <= MB rows.  A warp owns two output columns at a time; lane l multiplies elements 8l .. 8l + 7 (+ 256, ...) of the two weight rows with
// the same elements of every activation row (L1-resident), then the warp tree-sums.  The weight matrix is streamed exactly once per
// launch with 16-byte loads (VEC: K % 8 == 0 and 16-byte aligned rows; otherwise element by element).
template <typename WT, int EPI, int MB, bool VEC>
static __global__ void __launch_bounds__(256) gemm_skinny_kernel(GemmAnyArgs g) {
    const WT* __restrict__ W = any_batch_setup<WT>(g);
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    for (int n = warp * 2; n < g.N; n += nwarps * 2) {
        const bool two = n + 1 < g.N;
        const WT* w0 = W + (size_t)n * g.K;
        const WT* w1 = W + (size_t)(two ? n + 1 : n) * g.K;
        float acc0[MB], acc1[MB];
#pragma unroll
        for (int r = 0; r < MB; ++r) { acc0[r] = 0.f; acc1[r] = 0.f; }
        if (VEC) {
#pragma unroll 4      // four steps' weight loads (eight of 16 bytes per lane) in flight: a warp's two rows alone do not cover the memory latency
            for (int k = lane * 8; k < g.K; k += 256) {
                float a[8], b[8];
                load_w8(w0 + k, a);
                load_w8(w1 + k, b);
#pragma unroll
                for (int r = 0; r < MB; ++r)
                    if (r < g.M) {
                        const float4 x0 = *reinterpret_cast<const float4*>(g.A + (size_t)r * g.lda + k);
                        const float4 x1 = *reinterpret_cast<const float4*>(g.A + (size_t)r * g.lda + k + 4);
                        const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i) { acc0[r] = fmaf(x[i], a[i], acc0[r]); acc1[r] = fmaf(x[i], b[i], acc1[r]); }
                    }
            }
        } else {
            for (int k = lane; k < g.K; k += 32) {
                const float a = wt_to_f(w0[k]), b = wt_to_f(w1[k]);
#pragma unroll
                for (int r = 0; r < MB; ++r)
                    if (r < g.M) { const float x = g.A[(size_t)r * g.lda + k]; acc0[r] = fmaf(x, a, acc0[r]); acc1[r] = fmaf(x, b, acc1[r]); }
            }
        }
#pragma unroll
        for (int r = 0; r < MB; ++r) {
            const float v0 = warp_sum(acc0[r]), v1 = warp_sum(acc1[r]);
            if (EPI == AEPI_SWIGLU) {
                if (lane == 0 && r < g.M && two) g.C[(size_t)r * g.ldc + n / 2] = any_swiglu(g, v0, v1, n);
            } else if (lane == 0 && r < g.M) {
                g.C[(size_t)r * g.ldc + n] = any_epilogue<EPI>(g, v0, n);
                if (two) g.C[(size_t)r * g.ldc + n + 1] = any_epilogue<EPI>(g, v1, n + 1);
            }
        }
    }
}

// M <= MB rows, K % 8 == 0, 16-byte aligned rows.  A block owns 8 output columns; its 8 warps take the steps of 256 elements of K in
// turn (lane l: elements 8 l .. 8 l + 7 of a step).  A lane keeps the activations of its step for all rows in registers and multiplies them
// with its 8 elements of each of the 8 weight rows: an activation is read once per 8 columns (the two-column kernel reads it again for
// every pair of columns and, with 8 rows, spends its time waiting for those loads), and all 8 weight loads of a step are in flight together.
// The partial sums are tree-summed in the warp, then over the warps in a fixed order.
template <typename WT, int EPI, int MB>
static __global__ void __launch_bounds__(256) gemm_rows_kernel(GemmAnyArgs g) {
    constexpr int NC = 8;
    __shared__ float part[8][NC * MB];
    const WT* __restrict__ W = any_batch_setup<WT>(g);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n0 = blockIdx.x * NC;
    float acc[NC][MB];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int r = 0; r < MB; ++r) acc[c][r] = 0.f;
#pragma unroll(MB <= 2 ? 4 : 1)      // few rows leave registers for several steps' loads in flight
    for (int k = warp * 256 + lane * 8; k < g.K; k += 8 * 256) {
        float w[NC][8], x[MB][8];
#pragma unroll
        for (int c = 0; c < NC; ++c) load_w8(W + (size_t)min(n0 + c, g.N - 1) * g.K + k, w[c]);
#pragma unroll
        for (int r = 0; r < MB; ++r) {
            float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
            if (r < g.M) {
                x0 = *reinterpret_cast<const float4*>(g.A + (size_t)r * g.lda + k);
                x1 = *reinterpret_cast<const float4*>(g.A + (size_t)r * g.lda + k + 4);
            }
            x[r][0] = x0.x; x[r][1] = x0.y; x[r][2] = x0.z; x[r][3] = x0.w; x[r][4] = x1.x; x[r][5] = x1.y; x[r][6] = x1.z; x[r][7] = x1.w;
        }
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int r = 0; r < MB; ++r)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[c][r] = fmaf(x[r][i], w[c][i], acc[c][r]);
    }
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int r = 0; r < MB; ++r) {
            const float v = warp_sum(acc[c][r]);
            if (lane == 0) part[warp][c * MB + r] = v;
        }
    __syncthreads();
    if (threadIdx.x < NC * MB) {
        const int c = threadIdx.x / MB, r = threadIdx.x % MB, n = n0 + c;
        float v = 0.f;
#pragma unroll
        for (int wp = 0; wp < 8; ++wp) v += part[wp][threadIdx.x];
        if (EPI == AEPI_SWIGLU) {      // the thread of an even column also sums its odd neighbour (the up projection)
            if ((c & 1) == 0 && r < g.M && n + 1 < g.N) {
                float u = 0.f;
#pragma unroll
                for (int wp = 0; wp < 8; ++wp) u += part[wp][threadIdx.x + MB];
                g.C[(size_t)r * g.ldc + n / 2] = any_swiglu(g, v, u, n);
            }
        } else if (r < g.M && n < g.N) g.C[(size_t)r * g.ldc + n] = any_epilogue<EPI>(g, v, n);
    }
}

template <typename WT, int EPI, bool VEC>
inline void gemm_skinny_launch(cudaStream_t st, const GemmAnyArgs& g, int num_sms) {
    const dim3 blocks(std::max(1, std::min(ceil_div(g.N, 16), num_sms * 8)), 1, g.batch);
    if (g.M <= 1) gemm_skinny_kernel<WT, EPI, 1, VEC><<<blocks, 256, 0, st>>>(g);
    else if (g.M <= 2) gemm_skinny_kernel<WT, EPI, 2, VEC><<<blocks, 256, 0, st>>>(g);
    else if (g.M <= 4) gemm_skinny_kernel<WT, EPI, 4, VEC><<<blocks, 256, 0, st>>>(g);
    else gemm_skinny_kernel<WT, EPI, 8, VEC><<<blocks, 256, 0, st>>>(g);
}

template <typename WT, int EPI>
inline void gemm_any_launch(cudaStream_t st, const GemmAnyArgs& g, int num_sms) {
    if (g.M <= 8 && !g.row_offsets && !g.a_gather) {
        const bool vec = g.K % 8 == 0 && g.lda % 4 == 0 && (reinterpret_cast<uintptr_t>(g.A) & 15) == 0 && (reinterpret_cast<uintptr_t>(g.W) & 15) == 0 &&
                         (g.batch == 1 || (g.a_bs % 4 == 0 && g.w_bs % 8 == 0));
        const dim3 grid(ceil_div(g.N, 8), 1, g.batch);
        if (vec && (g.M >= 3 || g.K >= 1024)) {      // one or two rows of a short K leave most of the 8 warps without a step: the two-column kernel
            if (g.M <= 1) gemm_rows_kernel<WT, EPI, 1><<<grid, 256, 0, st>>>(g);
            else if (g.M <= 2) gemm_rows_kernel<WT, EPI, 2><<<grid, 256, 0, st>>>(g);
            else if (g.M <= 4) gemm_rows_kernel<WT, EPI, 4><<<grid, 256, 0, st>>>(g);
            else gemm_rows_kernel<WT, EPI, 8><<<grid, 256, 0, st>>>(g);
        } else if (vec) gemm_skinny_launch<WT, EPI, true>(st, g, num_sms);
        else gemm_skinny_launch<WT, EPI, false>(st, g, num_sms);
    } else {
        gemm_any_kernel<WT, EPI><<<dim3(ceil_div(g.N, 64), ceil_div(g.M, 64), g.batch), 256, 0, st>>>(g);
    }
}

// fp32_weights: W holds floats, else bf16
inline void gemm_any(cudaStream_t st, int epi, bool fp32_weights, const GemmAnyArgs& g_in, int num_sms) {
    GemmAnyArgs g = g_in;
    if (g.M == 0 || g.N == 0) return;
    g.glu = epi == AEPI_CLAMP_GLU ? 1 : 0;
    if (epi == AEPI_CLAMP_GLU) epi = AEPI_SWIGLU;
    AHA_REQUIRE(epi == AEPI_STORE || epi == AEPI_XIELU || epi == AEPI_SWIGLU || epi == AEPI_RELU2, "gemm_any: bad epilogue");
    AHA_REQUIRE(epi != AEPI_SWIGLU || g.N % 2 == 0, "gemm_any: the gate / up epilogue needs an even number of weight rows");
    AHA_REQUIRE(g.batch >= 1 && g.batch <= 65535, "gemm_any: bad batch count");
    if (fp32_weights) {
        if (epi == AEPI_STORE) gemm_any_launch<float, AEPI_STORE>(st, g, num_sms);
        else if (epi == AEPI_XIELU) gemm_any_launch<float, AEPI_XIELU>(st, g, num_sms);
        else if (epi == AEPI_RELU2) gemm_any_launch<float, AEPI_RELU2>(st, g, num_sms);
        else gemm_any_launch<float, AEPI_SWIGLU>(st, g, num_sms);
    } else {
        if (epi == AEPI_STORE) gemm_any_launch<__nv_bfloat16, AEPI_STORE>(st, g, num_sms);
        else if (epi == AEPI_XIELU) gemm_any_launch<__nv_bfloat16, AEPI_XIELU>(st, g, num_sms);
        else if (epi == AEPI_RELU2) gemm_any_launch<__nv_bfloat16, AEPI_RELU2>(st, g, num_sms);
        else gemm_any_launch<__nv_bfloat16, AEPI_SWIGLU>(st, g, num_sms);
    }
    AHA_CUDA_CHECK(cudaGetLastError());
}

}  // namespace aha
