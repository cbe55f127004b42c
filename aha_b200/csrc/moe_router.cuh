// moe_router.cuh -- routing of a mixture of experts by a learned router: scores = softmax of the router's logits over ALL experts, the
// `top` largest scores name a token's experts and weigh their outputs as they are (no renormalisation over the chosen ones).  A shared
// expert that every token runs is added behind a sigmoid gate, one number per token.
//
//   router_topk_kernel           a warp per token: softmax over the logits (fp32), then `top` rounds of arg-max (the earlier expert wins
//                                among equal scores), writing assignment a = token * top + choice -> expert and its weight
//   moe_weighted_combine_kernel  y[t] = sum_k weight[t][k] * rows[place(t, k)] + sigmoid(gate[t]) * shared[t]
// The ordering of assignments by expert for the grouped products is moe_table_route_kernel (moe_table.cuh) without a table.
#pragma once
#include "common.cuh"

namespace aha {

struct RouterArgs {
    const float* logits; int ld;     // [T, ld]: the router's logits in columns 0 .. experts - 1
    int T, experts, top;
    int* expert_of;                  // [T * top]
    float* weights; int ld_w;        // weight of choice k of token t at weights[t * ld_w + k] (may lie in the logits' rows, beyond the experts)
};

constexpr int kRouterWarps = 4;

static __global__ void __launch_bounds__(32 * kRouterWarps) router_topk_kernel(RouterArgs a) {
    extern __shared__ float router_sm[];      // [warps][experts]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = blockIdx.x * kRouterWarps + warp;
    if (t >= a.T) return;
    float* s = router_sm + (size_t)warp * a.experts;
    const float* z = a.logits + (size_t)t * a.ld;
    float mx = -INFINITY;
    for (int e = lane; e < a.experts; e += 32) { s[e] = z[e]; mx = fmaxf(mx, s[e]); }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < a.experts; e += 32) { s[e] = expf(s[e] - mx); sum += s[e]; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    __syncwarp();
    for (int k = 0; k < a.top; ++k) {
        float best = -1.f; int arg = a.experts;
        for (int e = lane; e < a.experts; e += 32)
            if (s[e] > best) { best = s[e]; arg = e; }      // ascending e: the first of equal scores stays
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0) {
            a.expert_of[(size_t)t * a.top + k] = arg;
            a.weights[(size_t)t * a.ld_w + k] = best * inv;
            s[arg] = -2.f;      // chosen: out of the next rounds
        }
        __syncwarp();
    }
}

inline void router_topk(cudaStream_t st, const RouterArgs& a) {
    if (a.T == 0) return;
    const size_t smem = (size_t)kRouterWarps * a.experts * sizeof(float);
    AHA_REQUIRE(smem <= 48 * 1024, "router: too many experts for the selection kernel");
    router_topk_kernel<<<ceil_div(a.T, kRouterWarps), 32 * kRouterWarps, smem, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

struct WeightedCombineArgs {
    const float* rows;               // [assignments, C] expert outputs
    const int* place_of;             // row of assignment a, or nullptr: row a
    const float* weights; int ld_w;  // see RouterArgs
    const float* shared;             // [T, C] the shared expert's output or nullptr
    const float* gate; int ld_gate;  // its gate's pre-activation of token t at gate[t * ld_gate]
    float* y;                        // [T, C]
    int C, top;
    size_t total;                    // T * C
};

static __global__ void moe_weighted_combine_kernel(WeightedCombineArgs a) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const size_t t = i / a.C; const int c = (int)(i % a.C);
    float s = 0.f;
    for (int k = 0; k < a.top; ++k) {
        const size_t r = a.place_of ? (size_t)a.place_of[t * a.top + k] : t * a.top + k;
        s = fmaf(a.weights[t * a.ld_w + k], a.rows[r * a.C + c], s);
    }
    if (a.shared) s = fmaf(sigmoid_f(a.gate[t * a.ld_gate]), a.shared[i], s);
    a.y[i] = s;
}

}  // namespace aha
