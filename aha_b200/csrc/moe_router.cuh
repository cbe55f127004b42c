// moe_router.cuh -- routing of a mixture of experts by a learned router: scores = softmax of the router's logits over ALL experts, the
// `top` largest scores name a token's experts and weigh their outputs.  A RouterRule says what else a design asks for: a learned
// correction added to the scores for the CHOICE only, experts in groups of neighbours of which only the best few groups may be
// chosen from, weights renormalised over the chosen experts, a factor on the weights.  A shared expert that every token runs is
// added, behind a sigmoid gate (one number per token) if the design has one.
//
//   router_fused_kernel          router product (fp32) + softmax + choice in one launch, see below; the two kernels after it serve sizes whose rows do
//                                not fit shared memory (the product is then a separate launch)
//   router_topk_kernel           a warp per token: softmax over the logits (fp32), then `top` rounds of arg-max (the earlier expert wins
//                                among equal scores), writing assignment a = token * top + choice -> expert and its weight
//   moe_weighted_combine_kernel  y[t] = sum_k weight[t][k] * rows[place(t, k)] + sigmoid(gate[t]) * shared[t]   (no gate: + shared[t])
// The ordering of assignments by expert for the grouped products is moe_table_route_kernel (moe_table.cuh) without a table.
#pragma once
#include "common.cuh"

namespace aha {


// How a token's experts are chosen from its softmax scores s and how they are weighed.
struct RouterRule {
    const float* correction = nullptr;   // [experts] added to the scores for the choice only (the weights use s itself)
    int group_count = 1, group_keep = 1; // experts form group_count equal groups of neighbours; a group's score is its largest choice score, and only
                                         // the group_keep best groups' experts can be chosen (group_keep >= group_count: no restriction)
    int renorm = 0;                      // 1: the chosen scores are divided by their sum (+ floor)
    float floor = 0.f;
    float scale = 1.f;                   // on the weights
};

// One warp.  s[experts] holds the token's softmax scores, ch[experts + group_count] is scratch (both in shared memory).  Writes the `top`
// chosen experts (the earlier expert wins among equal choice scores) and their weights.  The host guarantees that the kept groups hold at
// least `top` experts.
__device__ __forceinline__ void router_choose(const float* s, float* ch, int experts, int top, const RouterRule& rule, int lane, int* expert_out, float* weight_out) {
    for (int e = lane; e < experts; e += 32) ch[e] = s[e] + (rule.correction ? rule.correction[e] : 0.f);
    __syncwarp();
    if (rule.group_keep < rule.group_count) {
        float* gs = ch + experts;
        const int n = experts / rule.group_count;
        for (int g = lane; g < rule.group_count; g += 32) {
            float mx = -INFINITY;
            for (int i = 0; i < n; ++i) mx = fmaxf(mx, ch[g * n + i]);
            gs[g] = mx;
        }
        __syncwarp();
        for (int e = lane; e < experts; e += 32) {      // a group is kept if fewer than group_keep groups come before it (larger score, or equal and earlier)
            const int g = e / n;
            const float mine = gs[g];
            int before = 0;
            for (int o = 0; o < rule.group_count; ++o) before += (gs[o] > mine || (gs[o] == mine && o < g)) ? 1 : 0;
            if (before >= rule.group_keep) ch[e] = -INFINITY;
        }
        __syncwarp();
    }
    float sum = 0.f;      // lane 0's
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY; int arg = experts;
        for (int e = lane; e < experts; e += 32)
            if (ch[e] > best) { best = ch[e]; arg = e; }      // ascending e: the first of equal scores stays
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, off);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        arg = min(arg, experts - 1);
        if (lane == 0) {
            expert_out[k] = arg;
            const float w = s[arg];
            weight_out[k] = w;
            sum += w;
            ch[arg] = -INFINITY;      // chosen: out of the next rounds
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float f = rule.renorm ? rule.scale / (sum + rule.floor) : rule.scale;
        if (rule.renorm || rule.scale != 1.f)
            for (int k = 0; k < top; ++k) weight_out[k] *= f;
    }
}

struct RouterArgs {
    const float* logits; int ld;     // [T, ld]: the router's logits in columns 0 .. experts - 1
    int T, experts, top;
    int* expert_of;                  // [T * top]
    float* weights; int ld_w;        // weight of choice k of token t at weights[t * ld_w + k] (may lie in the logits' rows, beyond the experts)
    RouterRule rule;
};

constexpr int kRouterWarps = 4;

static __global__ void __launch_bounds__(32 * kRouterWarps) router_topk_kernel(RouterArgs a) {
    extern __shared__ float router_sm[];      // [warps][2 experts + groups]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = blockIdx.x * kRouterWarps + warp;
    if (t >= a.T) return;
    float* s = router_sm + (size_t)warp * (2 * a.experts + a.rule.group_count);
    const float* z = a.logits + (size_t)t * a.ld;
    float mx = -INFINITY;
    for (int e = lane; e < a.experts; e += 32) { s[e] = z[e]; mx = fmaxf(mx, s[e]); }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < a.experts; e += 32) { s[e] = expf(s[e] - mx); sum += s[e]; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < a.experts; e += 32) s[e] *= inv;
    __syncwarp();
    router_choose(s, s + a.experts, a.experts, a.top, a.rule, lane, a.expert_of + (size_t)t * a.top, a.weights + (size_t)t * a.ld_w);
}

inline void router_topk(cudaStream_t st, const RouterArgs& a) {
    if (a.T == 0) return;
    const size_t smem = (size_t)kRouterWarps * (2 * a.experts + a.rule.group_count) * sizeof(float);
    AHA_REQUIRE(smem <= 48 * 1024, "router: too many experts for the selection kernel");
    router_topk_kernel<<<ceil_div(a.T, kRouterWarps), 32 * kRouterWarps, smem, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

// The router product, the softmax and the choice in ONE launch: a block owns TOK tokens and keeps their rows in shared memory; its threads walk
// every weight row together (a few rows at a time), the warps' partial sums meet in shared memory, then warp r ranks token r.
// A token's sums run in an order that depends on K only, so its logits are the same whatever else is in the batch and whatever TOK is.
struct RouterFusedArgs {
    const float* x; int ldx;         // [T, K] what the router reads
    const float* w;                  // [n_out, K] fp32: the experts' rows, then (n_out = experts + 1) the shared gate's
    int T, K, experts, n_out, top;
    float* logits; int ld;           // [T, ld]: n_out logits, then the `top` weights of the chosen experts
    int* expert_of;                  // [T * top]
    RouterRule rule;
};

template <int TOK>
static __global__ void __launch_bounds__(256) router_fused_kernel(RouterFusedArgs a) {
    constexpr int EU = TOK == 1 ? 8 : 4;             // weight rows whose loads are in flight together
    extern __shared__ __align__(16) float rf_sm[];
    float* xs = rf_sm;                               // [TOK][K]
    float* lg = rf_sm + (size_t)TOK * a.K;           // [TOK][n_out]
    float* part = lg + (size_t)TOK * a.n_out;        // [8 warps][n_out][TOK]
    float* chs = part + (size_t)8 * a.n_out * TOK;   // [TOK][experts + groups] scratch of the choice
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, t0 = blockIdx.x * TOK, nt = min(TOK, a.T - t0);
    const bool vec = (a.K & 3) == 0 && (a.ldx & 3) == 0;
    for (int r = 0; r < TOK; ++r) {
        if (r < nt) {
            const float* src = a.x + (size_t)(t0 + r) * a.ldx;
            if (vec) for (int k = tid * 4; k < a.K; k += 1024) *reinterpret_cast<float4*>(xs + (size_t)r * a.K + k) = *reinterpret_cast<const float4*>(src + k);
            else for (int k = tid; k < a.K; k += 256) xs[(size_t)r * a.K + k] = src[k];
        } else for (int k = tid; k < a.K; k += 256) xs[(size_t)r * a.K + k] = 0.f;
    }
    __syncthreads();
    // the block's threads share every weight row (a thread takes every 256th piece of it) and EU rows at a time, so that a single block
    // -- a decode step has no more than one per token -- still has most of the matrix requested at once
    for (int e0 = 0; e0 < a.n_out; e0 += EU) {
        float acc[EU][TOK];
#pragma unroll
        for (int u = 0; u < EU; ++u)
#pragma unroll
            for (int r = 0; r < TOK; ++r) acc[u][r] = 0.f;
        if (vec) {
#pragma unroll 2
            for (int k = tid * 4; k < a.K; k += 1024) {
                float4 w4[EU];
#pragma unroll
                for (int u = 0; u < EU; ++u) w4[u] = *reinterpret_cast<const float4*>(a.w + (size_t)min(e0 + u, a.n_out - 1) * a.K + k);
#pragma unroll
                for (int r = 0; r < TOK; ++r) {
                    const float4 x4 = *reinterpret_cast<const float4*>(xs + (size_t)r * a.K + k);
#pragma unroll
                    for (int u = 0; u < EU; ++u) acc[u][r] = fmaf(x4.w, w4[u].w, fmaf(x4.z, w4[u].z, fmaf(x4.y, w4[u].y, fmaf(x4.x, w4[u].x, acc[u][r]))));
                }
            }
        } else {
            for (int k = tid; k < a.K; k += 256) {
                float wv[EU];
#pragma unroll
                for (int u = 0; u < EU; ++u) wv[u] = a.w[(size_t)min(e0 + u, a.n_out - 1) * a.K + k];
#pragma unroll
                for (int r = 0; r < TOK; ++r) {
                    const float xv = xs[(size_t)r * a.K + k];
#pragma unroll
                    for (int u = 0; u < EU; ++u) acc[u][r] = fmaf(xv, wv[u], acc[u][r]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < EU; ++u)
#pragma unroll
            for (int r = 0; r < TOK; ++r) {
                const float v = warp_sum(acc[u][r]);
                if (lane == 0 && e0 + u < a.n_out) part[((size_t)warp * a.n_out + e0 + u) * TOK + r] = v;
            }
    }
    __syncthreads();
    for (int idx = tid; idx < a.n_out * TOK; idx += 256) {      // the warps' parts in a fixed order
        const int e = idx / TOK, r = idx % TOK;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += part[((size_t)w * a.n_out + e) * TOK + r];
        lg[r * a.n_out + e] = v;
        if (r < nt) a.logits[(size_t)(t0 + r) * a.ld + e] = v;
    }
    __syncthreads();
    for (int r = warp; r < nt; r += 8) {
        float* s = lg + (size_t)r * a.n_out;
        const int t = t0 + r;
        float mx = -INFINITY;
        for (int e = lane; e < a.experts; e += 32) mx = fmaxf(mx, s[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < a.experts; e += 32) { s[e] = expf(s[e] - mx); sum += s[e]; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < a.experts; e += 32) s[e] *= inv;
        __syncwarp();
        router_choose(s, chs + (size_t)r * (a.experts + a.rule.group_count), a.experts, a.top, a.rule, lane, a.expert_of + (size_t)t * a.top,
                      a.logits + (size_t)t * a.ld + a.n_out);
    }
}

inline size_t router_fused_smem(int tok, int K, int n_out, int groups = 1) { return (size_t)tok * (K + 10 * n_out + groups) * sizeof(float); }
inline bool router_fused_supported(int K, int n_out, int groups = 1) { return router_fused_smem(8, K, n_out, groups) <= 200 * 1024; }

// decode-sized steps give every token a block of its own (the weight rows are then read once per token, which a few tokens can afford)
inline void router_fused(cudaStream_t st, const RouterFusedArgs& a) {
    if (a.T == 0) return;
    static bool attr = false;
    if (!attr) {
        AHA_CUDA_CHECK(cudaFuncSetAttribute(router_fused_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        AHA_CUDA_CHECK(cudaFuncSetAttribute(router_fused_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    if (a.T <= 8) router_fused_kernel<1><<<a.T, 256, router_fused_smem(1, a.K, a.n_out, a.rule.group_count), st>>>(a);
    else router_fused_kernel<8><<<ceil_div(a.T, 8), 256, router_fused_smem(8, a.K, a.n_out, a.rule.group_count), st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

struct WeightedCombineArgs {
    const float* rows;               // [assignments, C] expert outputs
    const int* place_of;             // row of assignment a, or nullptr: row a
    const float* weights; int ld_w;  // see RouterArgs
    const float* shared;             // [T, C] the shared expert's output or nullptr
    const float* gate; int ld_gate;  // its gate's pre-activation of token t at gate[t * ld_gate]; nullptr: the shared expert is added as it is
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
    if (a.shared) s = fmaf(a.gate ? sigmoid_f(a.gate[t * a.ld_gate]) : 1.f, a.shared[i], s);
    a.y[i] = s;
}

}  // namespace aha
