// moe_table.cuh -- routing of a mixture of experts whose choice is a lookup: row `token id` of an integer table names the token's
// experts, each with the same weight.  There is no router product and nothing to rank; what remains is bookkeeping for the grouped
// matrix products, done on the device because a decoded token's id may never have left it.
//
//   moe_table_route_kernel   assignment a = token * top + choice -> its expert; with `sort`: the assignments ordered by expert (stable, so the
//                            order never depends on thread timing), every expert's first row, the token row of every ordered assignment
//                            (the gather index of the first product) and every assignment's place in that order (for the combine)
//   moe_combine_kernel       y[t] = weight * sum over the token's choices of its experts' output rows
// With table == nullptr the first kernel only ORDERS assignments whose experts something else chose (moe_router.cuh).
#pragma once
#include "common.cuh"

namespace aha {

struct MoeRouteArgs {
    const uint32_t* tokens; int T;
    const int* table; int table_ld; int V;   // [V][table_ld], the first `top` entries of a row are used; nullptr: expert_of is given (a router chose)
    int top, experts;
    int* expert_of;      // [T * top]
    int* offsets;        // [experts + 1]   (sort)
    int* sorted_tok;     // [T * top] token row of the i-th ordered assignment   (sort)
    int* place_of;       // [T * top] place of assignment a in the order   (sort)
    int* error;          // set to 1 when a table entry names no expert
    int sort;
    int stage;           // 1: the ordering pass reads the assignments' experts from shared memory (they fit), 0: from global memory
};

static __global__ void __launch_bounds__(1024) moe_table_route_kernel(MoeRouteArgs a) {
    extern __shared__ int cnt[];     // [experts] counts, then [experts + 1] exclusive offsets, then (stage) [T * top] experts
    const int A = a.T * a.top, tid = threadIdx.x;
    int* eo = a.stage ? cnt + 2 * a.experts + 1 : a.expert_of;
    for (int e = tid; e < a.experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = tid; i < A; i += blockDim.x) {
        int e;
        if (a.table) {
            uint32_t tok = a.tokens[i / a.top];
            if (tok >= (uint32_t)a.V) tok = a.V - 1;
            e = a.table[(size_t)tok * a.table_ld + i % a.top];
        } else e = a.expert_of[i];
        if (e < 0 || e >= a.experts) { *a.error = 1; e = 0; }
        a.expert_of[i] = e;
        if (a.stage) eo[i] = e;
        if (a.sort) atomicAdd(&cnt[e], 1);       // integer counts: the result does not depend on the order
    }
    if (!a.sort) return;
    __syncthreads();
    int* off = cnt + a.experts;
    if (tid == 0) {
        int s = 0;
        for (int e = 0; e < a.experts; ++e) { off[e] = s; s += cnt[e]; }
        off[a.experts] = s;
    }
    __syncthreads();
    for (int e = tid; e <= a.experts; e += blockDim.x) a.offsets[e] = off[e];
    // a warp per expert walks the assignments in order: place = the expert's first row + how many of its assignments came before
    const int lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    for (int e = warp; e < a.experts; e += nw) {
        int run = off[e];
        for (int i0 = 0; i0 < A; i0 += 32) {
            const int i = i0 + lane;
            const bool mine = i < A && eo[i] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int p = run + __popc(m & ((1u << lane) - 1u));
                a.sorted_tok[p] = i / a.top;
                a.place_of[i] = p;
            }
            run += __popc(m);
        }
    }
}

inline void moe_table_route(cudaStream_t st, const MoeRouteArgs& a) {
    const int A = a.T * a.top;
    const int threads = a.sort ? 1024 : std::min(1024, std::max(32, (A + 31) / 32 * 32));
    MoeRouteArgs b = a;
    size_t smem = (2 * (size_t)a.experts + 1) * sizeof(int);
    b.stage = a.sort && smem + (size_t)A * sizeof(int) <= 48 * 1024 ? 1 : 0;
    if (b.stage) smem += (size_t)A * sizeof(int);
    moe_table_route_kernel<<<1, threads, smem, st>>>(b);
    AHA_CUDA_CHECK(cudaGetLastError());
}

// place_of == nullptr: assignment a's row is row a
static __global__ void moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ place_of, float* __restrict__ y, int C, int top, float weight, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / C; const int c = (int)(i % C);
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
        const size_t r = place_of ? (size_t)place_of[t * top + k] : t * top + k;
        s += rows[r * C + c];
    }
    y[i] = s * weight;
}

}  // namespace aha
