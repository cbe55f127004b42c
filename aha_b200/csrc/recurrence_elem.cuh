// recurrence_elem.cuh -- an ELEMENTWISE gated recurrence (minGRU): every channel carries one number per sequence,
//     S_t = (1 - z_t) S_{t-1} + z_t c_t,      z_t = sigmoid(a_t),      c_t = b_t + 1/2 (b_t >= 0) | sigmoid(b_t) (b_t < 0),
// where a_t, b_t are projections of the CURRENT token only, and the mixer's output is S_t * silu(g_t).  The gate and the candidate do not
// read the state, so the recurrence is linear in S: a run of tokens composes to S -> A S + B with A = prod (1 - z), and only PRODUCTS of
// numbers in (0, 1) appear (they shrink; nothing is divided).  The kernel uses that to run a long prompt portion side by side:
//
//   mingru_scan_kernel<TY>   grid (32-channel slice, entry), block (32 channels, TY token lanes).  A tile is TY x 16 consecutive tokens; lane
//                            ty walks its 16 tokens once from a zero state (keeping 1 - z and z c in registers) and leaves the composite
//                            (A, B) in shared memory; every thread then folds the composites before its own into the tile's incoming state,
//                            walks its 16 tokens again from there and writes S_t * silu(g_t).  TY = 1 is the plain serial walk (decoded
//                            tokens, short portions).  The state of a sequence is ONE fp32 per channel in its slot; an entry whose first
//                            position is 0 starts from zero, so a slot that is used again needs no clearing.
// Gates, candidates, products and the state are fp32.  A channel's result depends only on its own sequence.
#pragma once
#include "common.cuh"
#include "ragged.cuh"

namespace aha {

constexpr int kEgTok = 16;      // consecutive tokens a thread walks per tile

struct ElemScanArgs {
    const float* proj; int ld;          // [T, ld] projected rows (bias added)
    int z_off, c_off, g_off;            // first column of the gate, candidate and output-gate pre-activations
    int n;                              // channels
    float* state; size_t slot_stride;   // [slots][n]
    float* out; int ld_out;             // [T, ld_out]: S_t * silu(g_t)
    RaggedBatch rb;
};

__device__ __forceinline__ float mingru_candidate(float u) { return u >= 0.f ? u + 0.5f : sigmoid_f(u); }

template <int TY>
static __global__ void __launch_bounds__(32 * TY) mingru_scan_kernel(ElemScanArgs a) {
    __shared__ float sA[TY][32], sB[TY][32];
    const int tx = threadIdx.x, ty = threadIdx.y, c = blockIdx.x * 32 + tx, e = blockIdx.y;
    const int t0 = a.rb.ent_start[e], n = a.rb.ent_start[e + 1] - t0, pos0 = a.rb.ent_pos0[e], slot = a.rb.ent_slot[e];
    const bool live = c < a.n;
    float carry = (live && pos0 > 0) ? a.state[(size_t)slot * a.slot_stride + c] : 0.f;
    for (int tile = 0; tile < n; tile += TY * kEgTok) {
        const int s = tile + ty * kEgTok;
        const int cnt = live ? max(0, min(kEgTok, n - s)) : 0;
        const float* row0 = a.proj + (size_t)(t0 + s) * a.ld + c;
        float keep[kEgTok], add[kEgTok];
        float A = 1.f, B = 0.f;
#pragma unroll
        for (int k = 0; k < kEgTok; ++k) {
            keep[k] = 1.f; add[k] = 0.f;
            if (k < cnt) {
                const float* row = row0 + (size_t)k * a.ld;
                const float z = sigmoid_f(row[a.z_off]);
                keep[k] = 1.f - z;
                add[k] = z * mingru_candidate(row[a.c_off]);
                A *= keep[k];
                B = fmaf(keep[k], B, add[k]);
            }
        }
        float S = carry;
        if (TY > 1) {
            sA[ty][tx] = A; sB[ty][tx] = B;
            __syncthreads();
            float run = carry;
#pragma unroll
            for (int j = 0; j < TY; ++j) {
                if (j == ty) S = run;
                run = fmaf(sA[j][tx], run, sB[j][tx]);
            }
            carry = run;
            __syncthreads();      // the composites are rewritten by the next tile
        }
#pragma unroll
        for (int k = 0; k < kEgTok; ++k) {
            if (k < cnt) {
                S = fmaf(keep[k], S, add[k]);
                const float g = row0[(size_t)k * a.ld + a.g_off];
                a.out[(size_t)(t0 + s + k) * a.ld_out + c] = S * silu_f(g);
            }
        }
        if (TY == 1) carry = S;
    }
    if (live && ty == 0) a.state[(size_t)slot * a.slot_stride + c] = carry;
}

// longest: the most tokens an entry of the step brings.  Returns the launches.
inline int mingru_scan(cudaStream_t st, const ElemScanArgs& a, int longest) {
    if (a.rb.T == 0) return 0;
    const dim3 grid(ceil_div(a.n, 32), a.rb.E);
    if (longest <= kEgTok) mingru_scan_kernel<1><<<grid, dim3(32, 1), 0, st>>>(a);
    else if (longest <= 4 * kEgTok) mingru_scan_kernel<4><<<grid, dim3(32, 4), 0, st>>>(a);
    else mingru_scan_kernel<16><<<grid, dim3(32, 16), 0, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
    return 1;
}

}  // namespace aha
