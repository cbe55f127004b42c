// recurrence_elem.cuh -- an ELEMENTWISE gated recurrence (minGRU): every channel carries one number per sequence,
//     S_t = (1 - z_t) S_{t-1} + z_t c_t,      z_t = sigmoid(a_t),      c_t = b_t + 1/2 (b_t >= 0) | sigmoid(b_t) (b_t < 0),
// where a_t, b_t are projections of the CURRENT token only, and the mixer's output is S_t * silu(g_t).  The gate and the candidate do not
// read the state, so the recurrence is linear in S: a run of tokens composes to S -> A S + B with A = prod (1 - z), and only PRODUCTS of
// numbers in (0, 1) appear (they shrink; nothing is divided).  The kernel uses that to run a long prompt portion side by side:
//
//   mingru_scan_kernel<TY>   grid (channel slice, entry), block (32 channels, TY token lanes; or 16 channels and twice the lanes when that is what
//                            gives every SM a block).  A tile is (token lanes) x 16 consecutive tokens; a lane
//                            walks its 16 tokens once from a zero state (keeping 1 - z and z c in registers) and leaves the composite
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
    int cw = 32;                        // channels a block owns: 32, or 16 when 32-channel slices would leave SMs without a block (set by mingru_scan)
    RaggedBatch rb;
};

__device__ __forceinline__ float mingru_candidate(float u) { return u >= 0.f ? u + 0.5f : sigmoid_f(u); }

template <int TY>
static __global__ void __launch_bounds__(32 * TY) mingru_scan_kernel(ElemScanArgs a) {
    __shared__ float sA[TY][32], sB[TY][32];
    // the block's 32 TY threads are regrouped into (cw channels) x (32 TY / cw token lanes)
    const int CW = a.cw, lanes = 32 * TY / CW;
    const int lin = threadIdx.y * 32 + threadIdx.x;
    const int tx = lin % CW, ty = lin / CW, c = blockIdx.x * CW + tx, e = blockIdx.y;
    const int t0 = a.rb.ent_start[e], n = a.rb.ent_start[e + 1] - t0, pos0 = a.rb.ent_pos0[e], slot = a.rb.ent_slot[e];
    const bool live = c < a.n;
    float* sa = &sA[0][0]; float* sb = &sB[0][0];          // [lanes][CW]
    float carry = (live && pos0 > 0) ? a.state[(size_t)slot * a.slot_stride + c] : 0.f;
    for (int tile = 0; tile < n; tile += lanes * kEgTok) {
        const int s = tile + ty * kEgTok;
        const int cnt = live ? max(0, min(kEgTok, n - s)) : 0;
        const float* __restrict__ row0 = a.proj + (size_t)(t0 + s) * a.ld + c;
        // every load of the thread's tokens is issued before anything depends on one of them
        float zr[kEgTok], cr[kEgTok], gr[kEgTok];
#pragma unroll
        for (int k = 0; k < kEgTok; ++k) {
            const float* row = row0 + (size_t)k * a.ld;
            const bool on = k < cnt;
            zr[k] = on ? row[a.z_off] : 0.f; cr[k] = on ? row[a.c_off] : 0.f; gr[k] = on ? row[a.g_off] : 0.f;
        }
        float A = 1.f, B = 0.f;
#pragma unroll
        for (int k = 0; k < kEgTok; ++k) {
            if (k < cnt) {
                const float z = sigmoid_f(zr[k]);
                zr[k] = 1.f - z;                                   // what the state keeps,
                cr[k] = z * mingru_candidate(cr[k]);               // what the token adds
                A *= zr[k];
                B = fmaf(zr[k], B, cr[k]);
            }
        }
        float S = carry;
        if (TY > 1) {
            sa[ty * CW + tx] = A; sb[ty * CW + tx] = B;
            __syncthreads();
            float run = carry;
            for (int j = 0; j < lanes; ++j) {
                if (j == ty) S = run;
                run = fmaf(sa[j * CW + tx], run, sb[j * CW + tx]);
            }
            carry = run;
            __syncthreads();      // the composites are rewritten by the next tile
        }
        float* __restrict__ orow = a.out + (size_t)(t0 + s) * a.ld_out + c;
#pragma unroll
        for (int k = 0; k < kEgTok; ++k) {
            if (k < cnt) {
                S = fmaf(zr[k], S, cr[k]);
                orow[(size_t)k * a.ld_out] = S * silu_f(gr[k]);
            }
        }
        if (TY == 1) carry = S;
    }
    if (live && ty == 0) a.state[(size_t)slot * a.slot_stride + c] = carry;
}

// longest: the most tokens an entry of the step brings.  Returns the launches.
inline int mingru_scan(cudaStream_t st, ElemScanArgs a, int longest, int num_sms) {
    if (a.rb.T == 0) return 0;
    a.cw = 32;
    if (longest <= kEgTok) mingru_scan_kernel<1><<<dim3(ceil_div(a.n, 32), a.rb.E), dim3(32, 1), 0, st>>>(a);
    else if (longest <= 4 * kEgTok) mingru_scan_kernel<4><<<dim3(ceil_div(a.n, 32), a.rb.E), dim3(32, 4), 0, st>>>(a);
    else {
        if (ceil_div(a.n, 32) * a.rb.E < num_sms) a.cw = 16;
        mingru_scan_kernel<16><<<dim3(ceil_div(a.n, a.cw), a.rb.E), dim3(32, 16), 0, st>>>(a);
    }
    AHA_CUDA_CHECK(cudaGetLastError());
    return 1;
}

}  // namespace aha
