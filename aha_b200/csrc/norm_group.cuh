// norm_group.cuh -- row kernels of the layered engine's "sandwich" layers:
//
//   group_rmsnorm_kernel   RMS norm in groups: a row of C channels is cut into `groups` equal consecutive parts, each divided by its own
//                          sqrt(mean(part^2) + eps), then multiplied by a per-channel gain.  One block per (row, group).  Variants by
//                          arguments: gathered rows (the rows whose logits are wanted), a value formed on the way
//                          (in + skip_w[channel / skip_span] * skip) * silu(gate) -- a state-space layer's D x term and output gate --,
//                          and the residual update  out += mult * normed  (post-norm of a sublayer) instead of a store.
//   post_pre_norm_kernel   the residual update after a sublayer and the norm before the next one in one launch
//   sum_residual_norm_kernel  the end of a PARALLEL layer (both sublayers read one normed row): x += y_a + y_b, optionally a further row
//                          added after that (what a pass of looped layers starts from), and the next layer's norm, in one launch
//   short_conv_kernel      causal convolution over time on every channel, y_t = sum_j w[c][j] u_{t - taps + 1 + j} (+ bias) (silu) (+ u_t);
//                          the taps - 1 inputs before a step are the sequence's state ("tail") in its slot, zeros before position 0.
//                          An entry of one token moves its tail along in the same launch; short_conv_tail_kernel does it for longer entries.
//   norm_conv_single_kernel  decode steps (every entry one token): group norm, convolution with the tail and tail update in ONE launch.
//   add_row_vector_kernel  x[t] += vec  for every row (the vector added before a pass of looped layers)
//   gate_mul_kernel        y[t][c] *= sigmoid or silu of gate[t][c]
// Everything is fp32.
#pragma once
#include "common.cuh"
#include "ragged.cuh"

namespace aha {

struct GroupNormArgs {
    const float* in; int ld_in;
    const int* rows = nullptr;        // gather: block row r reads row rows[r] of `in` (and of gate / skip)
    const float* gate = nullptr; int ld_gate = 0;                         // value *= silu(gate)
    const float* skip = nullptr; int ld_skip = 0; const float* skip_w = nullptr; int skip_span = 1;   // value += skip_w[c / skip_span] * skip[c]
    const float* w;                   // [C] gain
    float eps;
    int C, groups;
    float* out; int ld_out;
    int sum_rows = 1;                 // > 1: the value of row r is the sum of rows r * sum_rows .. + sum_rows - 1 of `in` (the outputs of a token's experts), times in_scale
    float in_scale = 1.f;
    float mult = 1.f;                 // on the normed value (a residual multiplier, a logit scale)
    int add = 0;                      // 1: out += mult * normed (the residual sum), 0: out = mult * normed
};

static __global__ void group_rmsnorm_kernel(GroupNormArgs a) {
    __shared__ float red[32];
    const int r = blockIdx.x, g = blockIdx.y, n = a.C / a.groups, c0 = g * n;
    const size_t src = a.rows ? (size_t)a.rows[r] : (size_t)r;
    const float* x = a.in + src * a.ld_in;
    const float* gt = a.gate ? a.gate + src * a.ld_gate : nullptr;
    const float* sk = a.skip ? a.skip + src * a.ld_skip : nullptr;
    auto value = [&](int c) {
        float v;
        if (a.sum_rows > 1) {
            const float* xs = a.in + src * a.sum_rows * a.ld_in;
            v = 0.f;
            for (int k = 0; k < a.sum_rows; ++k) v += xs[(size_t)k * a.ld_in + c];
            v *= a.in_scale;
        } else v = x[c];
        if (sk) v = fmaf(a.skip_w[c / a.skip_span], sk[c], v);
        if (gt) v *= silu_f(gt[c]);
        return v;
    };
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = value(c0 + i); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float sc = a.mult / sqrtf(ss / (float)n + a.eps);
    float* o = a.out + (size_t)r * a.ld_out;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int c = c0 + i;
        const float v = value(c) * sc * a.w[c];
        o[c] = a.add ? o[c] + v : v;
    }
}

inline void group_rmsnorm(cudaStream_t st, const GroupNormArgs& a, int rows) {
    if (rows == 0) return;
    AHA_REQUIRE(a.groups >= 1 && a.C % a.groups == 0, "group norm: the channels do not divide into the groups");
    const int n = a.C / a.groups;
    const int threads = std::min(1024, std::max(64, (rows <= 8 ? (n / 2 + 31) : (n / 4 + 31)) / 32 * 32));
    group_rmsnorm_kernel<<<dim3(rows, a.groups), threads, 0, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

// The end of one sublayer and the start of the next in ONE launch (ungrouped norms, nothing between them):
//     x += mult * rms_norm(y) * w_post;     h = rms_norm(x) * w_pre
// One block per row; a thread rereads only what it wrote itself.
struct PostPreNormArgs {
    const float* y;            // [T, C] sublayer output
    float* x;                  // [T, C] residual stream, updated in place
    const float* w_post;       // [C]
    const float* w_pre;        // [C]
    float* h;                  // [T, C] what the next sublayer reads
    float eps, mult;
    int C;
    // (register kernel only) y formed on the way from a token's expert rows: y[t] = sum_k mix_w[t][k] * mix_rows[t * mix_top + k] (+ sigmoid(mix_gate[t]) *
    // mix_shared[t]) -- the combine step of routed experts in decode steps, in the order the combine kernel sums
    const float* mix_rows = nullptr; int mix_top = 0;
    const float* mix_w = nullptr; int mix_ldw = 0;
    const float* mix_shared = nullptr; const float* mix_gate = nullptr; int mix_ldg = 0;
};

static __global__ void post_pre_norm_kernel(PostPreNormArgs a) {
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    const float* __restrict__ y = a.y + r * a.C;
    float* x = a.x + r * a.C;
    float ss = 0.f;
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) ss = fmaf(y[c], y[c], ss);
    ss = block_sum(ss, red);
    const float sc = a.mult / sqrtf(ss / (float)a.C + a.eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) {
        const float v = x[c] + y[c] * sc * a.w_post[c];
        x[c] = v;
        s2 = fmaf(v, v, s2);
    }
    s2 = block_sum(s2, red);
    const float sc2 = 1.0f / sqrtf(s2 / (float)a.C + a.eps);
    float* h = a.h + r * a.C;
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) h[c] = x[c] * sc2 * a.w_pre[c];
}

// The same with a row's values in registers (C % 4 == 0, C <= 4 NV blockDim): y and x are read once, 16 bytes at a time.
template <int NV>
static __global__ void post_pre_norm_reg_kernel(PostPreNormArgs a) {
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    const int C4 = a.C >> 2;
    const float4* __restrict__ y4 = reinterpret_cast<const float4*>(a.y + r * a.C);
    float4* x4 = reinterpret_cast<float4*>(a.x + r * a.C);
    float4 yv[NV], xv[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        xv[i] = c < C4 ? x4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        if (!a.mix_rows) yv[i] = c < C4 ? y4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        else {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < C4) {
                for (int k = 0; k < a.mix_top; ++k) {
                    const float w = a.mix_w[r * a.mix_ldw + k];
                    const float4 v = reinterpret_cast<const float4*>(a.mix_rows + (r * a.mix_top + k) * a.C)[c];
                    s.x = fmaf(w, v.x, s.x); s.y = fmaf(w, v.y, s.y); s.z = fmaf(w, v.z, s.z); s.w = fmaf(w, v.w, s.w);
                }
                if (a.mix_shared) {
                    const float g = a.mix_gate ? sigmoid_f(a.mix_gate[r * a.mix_ldg]) : 1.f;
                    const float4 v = reinterpret_cast<const float4*>(a.mix_shared + r * a.C)[c];
                    s.x = fmaf(g, v.x, s.x); s.y = fmaf(g, v.y, s.y); s.z = fmaf(g, v.z, s.z); s.w = fmaf(g, v.w, s.w);
                }
            }
            yv[i] = s;
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) ss = fmaf(yv[i].x, yv[i].x, fmaf(yv[i].y, yv[i].y, fmaf(yv[i].z, yv[i].z, fmaf(yv[i].w, yv[i].w, ss))));
    ss = block_sum(ss, red);
    const float sc = a.mult / sqrtf(ss / (float)a.C + a.eps);
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < C4) {
            const float4 w = reinterpret_cast<const float4*>(a.w_post)[c];
            xv[i].x += yv[i].x * sc * w.x; xv[i].y += yv[i].y * sc * w.y; xv[i].z += yv[i].z * sc * w.z; xv[i].w += yv[i].w * sc * w.w;
            x4[c] = xv[i];
            s2 = fmaf(xv[i].x, xv[i].x, fmaf(xv[i].y, xv[i].y, fmaf(xv[i].z, xv[i].z, fmaf(xv[i].w, xv[i].w, s2))));
        }
    }
    s2 = block_sum(s2, red);
    const float sc2 = 1.0f / sqrtf(s2 / (float)a.C + a.eps);
    float4* h4 = reinterpret_cast<float4*>(a.h + r * a.C);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < C4) {
            const float4 w = reinterpret_cast<const float4*>(a.w_pre)[c];
            h4[c] = make_float4(xv[i].x * sc2 * w.x, xv[i].y * sc2 * w.y, xv[i].z * sc2 * w.z, xv[i].w * sc2 * w.w);
        }
    }
}

inline int post_pre_norm_threads(int C, int rows) { return rows <= 8 ? std::min(1024, std::max(128, (C / 4 + 31) / 32 * 32)) : 256; }      // a decode step has few blocks: more threads for each
// whether the register kernel (the only one that forms y from expert rows) takes this row size; the engine's buffers are 16-byte aligned
inline bool post_pre_norm_in_registers(int C, int rows) { return C % 4 == 0 && (C / 4 + post_pre_norm_threads(C, rows) - 1) / post_pre_norm_threads(C, rows) <= 8; }

inline void post_pre_norm(cudaStream_t st, const PostPreNormArgs& a, int rows) {
    if (rows == 0) return;
    const int threads = post_pre_norm_threads(a.C, rows);
    const int nv = (a.C / 4 + threads - 1) / threads;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool reg = post_pre_norm_in_registers(a.C, rows) && al(a.y) && al(a.x) && al(a.h) && al(a.w_post) && al(a.w_pre) && al(a.mix_rows) && al(a.mix_shared);
    AHA_REQUIRE(reg || !a.mix_rows, "post_pre_norm: expert rows are summed by the register kernel only");
    if (reg) {
        if (nv <= 1) post_pre_norm_reg_kernel<1><<<rows, threads, 0, st>>>(a);
        else if (nv <= 2) post_pre_norm_reg_kernel<2><<<rows, threads, 0, st>>>(a);
        else if (nv <= 4) post_pre_norm_reg_kernel<4><<<rows, threads, 0, st>>>(a);
        else post_pre_norm_reg_kernel<8><<<rows, threads, 0, st>>>(a);
    } else post_pre_norm_kernel<<<rows, threads, 0, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

// The end of a parallel layer and the start of the next in ONE launch:
//     x += y_a + y_b;   (trace: x as it is now goes there)   x += inject;   h = rms_norm(x) * w_next
// y_b may be formed on the way from a token's expert rows (as PostPreNormArgs::mix_*; no gate: the shared row is added as it is).  Every
// part but x and y_a is optional.  One block per row; with the row in registers (C % 4 == 0, C <= 4 NV blockDim) everything is read once.
struct SumResidualNormArgs {
    float* x;                  // [T, C] residual stream, updated in place
    const float* y_a;          // [T, C]
    const float* y_b = nullptr;
    const float* mix_rows = nullptr; int mix_top = 0;
    const float* mix_w = nullptr; int mix_ldw = 0;
    const float* mix_shared = nullptr; const float* mix_gate = nullptr; int mix_ldg = 0;
    float* trace = nullptr;    // [T, C]
    const float* inject = nullptr;   // [T, C]
    const float* w_next = nullptr;   // [C]; nullptr: no norm
    float* h = nullptr;        // [T, C]
    float eps = 0.f;
    int C = 0;
};

template <int NV>
static __global__ void sum_residual_norm_reg_kernel(SumResidualNormArgs a) {
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    const int C4 = a.C >> 2;
    float4* x4 = reinterpret_cast<float4*>(a.x + r * a.C);
    const float4* __restrict__ ya = reinterpret_cast<const float4*>(a.y_a + r * a.C);
    float4 xv[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        xv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < C4) {
            float4 v = x4[c];
            const float4 p = ya[c];
            float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.y_b) q = reinterpret_cast<const float4*>(a.y_b + r * a.C)[c];
            else if (a.mix_rows) {
                for (int k = 0; k < a.mix_top; ++k) {
                    const float w = a.mix_w[r * a.mix_ldw + k];
                    const float4 e = reinterpret_cast<const float4*>(a.mix_rows + (r * a.mix_top + k) * a.C)[c];
                    q.x = fmaf(w, e.x, q.x); q.y = fmaf(w, e.y, q.y); q.z = fmaf(w, e.z, q.z); q.w = fmaf(w, e.w, q.w);
                }
                if (a.mix_shared) {
                    const float g = a.mix_gate ? sigmoid_f(a.mix_gate[r * a.mix_ldg]) : 1.f;
                    const float4 e = reinterpret_cast<const float4*>(a.mix_shared + r * a.C)[c];
                    q.x = fmaf(g, e.x, q.x); q.y = fmaf(g, e.y, q.y); q.z = fmaf(g, e.z, q.z); q.w = fmaf(g, e.w, q.w);
                }
            }
            v.x += p.x + q.x; v.y += p.y + q.y; v.z += p.z + q.z; v.w += p.w + q.w;
            if (a.trace) reinterpret_cast<float4*>(a.trace + r * a.C)[c] = v;
            if (a.inject) {
                const float4 j = reinterpret_cast<const float4*>(a.inject + r * a.C)[c];
                v.x += j.x; v.y += j.y; v.z += j.z; v.w += j.w;
            }
            x4[c] = v;
            xv[i] = v;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    }
    if (!a.w_next) return;
    ss = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(ss / (float)a.C + a.eps);
    float4* h4 = reinterpret_cast<float4*>(a.h + r * a.C);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < C4) {
            const float4 w = reinterpret_cast<const float4*>(a.w_next)[c];
            h4[c] = make_float4(xv[i].x * sc * w.x, xv[i].y * sc * w.y, xv[i].z * sc * w.z, xv[i].w * sc * w.w);
        }
    }
}

// any C and alignment: a thread rereads only what it wrote itself
static __global__ void sum_residual_norm_kernel(SumResidualNormArgs a) {
    __shared__ float red[32];
    const size_t r = blockIdx.x;
    float* x = a.x + r * a.C;
    float ss = 0.f;
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) {
        float q = 0.f;
        if (a.y_b) q = a.y_b[r * a.C + c];
        else if (a.mix_rows) {
            for (int k = 0; k < a.mix_top; ++k) q = fmaf(a.mix_w[r * a.mix_ldw + k], a.mix_rows[(r * a.mix_top + k) * a.C + c], q);
            if (a.mix_shared) q = fmaf(a.mix_gate ? sigmoid_f(a.mix_gate[r * a.mix_ldg]) : 1.f, a.mix_shared[r * a.C + c], q);
        }
        float v = x[c] + (a.y_a[r * a.C + c] + q);
        if (a.trace) a.trace[r * a.C + c] = v;
        if (a.inject) v += a.inject[r * a.C + c];
        x[c] = v;
        ss = fmaf(v, v, ss);
    }
    if (!a.w_next) return;
    ss = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(ss / (float)a.C + a.eps);
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) a.h[r * a.C + c] = x[c] * sc * a.w_next[c];
}

inline void sum_residual_norm(cudaStream_t st, const SumResidualNormArgs& a, int rows) {
    if (rows == 0) return;
    const int threads = post_pre_norm_threads(a.C, rows);
    const int nv = (a.C / 4 + threads - 1) / threads;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool reg = post_pre_norm_in_registers(a.C, rows) && al(a.x) && al(a.y_a) && al(a.y_b) && al(a.mix_rows) && al(a.mix_shared) && al(a.trace) && al(a.inject) &&
                     al(a.w_next) && al(a.h);
    if (reg) {
        if (nv <= 1) sum_residual_norm_reg_kernel<1><<<rows, threads, 0, st>>>(a);
        else if (nv <= 2) sum_residual_norm_reg_kernel<2><<<rows, threads, 0, st>>>(a);
        else if (nv <= 4) sum_residual_norm_reg_kernel<4><<<rows, threads, 0, st>>>(a);
        else sum_residual_norm_reg_kernel<8><<<rows, threads, 0, st>>>(a);
    } else sum_residual_norm_kernel<<<rows, threads, 0, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

constexpr int kShortConvMaxTaps = 16;

struct ShortConvArgs {
    const float* in; int ld_in; int in_off;    // input channel c of packed token t: in[t * ld_in + in_off + c]
    int C, taps;
    const float* w;                            // [C, taps], the last column is the current token's
    const float* bias = nullptr;               // [C]
    float* tails; size_t tail_slot_stride;     // [slots][taps - 1][C]
    float* out; int ld_out; int out_off;
    int add_input = 0;                         // 1: out = in + conv(in)
    int silu = 0;                              // 1: silu(conv(in) + bias)
    RaggedBatch rb;
};

static __global__ void short_conv_kernel(ShortConvArgs a) {
    const int t = blockIdx.x;
    const int e = a.rb.tok_entry[t], pos = a.rb.tok_pos[t], local = t - a.rb.ent_start[e], slot = a.rb.ent_slot[e];
    const int nt = a.taps - 1;
    float* tail = a.tails + (size_t)slot * a.tail_slot_stride;
    const bool single = a.rb.ent_start[e + 1] - a.rb.ent_start[e] == 1;     // the thread of a channel is the only reader and writer of its tail
    const float* cur = a.in + (size_t)t * a.ld_in + a.in_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.C; c += gridDim.y * blockDim.x) {
        float y = a.bias ? a.bias[c] : 0.f;
        for (int j = 0; j < a.taps; ++j) {
            const int back = nt - j;
            float u;
            if (local - back >= 0) u = cur[c - (ptrdiff_t)back * a.ld_in];
            else if (pos - back < 0) u = 0.f;
            else u = tail[(size_t)(nt + local - back) * a.C + c];
            y = fmaf(a.w[(size_t)c * a.taps + j], u, y);
        }
        const float x = cur[c];
        if (single && nt > 0) {
            for (int r = 0; r + 1 < nt; ++r) tail[(size_t)r * a.C + c] = tail[(size_t)(r + 1) * a.C + c];
            tail[(size_t)(nt - 1) * a.C + c] = x;
        }
        if (a.silu) y = silu_f(y);
        if (a.add_input) y += x;
        a.out[(size_t)t * a.ld_out + a.out_off + c] = y;
    }
}

// One block row per entry of more than one token: new tail[r] = the input at local index n - (taps - 1) + r, from this step's rows where that
// index is >= 0, else from the old tail (shifted by n), else zero (before the sequence's start).  A thread reads all of its channel first.
static __global__ void short_conv_tail_kernel(ShortConvArgs a) {
    const int e = blockIdx.x;
    const int t0 = a.rb.ent_start[e], n = a.rb.ent_start[e + 1] - t0, pos0 = a.rb.ent_pos0[e], slot = a.rb.ent_slot[e];
    if (n == 1) return;
    const int nt = a.taps - 1;
    float* tail = a.tails + (size_t)slot * a.tail_slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.C; c += gridDim.y * blockDim.x) {
        float v[kShortConvMaxTaps];
#pragma unroll
        for (int r = 0; r < kShortConvMaxTaps; ++r) {
            if (r >= nt) break;
            const int li = n - nt + r;
            v[r] = li >= 0 ? a.in[(size_t)(t0 + li) * a.ld_in + a.in_off + c] : (pos0 + li < 0 ? 0.f : tail[(size_t)(r + n) * a.C + c]);
        }
#pragma unroll
        for (int r = 0; r < kShortConvMaxTaps; ++r) {
            if (r >= nt) break;
            tail[(size_t)r * a.C + c] = v[r];
        }
    }
}

// only_single: every entry of the step brings one token.  Returns the launches.
inline int short_conv(cudaStream_t st, const ShortConvArgs& a, bool only_single) {
    if (a.rb.T == 0) return 0;
    AHA_REQUIRE(a.taps >= 1 && a.taps <= kShortConvMaxTaps, "short convolution: between 1 and 16 taps");
    const int threads = 256, by = std::max(1, std::min(ceil_div(a.C, threads), a.rb.T <= 8 ? 64 : 4));
    short_conv_kernel<<<dim3(a.rb.T, by), threads, 0, st>>>(a);
    const bool tail_launch = a.taps > 1 && !only_single;
    if (tail_launch) short_conv_tail_kernel<<<dim3(a.rb.E, by), threads, 0, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
    return tail_launch ? 2 : 1;
}

// Decode steps: every entry is one token, so the convolution of a normed row needs only the slot's tail (which holds normed rows).
// One block per token: all groups' norms, then out = h + conv(h) and the tail moves along.  `scratch` is not needed: the normed row
// lives in shared memory ([C] floats).
struct NormConvArgs {
    const float* x; int C, groups; const float* w; float eps;       // the norm
    int taps; const float* cw; float* tails; size_t tail_slot_stride;   // the convolution ([C, taps]) and its state
    float* out;                                                     // [T, C]
    RaggedBatch rb;
};

static __global__ void norm_conv_single_kernel(NormConvArgs a) {
    extern __shared__ float hs[];      // [C] normed row
    __shared__ float red[32];
    __shared__ float inv[64];
    const int t = blockIdx.x, e = a.rb.tok_entry[t], pos = a.rb.tok_pos[t], slot = a.rb.ent_slot[e];
    const float* xr = a.x + (size_t)t * a.C;
    const int n = a.C / a.groups;
    for (int g0 = 0; g0 < a.groups; g0 += 64) {
        const int ng = min(64, a.groups - g0);
        for (int g = 0; g < ng; ++g) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = xr[(g0 + g) * n + i]; ss = fmaf(v, v, ss); }
            ss = block_sum(ss, red);
            if (threadIdx.x == 0) inv[g] = 1.0f / sqrtf(ss / (float)n + a.eps);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < ng * n; i += blockDim.x) { const int c = g0 * n + i; hs[c] = xr[c] * inv[i / n] * a.w[c]; }
        __syncthreads();
    }
    const int nt = a.taps - 1;
    float* tail = a.tails + (size_t)slot * a.tail_slot_stride;
    for (int c = threadIdx.x; c < a.C; c += blockDim.x) {
        const float h = hs[c];
        float y = a.cw[(size_t)c * a.taps + nt] * h;
        for (int j = 0; j < nt; ++j) {
            const int back = nt - j;
            if (pos - back >= 0) y = fmaf(a.cw[(size_t)c * a.taps + j], tail[(size_t)j * a.C + c], y);
        }
        for (int r = 0; r + 1 < nt; ++r) tail[(size_t)r * a.C + c] = tail[(size_t)(r + 1) * a.C + c];
        if (nt > 0) tail[(size_t)(nt - 1) * a.C + c] = h;
        a.out[(size_t)t * a.C + c] = h + y;
    }
}

static __global__ void add_row_vector_kernel(float* __restrict__ x, const float* __restrict__ vec, int C, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] += vec[i % C];
}

// y[t][c] *= act(gate[t * ld_gate + c]), act: 0 sigmoid, 1 silu
static __global__ void gate_mul_kernel(float* __restrict__ y, int ld_y, const float* __restrict__ gate, int ld_gate, int C, size_t total, int act) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / C; const int c = (int)(i % C);
    const float g = gate[t * ld_gate + c];
    y[t * ld_y + c] *= act == 0 ? sigmoid_f(g) : silu_f(g);
}

}  // namespace aha
