// attention_window.cuh -- the ragged attention path: sequences of unequal length in one launch, keys / values in the paged cache.
//
//   qkv_conv_norm_kernel   what happens between the q/k/v projection and the cache: an optional short causal convolution per channel
//                          (y_t = sum_j w[c][j] u_{t - taps + 1 + j}; the taps - 1 projected values before a step are the sequence's conv
//                          state), an optional RMS norm of q and of k over the WHOLE projection (all heads at once), then K (convolved,
//                          normed) and V (convolved) go to the cache at the token's position and q to a dense buffer
//   conv_tail_update_kernel  leaves the last taps - 1 projected values of every entry in its slot
//   qk_rotary_norm_kernel  the other prologue: rotary positions on interleaved pairs of the first coordinates of every q and k head (a frequency
//                          table from the host, angle = position * frequency in fp32), then an optional division of every head by its own
//                          root mean square (a unit norm, no gain); K and V go to the cache, q to a dense buffer
//   window_attn_kernel     softmax attention of query head h over kv head h / (H / G) with
//                              score(i, j) = q_i . k_j * scale - slope_h * (i - j),   visible: 0 <= i - j < window  (window 0: all j <= i)
//                          and an optional sigmoid output gate (a number per channel or one per head).  slope_h comes from a table, so any
//                          bias schedule can be passed.  `sink`: the softmax denominator holds an extra exp(0) -- a key of score 0 without
//                          a value, so a head may attend to nothing.
// Positions, scores, softmax weights and norms are fp32; the cache is fp32.  A token's result depends only on its own sequence.
#pragma once
#include <cmath>
#include <vector>

#include "common.cuh"
#include "ragged.cuh"

namespace aha {

constexpr int kConvMaxTaps = 16;

struct PagedKV {           // one layer's cache: K pages [page][G][kPage][D], V pages [page][G][kPage][Dv]
    float* k = nullptr;
    float* v = nullptr;
    int G = 0, D = 0, Dv = 0;
    int ldv = 0;           // floats between value rows; 0: Dv.  With v = k and ldv = D the values are the first Dv columns of the key rows (one array holds both)
    __device__ __forceinline__ float* k_row(int page, int g, int tok_in_page) const { return k + (((size_t)page * G + g) * kPage + tok_in_page) * D; }
    __device__ __forceinline__ float* v_row(int page, int g, int tok_in_page) const { return v + (((size_t)page * G + g) * kPage + tok_in_page) * (ldv ? ldv : Dv); }
};

struct QkvPrepArgs {
    const float* proj; int ld;       // [T, ld] projected rows (bias added)
    int q_off, k_off, v_off;         // column of the first q / k / v channel in a row
    int Cq, Ck, Cv;                  // channels (Ck = Cv = 0: the layer reads another layer's cache)
    int taps;                        // 0 / 1: no convolution
    const float *wq, *wk, *wv;       // [C, taps]
    float* tails;                    // [slots][taps - 1][Cq + Ck + Cv]
    size_t tail_slot_stride;
    const float *q_norm, *k_norm;    // [Cq], [Ck] or nullptr
    float eps;
    float* q_out;                    // [T, Cq]
    PagedKV kv;
    RaggedBatch rb;
};

// projected value of channel (off + c) `back` tokens before packed token t, taken from this step's rows or from the slot's tail
__device__ __forceinline__ float conv_input(const QkvPrepArgs& a, int t, int local, int pos, const float* tail, int ctot, int coff, int off, int c, int back) {
    if (local - back >= 0) return a.proj[(size_t)(t - back) * a.ld + off + c];
    if (pos - back < 0) return 0.f;                                  // before the sequence's start
    return tail[(size_t)(a.taps - 1 + local - back) * ctot + coff + c];
}

template <int THREADS>
static __global__ void __launch_bounds__(THREADS) qkv_conv_norm_kernel(QkvPrepArgs a) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int e = a.rb.tok_entry[t], pos = a.rb.tok_pos[t], local = t - a.rb.ent_start[e], slot = a.rb.ent_slot[e];
    const int ctot = a.Cq + a.Ck + a.Cv;
    const float* tail = a.tails ? a.tails + (size_t)slot * a.tail_slot_stride : nullptr;
    const bool conv = a.taps > 1;
    // an entry of ONE token (a decoded token) moves its slot's tail along right here: the thread that convolves a channel is the only
    // reader and writer of that channel's tail, so no second launch is needed for it
    const bool single = conv && a.rb.ent_start[e + 1] - a.rb.ent_start[e] == 1;
    auto value = [&](const float* w, int coff, int off, int c) {
        if (!conv) return a.proj[(size_t)t * a.ld + off + c];
        float y = 0.f;
        for (int j = 0; j < a.taps; ++j) y = fmaf(w[(size_t)c * a.taps + j], conv_input(a, t, local, pos, tail, ctot, coff, off, c, a.taps - 1 - j), y);
        if (single) {
            float* tl = a.tails + (size_t)slot * a.tail_slot_stride + coff + c;
            for (int r = 0; r + 2 < a.taps; ++r) tl[(size_t)r * ctot] = tl[(size_t)(r + 1) * ctot];
            tl[(size_t)(a.taps - 2) * ctot] = a.proj[(size_t)t * a.ld + off + c];
        }
        return y;
    };
    // q
    {
        float ss = 0.f;
        float* qo = a.q_out + (size_t)t * a.Cq;
        for (int c = threadIdx.x; c < a.Cq; c += blockDim.x) { const float y = value(a.wq, 0, a.q_off, c); qo[c] = y; ss = fmaf(y, y, ss); }
        if (a.q_norm) {
            ss = block_sum(ss, red);
            const float inv = 1.0f / sqrtf(ss / (float)a.Cq + a.eps);
            for (int c = threadIdx.x; c < a.Cq; c += blockDim.x) qo[c] = qo[c] * inv * a.q_norm[c];
        }
    }
    if (a.Ck == 0) return;
    const int page = a.rb.page_tables[(size_t)slot * a.rb.max_pages + (pos >> kPageShift)], tip = pos & (kPage - 1);
    {
        float ss = 0.f;
        for (int c = threadIdx.x; c < a.Ck; c += blockDim.x) {
            const float y = value(a.wk, a.Cq, a.k_off, c);
            a.kv.k_row(page, c / a.kv.D, tip)[c % a.kv.D] = y;
            ss = fmaf(y, y, ss);
        }
        if (a.k_norm) {
            ss = block_sum(ss, red);
            const float inv = 1.0f / sqrtf(ss / (float)a.Ck + a.eps);
            for (int c = threadIdx.x; c < a.Ck; c += blockDim.x) { float* p = a.kv.k_row(page, c / a.kv.D, tip) + c % a.kv.D; *p = *p * inv * a.k_norm[c]; }
        }
    }
    for (int c = threadIdx.x; c < a.Cv; c += blockDim.x) a.kv.v_row(page, c / a.kv.Dv, tip)[c % a.kv.Dv] = value(a.wv, a.Cq + a.Ck, a.v_off, c);
}

// One block per entry: new tail[r] = projected value at local index n - (taps - 1) + r, from this step's rows where that index is >= 0, else
// from the old tail (shifted by n), else zero (before the sequence's start).  A thread reads all it needs of its channel before it writes.
static __global__ void __launch_bounds__(256) conv_tail_update_kernel(QkvPrepArgs a) {
    const int e = blockIdx.x;
    const int t0 = a.rb.ent_start[e], n = a.rb.ent_start[e + 1] - t0, pos0 = a.rb.ent_pos0[e], slot = a.rb.ent_slot[e];
    if (n == 1) return;      // done by the convolution kernel
    const int ctot = a.Cq + a.Ck + a.Cv, nt = a.taps - 1;
    float* tail = a.tails + (size_t)slot * a.tail_slot_stride;
    for (int c = threadIdx.x; c < ctot; c += blockDim.x) {
        const int off = c < a.Cq ? a.q_off + c : (c < a.Cq + a.Ck ? a.k_off + c - a.Cq : a.v_off + c - a.Cq - a.Ck);
        float v[kConvMaxTaps];
#pragma unroll
        for (int r = 0; r < kConvMaxTaps; ++r) {
            if (r >= nt) break;
            const int li = n - nt + r;
            v[r] = li >= 0 ? a.proj[(size_t)(t0 + li) * a.ld + off] : (pos0 + li < 0 ? 0.f : tail[(size_t)(r + n) * ctot + c]);
        }
#pragma unroll
        for (int r = 0; r < kConvMaxTaps; ++r) {
            if (r >= nt) break;
            tail[(size_t)r * ctot + c] = v[r];
        }
    }
}

struct RotaryPrepArgs {
    const float* proj; int ld;       // [T, ld] projected rows
    int q_off, k_off, v_off;
    int H, G, D, Dv;
    const float* freq; int n_freq;   // coordinates (2i, 2i + 1), i < n_freq, of every head turn by position * freq[i]; the rest pass
    int unit_norm; float eps;        // 1: after the rotation every q and k head is divided by sqrt(mean(head^2) + eps)
    float* q_out;                    // [T, H * D]
    PagedKV kv;
    RaggedBatch rb;
};

// One block per token.  cos / sin of the token's angles are formed once (shared memory); a warp takes a head of q or k at a time, a lane a
// pair of coordinates.
static __global__ void __launch_bounds__(256) qk_rotary_norm_kernel(RotaryPrepArgs a) {
    extern __shared__ float rot_cs[];      // [n_freq] cos, [n_freq] sin
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int e = a.rb.tok_entry[t], pos = a.rb.tok_pos[t], slot = a.rb.ent_slot[e];
    const float fpos = (float)pos;
    for (int i = tid; i < a.n_freq; i += blockDim.x) {
        float sn, cs;
        sincosf(fpos * a.freq[i], &sn, &cs);
        rot_cs[i] = cs; rot_cs[a.n_freq + i] = sn;
    }
    __syncthreads();
    const int page = a.rb.page_tables[(size_t)slot * a.rb.max_pages + (pos >> kPageShift)], tip = pos & (kPage - 1);
    const float* row = a.proj + (size_t)t * a.ld;
    const int pairs = (a.D + 1) / 2;
    for (int item = warp; item < a.H + a.G; item += nw) {
        const bool isq = item < a.H;
        const float* src = isq ? row + a.q_off + (size_t)item * a.D : row + a.k_off + (size_t)(item - a.H) * a.D;
        float* dst = isq ? a.q_out + (size_t)t * a.H * a.D + (size_t)item * a.D : a.kv.k_row(page, item - a.H, tip);
        float ss = 0.f;
        for (int j = lane; j < pairs; j += 32) {
            const bool two = 2 * j + 1 < a.D;
            float u = src[2 * j], v = two ? src[2 * j + 1] : 0.f;
            if (j < a.n_freq) {
                const float cs = rot_cs[j], sn = rot_cs[a.n_freq + j];
                const float ru = u * cs - v * sn, rv = v * cs + u * sn;
                u = ru; v = rv;
            }
            dst[2 * j] = u;
            if (two) dst[2 * j + 1] = v;
            ss = fmaf(u, u, fmaf(v, v, ss));
        }
        if (a.unit_norm) {
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)a.D + a.eps);
            for (int j = lane; j < pairs; j += 32) {       // a lane rereads what it wrote itself
                dst[2 * j] *= inv;
                if (2 * j + 1 < a.D) dst[2 * j + 1] *= inv;
            }
        }
    }
    for (int c = tid; c < a.G * a.Dv; c += blockDim.x) a.kv.v_row(page, c / a.Dv, tip)[c % a.Dv] = row[a.v_off + c];
}

inline int qk_rotary_prepare(cudaStream_t st, const RotaryPrepArgs& a) {
    if (a.rb.T == 0) return 0;
    AHA_REQUIRE(2 * a.n_freq <= a.D, "rotary: more rotated coordinates than the head has");
    qk_rotary_norm_kernel<<<a.rb.T, 256, 2 * (size_t)std::max(1, a.n_freq) * sizeof(float), st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
    return 1;
}

// Rotary frequencies f_i = base^(-2i / dims), i < dims / 2, optionally rescaled band by band (host, double): with wavelength 2 pi / f, waves
// shorter than original / high are kept, waves longer than original / low are divided by `factor`, and between the two the frequency moves
// linearly in s = (original / wavelength - low) / (high - low) from f / factor (s = 0) to f (s = 1).  factor <= 0: no rescaling.
inline void banded_rotary_frequencies(int dims, double base, double factor, double low, double high, double original, std::vector<float>& freq) {
    const double pi = 3.14159265358979323846;
    freq.resize(dims / 2);
    for (int i = 0; i < dims / 2; ++i) {
        double f = std::pow(base, -2.0 * i / dims);
        if (factor > 0) {
            const double wl = 2.0 * pi / f;
            if (wl > original / low) f = f / factor;
            else if (!(wl < original / high)) {
                const double s = (original / wl - low) / (high - low);
                f = (1.0 - s) * f / factor + s * f;
            }
        }
        freq[i] = (float)f;
    }
}

struct WindowAttnArgs {
    const float* q;          // [T, H*D]
    PagedKV kv;
    const float* slopes;     // [H] distance penalty per head (0 = none)
    float scale;
    int window;              // 0 = every earlier position
    const float* gate; int gate_ld;   // raw gate pre-activations [T, .] (column h*Dv + c) or nullptr
    int gate_per_head = 0;   // 1: the gate has ONE number per head (column h)
    int sink = 0;            // 1: one is added to the softmax denominator (a key of score 0 that has no value)
    const float* sink_logit = nullptr;   // [H] with sink == 1: the extra key's score is this learned number of the head (unscaled) instead of 0
    float* out;              // [T, H*Dv]
    int H;
    RaggedBatch rb;
    int skip_from_n = 0;     // > 0: tokens of entries that bring at least this many tokens are left to another kernel
    // split launches (decode-sized steps): the visible keys of a token are cut into `nsplit` chunks of `chunk` keys, one block each
    float* part = nullptr;   // [T][H][nsplit][2 + Dv]: running max, sum of weights, un-normalised weighted values
    int nsplit = 1, chunk = 0;
};

constexpr int kWinAttnThreads = 128;
constexpr int kWinAttnMaxAcc = 4;    // Dv <= 4 * 128
constexpr int kWinSplitMaxTokens = 32, kWinMaxSplits = 32, kWinSplitKeys = 64;

// One block per (token, head[, chunk of keys]).  Scores: a warp takes four keys at a time, its lanes run over the head dimension (one
// coalesced read of each key row), so a tile of 128 keys costs 8 rounds per warp; softmax over the tile across the block; values: thread
// c owns output channel c (+ 128, ...) and walks the tile's value rows, which are contiguous across the threads.
template <bool SPLIT>
static __global__ void __launch_bounds__(kWinAttnThreads) window_attn_kernel(WindowAttnArgs a) {
    extern __shared__ float sm[];
    const int D = a.kv.D, Dv = a.kv.Dv;
    float* qs = sm;                 // [D]
    float* sc = sm + D;             // [threads]
    float* red = sc + kWinAttnThreads;   // [32]
    __shared__ int pgs[kWinAttnThreads / kPage + 1];      // physical pages of the tile's keys
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = h / (a.H / a.kv.G);
    const int e = a.rb.tok_entry[t], i = a.rb.tok_pos[t], slot = a.rb.ent_slot[e];
    if (!SPLIT && a.skip_from_n > 0 && a.rb.ent_start[e + 1] - a.rb.ent_start[e] >= a.skip_from_n) return;
    const int* pt = a.rb.page_tables + (size_t)slot * a.rb.max_pages;
    const float slope = a.slopes ? a.slopes[h] : 0.f;
    int ja = a.window > 0 ? max(0, i - a.window + 1) : 0, jb = i + 1;          // visible keys [ja, jb)
    float* P = nullptr;
    if (SPLIT) {
        ja += blockIdx.z * a.chunk;
        jb = min(ja + a.chunk, jb);
        P = a.part + (((size_t)t * a.H + h) * a.nsplit + blockIdx.z) * (size_t)(2 + Dv);
        if (ja >= jb) { if (tid == 0) { P[0] = -INFINITY; P[1] = 0.f; } return; }
    }
    for (int d = tid; d < D; d += kWinAttnThreads) qs[d] = a.q[(size_t)t * a.H * D + h * D + d];
    __syncthreads();
    float m = -INFINITY, l = 0.f;
    float acc[kWinAttnMaxAcc];
#pragma unroll
    for (int r = 0; r < kWinAttnMaxAcc; ++r) acc[r] = 0.f;
    for (int jt = ja; jt < jb; jt += kWinAttnThreads) {
        const int nj = min(kWinAttnThreads, jb - jt), pg0 = jt >> kPageShift;
        if (tid <= ((jt + nj - 1) >> kPageShift) - pg0) pgs[tid] = pt[pg0 + tid];
        __syncthreads();
        for (int k0 = warp * 4; k0 < nj; k0 += 16) {
            const float* kr[4];
            float dot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = jt + min(k0 + u, nj - 1);
                kr[u] = a.kv.k_row(pgs[(j >> kPageShift) - pg0], g, j & (kPage - 1));
            }
            for (int d = lane; d < D; d += 32) {
                const float qd = qs[d];
#pragma unroll
                for (int u = 0; u < 4; ++u) dot[u] = fmaf(qd, kr[u][d], dot[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float v = warp_sum(dot[u]);
                if (lane == 0 && k0 + u < nj) sc[k0 + u] = v * a.scale - slope * (float)(i - (jt + k0 + u));
            }
        }
        __syncthreads();
        const float s = tid < nj ? sc[tid] : -INFINITY;
        const float m_new = fmaxf(m, block_max(s, red));
        const float p = tid < nj ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);          // m = -inf on the first tile: 0
        sc[tid] = p;
        const float psum = block_sum(p, red);          // its barriers publish sc
        l = l * corr + psum;
        m = m_new;
#pragma unroll
        for (int r = 0; r < kWinAttnMaxAcc; ++r) {
            const int c = tid + r * kWinAttnThreads;
            if (c < Dv) {
                float o = acc[r] * corr;
#pragma unroll 8
                for (int jj = 0; jj < nj; ++jj) {
                    const int jk = jt + jj;
                    o = fmaf(sc[jj], a.kv.v_row(pgs[(jk >> kPageShift) - pg0], g, jk & (kPage - 1))[c], o);
                }
                acc[r] = o;
            }
        }
        __syncthreads();     // sc is rewritten by the next tile
    }
    if (SPLIT) {
        if (tid == 0) { P[0] = m; P[1] = l; }
#pragma unroll
        for (int r = 0; r < kWinAttnMaxAcc; ++r) {
            const int c = tid + r * kWinAttnThreads;
            if (c < Dv) P[2 + c] = acc[r];
        }
        return;
    }
    float inv = 1.0f / l;
    if (a.sink) {                      // bring the sums to max(m, sink score), the maximum once the sink takes part
        const float sk = a.sink_logit ? a.sink_logit[h] : 0.f;
        const float M = fmaxf(m, sk), w = expf(m - M);
        inv = w / (l * w + expf(sk - M));
    }
#pragma unroll
    for (int r = 0; r < kWinAttnMaxAcc; ++r) {
        const int c = tid + r * kWinAttnThreads;
        if (c < Dv) {
            float o = acc[r] * inv;
            if (a.gate) o *= sigmoid_f(a.gate[(size_t)t * a.gate_ld + (a.gate_per_head ? h : h * Dv + c)]);
            a.out[(size_t)t * a.H * Dv + h * Dv + c] = o;
        }
    }
}

// merges the chunks of a (token, head): weights exp(m_s - M) / L bring every partial sum to the common maximum.  The weights are formed
// once (a thread per chunk), so that the sum over the chunks is a chain of multiply-adds whose loads are all in flight together.
constexpr int kWinMergeMaxSplits = 128;
static __global__ void __launch_bounds__(kWinAttnThreads) window_attn_merge_kernel(WindowAttnArgs a) {
    __shared__ float wsm[kWinMergeMaxSplits];
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y, Dv = a.kv.Dv, tid = threadIdx.x;
    const float* P = a.part + ((size_t)t * a.H + h) * a.nsplit * (size_t)(2 + Dv);
    const bool mine = tid < a.nsplit;
    const float ms = mine ? P[(size_t)tid * (2 + Dv)] : -INFINITY, ls = mine ? P[(size_t)tid * (2 + Dv) + 1] : 0.f;
    float M = block_max(ms, red);
    const float sk = a.sink && a.sink_logit ? a.sink_logit[h] : 0.f;
    if (a.sink) M = fmaxf(M, sk);
    const float wgt = ls > 0.f ? expf(ms - M) : 0.f;
    const float L = block_sum(ls * wgt, red) + (a.sink ? expf(sk - M) : 0.f);
    if (mine) wsm[tid] = wgt / L;
    __syncthreads();
    // a block sums ONE slice of 128 channels (blockIdx.z): a single decoded token still spreads over heads x slices blocks, and a thread's
    // loads of several chunks are in flight together (a chunk without visible keys left no values: its weight is 0 and nothing is read)
    const int c = tid + blockIdx.z * kWinAttnThreads;
    if (c >= Dv) return;
    float o = 0.f;
#pragma unroll 8
    for (int s = 0; s < a.nsplit; ++s) {
        const float w = wsm[s];
        const float v = w != 0.f ? P[(size_t)s * (2 + Dv) + 2 + c] : 0.f;
        o = fmaf(v, w, o);
    }
    if (a.gate) o *= sigmoid_f(a.gate[(size_t)t * a.gate_ld + (a.gate_per_head ? h : h * Dv + c)]);
    a.out[(size_t)t * a.H * Dv + h * Dv + c] = o;
}

// only_single: every entry of the step brings one token (the tails are moved along by the convolution kernel).  Returns the launches.
inline int qkv_prepare(cudaStream_t st, const QkvPrepArgs& a, bool only_single) {
    if (a.rb.T == 0) return 0;
    AHA_REQUIRE(a.taps <= kConvMaxTaps, "short convolution: more than 16 taps");
    if (a.rb.T <= 8) qkv_conv_norm_kernel<1024><<<a.rb.T, 1024, 0, st>>>(a);      // a decode step has few blocks: more threads for each
    else qkv_conv_norm_kernel<256><<<a.rb.T, 256, 0, st>>>(a);
    const bool tail_launch = a.taps > 1 && !only_single;
    if (tail_launch) conv_tail_update_kernel<<<a.rb.E, 256, 0, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
    return tail_launch ? 2 : 1;
}

inline size_t window_attn_part_floats(int H, int Dv) { return (size_t)kWinSplitMaxTokens * H * kWinMaxSplits * (2 + Dv); }

// kv_span: an upper bound of the keys any token of the step sees (the window, or the longest sequence of the step); `part` != nullptr
// and a decode-sized step: the keys are cut into chunks, one block each, and merged.  Returns the launches.
inline int window_attn(cudaStream_t st, WindowAttnArgs a, int kv_span) {
    if (a.rb.T == 0) return 0;
    AHA_REQUIRE(a.kv.Dv <= kWinAttnMaxAcc * kWinAttnThreads, "window attention: value head size above 512");
    const size_t smem = ((size_t)a.kv.D + kWinAttnThreads + 32) * sizeof(float);
    if (a.part && a.rb.T <= kWinSplitMaxTokens && kv_span > kWinAttnThreads) {
        a.nsplit = std::min(kWinMaxSplits, ceil_div(kv_span, kWinSplitKeys));      // short chunks: a block walks its keys in order
        a.chunk = ceil_div(ceil_div(kv_span, a.nsplit), kPage) * kPage;
        a.skip_from_n = 0;
        window_attn_kernel<true><<<dim3(a.rb.T, a.H, a.nsplit), kWinAttnThreads, smem, st>>>(a);
        window_attn_merge_kernel<<<dim3(a.rb.T, a.H, ceil_div(a.kv.Dv, kWinAttnThreads)), kWinAttnThreads, 0, st>>>(a);
        AHA_CUDA_CHECK(cudaGetLastError());
        return 2;
    }
    window_attn_kernel<false><<<dim3(a.rb.T, a.H), kWinAttnThreads, smem, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
    return 1;
}

}  // namespace aha
