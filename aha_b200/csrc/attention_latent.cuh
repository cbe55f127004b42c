// attention_latent.cuh -- what is special about latent attention: every token leaves ONE low-rank latent c (RMS-normed) and ONE rotated
// key part in the cache, shared by all heads; a head's keys and values are W_uk c and W_uv c.  The engine never expands them: with
//     score = q_plain . (W_uk c) + q_rot . k_rot = (W_uk^T q_plain) . c + q_rot . k_rot
// a head's query becomes [W_uk^T q_plain | q_rot] against the cached row [c | k_rot], and its output W_uv (sum_j p_j c_j): ordinary
// attention of many query heads over a single key / value head whose values are the first `rank` columns of its keys.  The two
// per-head products are batched matrix products (gemm_any.cuh), the attention itself is the ragged kernel of attention_window.cuh.
//
//   latent_prep_kernel   per token: RMS norm of the latent (gain per channel) and rotary embedding of the shared key part into the page
//                        of the token's position; rotary embedding of every head's rotated query part into the absorbed-query buffer;
//                        optionally the RMS norm of a query latent in place (queries that are expanded from a latent of their own).
// Rotary: interleaved pairs (2i, 2i + 1) of the first 2 * n_freq coordinates turn by pos * freq[i]; cos and sin carry `mult` (YaRN's
// attention factor); further coordinates pass unchanged.  Angles are fp32 products, cos / sin the accurate functions.
#pragma once
#include <cmath>
#include <vector>

#include "attention_window.cuh"
#include "gemm_any.cuh"      // load_w8 / wt_to_f: weights as bf16 or fp32

namespace aha {

// Rotary frequencies with optional YaRN interpolation (host, double): dims rotated coordinates, base; factor > 0: frequencies whose
// wavelength exceeds the original context are divided by `factor`, short ones kept, a linear ramp between the coordinates whose
// wavelengths fit `fast` and `slow` times into `original`; cos / sin are multiplied by 0.1 ln(factor) + 1.
inline void yarn_frequencies(int dims, double base, double factor, double original, double fast, double slow, std::vector<float>& freq, float& mult) {
    const int n = dims / 2;
    freq.resize(n);
    mult = 1.f;
    const double pi = 3.14159265358979323846;
    auto dim_of = [&](double turns) { return dims * std::log(original / (2.0 * pi * turns)) / (2.0 * std::log(base)); };
    double lo = 0, hi = 0;
    if (factor > 0) {
        lo = std::max(std::floor(dim_of(fast)), 0.0);
        hi = std::min(std::ceil(dim_of(slow)), (double)(dims - 1));
        mult = (float)(0.1 * std::log(factor) + 1.0);
    }
    for (int i = 0; i < n; ++i) {
        const double f = std::pow(base, -2.0 * i / dims);
        if (factor > 0) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            freq[i] = (float)(f / factor * ramp + f * (1.0 - ramp));
        } else freq[i] = (float)f;
    }
}

struct LatentPrepArgs {
    float* proj; int ld;            // [T, ld] projected rows
    int q_off, dkv_off;             // first query column (heads x (dim + rot)), first latent column (rank + rot)
    int H, D, R, rank;
    const float* c_norm; float eps; // [rank]
    const float* freq; int n_freq; float mult;
    float* q_abs; int ld_q;         // [T, H * (rank + R)]: the rotated query part goes to columns h * (rank + R) + rank ...
    PagedKV kv;                     // G = 1, D = rank + R
    RaggedBatch rb;
    // a query latent that is normed on the way (in place, gain per channel): columns ql_off .. ql_off + ql_rank - 1 of the projected rows; 0: none
    int ql_off = 0, ql_rank = 0; const float* ql_norm = nullptr;
    int skip_q = 0;                 // 1: the queries' rotated parts are left alone (they do not exist yet: latent_absorb_kernel turns them later)
};

static __global__ void latent_prep_kernel(LatentPrepArgs a) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int e = a.rb.tok_entry[t], pos = a.rb.tok_pos[t], slot = a.rb.ent_slot[e];
    const float* row = a.proj + (size_t)t * a.ld;
    const int page = a.rb.page_tables[(size_t)slot * a.rb.max_pages + (pos >> kPageShift)];
    float* krow = a.kv.k_row(page, 0, pos & (kPage - 1));
    const float* d = row + a.dkv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) ss = fmaf(d[i], d[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)a.rank + a.eps);
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) krow[i] = d[i] * inv * a.c_norm[i];
    if (a.ql_rank > 0) {
        float* ql = a.proj + (size_t)t * a.ld + a.ql_off;
        float sq = 0.f;
        for (int i = threadIdx.x; i < a.ql_rank; i += blockDim.x) sq = fmaf(ql[i], ql[i], sq);
        sq = block_sum(sq, red);
        const float iq = 1.0f / sqrtf(sq / (float)a.ql_rank + a.eps);
        for (int i = threadIdx.x; i < a.ql_rank; i += blockDim.x) ql[i] = ql[i] * iq * a.ql_norm[i];
    }
    // rotated parts: item (0, pair) is the shared key part, item (1 + h, pair) head h's query part; pairs beyond n_freq are single pass-through coordinates
    const int half = a.n_freq, rest = a.R - 2 * half, per = half + rest;
    const float fpos = (float)pos;
    for (int idx = threadIdx.x; idx < (a.skip_q ? 1 : 1 + a.H) * per; idx += blockDim.x) {
        const int item = idx / per, j = idx % per;
        const float* src = item == 0 ? d + a.rank : row + a.q_off + (size_t)(item - 1) * (a.D + a.R) + a.D;
        float* dst = item == 0 ? krow + a.rank : a.q_abs + (size_t)t * a.ld_q + (size_t)(item - 1) * (a.rank + a.R) + a.rank;
        if (j < half) {
            float sn, cs;
            sincosf(fpos * a.freq[j], &sn, &cs);
            sn *= a.mult; cs *= a.mult;
            const float u = src[2 * j], v = src[2 * j + 1];
            dst[2 * j] = u * cs - v * sn;
            dst[2 * j + 1] = v * cs + u * sn;
        } else {
            const int c = 2 * half + (j - half);
            dst[c] = src[c];
        }
    }
}

}  // namespace aha

namespace aha {

// ---------------------------------------------------------------------------------------------------------------------------------
// Prompt portions.  The absorbed form costs (2 rank + R) multiply-adds per (query, key, head); with the keys and values of the
// sequence expanded once per portion (one matrix product of its cached latents with [W_uk; W_uv], on the tensor cores in serving mode)
// a pair costs D + R + Dv, a third of that for the usual sizes, and a head's keys are contiguous rows.  So an entry of many tokens runs
//   latent_gather_kernel   the sequence's cached rows [latent | rotated key part], positions 0 .. S - 1, from its pages into a dense buffer
//   (Linear)               kv[s] = [W_uk; W_uv] latent[s]
//   latent_flash_kernel    causal softmax attention per head, fp32 on the CUDA cores, never materialising n x S: a block owns 64 queries
//                          of one head and walks the keys in tiles of 64; thread (ty, tx) of 16 x 16 holds the scores of queries
//                          4 ty .. 4 ty + 3 against keys tx + 16 i, then the outputs of the same queries in columns tx + 16 j, so the
//                          running maximum and sum of a query never leave its threads (the 16 threads of a row meet by shuffles)
// while decoded tokens and short portions stay on the absorbed form above.
// rows of positions s0 .. s0 + S - 1 (s0 > 0: a sliding window needs nothing before its first query's first key)
static __global__ void latent_gather_kernel(PagedKV kv, const int* __restrict__ page_table, float* __restrict__ out, int s0, int S) {
    const int s = blockIdx.x;
    if (s >= S) return;
    const float* row = kv.k_row(page_table[(s0 + s) >> kPageShift], 0, (s0 + s) & (kPage - 1));
    for (int i = threadIdx.x; i < kv.D; i += blockDim.x) out[(size_t)s * kv.D + i] = row[i];
}

struct LatentFlashArgs {
    const float* q_plain; int ld_qp; int qp_head_stride;   // [T, .]: head h's unrotated query part at column h * qp_head_stride
    const float* q_rot; int ld_qr; int qr_head_stride;     // [T, .]: head h's rotated part at column h * qr_head_stride
    const float* kx; int ld_k; int k_head_stride;          // [S, .] expanded keys (unrotated part), head h at column h * k_head_stride
    const float* vx; int ld_v; int v_head_stride;          // [S, .] expanded values
    const float* k_rot; int ld_kr;                         // [S, .] rotated key part shared by the heads
    float* out; int ld_o;                                  // [T, H * Dv]
    int t0, n, pos0;                                       // the entry's packed rows t0 .. t0 + n - 1 are positions pos0 .. pos0 + n - 1 (counted from the
                                                           // first expanded key, which need not be the sequence's first token)
    int D, R, Dv;
    float scale;
    int window = 0;                                        // > 0: query i sees keys j with 0 <= i - j < window
    const float* sink = nullptr;                           // [H]: the softmax denominator of head h also holds exp(sink[h]) (no key, no value, not scaled)
};

constexpr int kLfBQ = 64, kLfBK = 64, kLfThreads = 256;

__device__ __forceinline__ void lf_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void lf_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Key and value tiles come in by cp.async, all of a tile's copies in flight at once, in two groups that alternate: the next key tile is
// requested as soon as the scores of this one are formed (it arrives under the value pass), the next value tile after the value pass (it
// arrives under the next scores), so one buffer each is enough.  vec: every row piece is 16-byte aligned (sizes and strides multiples of 4).
template <int NV>      // value columns per thread: Dv <= 16 NV
static __global__ void __launch_bounds__(kLfThreads) latent_flash_kernel(LatentFlashArgs a, int vec) {
    extern __shared__ __align__(16) float lf_sm[];
    const int Dq = a.D + a.R, ldq = (Dq + 3) / 4 * 4 + 4, ldv = (a.Dv + 3) / 4 * 4;     // (ldq: the 16 threads of a row read different banks when Dq % 8 == 0)
    float* Qs = lf_sm;                          // [64][ldq], scaled
    float* Ks = Qs + kLfBQ * ldq;               // [64][ldq]
    float* Vs = Ks + kLfBK * ldq;               // [64][ldv]
    float* Ps = Vs + kLfBK * ldv;               // [64][64 + 4]
    constexpr int ldp = kLfBK + 4;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4, h = blockIdx.y;
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kLfBQ, nq = min(kLfBQ, a.n - q0);      // the tiles with the most keys start first
    const int last_pos = a.pos0 + q0 + nq - 1;                 // the tile's last query sees keys 0 .. last_pos
    auto load_k = [&](int k0) {
        const int nk = min(kLfBK, last_pos + 1 - k0);
        if (nk > 0) {
            if (vec) {
                const int D4 = a.D >> 2, C4 = Dq >> 2;
                for (int idx = tid; idx < nk * C4; idx += kLfThreads) {
                    const int r = idx / C4, c = idx % C4;
                    const size_t sr = (size_t)(k0 + r);
                    lf_cp16(Ks + r * ldq + 4 * c, c < D4 ? a.kx + sr * a.ld_k + (size_t)h * a.k_head_stride + 4 * c : a.k_rot + sr * a.ld_kr + 4 * (c - D4));
                }
            } else {
                for (int idx = tid; idx < nk * Dq; idx += kLfThreads) {
                    const int r = idx / Dq, d = idx % Dq;
                    const size_t sr = (size_t)(k0 + r);
                    lf_cp4(Ks + r * ldq + d, d < a.D ? a.kx + sr * a.ld_k + (size_t)h * a.k_head_stride + d : a.k_rot + sr * a.ld_kr + d - a.D);
                }
            }
            for (int idx = tid; idx < (kLfBK - nk) * ldq; idx += kLfThreads) Ks[nk * ldq + idx] = 0.f;     // rows past the last key
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto load_v = [&](int k0) {
        const int nk = min(kLfBK, last_pos + 1 - k0);
        if (nk > 0) {
            if (vec) {
                const int C4 = a.Dv >> 2;
                for (int idx = tid; idx < nk * C4; idx += kLfThreads) {
                    const int r = idx / C4, c = idx % C4;
                    lf_cp16(Vs + r * ldv + 4 * c, a.vx + (size_t)(k0 + r) * a.ld_v + (size_t)h * a.v_head_stride + 4 * c);
                }
            } else {
                for (int idx = tid; idx < nk * a.Dv; idx += kLfThreads) {
                    const int r = idx / a.Dv, c = idx % a.Dv;
                    lf_cp4(Vs + r * ldv + c, a.vx + (size_t)(k0 + r) * a.ld_v + (size_t)h * a.v_head_stride + c);
                }
            }
            for (int idx = tid; idx < (kLfBK - nk) * ldv; idx += kLfThreads) Vs[nk * ldv + idx] = 0.f;     // a weight of zero must meet a finite value
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // keys before the window of the tile's first query are never visited
    const int k_begin = a.window > 0 ? max(0, a.pos0 + q0 - a.window + 1) / kLfBK * kLfBK : 0;
    load_k(k_begin);
    load_v(k_begin);
    for (int idx = tid; idx < kLfBQ * ldq; idx += kLfThreads) {
        const int r = idx / ldq, d = idx % ldq;
        float v = 0.f;
        if (r < nq && d < Dq) {
            const size_t t = (size_t)(a.t0 + q0 + r);
            v = (d < a.D ? a.q_plain[t * a.ld_qp + (size_t)h * a.qp_head_stride + d] : a.q_rot[t * a.ld_qr + (size_t)h * a.qr_head_stride + d - a.D]) * a.scale;
        }
        Qs[idx] = v;
        if (d >= Dq) Ks[idx] = 0.f;             // the padding columns of the key rows are never copied to
    }
    float m[4], l[4], o[4][NV];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) o[i][j] = 0.f;
    }
    for (int k0 = k_begin; k0 <= last_pos; k0 += kLfBK) {
        const int nk = min(kLfBK, last_pos + 1 - k0);
        asm volatile("cp.async.wait_group 1;" ::: "memory");      // this tile's keys (its values may still be on their way)
        __syncthreads();
        // scores of queries 4 ty + i against keys tx + 16 u
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int u = 0; u < 4; ++u) s[i][u] = 0.f;
        for (int d = 0; d < ldq - 4; d += 4) {
            float4 qv[4], kv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(Qs + (4 * ty + i) * ldq + d);
#pragma unroll
            for (int u = 0; u < 4; ++u) kv[u] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * u) * ldq + d);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    s[i][u] = fmaf(qv[i].w, kv[u].w, fmaf(qv[i].z, kv[u].z, fmaf(qv[i].y, kv[u].y, fmaf(qv[i].x, kv[u].x, s[i][u]))));
        }
        __syncthreads();                                           // every thread has read the key tile: the next one may come in
        load_k(k0 + kLfBK);
        // causal mask, running softmax of each query row (its 16 threads are the lanes of one half warp)
        float corr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qpos = a.pos0 + q0 + 4 * ty + i;
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = k0 + tx + 16 * u;
                if (j > qpos || tx + 16 * u >= nk || (a.window > 0 && qpos - j >= a.window)) s[i][u] = -INFINITY;
                mx = fmaxf(mx, s[i][u]);
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m[i], mx);
            float ps = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float p = m_new == -INFINITY ? 0.f : expf(s[i][u] - m_new);     // a row of a partial tile may see no key at all
                Ps[(4 * ty + i) * ldp + tx + 16 * u] = p;
                ps += p;
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            corr[i] = m_new == -INFINITY ? 1.f : expf(m[i] - m_new);
            l[i] = l[i] * corr[i] + ps;
            m[i] = m_new;
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");      // this tile's values (the next keys may still be on their way)
        __syncthreads();                                           // ... and the weights are in shared memory
        // outputs of the same queries, columns tx + 16 j
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < NV; ++j) o[i][j] *= corr[i];
        for (int k = 0; k < nk; k += 4) {
            float4 pv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pv[i] = *reinterpret_cast<const float4*>(Ps + (4 * ty + i) * ldp + k);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                float vv[NV];
#pragma unroll
                for (int j = 0; j < NV; ++j) vv[j] = (tx + 16 * j < a.Dv) ? Vs[(k + kk) * ldv + tx + 16 * j] : 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float p = kk == 0 ? pv[i].x : (kk == 1 ? pv[i].y : (kk == 2 ? pv[i].z : pv[i].w));
#pragma unroll
                    for (int j = 0; j < NV; ++j) o[i][j] = fmaf(p, vv[j], o[i][j]);
                }
            }
        }
        __syncthreads();                                           // every thread has read the values and the weights
        load_v(k0 + kLfBK);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = 4 * ty + i;
        if (r >= nq) continue;
        float inv = 1.0f / l[i];
        if (a.sink) {                  // bring the sums to max(m, sink), the maximum once the sink takes part
            const float sk = a.sink[h], M = fmaxf(m[i], sk), w = expf(m[i] - M);
            inv = w / (l[i] * w + expf(sk - M));
        }
        float* orow = a.out + (size_t)(a.t0 + q0 + r) * a.ld_o + (size_t)h * a.Dv;
#pragma unroll
        for (int j = 0; j < NV; ++j)
            if (tx + 16 * j < a.Dv) orow[tx + 16 * j] = o[i][j] * inv;
    }
}

inline size_t latent_flash_smem(int D, int R, int Dv) {
    const int ldq = (D + R + 3) / 4 * 4 + 4;
    return ((size_t)(kLfBQ + kLfBK) * ldq + (size_t)kLfBK * ((Dv + 3) / 4 * 4) + (size_t)kLfBQ * (kLfBK + 4)) * sizeof(float);
}
inline bool latent_flash_supported(int D, int R, int Dv) { return Dv <= 256 && latent_flash_smem(D, R, Dv) <= 200 * 1024; }

inline void latent_flash(cudaStream_t st, const LatentFlashArgs& a, int H) {
    const size_t smem = latent_flash_smem(a.D, a.R, a.Dv);
    const dim3 grid(ceil_div(a.n, kLfBQ), H);
    static bool attr = false;
    if (!attr) {
        AHA_CUDA_CHECK(cudaFuncSetAttribute(latent_flash_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        AHA_CUDA_CHECK(cudaFuncSetAttribute(latent_flash_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        AHA_CUDA_CHECK(cudaFuncSetAttribute(latent_flash_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr = true;
    }
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec = (a.D % 4 == 0 && a.R % 4 == 0 && a.Dv % 4 == 0 && a.ld_k % 4 == 0 && a.k_head_stride % 4 == 0 && a.ld_v % 4 == 0 && a.v_head_stride % 4 == 0 &&
                     a.ld_kr % 4 == 0 && al(a.kx) && al(a.vx) && al(a.k_rot)) ? 1 : 0;
    if (a.Dv <= 64) latent_flash_kernel<4><<<grid, kLfThreads, smem, st>>>(a, vec);
    else if (a.Dv <= 128) latent_flash_kernel<8><<<grid, kLfThreads, smem, st>>>(a, vec);
    else latent_flash_kernel<16><<<grid, kLfThreads, smem, st>>>(a, vec);
    AHA_CUDA_CHECK(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Decode-sized steps.  All heads of a token read the SAME cached rows, so a block owns (token, chunk of keys) for sixteen heads at a
// time instead of one: a key row is fetched once for them.  Scores: thread (key, slice) of 32 x 8 takes every eighth 16-byte piece of the
// key's row (the eight threads of a key read 128 consecutive bytes at a time) and holds the partial dot products of all sixteen heads,
// summed over the slices by shuffles; softmax of a head over the tile by one warp (a lane per key); values: thread c owns latent channels
// c and c + 256 for all sixteen heads.  Chunks are short (a few tiles) and many, so that a single decoded token still fills the GPU.  Partial results (running maximum, sum, un-normalised values per head and chunk) have the layout of
// window_attn_kernel<true>, so window_attn_merge_kernel joins the chunks.
constexpr int kLdThreads = 256, kLdKeys = 32, kLdHG = 16, kLdMaxSplits = 64;

struct LatentDecodeArgs {
    const float* q; int ld_q;        // [T, H * Dk] absorbed queries
    PagedKV kv;                      // G = 1, D = Dk, Dv = rank (values alias the keys)
    float scale;
    float* part; int nsplit, chunk;  // see WindowAttnArgs
    int H;
    int window;                      // > 0: token i sees keys j with 0 <= i - j < window
    RaggedBatch rb;
};

static __global__ void __launch_bounds__(kLdThreads) latent_decode_attn_kernel(LatentDecodeArgs a) {
    extern __shared__ __align__(16) float ld_sm[];
    const int Dk = a.kv.D, Dv = a.kv.Dv;
    float* qs = ld_sm;                          // [16][Dk], scaled
    float* sc = qs + kLdHG * Dk;                // [16][64]
    float* hm = sc + kLdHG * kLdKeys;           // [16] running maximum, [16] running sum, [16] rescale factor of the tile
    float* hl = hm + kLdHG;
    float* hc = hl + kLdHG;
    __shared__ int pgs[kLdKeys / kPage + 2];
    const int t = blockIdx.x, z = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e = a.rb.tok_entry[t], i = a.rb.tok_pos[t], slot = a.rb.ent_slot[e];
    const int* pt = a.rb.page_tables + (size_t)slot * a.rb.max_pages;
    const int ja = (a.window > 0 ? max(0, i - a.window + 1) : 0) + z * a.chunk, jb = min(ja + a.chunk, i + 1);
    const bool vec = (Dk & 3) == 0;
    for (int g0 = 0; g0 < a.H; g0 += kLdHG) {
        const int hg = min(kLdHG, a.H - g0);
        if (ja >= jb) {                         // nothing visible in this chunk
            if (tid < hg) { float* P = a.part + (((size_t)t * a.H + g0 + tid) * a.nsplit + z) * (size_t)(2 + Dv); P[0] = -INFINITY; P[1] = 0.f; }
            continue;
        }
        for (int idx = tid; idx < hg * Dk; idx += kLdThreads) qs[idx] = a.q[(size_t)t * a.ld_q + (size_t)g0 * Dk + idx] * a.scale;
        if (tid < kLdHG) { hm[tid] = -INFINITY; hl[tid] = 0.f; }
        float acc[2][kLdHG];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int h = 0; h < kLdHG; ++h) acc[r][h] = 0.f;
        __syncthreads();
        for (int jt = ja; jt < jb; jt += kLdKeys) {
            const int nj = min(kLdKeys, jb - jt), pg0 = jt >> kPageShift;
            if (tid <= ((jt + nj - 1) >> kPageShift) - pg0) pgs[tid] = pt[pg0 + tid];
            __syncthreads();
            {
                const int key = tid >> 3, ds = tid & 7;
                float s[kLdHG];
#pragma unroll
                for (int h = 0; h < kLdHG; ++h) s[h] = 0.f;
                if (key < nj) {
                    const int j = jt + key;
                    const float* kr = a.kv.k_row(pgs[(j >> kPageShift) - pg0], 0, j & (kPage - 1));
                    if (vec) {
#pragma unroll 4
                        for (int d = 4 * ds; d < Dk; d += 32) {
                            const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
                            for (int h = 0; h < kLdHG; ++h) {
                                if (h < hg) {
                                    const float4 q4 = *reinterpret_cast<const float4*>(qs + h * Dk + d);
                                    s[h] = fmaf(q4.w, k4.w, fmaf(q4.z, k4.z, fmaf(q4.y, k4.y, fmaf(q4.x, k4.x, s[h]))));
                                }
                            }
                        }
                    } else {
                        for (int d = ds; d < Dk; d += 8) {
                            const float kd = kr[d];
#pragma unroll
                            for (int h = 0; h < kLdHG; ++h)
                                if (h < hg) s[h] = fmaf(qs[h * Dk + d], kd, s[h]);
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < kLdHG; ++h) {
                    float v = s[h];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    if (ds == 0 && h < hg) sc[h * kLdKeys + key] = key < nj ? v : -INFINITY;
                }
            }
            __syncthreads();
            for (int h = warp; h < hg; h += kLdThreads / 32) {
                const float s0 = sc[h * kLdKeys + lane];
                const float m_old = hm[h], m_new = fmaxf(m_old, warp_max(s0));      // every tile holds at least one visible key
                const float p0 = expf(s0 - m_new);
                const float ps = warp_sum(p0);
                sc[h * kLdKeys + lane] = p0;
                if (lane == 0) { const float c = expf(m_old - m_new); hc[h] = c; hl[h] = hl[h] * c + ps; hm[h] = m_new; }
            }
            __syncthreads();
            {
                const int c0 = tid, c1 = tid + kLdThreads;
#pragma unroll
                for (int h = 0; h < kLdHG; ++h) { const float f = h < hg ? hc[h] : 0.f; acc[0][h] *= f; acc[1][h] *= f; }
#pragma unroll 8
                for (int jj = 0; jj < nj; ++jj) {      // both columns' loads of eight keys in flight together
                    const int j = jt + jj;
                    const float* vr = a.kv.v_row(pgs[(j >> kPageShift) - pg0], 0, j & (kPage - 1));
                    const float v0 = c0 < Dv ? vr[c0] : 0.f, v1 = c1 < Dv ? vr[c1] : 0.f;
#pragma unroll
                    for (int h = 0; h < kLdHG; ++h) {
                        const float p = h < hg ? sc[h * kLdKeys + jj] : 0.f;
                        acc[0][h] = fmaf(p, v0, acc[0][h]);
                        acc[1][h] = fmaf(p, v1, acc[1][h]);
                    }
                }
            }
            __syncthreads();       // sc, hc and pgs are rewritten by the next tile
        }
#pragma unroll
        for (int h = 0; h < kLdHG; ++h) {
            if (h < hg) {
                float* P = a.part + (((size_t)t * a.H + g0 + h) * a.nsplit + z) * (size_t)(2 + Dv);
                if (tid == 0) { P[0] = hm[h]; P[1] = hl[h]; }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int c = tid + r * kLdThreads;
                    if (c < Dv) P[2 + c] = acc[r][h];
                }
            }
        }
        __syncthreads();           // qs, hm, hl are rewritten by the next group of heads
    }
}

// Decode-sized steps: the absorbed query of every (token, head),
//     q_abs[t][h] = [ W_uk(h)^T q_plain[t][h] | rot(q_rot[t][h], pos_t) ],
// in ONE launch (where the queries come through a latent of their own the rotary embedding cannot run before their expansion, and a launch
// of its own would only move R numbers per head).
constexpr int kAbsorbMaxTokens = 8, kAbsorbThreads = 128, kAbsorbRows = 64;

struct LatentAbsorbArgs {
    const float* q; int ld; int q_off;     // [T, ld]: head h's query [D unrotated | R rotated] at column q_off + h * (D + R)
    const void* uk_t;                      // [H * rank, D]: row h * rank + r is column r of the head's W_uk rows (bf16 or fp32)
    float* q_abs; int ld_q;                // [T, H * (rank + R)]
    const float* freq; int n_freq; float mult;
    const int* tok_pos;
    int T, H, D, R, rank;
};

// A block owns (head, 64 rows of the head's transposed W_uk).  Sixteen lanes share a row (a lane takes every sixteenth 16-byte piece of it: the
// half warp reads 256 consecutive bytes), a warp walks two rows at a time and four such pairs with all their loads in flight; the unrotated
// query parts of all tokens of the step sit in shared memory, so the matrix is read once per step.  Block (h, 0) also turns the pairs.
template <typename WT>
static __global__ void __launch_bounds__(kAbsorbThreads) latent_absorb_kernel(LatentAbsorbArgs a) {
    extern __shared__ __align__(16) float ab_sm[];      // [T][D]
    const int h = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 15, half = lane >> 4;
    for (int idx = threadIdx.x; idx < a.T * a.D; idx += kAbsorbThreads) {
        const int t = idx / a.D, k = idx % a.D;
        ab_sm[idx] = a.q[(size_t)t * a.ld + a.q_off + (size_t)h * (a.D + a.R) + k];
    }
    __syncthreads();
    const WT* W = reinterpret_cast<const WT*>(a.uk_t) + (size_t)h * a.rank * a.D;
    const int r_base = blockIdx.y * kAbsorbRows + warp * (kAbsorbRows / 4) + half;      // this lane's rows: r_base + 2 i, i < 8
    const bool vec = (a.D & 7) == 0;
    for (int i0 = 0; i0 < kAbsorbRows / 8; i0 += 4) {
        float acc[4][kAbsorbMaxTokens];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int t = 0; t < kAbsorbMaxTokens; ++t) acc[u][t] = 0.f;
        if (vec) {
            for (int k = 8 * sub; k < a.D; k += 128) {
                float wv[4][8];
#pragma unroll
                for (int u = 0; u < 4; ++u) load_w8(W + (size_t)min(r_base + 2 * (i0 + u), a.rank - 1) * a.D + k, wv[u]);
#pragma unroll
                for (int t = 0; t < kAbsorbMaxTokens; ++t)
                    if (t < a.T) {
                        const float4 x0 = *reinterpret_cast<const float4*>(ab_sm + t * a.D + k), x1 = *reinterpret_cast<const float4*>(ab_sm + t * a.D + k + 4);
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            acc[u][t] = fmaf(x1.w, wv[u][7], fmaf(x1.z, wv[u][6], fmaf(x1.y, wv[u][5], fmaf(x1.x, wv[u][4],
                                        fmaf(x0.w, wv[u][3], fmaf(x0.z, wv[u][2], fmaf(x0.y, wv[u][1], fmaf(x0.x, wv[u][0], acc[u][t]))))))));
                    }
            }
        } else {
            for (int k = sub; k < a.D; k += 16) {
                float wk[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) wk[u] = wt_to_f(W[(size_t)min(r_base + 2 * (i0 + u), a.rank - 1) * a.D + k]);
#pragma unroll
                for (int t = 0; t < kAbsorbMaxTokens; ++t)
                    if (t < a.T) {
                        const float x = ab_sm[t * a.D + k];
#pragma unroll
                        for (int u = 0; u < 4; ++u) acc[u][t] = fmaf(x, wk[u], acc[u][t]);
                    }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int r = r_base + 2 * (i0 + u);
#pragma unroll
            for (int t = 0; t < kAbsorbMaxTokens; ++t)
                if (t < a.T) {      // (uniform over the warp)
                    float v = acc[u][t];
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    if (sub == 0 && r < a.rank) a.q_abs[(size_t)t * a.ld_q + (size_t)h * (a.rank + a.R) + r] = v;
                }
        }
    }
    if (blockIdx.y == 0) {
        const int hf = a.n_freq, rest = a.R - 2 * hf, per = hf + rest;
        for (int idx = threadIdx.x; idx < a.T * per; idx += kAbsorbThreads) {
            const int t = idx / per, j = idx % per;
            const float* src = a.q + (size_t)t * a.ld + a.q_off + (size_t)h * (a.D + a.R) + a.D;
            float* dst = a.q_abs + (size_t)t * a.ld_q + (size_t)h * (a.rank + a.R) + a.rank;
            if (j < hf) {
                float sn, cs;
                sincosf((float)a.tok_pos[t] * a.freq[j], &sn, &cs);
                sn *= a.mult; cs *= a.mult;
                const float u = src[2 * j], v = src[2 * j + 1];
                dst[2 * j] = u * cs - v * sn;
                dst[2 * j + 1] = v * cs + u * sn;
            } else {
                const int c = 2 * hf + (j - hf);
                dst[c] = src[c];
            }
        }
    }
}

inline bool latent_absorb_supported(int T, int D) { return T <= kAbsorbMaxTokens && (size_t)T * D * sizeof(float) <= 48 * 1024; }
inline void latent_absorb(cudaStream_t st, const LatentAbsorbArgs& a, bool fp32_weights) {
    const dim3 grid(a.H, ceil_div(a.rank, kAbsorbRows));
    const size_t smem = (size_t)a.T * a.D * sizeof(float);
    if (fp32_weights) latent_absorb_kernel<float><<<grid, kAbsorbThreads, smem, st>>>(a);
    else latent_absorb_kernel<__nv_bfloat16><<<grid, kAbsorbThreads, smem, st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

inline size_t latent_decode_smem(int Dk) { return ((size_t)kLdHG * Dk + kLdHG * kLdKeys + 3 * kLdHG) * sizeof(float); }
inline bool latent_decode_supported(int Dk, int Dv) { return Dv <= 2 * kLdThreads && latent_decode_smem(Dk) <= 160 * 1024; }

// kv_span: an upper bound of the keys any token of the step sees.  w: q, kv, scale, part, out, H, rb as for window_attn.  Returns the launches.
inline int latent_decode_attn(cudaStream_t st, WindowAttnArgs w, int kv_span, int num_sms = 148) {
    // the partial results of T tokens fit the workspace of window_attn (kWinSplitMaxTokens tokens x kWinMaxSplits chunks)
    // a block walks tiles of kLdKeys keys; when full tiles would leave most SMs without a block (one or two decoded tokens, a short window) the
    // chunks are half tiles, twice as many
    const int keys = w.rb.T * ceil_div(kv_span, kLdKeys) >= num_sms ? kLdKeys : kLdKeys / 2;
    w.nsplit = std::max(1, std::min({kLdMaxSplits, ceil_div(kv_span, keys), kWinSplitMaxTokens * kWinMaxSplits / std::max(1, w.rb.T)}));
    w.chunk = ceil_div(ceil_div(kv_span, w.nsplit), keys) * keys;
    w.skip_from_n = 0;
    LatentDecodeArgs a{};
    a.q = w.q; a.ld_q = w.H * w.kv.D; a.kv = w.kv; a.scale = w.scale; a.part = w.part; a.nsplit = w.nsplit; a.chunk = w.chunk; a.H = w.H; a.window = w.window; a.rb = w.rb;
    static bool attr = false;
    if (!attr) { AHA_CUDA_CHECK(cudaFuncSetAttribute(latent_decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)); attr = true; }
    latent_decode_attn_kernel<<<dim3(w.rb.T, w.nsplit), kLdThreads, latent_decode_smem(w.kv.D), st>>>(a);
    window_attn_merge_kernel<<<dim3(w.rb.T, w.H, ceil_div(w.kv.Dv, kWinAttnThreads)), kWinAttnThreads, 0, st>>>(w);
    AHA_CUDA_CHECK(cudaGetLastError());
    return 2;
}

}  // namespace aha
