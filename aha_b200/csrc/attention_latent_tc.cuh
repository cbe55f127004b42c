// attention_latent_tc.cuh -- latent attention's prompt portions on the tensor cores (serving mode): the expanded keys of a head are
// [W_uk c | rotated part] (dim + rot_dim values, e.g. 128 + 64) and its values W_uv c (vdim), so a head is ordinary causal attention
// with key rows longer than value rows.  flash_attn_tc_kernel takes that as HDQ != HD; what is special here is only the pass that packs
//     q   [head][token][HDQ]   from the projected unrotated part and the rotated part (two buffers), zero-padded to HDQ
//     k   [head][key][HDQ]     from the expanded keys and the ONE rotated key part all heads share, zero-padded
//     v^T [head][HD][keys padded to 64]
// into fp16 hi | lo halves (three-term products hi*hi + hi*lo + lo*hi, as everywhere on the tensor cores here).  Zero padding of the
// key / query rows adds nothing to a score.  Served: vdim 64 or 128, dim + rot_dim up to 192; other sizes stay on latent_flash_kernel.
#pragma once
#include "attention_latent.cuh"
#include "attention_tc.cuh"

namespace aha {

struct LatentSplitArgs {
    LatentFlashArgs f;
    __half *q_hi, *q_lo, *k_hi, *k_lo, *vt_hi, *vt_lo;
    int H, S, s_pad, HDQ, HD;
};

// blockIdx.y: 0 = q rows, 1 = k rows (a thread packs pairs of columns), 2 = v^T (a thread packs a pair of keys of one channel)
static __global__ void latent_split_tc_kernel(LatentSplitArgs s) {
    const LatentFlashArgs& a = s.f;
    const int which = blockIdx.y, Dq = a.D + a.R;
    const size_t stride = (size_t)gridDim.x * blockDim.x, start = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (which < 2) {
        const int rows_per_head = which == 0 ? a.n : s.S, half_cols = s.HDQ / 2;
        const size_t total = (size_t)s.H * rows_per_head * half_cols;
        for (size_t idx = start; idx < total; idx += stride) {
            const int p = (int)(idx % half_cols);
            const size_t row = idx / half_cols;
            const int head = (int)(row / rows_per_head), r = (int)(row % rows_per_head);
            float x[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int d = 2 * p + e;
                float v = 0.f;
                if (d < Dq) {
                    if (which == 0) {
                        const size_t t = (size_t)(a.t0 + r);
                        v = d < a.D ? a.q_plain[t * a.ld_qp + (size_t)head * a.qp_head_stride + d] : a.q_rot[t * a.ld_qr + (size_t)head * a.qr_head_stride + d - a.D];
                    } else {
                        v = d < a.D ? a.kx[(size_t)r * a.ld_k + (size_t)head * a.k_head_stride + d] : a.k_rot[(size_t)r * a.ld_kr + d - a.D];
                    }
                }
                x[e] = v;
            }
            uint32_t hi, lo;
            split2(x[0], x[1], hi, lo);
            __half* oh = which == 0 ? s.q_hi : s.k_hi;
            __half* ol = which == 0 ? s.q_lo : s.k_lo;
            reinterpret_cast<uint32_t*>(oh)[row * half_cols + p] = hi;
            reinterpret_cast<uint32_t*>(ol)[row * half_cols + p] = lo;
        }
    } else {
        const int half_keys = s.s_pad / 2;
        const size_t total = (size_t)s.H * half_keys * s.HD;
        for (size_t idx = start; idx < total; idx += stride) {       // the channel runs fastest: the reads are contiguous
            const int c = (int)(idx % s.HD);
            const size_t rest = idx / s.HD;
            const int sp = (int)(rest % half_keys), head = (int)(rest / half_keys);
            float x[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = 2 * sp + e;
                x[e] = (key < s.S && c < a.Dv) ? a.vx[(size_t)key * a.ld_v + (size_t)head * a.v_head_stride + c] : 0.f;
            }
            uint32_t hi, lo;
            split2(x[0], x[1], hi, lo);
            const size_t o = ((size_t)head * s.HD + c) * half_keys + sp;
            reinterpret_cast<uint32_t*>(s.vt_hi)[o] = hi;
            reinterpret_cast<uint32_t*>(s.vt_lo)[o] = lo;
        }
    }
}

inline bool latent_flash_tc_supported(int D, int R, int Dv) { return (Dv == 64 || Dv == 128) && D + R <= (Dv == 128 ? 192 : 128); }
inline int latent_flash_tc_hdq(int D, int R, int Dv) { const int q = (D + R + 63) / 64 * 64; return std::max(q, Dv == 128 ? 128 : 64); }
// workspace halfs for an entry of n queries over S keys
inline size_t latent_flash_tc_ws_halfs(int H, int n, int S, int D, int R, int Dv) {
    const int HDQ = latent_flash_tc_hdq(D, R, Dv);
    return 2 * ((size_t)H * n * HDQ + (size_t)H * S * HDQ + (size_t)H * Dv * flash_tc_skv_pad(S));
}

template <int HD, int HDQ, bool WIN>
inline void latent_flash_tc_launch(cudaStream_t st, const LatentFlashArgs& a, int H, int S, __half* ws) {
    const int pad = flash_tc_skv_pad(S);
    LatentSplitArgs sp;
    sp.f = a; sp.H = H; sp.S = S; sp.s_pad = pad; sp.HDQ = HDQ; sp.HD = HD;
    const size_t nq = (size_t)H * a.n * HDQ, nk = (size_t)H * S * HDQ, nv = (size_t)H * HD * pad;
    sp.q_hi = ws; sp.q_lo = ws + nq; sp.k_hi = ws + 2 * nq; sp.k_lo = sp.k_hi + nk; sp.vt_hi = sp.k_lo + nk; sp.vt_lo = sp.vt_hi + nv;
    const unsigned blocks = (unsigned)std::min<size_t>(148 * 16, std::max<size_t>(1, (nk / 2 + 255) / 256));
    latent_split_tc_kernel<<<dim3(blocks, 3), 256, 0, st>>>(sp);
    AHA_CUDA_CHECK(cudaGetLastError());
    const CUtensorMap tqh = make_tmap_f16_box(sp.q_hi, (uint64_t)H * a.n, HDQ, kFaBQ), tql = make_tmap_f16_box(sp.q_lo, (uint64_t)H * a.n, HDQ, kFaBQ);
    const CUtensorMap tkh = make_tmap_f16_box(sp.k_hi, (uint64_t)H * S, HDQ, kFaBKV), tkl = make_tmap_f16_box(sp.k_lo, (uint64_t)H * S, HDQ, kFaBKV);
    const CUtensorMap tvh = make_tmap_f16_box(sp.vt_hi, (uint64_t)H * HD, (uint64_t)pad, HD), tvl = make_tmap_f16_box(sp.vt_lo, (uint64_t)H * HD, (uint64_t)pad, HD);
    FlashTcArgs m;
    m.out = a.out; m.o_tok_stride = (size_t)a.ld_o; m.o_head_stride = (size_t)HD; m.out_hi = nullptr; m.out_lo = nullptr;
    m.Sq = a.n; m.Skv = S; m.q0 = a.t0; m.groups = 1; m.scaling = a.scale; m.window = a.window;
    if (a.sink) { m.sink = 1; m.sink_logit = a.sink; }
    static bool attr = false;      // (the instances the library's start-up does not know)
    if (!attr) { AHA_CUDA_CHECK(cudaFuncSetAttribute(flash_attn_tc_kernel<HD, true, WIN, HDQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)flash_tc_smem_bytes<HD, HDQ>())); attr = true; }
    flash_attn_tc_kernel<HD, true, WIN, HDQ><<<dim3(ceil_div(a.n, kFaBQ), H), kFaThreads, flash_tc_smem_bytes<HD, HDQ>(), st>>>(tqh, tql, tkh, tkl, tvh, tvl, m);
    AHA_CUDA_CHECK(cudaGetLastError());
}

// a: as for latent_flash (the entry's queries, the expanded keys / values of positions 0 .. S - 1).  A sliding window or a sink runs the
// kernel's windowed instances (window 0: every earlier key).  Returns the launches.
inline int latent_flash_tc(cudaStream_t st, const LatentFlashArgs& a, int H, __half* ws) {
    const int S = a.pos0 + a.n, HDQ = latent_flash_tc_hdq(a.D, a.R, a.Dv);
    if (a.window > 0 || a.sink) {
        if (a.Dv == 128) { if (HDQ == 128) latent_flash_tc_launch<128, 128, true>(st, a, H, S, ws); else latent_flash_tc_launch<128, 192, true>(st, a, H, S, ws); }
        else { if (HDQ == 64) latent_flash_tc_launch<64, 64, true>(st, a, H, S, ws); else latent_flash_tc_launch<64, 128, true>(st, a, H, S, ws); }
        return 2;
    }
    if (a.Dv == 128) { if (HDQ == 128) latent_flash_tc_launch<128, 128, false>(st, a, H, S, ws); else latent_flash_tc_launch<128, 192, false>(st, a, H, S, ws); }
    else { if (HDQ == 64) latent_flash_tc_launch<64, 64, false>(st, a, H, S, ws); else latent_flash_tc_launch<64, 128, false>(st, a, H, S, ws); }
    return 2;
}

}  // namespace aha
