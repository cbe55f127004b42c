// seq_engine.cu -- the layered sequence engine (see seq_engine.h): a model is a list of layers read from config.json, each a mixer and
// an optional feed-forward inside one of three layer templates (chosen by the config's "architecture"):
//     post-norm   x += norm1(mixer(x));   x += norm2(ff(x))                      norms with ONE scalar gain on the sublayer outputs
//     sandwich    x += m * norm1b(mixer(u)),  u = h + conv1(h),  h = norm1(x)    and the same around the feed-forward: RMS norms in groups with a
//                 gain per channel before AND after each sublayer, a short causal convolution over time on what the sublayer reads (its last
//                 inputs are state of the sequence), a residual multiplier m; a span of layers may run several times in a row with the same
//                 weights ("loop"), every pass with a state of its own and a learned vector added to the stream before it
//     parallel    x += mixer(h) + ff(h),  h = norm1(x)                           ONE norm (gain stored as an offset from one) whose output both sublayers
//                 read; a learned position vector joins the scaled embedding; in a loop the embedding output is added to the stream again
//                 before every pass but the first
// run by ONE ragged step function: the tokens of all entries of a step are packed into [T, width] fp32 rows, every Linear is one
// GEMM over all rows, and the mixers' sequence kernels (recurrence.cuh, attention_window.cuh) take the RaggedBatch description.
// Mixers and feed-forwards are looked up by name in a registry, each with its sizes and constants read from its config entry:
//     "hgrn2"      gated linear recurrence, matrix state per head in the slot pool            (recurrence.cuh)
//     "attention"  windowed softmax attention with a linear distance penalty, q/k/v bias, short convolution, whole-projection
//                  q/k norm, sigmoid output gate, optional reuse of an earlier layer's cache     (attention_window.cuh)
//     "dense"      W_down xIELU(W_up x)
//     "gla"        gated linear attention: keyed diagonal recurrence, decay from a low-rank projection                (recurrence.cuh, ssm.cuh)
//     "mamba2"     selective state space: convolved x / B / C, scalar decay per head, gate before a grouped norm        (recurrence.cuh, ssm.cuh)
//     "latent_attention"  softmax attention over one cached latent + one rotated key part per token (YaRN rotary)       (attention_latent.cuh)
//     "moe"        gated experts chosen by a table row of the token id, grouped matrix products                         (moe_table.cuh)
// A design may bind a name to a variant of its own ("<architecture>:<name>" is looked up first).  The Lupolorn design (sandwich template
// without convolution or groups, the embedding table also the output projection) has
//     "mingru"     elementwise gated recurrence, one fp32 per channel and sequence in the slot pool                      (recurrence_elem.cuh)
//     "attention"  causal attention with rotary positions (frequencies rescaled band by band), unit-RMS queries and keys, a softmax
//                  whose denominator holds an extra 1, one sigmoid gate per head                                          (attention_window.cuh)
//     "latent_attention"  as above without a rotated part: queries through a normed latent of their own, a sliding window
//     "dense"      W_down relu(W_up x)^2
//     "moe"        softmax router, the `top` best scores weigh their experts unrenormalised, a shared expert behind a sigmoid gate  (moe_router.cuh)
// The Gomerax design (parallel template, the embedding table also the output projection) has
//     "latent_attention"  as above with a query latent, a rotated part (plain rotary frequencies), a sliding window and a learned sink per head in
//                  the softmax denominator
//     "dense"      W_down (silu(W_gate h) * W_up h), biases on all three
//     "moe"        softmax router; a learned correction enters the choice only, experts are chosen from the best groups of neighbours, weights are
//                  renormalised over the chosen experts and scaled; experts and the shared expert are clamped gated units      (moe_router.cuh)
// Memory: one free list of 32-token pages serves every layer that owns keys / values (K pages [page][G][32][D], V pages
// [page][G][32][Dv], fp32); a sequence additionally owns a state slot (recurrent states, convolution tails, sampler state).
// Precision: the residual stream, norms, gates, recurrent state, scores and softmax are fp32 in both modes; the Linear layers
// multiply bf16 weights (serving mode) or the same values widened to fp32 (exact mode) with fp32 accumulation.
#include "seq_engine.h"

#include <algorithm>
#include <functional>
#include <memory>

#include "attention_latent_tc.cuh"
#include "attention_tc.cuh"
#include "attention_window.cuh"
#include "gemm_any.cuh"
#include "gemm_tc.cuh"
#include "json.hpp"
#include "kernels_common.cuh"
#include "moe_router.cuh"
#include "moe_table.cuh"
#include "norm_group.cuh"
#include "recurrence.cuh"
#include "recurrence_elem.cuh"
#include "runtime.cuh"
#include "sampling.cuh"
#include "ssm.cuh"

namespace aha {
namespace {

inline double softplus_d(double z) { return std::log1p(std::exp(-std::fabs(z))) + std::max(z, 0.0); }

struct LinearAny {
    void* w = nullptr;    // [N, K] bf16 or fp32
    float* b = nullptr;   // [N] or nullptr
    int N = 0, K = 0;
    CUtensorMap tmap, tmap256;   // TMA descriptors of the bf16 matrix for the tcgen05 kernels (128- and 256-row boxes), built on first use
    bool has_tmap = false, has_tmap256 = false;
};

constexpr int kTcMinRows = 32;    // fewer rows than this run on the CUDA cores (a 128-row tensor-core tile would be mostly padding)
constexpr int kGraphMaxTokens = 8;   // launches of at most this many tokens (decode steps) are replayed from CUDA graphs
constexpr int kLatentExpandMinTokens = 32;   // a prompt portion of at least this many tokens runs latent attention over expanded keys / values
constexpr int kTcAttnMinTokens = 32; // a prompt portion of at least this many tokens runs its attention on the tcgen05 flash kernel (serving mode, head size 64 / 128)

struct Engine;

// What a sublayer sees of a step: the packed rows and the engine's scratch.
struct StepView {
    Engine* eng;
    RaggedBatch rb;
    const float* x;     // [T, width] sublayer input (the residual stream)
    float* y;           // [T, width] sublayer output (before its norm)
    const int* h_ent_start;   // host copies of rb.ent_start / ent_pos0 / ent_slot
    const int* h_ent_pos0;
    const int* h_ent_slot;
    int span;           // a power of two >= the tokens the longest sequence of the step holds after it (part of a replayed graph's key)
};

struct Sublayer {
    virtual ~Sublayer() {}
    virtual void run(const StepView& v) = 0;
    virtual int proj_cols() const = 0;     // widest intermediate row this sublayer needs in Engine::proj
    virtual int inner_cols() const = 0;    // ... in Engine::inner
    virtual int q_cols() const { return 0; }
    virtual size_t attn_part_floats() const { return 0; }     // workspace of the split attention launches
    virtual size_t seg_state_floats() const { return 0; }     // scratch of a recurrence that cuts long prompt portions into segments: states,
    virtual size_t seg_decay_floats() const { return 0; }     // ... and the segments' decay products
    virtual uint64_t kv_bytes_per_token() const { return 0; }
    virtual size_t route_ints() const { return 0; }           // integer scratch of a routed feed-forward
    virtual size_t expand_gather_floats() const { return 0; } // latent attention's prompt path: a sequence's cached rows, dense,
    virtual size_t expand_kv_floats() const { return 0; }     // ... its expanded keys and values,
    virtual size_t expand_out_floats() const { return 0; }    // ... the attention output of a step
    virtual size_t expand_split_halfs() const { return 0; }   // ... and the 16-bit halves of the rows that are expanded on the tensor cores
};

struct Engine final : SeqEngine {
    Ctx& c;
    SeqEngineOptions opt;
    int W = 0, V = 0, L = 0;
    float eps = 1e-6f;
    bool fp32 = false;
    // weights
    void* embed = nullptr;
    LinearAny head;
    float* final_gain = nullptr;
    // one RUN of a layer: a layer inside a loop appears once per pass, with the same weights and its own mixer object (state, cache)
    struct LayerRec {
        std::unique_ptr<Sublayer> mixer, ff;
        float *gain1 = nullptr, *gain2 = nullptr;                   // post-norm template: scalar gains
        float *pre1 = nullptr, *pre2 = nullptr, *post1 = nullptr, *post2 = nullptr;   // sandwich template: [W] gains before / after the sublayers
        float *conv1 = nullptr, *conv2 = nullptr;                   // [W, taps] input convolutions
        float *tails1 = nullptr, *tails2 = nullptr;                 // [slots][taps - 1][W] their state, per run
        int pass = -1;                                              // >= 0: the run opens this pass of the loop (loop_step row added first)
        bool reinject = false;                                      // parallel template: the run opens a pass after the first, the embedding output is added first
    };
    std::vector<LayerRec> layers;
    bool sandwich = false;
    bool parallel = false;         // the parallel template (one norm per layer, both sublayers read it, their outputs are summed into the stream)
    float gain_offset = 0.f;       // norm gains are stored as offsets from this number
    float* pos_table = nullptr; int max_positions = 0;   // [max_positions, W] learned position rows added to the embedding
    float* x0 = nullptr;           // [T, W] the embedding output of the step, kept for the passes of a loop that add it again
    float* y2 = nullptr;           // [T, W] parallel template: the feed-forward's output beside the mixer's
    std::string design;            // config.json's "architecture", lower case
    int norm_groups = 1, conv_taps = 0;
    float resid_mult = 1.f, embed_scale = 1.f, logit_scale = 1.f;
    float* final_w = nullptr;      // sandwich: [W] gain of the final norm
    float* loop_step = nullptr;    // [passes, W]
    float *hnorm = nullptr, *hin = nullptr;   // [T, W] normed rows, sublayer input
    // a sublayer may leave its output as `out_rows` rows per token that are still to be summed and scaled (a token's experts in decode steps):
    // the norm + residual kernel that follows does it on the way
    const float* out_src = nullptr; int out_rows = 1; float out_scale = 1.f;
    int* route_buf = nullptr;
    float *lat_gather = nullptr, *lat_kv = nullptr, *lat_out = nullptr;   // latent attention scratch (see Sublayer::expand_*)
    // weights that several runs share are loaded once
    std::map<std::string, LinearAny> lin_cache;
    std::map<std::string, float*> vec_cache;
    std::map<std::string, int*> int_cache;
    float* vec(const WeightTable& wt, const std::string& name, size_t n) {
        auto it = vec_cache.find(name);
        if (it != vec_cache.end()) return it->second;
        return vec_cache[name] = upload_vec(c, wt, name, n);
    }
    // a norm gain as the kernels apply it: gain_offset + the stored vector
    float* gain_vec(const WeightTable& wt, const std::string& name, size_t n) {
        if (gain_offset == 0.f) return vec(wt, name, n);
        const std::string key = name + " (+offset)";
        auto it = vec_cache.find(key);
        if (it != vec_cache.end()) return it->second;
        std::vector<float> v = wt.vec_f32(name, n);
        for (auto& g : v) g += gain_offset;
        return vec_cache[key] = upload(c, v);
    }
    std::vector<Sublayer*> mixer_of_layer;   // for kv_from lookups while building
    uint64_t wbytes = 0;
    // pools
    int num_pages = 0, max_pages = 0, slots = 0;
    std::vector<int> free_pages;
    std::vector<std::vector<int>> h_tables;   // [slot][mapped pages]
    int* d_tables = nullptr;
    struct Seq { bool live = false; int pos = 0; bool samp_active = false; SampleArgs samp{}; int samp_epoch = 0; };
    std::vector<Seq> seqs;
    // step scratch
    int Tmax = 0, Rmax = 0;
    float *x = nullptr, *y = nullptr, *proj = nullptr, *inner = nullptr, *qbuf = nullptr, *hn = nullptr, *logits = nullptr, *attn_part = nullptr, *seg_state = nullptr, *seg_decay = nullptr;
    int* d_meta = nullptr; int* h_meta = nullptr; size_t meta_ints = 0;
    cudaEvent_t ev_meta = nullptr; bool meta_pending = false;
    // sampler state per slot
    DecodeState* d_states = nullptr; uint32_t* d_hist = nullptr; int hist_cap = 0; uint32_t* d_tok = nullptr;
    float *pmax = nullptr, *sample_work = nullptr; int* pidx = nullptr; int* d_sample_err = nullptr; int n_pcand = 64;
    // trace
    bool trace = false; float* trace_buf = nullptr; int trace_T = 0;

    // per-family device timing of a step (profile()): CUDA events around every launch family, summed over the layers
    struct Prof { double ms = 0, flops = 0, bytes = 0; int launches = 0; };
    bool profiling = false;
    std::map<std::string, Prof> prof;
    std::vector<cudaEvent_t> prof_ev;
    struct ProfSpan { std::string name; size_t ev; double flops, bytes; };
    std::vector<ProfSpan> prof_spans;
    void tic(const char* name, double flops, double bytes) {
        if (!profiling) return;
        const size_t i = 2 * prof_spans.size();
        while (prof_ev.size() < i + 2) { cudaEvent_t e; AHA_CUDA_CHECK(cudaEventCreate(&e)); prof_ev.push_back(e); }
        AHA_CUDA_CHECK(cudaEventRecord(prof_ev[i], c.stream));
        prof_spans.push_back({name, i, flops, bytes});
    }
    void toc() { if (profiling) AHA_CUDA_CHECK(cudaEventRecord(prof_ev[prof_spans.back().ev + 1], c.stream)); }
    void prof_collect() {
        AHA_CUDA_CHECK(cudaStreamSynchronize(c.stream));
        for (auto& sp : prof_spans) {
            float ms = 0.f;
            AHA_CUDA_CHECK(cudaEventElapsedTime(&ms, prof_ev[sp.ev], prof_ev[sp.ev + 1]));
            Prof& p = prof[sp.name];
            p.ms += ms; p.flops += sp.flops; p.bytes += sp.bytes; p.launches += 1;
        }
        prof_spans.clear();
    }

    int sampler_epochs = 0;
    Engine(Ctx& ctx, const SeqEngineOptions& o) : c(ctx), opt(o) {}
    ~Engine() override { clear_graphs(); for (auto e : prof_ev) cudaEventDestroy(e); if (h_meta) cudaFreeHost(h_meta); if (ev_meta) cudaEventDestroy(ev_meta); }

    // ---------------------------------------------------------------- weights
    // rows of several [N_i, K] tensors stacked into one matrix in the engine's storage type; absent bias parts are zeros
    // pad_to > 1: zero rows are appended until N is a multiple of it (so that the tensor-core kernels take the matrix)
    LinearAny load_linear(const WeightTable& wt, const std::vector<std::string>& names, const std::vector<int>& rows, int K, const std::vector<std::string>& biases, int pad_to = 1) {
        std::string key = std::to_string(pad_to) + "|";
        for (auto& nm : names) key += nm + "|";
        auto hit = lin_cache.find(key);
        if (hit != lin_cache.end()) return hit->second;
        LinearAny Lw = load_linear_uncached(wt, names, rows, K, biases, pad_to);
        lin_cache[key] = Lw;
        return Lw;
    }
    LinearAny load_linear_uncached(const WeightTable& wt, const std::vector<std::string>& names, const std::vector<int>& rows, int K, const std::vector<std::string>& biases, int pad_to) {
        LinearAny Lw;
        Lw.K = K;
        for (int r : rows) Lw.N += r;
        Lw.N = (Lw.N + pad_to - 1) / pad_to * pad_to;
        const size_t n = (size_t)Lw.N * K;
        bool any_bias = false;
        for (auto& b : biases) any_bias = any_bias || (!b.empty() && wt.has(b));
        if (fp32) {
            std::vector<float> st(n, 0.f);
            size_t o = 0;
            for (size_t i = 0; i < names.size(); ++i) {
                wt.expect(names[i], {rows[i], K});
                const aha_tensor_desc& d = wt.get(names[i]);
                const size_t ne = (size_t)rows[i] * K;
                if (d.dtype == AHA_BF16) { const uint16_t* s = reinterpret_cast<const uint16_t*>(d.data); for (size_t k = 0; k < ne; ++k) st[o + k] = bf16_bits_to_float(s[k]); }
                else for (size_t k = 0; k < ne; ++k) st[o + k] = WeightTable::at(d, k);
                o += ne;
            }
            Lw.w = upload(c, st);
        } else {
            std::vector<uint16_t> st(n, 0);
            size_t o = 0;
            for (size_t i = 0; i < names.size(); ++i) {
                wt.expect(names[i], {rows[i], K});
                const aha_tensor_desc& d = wt.get(names[i]);
                const size_t ne = (size_t)rows[i] * K;
                if (d.dtype == AHA_BF16) std::memcpy(st.data() + o, d.data, ne * 2);
                else for (size_t k = 0; k < ne; ++k) {   // round to nearest even
                    float f = WeightTable::at(d, k); uint32_t u; std::memcpy(&u, &f, 4);
                    st[o + k] = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
                }
                o += ne;
            }
            Lw.w = upload(c, st);
        }
        if (any_bias) {
            std::vector<float> b((size_t)Lw.N, 0.f);
            size_t o = 0;
            for (size_t i = 0; i < names.size(); ++i) {
                if (i < biases.size() && !biases[i].empty() && wt.has(biases[i])) { auto v = wt.vec_f32(biases[i], rows[i]); std::copy(v.begin(), v.end(), b.begin() + o); }
                o += rows[i];
            }
            Lw.b = upload(c, b);
        }
        return Lw;
    }
    // A matrix [N, K] in the engine's storage type whose row n is row src[n].second of tensor src[n].first ([., K]): stacks, interleavings.
    // bias_src (optional, one entry per row): element .second of vector .first is the row's bias
    LinearAny load_rows(const WeightTable& wt, const std::string& key, const std::vector<std::pair<const aha_tensor_desc*, int>>& src, int K,
                        const std::vector<std::pair<const aha_tensor_desc*, int>>* bias_src = nullptr) {
        auto hit = lin_cache.find(key);
        if (hit != lin_cache.end()) return hit->second;
        LinearAny Lw;
        Lw.K = K; Lw.N = (int)src.size();
        const size_t esz = fp32 ? 4 : 2;
        std::vector<uint8_t> st((size_t)Lw.N * K * esz);
        for (size_t n = 0; n < src.size(); ++n) {
            const aha_tensor_desc& d = *src[n].first;
            const size_t base = (size_t)src[n].second * K;
            AHA_REQUIRE(base + K <= WeightTable::numel(d), std::string("weight '") + (d.name ? d.name : "?") + "' is smaller than the config says");
            if (fp32) {
                float* o = reinterpret_cast<float*>(st.data()) + n * K;
                for (int k = 0; k < K; ++k) o[k] = WeightTable::at(d, base + k);
            } else {
                uint16_t* o = reinterpret_cast<uint16_t*>(st.data()) + n * K;
                if (d.dtype == AHA_BF16) std::memcpy(o, reinterpret_cast<const uint16_t*>(d.data) + base, (size_t)K * 2);
                else for (int k = 0; k < K; ++k) { float f = WeightTable::at(d, base + k); uint32_t u; std::memcpy(&u, &f, 4); o[k] = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16); }
            }
        }
        Lw.w = upload(c, st);
        if (bias_src) {
            AHA_REQUIRE(bias_src->size() == src.size(), "load_rows: one bias entry per row");
            std::vector<float> b(src.size());
            for (size_t n = 0; n < src.size(); ++n) {
                const aha_tensor_desc& d = *(*bias_src)[n].first;
                AHA_REQUIRE((size_t)(*bias_src)[n].second < WeightTable::numel(d), std::string("bias '") + (d.name ? d.name : "?") + "' is smaller than the config says");
                b[n] = WeightTable::at(d, (size_t)(*bias_src)[n].second);
            }
            Lw.b = upload(c, b);
        }
        lin_cache[key] = Lw;
        return Lw;
    }
    // batched / grouped products on the CUDA cores (gemm_any.cuh): g carries the batch description, the weights' type is the engine's
    void gemm_batched(const char* family, int epi, GemmAnyArgs g, double flops, double bytes) {
        tic(family, flops, bytes);
        gemm_any(c.stream, epi, fp32, g, c.num_sms);
        c.cnt.kernels++;
        toc();
    }
    // y = epilogue(x W^T + b).  Serving mode with enough rows and a shape that tiles: the library's tcgen05 kernels on bf16 operands -- the
    // fp32 activations are split into bf16 hi + lo halves (16 significant bits), W is the bf16 checkpoint matrix, accumulation is fp32 in
    // TMEM.  Otherwise (exact mode, decode steps, odd sizes): the CUDA-core kernels of gemm_any.cuh.
    bool on_tensor_cores(int M, const LinearAny& Wt, int lda, int ldc) const {
        return !fp32 && opt.gemm_impl != 1 && M >= kTcMinRows && gemm_tc_supported(M, Wt.N, Wt.K) && lda % 4 == 0 && ldc % 4 == 0;
    }
    void gemm(int epi, const float* A, int lda, LinearAny& Wt, float* C, int ldc, int M, float a0 = 0.f, float a1 = 0.f) {
        tic(on_tensor_cores(M, Wt, lda, ldc) ? "linear (tcgen05, bf16 hi+lo)" : (M <= 8 ? "linear (decode rows, weights streamed once)" : "linear (CUDA cores)"),
            2.0 * M * Wt.N * Wt.K, (double)Wt.N * Wt.K * (fp32 ? 4 : 2) + 4.0 * M * (Wt.K + Wt.N));
        gemm_dispatch(epi, A, lda, Wt, C, ldc, M, a0, a1);
        toc();
    }
    void gemm_dispatch(int epi, const float* A, int lda, LinearAny& Wt, float* C, int ldc, int M, float a0, float a1) {
        if (on_tensor_cores(M, Wt, lda, ldc)) {
            const size_t halfs = (size_t)M * Wt.K;
            __half* hi = c.split_buf(halfs);
            __half* lo = hi + c.split_cap;
            split_f32_to_bf16x2_kernel<<<(unsigned)((halfs / 4 + 255) / 256), 256, 0, c.stream>>>(A, lda, reinterpret_cast<__nv_bfloat16*>(hi), reinterpret_cast<__nv_bfloat16*>(lo), M, Wt.K);
            c.cnt.kernels++;
            if (!Wt.has_tmap) { Wt.tmap = make_tmap_f16(Wt.w, (uint64_t)Wt.N, (uint64_t)Wt.K); Wt.has_tmap = true; }   // 16-bit elements: the copy is bitwise
            GemmTcArgs t{};
            t.bias = Wt.b; t.resid = nullptr; t.ldr = 0; t.C = C; t.ldc = ldc; t.M = M; t.N = Wt.N; t.K = Wt.K;
            t.act = epi == AEPI_XIELU ? ACT_XIELU : (epi == AEPI_RELU2 ? ACT_RELU2 : (epi == AEPI_CLAMP_GLU ? ACT_CLAMP_GLU : ACT_NONE));
            t.act_a = a0; t.act_b = a1; t.bf16 = 1; t.group_m = std::max(1, c.gemm_group_m);
            const int e = (epi == AEPI_XIELU || epi == AEPI_RELU2) ? EPI_ACT : ((epi == AEPI_SWIGLU || epi == AEPI_CLAMP_GLU) ? EPI_SWIGLU : EPI_STORE);
            if (c.gemm_pair && Wt.N >= 256 && M >= 1024) gemm_tc3_launch(c.stream, e, hi, lo, Wt.tmap, t, c.num_sms);
            else if (c.gemm_wide && Wt.N >= 256) {
                if (!Wt.has_tmap256) { Wt.tmap256 = make_tmap_f16_rows(Wt.w, (uint64_t)Wt.N, (uint64_t)Wt.K, 256); Wt.has_tmap256 = true; }
                gemm_tc2_launch(c.stream, e, hi, lo, Wt.tmap256, t, c.num_sms);
            } else gemm_tc_launch(c.stream, e, hi, lo, Wt.tmap, t);
            c.cnt.kernels++;
            return;
        }
        GemmAnyArgs g{};
        g.A = A; g.lda = lda; g.W = Wt.w; g.bias = Wt.b; g.C = C; g.ldc = ldc; g.M = M; g.N = Wt.N; g.K = Wt.K; g.act_a = a0; g.act_b = a1;
        gemm_any(c.stream, epi, fp32, g, c.num_sms);
        c.cnt.kernels++;
    }

    // ---------------------------------------------------------------- SeqEngine
    int vocab() const override { return V; }
    int max_seqs() const override { return slots; }
    int page_tokens() const override { return kPage; }
    size_t free_tokens() const override { return free_pages.size() * (size_t)kPage; }
    uint64_t weight_bytes() const override { return wbytes; }
    uint64_t kv_bytes_per_token() const override { uint64_t b = 0; for (auto& l : layers) b += l.mixer->kv_bytes_per_token(); return b; }
    bool live(int slot) const override { return slot >= 0 && slot < slots && seqs[slot].live; }
    int position(int slot) const override { AHA_REQUIRE(live(slot), "sequence slot is not live"); return seqs[slot].pos; }
    int admit() override {
        for (int s = 0; s < slots; ++s)
            if (!seqs[s].live) { seqs[s] = Seq{}; seqs[s].live = true; return s; }
        throw std::runtime_error("aha_b200: all " + std::to_string(slots) + " sequence slots are live");
    }
    void release(int slot) override {
        AHA_REQUIRE(live(slot), "sequence slot is not live");
        for (int p : h_tables[slot]) free_pages.push_back(p);
        h_tables[slot].clear();
        seqs[slot] = Seq{};
    }
    void release_all() override { for (int s = 0; s < slots; ++s) if (seqs[s].live) release(s); }
    void set_sampler(int slot, const aha_gen_params& p) override {
        AHA_REQUIRE(live(slot), "sequence slot is not live");
        Seq& q = seqs[slot];
        q.samp_epoch = ++sampler_epochs;
        const int mode = sampling_mode(p);
        const bool pen = !(p.repeat_penalty == 1.0f || p.repeat_last_n == 0);
        q.samp_active = mode != SAMPLE_ARGMAX || pen;
        DecodeState st{};
        AHA_CUDA_CHECK(cudaMemcpyAsync(d_states + slot, &st, sizeof(st), cudaMemcpyHostToDevice, c.stream));
        AHA_CUDA_CHECK(cudaStreamSynchronize(c.stream));   // `st` is a stack temporary
        if (!q.samp_active) return;
        AHA_REQUIRE(V <= kSampleThreads * kSampleChunk, "vocabulary too large for the device sampler");
        AHA_REQUIRE(!(mode == SAMPLE_TOPK || mode == SAMPLE_TOPK_TOPP) || p.top_k >= V || p.top_k <= kSampleMaxTopK, "top_k > 1024 is not supported by the device sampler");
        SampleArgs a{};
        a.work = sample_work; a.V = V; a.mode = mode;
        a.inv_temp = mode == SAMPLE_ARGMAX ? 1.0f : (float)(1.0 / (double)p.temperature);
        a.top_p = p.top_p; a.top_k = p.top_k; a.penalty = p.repeat_penalty; a.last_n = p.repeat_last_n;
        sampler_key_from_seed(p.seed, a.key);
        a.st = d_states + slot; a.history = d_hist + (size_t)slot * hist_cap; a.hist_cap = hist_cap; a.token_out = d_tok + slot; a.error = d_sample_err;
        a.overwrite = 1;
        q.samp = a;
    }
    void set_trace(bool on) override {
        if (on && !trace_buf) trace_buf = c.alloc<float>((size_t)L * Tmax * W);
        trace = on;
    }
    size_t read_trace(int layer, float* out, size_t cap) override {
        AHA_REQUIRE(trace_buf && layer >= 0 && layer < L, "no trace recorded for this layer");
        const size_t n = (size_t)trace_T * W;
        AHA_REQUIRE(cap >= n, "trace buffer too small");
        AHA_CUDA_CHECK(cudaStreamSynchronize(c.stream));
        AHA_CUDA_CHECK(cudaMemcpy(out, trace_buf + (size_t)layer * Tmax * W, n * sizeof(float), cudaMemcpyDeviceToHost));
        return n;
    }

    // ---------------------------------------------------------------- the step
    struct Piece { int ent, off, cnt; };

    void step(const SeqStepEntry* ents, int n, float* logits_out, uint32_t* tokens_out) override {
        AHA_REQUIRE(n >= 1 && ents, "step: no entries");
        std::vector<char> seen(slots, 0);
        std::vector<size_t> row_base(n + 1, 0);
        for (int i = 0; i < n; ++i) {
            const SeqStepEntry& e = ents[i];
            AHA_REQUIRE(live(e.slot), "step: entry names a slot that is not live");
            AHA_REQUIRE(!seen[e.slot], "step: a sequence appears twice in one step");
            seen[e.slot] = 1;
            AHA_REQUIRE(e.n >= 1, "step: an entry brings no tokens");
            AHA_REQUIRE(e.tokens || e.n == 1, "step: a fed-back token is a single token");
            for (int k = 0; k < e.n_want; ++k) AHA_REQUIRE(e.want[k] >= 0 && e.want[k] < e.n && (k == 0 || e.want[k] > e.want[k - 1]), "step: `want` must be ascending indices into the entry's tokens");
            if (e.tokens) for (int k = 0; k < e.n; ++k) AHA_REQUIRE(e.tokens[k] < (uint32_t)V, "step: token id outside the vocabulary");
            row_base[i + 1] = row_base[i] + (size_t)e.n_want;
        }
        // the scheduler's cut: launches of at most Tmax packed tokens; an entry that does not fit goes on in the next launch
        std::vector<Piece> cur;
        int used = 0;
        for (int i = 0; i < n; ++i) {
            int off = 0;
            while (off < ents[i].n) {
                if (used == Tmax) { launch(ents, cur, row_base, logits_out); cur.clear(); used = 0; }
                const int cnt = std::min(ents[i].n - off, Tmax - used);
                cur.push_back({i, off, cnt});
                used += cnt; off += cnt;
            }
        }
        if (!cur.empty()) launch(ents, cur, row_base, logits_out);
        if (tokens_out) {
            std::vector<uint32_t> h(slots);
            AHA_CUDA_CHECK(cudaMemcpyAsync(h.data(), d_tok, slots * sizeof(uint32_t), cudaMemcpyDeviceToHost, c.stream));
            AHA_CUDA_CHECK(cudaStreamSynchronize(c.stream));
            for (int i = 0; i < n; ++i) tokens_out[i] = ents[i].sample ? h[ents[i].slot] : 0u;
            int err = 0;
            AHA_CUDA_CHECK(cudaMemcpy(&err, d_sample_err, sizeof(int), cudaMemcpyDeviceToHost));
            if (err) { cudaMemset(d_sample_err, 0, sizeof(int)); throw std::runtime_error("sampler: the token weights are all zero or not finite"); }
        } else if (logits_out) {
            AHA_CUDA_CHECK(cudaStreamSynchronize(c.stream));
        }
    }

    void map_pages(int slot, int n_tokens) {
        const int need = ceil_div(n_tokens, kPage);
        std::vector<int>& tb = h_tables[slot];
        const int first = (int)tb.size();
        if (need <= first) return;
        AHA_REQUIRE((size_t)(need - first) <= free_pages.size(), "the KV pool is exhausted: " + std::to_string(num_pages * kPage) + " tokens are held by live sequences");
        while ((int)tb.size() < need) { tb.push_back(free_pages.back()); free_pages.pop_back(); }
        AHA_CUDA_CHECK(cudaMemcpyAsync(d_tables + (size_t)slot * max_pages + first, tb.data() + first, (size_t)(need - first) * sizeof(int), cudaMemcpyHostToDevice, c.stream));
        AHA_CUDA_CHECK(cudaStreamSynchronize(c.stream));   // pageable source
    }

    void launch(const SeqStepEntry* ents, const std::vector<Piece>& pieces, const std::vector<size_t>& row_base, float* logits_out) {
        cudaStream_t st = c.stream;
        const int E = (int)pieces.size();
        int T = 0;
        for (auto& p : pieces) T += p.cnt;
        if (pos_table)
            for (auto& p : pieces) AHA_REQUIRE(seqs[ents[p.ent].slot].pos + p.cnt <= max_positions, "step: a sequence would grow beyond the model's " + std::to_string(max_positions) + " learned positions");
        for (auto& p : pieces) map_pages(ents[p.ent].slot, seqs[ents[p.ent].slot].pos + p.cnt);
        // ---- metadata: tokens | fb_slot | tok_entry | tok_pos | ent_start | ent_pos0 | ent_slot | rows
        if (meta_pending) { AHA_CUDA_CHECK(cudaEventSynchronize(ev_meta)); meta_pending = false; }
        int* hm = h_meta;
        int* tokens = hm; int* fb = tokens + Tmax; int* tok_entry = fb + Tmax; int* tok_pos = tok_entry + Tmax;
        int* ent_start = tok_pos + Tmax; int* ent_pos0 = ent_start + (slots + 1); int* ent_slot = ent_pos0 + slots; int* rows = ent_slot + slots;
        struct OutRow { size_t out; };           // logits_out row of a wanted packed row
        std::vector<size_t> want_out;
        std::vector<int> sample_slots;
        int t = 0, nrows = 0;
        bool any_fb = false;
        for (int i = 0; i < E; ++i) {
            const Piece& p = pieces[i];
            const SeqStepEntry& e = ents[p.ent];
            const int pos0 = seqs[e.slot].pos;
            ent_start[i] = t; ent_pos0[i] = pos0; ent_slot[i] = e.slot;
            for (int k = 0; k < p.cnt; ++k) {
                tokens[t + k] = e.tokens ? (int)e.tokens[p.off + k] : 0;
                fb[t + k] = e.tokens ? -1 : e.slot;
                any_fb = any_fb || !e.tokens;
                tok_entry[t + k] = i; tok_pos[t + k] = pos0 + k;
            }
            for (int k = 0; k < e.n_want; ++k)
                if (e.want[k] >= p.off && e.want[k] < p.off + p.cnt) { rows[nrows++] = t + e.want[k] - p.off; want_out.push_back(row_base[p.ent] + k); }
            t += p.cnt;
        }
        ent_start[E] = T;
        int span = 128;
        for (int i = 0; i < E; ++i) while (span < ent_pos0[i] + (ent_start[i + 1] - ent_start[i])) span *= 2;
        cur_span = span;
        const int n_want_rows = nrows;
        for (int i = 0, tt = 0; i < E; ++i) {     // sampled rows come after the wanted ones
            const Piece& p = pieces[i];
            const SeqStepEntry& e = ents[p.ent];
            tt += p.cnt;
            if (e.sample && p.off + p.cnt == e.n) { rows[nrows++] = tt - 1; sample_slots.push_back(e.slot); }
        }
        AHA_CUDA_CHECK(cudaMemcpyAsync(d_meta, h_meta, meta_ints * sizeof(int), cudaMemcpyHostToDevice, st));
        AHA_CUDA_CHECK(cudaEventRecord(ev_meta, st));
        meta_pending = true;
        int* dm = d_meta;
        RaggedBatch rb;
        rb.T = T; rb.E = E;
        rb.tokens = reinterpret_cast<const uint32_t*>(dm);
        const int* d_fb = dm + Tmax;
        rb.tok_entry = dm + 2 * Tmax; rb.tok_pos = dm + 3 * Tmax;
        rb.ent_start = dm + 4 * Tmax; rb.ent_pos0 = rb.ent_start + (slots + 1); rb.ent_slot = rb.ent_pos0 + slots;
        const int* d_rows = rb.ent_slot + slots;
        rb.page_tables = d_tables; rb.max_pages = max_pages;
        // ---- device work.  Decode-sized launches are replayed from a CUDA graph keyed by everything the launch arguments depend on.
        const bool graphable = opt.use_graph && !trace && !profiling && T <= kGraphMaxTokens && nrows <= Rmax;
        if (graphable) {
            std::vector<int> key{T, E, n_want_rows, any_fb ? 1 : 0, span};
            for (int sl : sample_slots) { key.push_back(sl); key.push_back(seqs[sl].samp_epoch); }
            StepGraph* g = nullptr;
            for (auto& e : graphs) if (e.key == key) { g = &e; break; }
            if (!g) {
                if (graphs.size() >= 64) clear_graphs();
                const uint64_t k0 = c.cnt.kernels;
                cudaGraph_t cg = nullptr;
                AHA_CUDA_CHECK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
                try { device_work(rb, d_fb, any_fb, d_rows, nrows, n_want_rows, sample_slots, nullptr, nullptr); }
                catch (...) { cudaStreamEndCapture(st, &cg); if (cg) cudaGraphDestroy(cg); throw; }
                AHA_CUDA_CHECK(cudaStreamEndCapture(st, &cg));
                StepGraph e{key, nullptr, c.cnt.kernels - k0};
                c.cnt.kernels = k0;
                const cudaError_t err = cudaGraphInstantiate(&e.exec, cg, 0);
                cudaGraphDestroy(cg);
                AHA_CUDA_CHECK(err);
                graphs.push_back(e);
                g = &graphs.back();
            }
            AHA_CUDA_CHECK(cudaGraphLaunch(g->exec, st));
            c.cnt.graphs++; c.cnt.kernels += g->kernels;
            if (logits_out)
                for (int r = 0; r < n_want_rows; ++r)
                    AHA_CUDA_CHECK(cudaMemcpyAsync(logits_out + want_out[r] * (size_t)V, logits + (size_t)r * V, (size_t)V * sizeof(float), cudaMemcpyDeviceToHost, st));
        } else {
            device_work(rb, d_fb, any_fb, d_rows, nrows, n_want_rows, sample_slots, logits_out, &want_out);
        }
        for (auto& p : pieces) seqs[ents[p.ent].slot].pos += p.cnt;
    }

    int cur_span = 128;
    struct StepGraph { std::vector<int> key; cudaGraphExec_t exec; uint64_t kernels; };
    std::vector<StepGraph> graphs;
    void clear_graphs() { for (auto& g : graphs) if (g.exec) cudaGraphExecDestroy(g.exec); graphs.clear(); }

    // embed -> layers -> final norm + head (+ sampler) for `nrows` gathered rows.  want_out == nullptr (graph capture): no copies to the host and a
    // single head chunk; else the wanted rows are copied out chunk by chunk.
    void device_work(const RaggedBatch& rb, const int* d_fb, bool any_fb, const int* d_rows, int nrows, int n_want_rows, const std::vector<int>& sample_slots,
                     float* logits_out, const std::vector<size_t>* want_out) {
        cudaStream_t st = c.stream;
        const int T = rb.T;
        pre_ready = nullptr; mix_pending = false;
        if (any_fb) { feedback_tokens_kernel<<<ceil_div(T, 256), 256, 0, st>>>(reinterpret_cast<uint32_t*>(d_meta), d_fb, d_states, T); c.cnt.kernels++; }
        if (fp32) embed_gather_any_kernel<float><<<T, 128, 0, st>>>(rb.tokens, reinterpret_cast<const float*>(embed), x, W, V, embed_scale, pos_table, rb.tok_pos, max_positions, x0);
        else embed_gather_any_kernel<__nv_bfloat16><<<T, 128, 0, st>>>(rb.tokens, reinterpret_cast<const __nv_bfloat16*>(embed), x, W, V, embed_scale, pos_table, rb.tok_pos, max_positions, x0);
        c.cnt.kernels++;
        const int norm_threads = T <= 8 ? std::min(1024, std::max(256, (W / 2 + 31) / 32 * 32)) : 256;      // a decode step has few blocks: more threads for each
        StepView v{this, rb, x, y, h_meta + 4 * Tmax, h_meta + 4 * Tmax + (slots + 1), h_meta + 4 * Tmax + (slots + 1) + slots, cur_span};
        if (parallel) {      // the first layer's norm; every later one rides with the residual update before it
            tic("norm", 4.0 * T * W, 8.0 * T * W);
            GroupNormArgs n{};
            n.in = x; n.ld_in = W; n.w = layers[0].pre1; n.eps = eps; n.C = W; n.groups = 1; n.out = hnorm; n.ld_out = W;
            group_rmsnorm(st, n, T); c.cnt.kernels++;
            toc();
        }
        for (int l = 0; l < L; ++l) {
            LayerRec& Ly = layers[l];
            if (parallel) {
                v.x = hnorm; v.y = y;
                Ly.mixer->run(v);
                if (Ly.ff) { v.y = y2; Ly.ff->run(v); }
                const LayerRec* nx = l + 1 < L ? &layers[l + 1] : nullptr;
                tic("residual sum + next norm", 6.0 * T * W, (nx ? 20.0 : 12.0) * T * W);
                SumResidualNormArgs a{};
                a.x = x; a.y_a = y; a.eps = eps; a.C = W;
                if (mix_pending) {
                    a.mix_rows = mix.rows; a.mix_top = mix.top; a.mix_w = mix.weights; a.mix_ldw = mix.ld_w; a.mix_shared = mix.shared; a.mix_gate = mix.gate; a.mix_ldg = mix.ld_gate;
                    mix_pending = false;
                } else if (Ly.ff) a.y_b = y2;
                if (trace) a.trace = trace_buf + (size_t)l * Tmax * W;
                if (nx) { a.inject = nx->reinject ? x0 : nullptr; a.w_next = nx->pre1; a.h = hnorm; }
                sum_residual_norm(st, a, T); c.cnt.kernels++;
                toc();
                continue;
            }
            if (sandwich) {
                if (Ly.pass >= 0) {
                    add_row_vector_kernel<<<(unsigned)(((size_t)T * W + 255) / 256), 256, 0, st>>>(x, loop_step + (size_t)Ly.pass * W, W, (size_t)T * W); c.cnt.kernels++;
                }
                // (the norm before a sublayer rides with the residual update before it where nothing stands between the two)
                const LayerRec* nx = l + 1 < L ? &layers[l + 1] : nullptr;
                const float* next_pre = nx && nx->pass < 0 && !nx->conv1 ? nx->pre1 : nullptr;
                v.x = sublayer_input(rb, Ly.pre1, Ly.conv1, Ly.tails1);
                Ly.mixer->run(v);
                sublayer_output(T, Ly.post1, Ly.ff ? (Ly.conv2 ? nullptr : Ly.pre2) : next_pre);
                if (Ly.ff) {
                    v.x = sublayer_input(rb, Ly.pre2, Ly.conv2, Ly.tails2);
                    Ly.ff->run(v);
                    sublayer_output(T, Ly.post2, next_pre);
                }
                if (trace) AHA_CUDA_CHECK(cudaMemcpyAsync(trace_buf + (size_t)l * Tmax * W, x, (size_t)T * W * sizeof(float), cudaMemcpyDeviceToDevice, st));
                continue;
            }
            Ly.mixer->run(v);
            tic("norm + residual", 4.0 * T * W, 12.0 * T * W);
            scalar_rmsnorm_add_kernel<<<T, norm_threads, 0, st>>>(x, y, Ly.gain1, eps, W); c.cnt.kernels++;
            toc();
            if (Ly.ff) {
                Ly.ff->run(v);
                tic("norm + residual", 4.0 * T * W, 12.0 * T * W);
                scalar_rmsnorm_add_kernel<<<T, norm_threads, 0, st>>>(x, y, Ly.gain2, eps, W); c.cnt.kernels++;
                toc();
            }
            if (trace) AHA_CUDA_CHECK(cudaMemcpyAsync(trace_buf + (size_t)l * Tmax * W, x, (size_t)T * W * sizeof(float), cudaMemcpyDeviceToDevice, st));
        }
        trace_T = T;
        AHA_CUDA_CHECK(cudaGetLastError());
        for (int r0 = 0; r0 < nrows; r0 += Rmax) {
            const int nr = std::min(Rmax, nrows - r0);
            if (sandwich || parallel) {
                GroupNormArgs n{};
                n.in = x; n.ld_in = W; n.rows = d_rows + r0; n.w = final_w; n.eps = eps; n.C = W; n.groups = norm_groups; n.out = hn; n.ld_out = W; n.mult = logit_scale;
                group_rmsnorm(st, n, nr);
            } else scalar_rmsnorm_rows_kernel<<<nr, 256, 0, st>>>(x, d_rows + r0, final_gain, eps, hn, W);
            c.cnt.kernels++;
            gemm(AEPI_STORE, hn, W, head, logits, V, nr);
            for (int r = 0; r < nr; ++r) {
                const int gr = r0 + r;
                const float* lg = logits + (size_t)r * V;
                if (gr < n_want_rows) {
                    if (logits_out) AHA_CUDA_CHECK(cudaMemcpyAsync(logits_out + (*want_out)[gr] * (size_t)V, lg, (size_t)V * sizeof(float), cudaMemcpyDeviceToHost, st));
                } else {
                    const int slot = sample_slots[gr - n_want_rows];
                    argmax_partial_kernel<<<n_pcand, 256, 0, st>>>(lg, V, pmax, pidx);
                    argmax_final_kernel<<<1, 32, 0, st>>>(pmax, pidx, n_pcand, d_tok + slot, d_states + slot, d_hist + (size_t)slot * hist_cap, hist_cap, 1);
                    c.cnt.kernels += 2;
                    if (seqs[slot].samp_active) {   // the sampled token replaces the ArgMax one that was just pushed
                        SampleArgs a = seqs[slot].samp;
                        a.logits = lg;
                        sample_kernel<<<1, kSampleThreads, 0, st>>>(a);
                        c.cnt.kernels++;
                    }
                }
            }
            if (r0 + nr < nrows) AHA_CUDA_CHECK(cudaStreamSynchronize(st));   // the logits buffer is reused by the next chunk only after its copies have left
        }
        AHA_CUDA_CHECK(cudaGetLastError());
    }

    // sandwich template: what a sublayer reads, h + conv(h) with h = group norm of the stream.  Decode steps (every entry one token): one launch.
    const float* sublayer_input(const RaggedBatch& rb, const float* gain, const float* conv_w, float* tails) {
        cudaStream_t st = c.stream;
        const int T = rb.T;
        if (pre_ready == gain && !conv_w) { pre_ready = nullptr; return hnorm; }      // formed by the launch that ended the sublayer before
        pre_ready = nullptr;
        const size_t tail_stride = (size_t)std::max(0, conv_taps - 1) * W;
        tic("norm + input convolution", (2.0 * conv_taps + 4.0) * T * W, 4.0 * T * W * (conv_w ? 4.0 : 2.0));
        const float* res;
        if (conv_w && rb.E == T && (size_t)W * sizeof(float) <= 160 * 1024) {
            NormConvArgs a{};
            a.x = x; a.C = W; a.groups = norm_groups; a.w = gain; a.eps = eps; a.taps = conv_taps; a.cw = conv_w; a.tails = tails; a.tail_slot_stride = tail_stride;
            a.out = hin; a.rb = rb;
            static bool attr = false;
            if (!attr) { AHA_CUDA_CHECK(cudaFuncSetAttribute(norm_conv_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)); attr = true; }
            norm_conv_single_kernel<<<T, std::min(1024, std::max(128, (W / 2 + 31) / 32 * 32)), (size_t)W * sizeof(float), st>>>(a);
            c.cnt.kernels++;
            res = hin;
        } else {
            GroupNormArgs n{};
            n.in = x; n.ld_in = W; n.w = gain; n.eps = eps; n.C = W; n.groups = norm_groups; n.out = hnorm; n.ld_out = W;
            group_rmsnorm(st, n, T); c.cnt.kernels++;
            res = hnorm;
            if (conv_w) {
                ShortConvArgs a{};
                a.in = hnorm; a.ld_in = W; a.in_off = 0; a.C = W; a.taps = conv_taps; a.w = conv_w; a.tails = tails; a.tail_slot_stride = tail_stride;
                a.out = hin; a.ld_out = W; a.out_off = 0; a.add_input = 1; a.rb = rb;
                c.cnt.kernels += short_conv(st, a, rb.E == T);
                res = hin;
            }
        }
        AHA_CUDA_CHECK(cudaGetLastError());
        toc();
        return res;
    }
    // ... and what it leaves: x += m * group norm(y) * gain
    const float* pre_ready = nullptr;      // the gain of the pre-norm whose result hnorm already holds
    // routed experts of a decode-sized step may leave their weighted sum to the launch that follows (see PostPreNormArgs::mix_*)
    WeightedCombineArgs mix{}; bool mix_pending = false;
    bool can_defer_mix(int T) const { return parallel || (sandwich && norm_groups == 1 && post_pre_norm_in_registers(W, T)); }
    void sublayer_output(int T, const float* gain, const float* next_pre = nullptr) {
        const bool fuse = next_pre && norm_groups == 1 && !out_src;
        if (mix_pending && !fuse) {          // nothing to ride with (the last sublayer of the model): the combine kernel after all
            moe_weighted_combine_kernel<<<(unsigned)((mix.total + 255) / 256), 256, 0, c.stream>>>(mix);
            c.cnt.kernels++;
            mix_pending = false;
        }
        if (fuse) {
            tic("norm + residual + next norm", 8.0 * T * W, 20.0 * T * W);
            PostPreNormArgs a{};
            a.y = y; a.x = x; a.w_post = gain; a.w_pre = next_pre; a.h = hnorm; a.eps = eps; a.mult = resid_mult; a.C = W;
            if (mix_pending) {
                a.mix_rows = mix.rows; a.mix_top = mix.top; a.mix_w = mix.weights; a.mix_ldw = mix.ld_w; a.mix_shared = mix.shared; a.mix_gate = mix.gate; a.mix_ldg = mix.ld_gate;
                mix_pending = false;
            }
            post_pre_norm(c.stream, a, T);
            c.cnt.kernels++;
            pre_ready = next_pre;
            toc();
            return;
        }
        tic("norm + residual", 4.0 * T * W, 12.0 * T * W);
        GroupNormArgs n{};
        n.in = y; n.ld_in = W; n.w = gain; n.eps = eps; n.C = W; n.groups = norm_groups; n.out = x; n.ld_out = W; n.mult = resid_mult; n.add = 1;
        if (out_src) { n.in = out_src; n.sum_rows = out_rows; n.in_scale = out_scale; out_src = nullptr; }
        group_rmsnorm(c.stream, n, T); c.cnt.kernels++;
        toc();
    }

    int prof_n = 0, prof_tps = 0, prof_ctx = 0;   // shape of the profiled step
    double prof_pairs(int window) const {          // (query, key) pairs an attention layer with this window visits
        double k = 0;
        for (int t = 0; t < prof_tps; ++t) k += window > 0 ? std::min(prof_ctx + t + 1, window) : prof_ctx + t + 1;
        return k * prof_n;
    }
    double prof_unique(int window) const {         // distinct cached positions it reads
        const int all = prof_ctx + prof_tps;
        return (double)prof_n * (window > 0 ? std::min(all, window + prof_tps - 1) : all);
    }

    // Device-timed steps on synthetic tokens: n_seqs sequences, each feeding tokens_per_seq tokens at context ctx (positions are set, the cache holds
    // whatever it holds: timing only).  Leaves every slot free.  Returns JSON.
    std::string profile(int n_seqs, int tokens_per_seq, int ctx, int warmup, int iters) override {
        AHA_REQUIRE(n_seqs >= 1 && n_seqs <= slots && tokens_per_seq >= 1 && ctx >= 0 && iters >= 1, "profile: bad arguments");
        AHA_REQUIRE((size_t)n_seqs * ceil_div(ctx + tokens_per_seq, kPage) <= (size_t)num_pages, "profile: the KV pool is too small for this context");
        release_all();
        std::vector<std::vector<uint32_t>> toks(n_seqs);
        std::vector<SeqStepEntry> ents(n_seqs);
        for (int i = 0; i < n_seqs; ++i) {
            ents[i].slot = admit();
            toks[i].resize(tokens_per_seq);
            for (int k = 0; k < tokens_per_seq; ++k) toks[i][k] = (uint32_t)((i * 7919 + k * 31 + 1) % V);
            ents[i].tokens = toks[i].data(); ents[i].n = tokens_per_seq; ents[i].sample = true;
            map_pages(ents[i].slot, ctx + tokens_per_seq);
        }
        std::vector<uint32_t> out(n_seqs);
        auto one = [&] { for (auto& e : ents) seqs[e.slot].pos = ctx; step(ents.data(), n_seqs, nullptr, out.data()); };
        cudaEvent_t e0, e1;
        AHA_CUDA_CHECK(cudaEventCreate(&e0)); AHA_CUDA_CHECK(cudaEventCreate(&e1));
        for (int i = 0; i < std::max(3, warmup); ++i) one();
        const uint64_t k0 = c.cnt.kernels, g0 = c.cnt.graphs;
        AHA_CUDA_CHECK(cudaEventRecord(e0, c.stream));
        for (int i = 0; i < iters; ++i) one();
        AHA_CUDA_CHECK(cudaEventRecord(e1, c.stream));
        AHA_CUDA_CHECK(cudaEventSynchronize(e1));
        float ms = 0.f;
        AHA_CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
        const double launches = (double)(c.cnt.kernels - k0) / iters, graphs_per = (double)(c.cnt.graphs - g0) / iters;
        // the same steps with events around every launch family
        prof.clear();
        prof_n = n_seqs; prof_tps = tokens_per_seq; prof_ctx = ctx;
        profiling = true;
        const int pit = std::min(iters, 5);
        try { for (int i = 0; i < pit; ++i) { one(); prof_collect(); } } catch (...) { profiling = false; prof_spans.clear(); throw; }
        profiling = false;
        release_all();
        cudaEventDestroy(e0); cudaEventDestroy(e1);
        std::string j = "{\"ms_per_step\": " + std::to_string(ms / iters) + ", \"tokens_per_step\": " + std::to_string(n_seqs * tokens_per_seq) +
                        ", \"kernels_per_step\": " + std::to_string(launches) + ", \"graph_launches_per_step\": " + std::to_string(graphs_per) + ", \"families\": {";
        bool first = true;
        for (auto& kv : prof) {
            if (!first) j += ", ";
            first = false;
            j += "\"" + kv.first + "\": {\"ms\": " + std::to_string(kv.second.ms / pit) + ", \"flops\": " + std::to_string(kv.second.flops / pit) + ", \"bytes\": " +
                 std::to_string(kv.second.bytes / pit) + ", \"launches\": " + std::to_string(kv.second.launches / pit) + "}";
        }
        return j + "}}";
    }
};

// segments for a recurrence whose longest entry is long (see recurrence.cuh): the longest segments that still give every SM four blocks
inline void choose_segments(Engine& E, const StepView& v, Hgrn2Args& a) {
    int longest = 0;
    for (int e = 0; e < v.rb.E; ++e) longest = std::max(longest, v.h_ent_start[e + 1] - v.h_ent_start[e]);
    if (longest >= kSegMinEntry && E.seg_state && E.opt.seq_impl == 0 && a.D <= 256) {
        const int per_seg = a.H * ((a.Dv + kScanCols - 1) / kScanCols);
        int L = kSegLen;
        while (L < kSegLenMax && (longest / (2 * L)) * per_seg >= 4 * E.c.num_sms) L *= 2;
        if (longest > L) { a.seg_state = E.seg_state; a.seg_decay = E.seg_decay; a.seg_len = L; a.seg_max = (longest + L - 1) / L; }
    }
}

// ------------------------------------------------------------------------------------------------------------------------------
struct Hgrn2Mixer final : Sublayer {
    Engine& E;
    int H, D, Dv;
    LinearAny in, out;
    float *lower = nullptr, *norm_w = nullptr, *state = nullptr;
    size_t slot_stride = 0;
    Hgrn2Mixer(Engine& e, const Json& mx, const WeightTable& wt, const std::string& p) : E(e) {
        H = mx.integer("heads"); D = mx.integer("dim"); Dv = mx.integer("vdim");
        AHA_REQUIRE(H >= 1 && D >= 1 && Dv >= 1, "hgrn2: bad sizes");
        in = E.load_linear(wt, {p + "q", p + "f", p + "v"}, {H * D, H * D, H * Dv}, E.W, {"", p + "f.b", ""});
        out = E.load_linear(wt, {p + "o"}, {E.W}, H * Dv, {});
        lower = upload_vec(E.c, wt, p + "lower", (size_t)H * D);
        norm_w = upload_vec(E.c, wt, p + "norm", (size_t)Dv);
        slot_stride = (size_t)H * D * Dv;
        state = E.c.alloc<float>(slot_stride * E.slots);
        AHA_CUDA_CHECK(cudaMemset(state, 0, slot_stride * E.slots * sizeof(float)));
        const size_t smem = hgrn2_scan_smem(D, Dv);
        AHA_REQUIRE((D <= 256 && E.opt.seq_impl != 1) || smem <= 200 * 1024, "hgrn2: dim x vdim state does not fit shared memory");
        AHA_CUDA_CHECK(cudaFuncSetAttribute(hgrn2_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    int proj_cols() const override { return in.N; }
    int inner_cols() const override { return H * Dv; }
    int max_segments() const { return E.Tmax / kSegLen + E.slots; }      // of one step: every entry has at most one segment that is not full
    size_t seg_state_floats() const override { return E.Tmax >= kSegMinEntry ? (size_t)max_segments() * slot_stride : 0; }
    size_t seg_decay_floats() const override { return E.Tmax >= kSegMinEntry ? (size_t)max_segments() * H * D : 0; }
    void run(const StepView& v) override {
        const int T = v.rb.T;
        E.gemm(AEPI_STORE, v.x, E.W, in, E.proj, in.N, T);
        Hgrn2Args a{};
        a.qfv = E.proj; a.ld = in.N; a.lower = lower; a.norm_w = norm_w; a.eps = E.eps; a.state = state; a.slot_stride = slot_stride;
        a.out = E.inner; a.H = H; a.D = D; a.Dv = Dv; a.rb = v.rb;
        choose_segments(E, v, a);      // long prompt portions: segments scanned side by side
        E.tic("hgrn2 recurrence", 4.0 * T * H * D * Dv, 4.0 * T * (in.N + H * Dv) + 8.0 * v.rb.E * slot_stride);
        E.c.cnt.kernels += hgrn2_scan(E.c.stream, a, E.opt.seq_impl);
        E.toc();
        E.gemm(AEPI_STORE, E.inner, H * Dv, out, v.y, E.W, T);
    }
};

// What differs between the designs' "attention" mixers; everything else (sizes, window, scale, convolution, biases, cache reuse) comes from the
// layer's config entry and the checkpoint's tensors.
struct AttentionFlavor {
    bool distance_penalty = true;   // score -= 2^(-8 (h + 1) / H) * (i - j)
    bool rotary = false;            // rotary positions from the layer's "rot" entry, then ...
    bool unit_qk = false;           // ... every q and k head divided by its own root mean square (instead of whole-projection norms with gains)
    bool sink = false;              // softmax denominator + 1
    bool head_gate = false;         // the output gate '.g' has one row per head (else one per output channel, if the tensor exists)
};

struct WindowAttentionMixer final : Sublayer {
    Engine& E;
    AttentionFlavor fl;
    int H, G, D, Dv, taps = 0, window = 0, kv_from = -1, n_freq = 0;
    float* freq = nullptr;
    float scale = 1.f;
    LinearAny in, out;
    int q_off = 0, k_off = 0, v_off = 0, g_off = -1;
    float *wq = nullptr, *wk = nullptr, *wv = nullptr, *q_norm = nullptr, *k_norm = nullptr, *slopes = nullptr, *tails = nullptr;
    size_t tail_stride = 0;
    PagedKV kv;          // own pages, or the owner's when kv_from >= 0
    bool owns_kv = true;
    WindowAttentionMixer(Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int layer_index, AttentionFlavor flavor = AttentionFlavor()) : E(e), fl(flavor) {
        H = mx.integer("heads"); G = mx.integer_or("kv_heads", H); D = mx.integer("dim"); Dv = mx.integer_or("vdim", D);
        AHA_REQUIRE(H >= 1 && G >= 1 && H % G == 0, "attention: heads must be a multiple of kv_heads");
        scale = (float)mx.number("scale");
        taps = mx.integer_or("conv", 0);
        window = mx.has("mask") ? mx.at("mask").integer("size") : 0;
        AHA_REQUIRE(window >= 0, "attention: mask.size must be positive");
        kv_from = mx.integer_or("kv_from", -1);
        owns_kv = kv_from < 0;
        const bool gate = fl.head_gate || wt.has(p + "g");
        std::vector<std::string> names{p + "q"}, biases{p + "q.b"};
        std::vector<int> rows{H * D};
        int col = H * D;
        if (owns_kv) {
            k_off = col; names.push_back(p + "k"); biases.push_back(p + "k.b"); rows.push_back(G * D); col += G * D;
            v_off = col; names.push_back(p + "v"); biases.push_back(p + "v.b"); rows.push_back(G * Dv); col += G * Dv;
        }
        if (gate) { g_off = col; names.push_back(p + "g"); biases.push_back(""); rows.push_back(fl.head_gate ? H : H * Dv); col += rows.back(); }
        in = E.load_linear(wt, names, rows, E.W, biases, fl.head_gate ? 32 : 1);      // (a row per head rarely tiles for the tensor cores: zero rows are appended)
        out = E.load_linear(wt, {p + "o"}, {E.W}, H * Dv, {});
        if (fl.rotary || fl.unit_qk) {
            AHA_REQUIRE(owns_kv, "attention: a layer with rotary positions owns its keys and values");
            std::vector<float> fr;
            if (fl.rotary && mx.has("rot")) {
                const Json& rot = mx.at("rot");
                const int dims = rot.integer_or("dims", D);
                AHA_REQUIRE(dims >= 0 && dims <= D && dims % 2 == 0, "attention: rot.dims must be even and at most dim");
                if (dims > 0) {
                    if (rot.has("scaling")) {
                        const Json& sc = rot.at("scaling");
                        banded_rotary_frequencies(dims, rot.number("base"), sc.number("factor"), sc.number("low"), sc.number("high"), sc.number("original"), fr);
                    } else banded_rotary_frequencies(dims, rot.number("base"), 0.0, 1.0, 1.0, 1.0, fr);
                }
            }
            n_freq = (int)fr.size();
            if (fr.empty()) fr.push_back(0.f);
            freq = upload(E.c, fr);
        }
        if (wt.has(p + "q.norm")) q_norm = upload_vec(E.c, wt, p + "q.norm", (size_t)H * D);
        if (owns_kv && wt.has(p + "k.norm")) k_norm = upload_vec(E.c, wt, p + "k.norm", (size_t)G * D);
        if (taps > 1) {
            AHA_REQUIRE(taps <= kConvMaxTaps, "attention: conv has more than 16 taps");
            wq = upload_vec(E.c, wt, p + "q.conv", (size_t)H * D * taps);
            if (owns_kv) { wk = upload_vec(E.c, wt, p + "k.conv", (size_t)G * D * taps); wv = upload_vec(E.c, wt, p + "v.conv", (size_t)G * Dv * taps); }
            tail_stride = (size_t)(taps - 1) * (H * D + (owns_kv ? G * D + G * Dv : 0));
            tails = E.c.alloc<float>(tail_stride * E.slots);
            AHA_CUDA_CHECK(cudaMemset(tails, 0, tail_stride * E.slots * sizeof(float)));
        }
        if (fl.distance_penalty) {
            std::vector<float> sl(H);
            for (int h = 0; h < H; ++h) sl[h] = (float)std::exp2(-8.0 * (double)(h + 1) / (double)H);
            slopes = upload(E.c, sl);
        }
        if (owns_kv) {
            kv.G = G; kv.D = D; kv.Dv = Dv;
            const size_t nk = (size_t)E.num_pages * G * kPage * D, nv = (size_t)E.num_pages * G * kPage * Dv;
            kv.k = E.c.alloc<float>(nk); kv.v = E.c.alloc<float>(nv);
            AHA_CUDA_CHECK(cudaMemset(kv.k, 0, nk * sizeof(float)));
            AHA_CUDA_CHECK(cudaMemset(kv.v, 0, nv * sizeof(float)));
        } else {
            AHA_REQUIRE(kv_from < layer_index, "attention: kv_from must name an earlier layer");
            auto* src = dynamic_cast<WindowAttentionMixer*>(E.mixer_of_layer[kv_from]);
            AHA_REQUIRE(src && src->owns_kv, "attention: kv_from must name an attention layer with keys and values of its own");
            AHA_REQUIRE(src->G == G && src->D == D && src->Dv == Dv, "attention: kv_from layer has other key / value sizes");
            kv = src->kv;
        }
    }
    int proj_cols() const override { return in.N; }
    int inner_cols() const override { return H * Dv; }
    int q_cols() const override { return H * D; }
    size_t attn_part_floats() const override { return window_attn_part_floats(H, Dv); }
    uint64_t kv_bytes_per_token() const override { return owns_kv ? 4ull * G * (D + Dv) : 0; }
    void run(const StepView& v) override {
        const int T = v.rb.T;
        E.gemm(AEPI_STORE, v.x, E.W, in, E.proj, in.N, T);
        if (fl.rotary || fl.unit_qk) {
            RotaryPrepArgs a{};
            a.proj = E.proj; a.ld = in.N; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.H = H; a.G = G; a.D = D; a.Dv = Dv;
            a.freq = freq; a.n_freq = n_freq; a.unit_norm = fl.unit_qk ? 1 : 0; a.eps = E.eps; a.q_out = E.qbuf; a.kv = kv; a.rb = v.rb;
            E.tic("rotary + q/k unit norm + cache write", 8.0 * T * (H + G) * D, 4.0 * T * (2.0 * H * D + 2.0 * G * D + 2.0 * G * Dv));
            E.c.cnt.kernels += qk_rotary_prepare(E.c.stream, a);
            E.toc();
        } else {
            QkvPrepArgs a{};
            a.proj = E.proj; a.ld = in.N; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
            a.Cq = H * D; a.Ck = owns_kv ? G * D : 0; a.Cv = owns_kv ? G * Dv : 0;
            a.taps = taps; a.wq = wq; a.wk = wk; a.wv = wv; a.tails = tails; a.tail_slot_stride = tail_stride;
            a.q_norm = q_norm; a.k_norm = k_norm; a.eps = E.eps; a.q_out = E.qbuf; a.kv = kv; a.rb = v.rb;
            E.tic("conv + q/k norm + cache write", 2.0 * T * (a.Cq + a.Ck + a.Cv) * std::max(1, taps), 4.0 * T * (2.0 * a.Cq + 2.0 * a.Ck + 2.0 * a.Cv));
            E.c.cnt.kernels += qkv_prepare(E.c.stream, a, v.rb.E == T);
            E.toc();
        }
        WindowAttnArgs w{};
        w.q = E.qbuf; w.kv = kv; w.slopes = slopes; w.scale = scale; w.window = window;
        w.gate = g_off >= 0 ? E.proj + g_off : nullptr; w.gate_ld = in.N; w.gate_per_head = fl.head_gate ? 1 : 0; w.sink = fl.sink ? 1 : 0;
        w.out = E.inner; w.H = H; w.rb = v.rb;
        w.part = E.opt.seq_impl == 1 ? nullptr : E.attn_part;
        // prompt portions on the tensor cores (one launch pair per entry), everything else -- decoded tokens, short portions, exact mode,
        // other head sizes -- on the CUDA-core kernel, which skips the entries the tensor cores took
        const bool tc = !E.fp32 && E.opt.seq_impl != 1 && D == Dv && (D == 64 || D == 128);
        int tc_tokens = 0;
        E.tic(window > 0 ? "window attention" : "causal attention", 2.0 * E.prof_pairs(window) * H * (D + Dv), 4.0 * (T * (double)H * (D + Dv) + E.prof_unique(window) * G * (D + Dv)));
        if (tc)
            for (int e = 0; e < v.rb.E; ++e) {
                const int n = v.h_ent_start[e + 1] - v.h_ent_start[e], pos0 = v.h_ent_pos0[e];
                if (n < kTcAttnMinTokens) continue;
                FlashArgs f{};
                f.q = E.qbuf; f.q_tok_stride = (size_t)H * D; f.q_head_stride = D;
                f.kv.k = kv.k; f.kv.v = kv.v; f.kv.page_table = v.rb.page_tables + (size_t)v.h_ent_slot[e] * v.rb.max_pages; f.kv.page_shift = kPageShift;
                f.kv.page_stride = (size_t)G * kPage * D; f.kv.tok_stride = D; f.kv.head_stride = (size_t)kPage * D;
                f.out = E.inner; f.o_tok_stride = (size_t)H * Dv; f.o_head_stride = Dv;
                f.kv0 = window > 0 ? std::max(0, pos0 - window + 1) : 0;      // keys before the first query's window are not staged
                f.Sq = n; f.Skv = pos0 + n - f.kv0; f.q0 = v.h_ent_start[e]; f.groups = H / G; f.scaling = scale;
                FlashWindow fw;
                fw.window = window; fw.slopes = slopes; fw.gate_tok_stride = in.N; fw.sink = w.sink;
                if (fl.head_gate) fw.gate_head = w.gate; else fw.gate = w.gate;
                if (D == 64) flash_attn_tc<64>(E.c.stream, f, H, true, E.c.split_buf((flash_tc_ws_halfs<64>(f, H) + 1) / 2), &fw);
                else flash_attn_tc<128>(E.c.stream, f, H, true, E.c.split_buf((flash_tc_ws_halfs<128>(f, H) + 1) / 2), &fw);
                E.c.cnt.kernels += 2;
                tc_tokens += n;
            }
        if (tc_tokens < T) {
            w.skip_from_n = tc ? kTcAttnMinTokens : 0;
            E.c.cnt.kernels += window_attn(E.c.stream, w, window > 0 ? std::min(window, v.span) : v.span);
        }
        E.toc();
        E.gemm(AEPI_STORE, E.inner, H * Dv, out, v.y, E.W, T);
    }
};

struct DenseFF final : Sublayer {
    Engine& E;
    int ff;
    LinearAny up, down;
    float alpha_p = 0.f, alpha_n = 0.f;
    int act;      // AEPI_XIELU (two learned parameters in '.act') or AEPI_RELU2
    DenseFF(Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p, int activation = AEPI_XIELU) : E(e), act(activation) {
        ff = cfg.integer("ff");
        up = E.load_linear(wt, {p + "up"}, {ff}, E.W, {});
        down = E.load_linear(wt, {p + "down"}, {E.W}, ff, {});
        if (act == AEPI_XIELU) {
            auto a = wt.vec_f32(p + "act", 2);
            alpha_p = (float)softplus_d(a[0]);
            alpha_n = (float)(0.5 + softplus_d(a[1]));
        }
    }
    int proj_cols() const override { return ff; }
    int inner_cols() const override { return 0; }
    void run(const StepView& v) override {
        E.gemm(act, v.x, E.W, up, E.proj, ff, v.rb.T, alpha_p, alpha_n);
        E.gemm(AEPI_STORE, E.proj, ff, down, v.y, E.W, v.rb.T);
    }
};

// W_down (silu(W_gate h) * (W_up h)) with optional biases on all three ('.gate.b', '.up.b', '.down.b').  The gate and up rows are interleaved into
// one matrix, so that the gated unit is the product's epilogue.
struct GatedDenseFF final : Sublayer {
    Engine& E;
    int ff;
    LinearAny gu, down;
    GatedDenseFF(Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) : E(e) {
        ff = cfg.integer("ff");
        AHA_REQUIRE(ff >= 1, "dense: bad size");
        wt.expect(p + "gate", {ff, E.W}); wt.expect(p + "up", {ff, E.W});
        std::vector<std::pair<const aha_tensor_desc*, int>> rows, bias;
        const bool has_bias = wt.has(p + "gate.b") && wt.has(p + "up.b");
        for (int j = 0; j < ff; ++j) {
            rows.push_back({&wt.get(p + "gate"), j}); rows.push_back({&wt.get(p + "up"), j});
            if (has_bias) { bias.push_back({&wt.get(p + "gate.b"), j}); bias.push_back({&wt.get(p + "up.b"), j}); }
        }
        gu = E.load_rows(wt, p + "gate/up", rows, E.W, has_bias ? &bias : nullptr);
        down = E.load_linear(wt, {p + "down"}, {E.W}, ff, {p + "down.b"});
    }
    int proj_cols() const override { return ff; }
    int inner_cols() const override { return 0; }
    void run(const StepView& v) override {
        E.gemm(AEPI_SWIGLU, v.x, E.W, gu, E.proj, ff, v.rb.T);
        E.gemm(AEPI_STORE, E.proj, ff, down, v.y, E.W, v.rb.T);
    }
};

// Gated linear attention: q = W_q h / sqrt(dim), k = W_k h, v = W_v h, a decay per key channel alpha = sigmoid(z)^(1 / tau) with
// z = W_a2 (W_a1 h) + b (a low-rank projection); per head S <- diag(alpha) S + k v^T, o = S^T q; o is RMS-normed per head (gain over vdim
// shared by the heads), multiplied by silu(W_g h) and projected by W_o.  The state is fp32 in the slot pool.
struct GlaMixer final : Sublayer {
    Engine& E;
    int H, D, Dv, r;
    float tau;
    LinearAny in, a2, out;
    float *norm_w = nullptr, *state = nullptr;
    size_t slot_stride = 0;
    int ld = 0, z_off = 0, a1_off = 0;
    GlaMixer(Engine& e, const Json& mx, const WeightTable& wt, const std::string& p) : E(e) {
        H = mx.integer("heads"); D = mx.integer("dim"); Dv = mx.integer("vdim"); tau = (float)mx.number("tau");
        AHA_REQUIRE(H >= 1 && D >= 1 && Dv >= 1 && tau > 0.f, "gla: bad sizes");
        const aha_tensor_desc& d1 = wt.get(p + "a1");
        AHA_REQUIRE(d1.rank == 2, "gla: a1 must be a matrix");
        r = (int)d1.shape[0];
        // the first factor of the low-rank decay projection rides along with q | k | v | g (rows padded so that the tensor-core kernels take the matrix)
        in = E.load_linear(wt, {p + "q", p + "k", p + "v", p + "g", p + "a1"}, {H * D, H * D, H * Dv, H * Dv, r}, E.W, {}, 32);
        a2 = E.load_linear(wt, {p + "a2"}, {H * D}, r, {p + "a2.b"});
        out = E.load_linear(wt, {p + "o"}, {E.W}, H * Dv, {});
        norm_w = E.vec(wt, p + "norm", (size_t)Dv);
        a1_off = 2 * H * D + 2 * H * Dv;
        z_off = in.N;
        ld = (in.N + H * D + 3) / 4 * 4;
        slot_stride = (size_t)H * D * Dv;
        state = E.c.alloc<float>(slot_stride * E.slots);
        AHA_CUDA_CHECK(cudaMemset(state, 0, slot_stride * E.slots * sizeof(float)));
        AHA_REQUIRE((D <= 256 && E.opt.seq_impl != 1) || hgrn2_scan_smem(D, Dv) <= 200 * 1024, "gla: dim x vdim state does not fit shared memory");
        AHA_CUDA_CHECK(cudaFuncSetAttribute(hgrn2_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    int proj_cols() const override { return ld; }
    int inner_cols() const override { return H * Dv; }
    int max_segments() const { return E.Tmax / kSegLen + E.slots; }
    size_t seg_state_floats() const override { return E.Tmax >= kSegMinEntry ? (size_t)max_segments() * slot_stride : 0; }
    size_t seg_decay_floats() const override { return E.Tmax >= kSegMinEntry ? (size_t)max_segments() * H * D : 0; }
    void run(const StepView& v) override {
        const int T = v.rb.T, HD = H * D;
        E.gemm(AEPI_STORE, v.x, E.W, in, E.proj, ld, T);
        E.gemm(AEPI_STORE, E.proj + a1_off, ld, a2, E.proj + z_off, ld, T);
        E.tic("linear recurrence", 4.0 * T * H * D * Dv, 4.0 * T * (3.0 * HD + 3.0 * H * Dv) + 8.0 * v.rb.E * slot_stride);
        gla_gates_kernel<<<(unsigned)(((size_t)T * HD + 255) / 256), 256, 0, E.c.stream>>>(E.proj, ld, 0, z_off, HD, 1.0f / sqrtf((float)D), 1.0f / tau, (size_t)T * HD);
        E.c.cnt.kernels++;
        Hgrn2Args a{};
        a.qfv = E.proj; a.ld = ld; a.q_off = 0; a.k_off = HD; a.f_off = z_off; a.v = E.proj; a.ld_v = ld; a.v_off = 2 * HD; a.gates_done = 1;
        a.norm_w = norm_w; a.eps = E.eps; a.out_gate = E.proj + 2 * HD + H * Dv; a.out_gate_ld = ld;
        a.state = state; a.slot_stride = slot_stride; a.out = E.inner; a.H = H; a.D = D; a.Dv = Dv; a.rb = v.rb;
        choose_segments(E, v, a);
        E.c.cnt.kernels += hgrn2_scan(E.c.stream, a, E.opt.seq_impl);
        E.toc();
        E.gemm(AEPI_STORE, E.inner, H * Dv, out, v.y, E.W, T);
    }
};

// Mamba-2: W_in h = [z | x | B | C | dt]; x, B, C pass a short causal convolution (bias, silu); dt = softplus(dt + dt_bias); per head (with the
// B and C of its group) S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; y * silu(z) is RMS-normed in groups, then W_o.  The recurrence
// is the keyed diagonal scan with the scalar decay repeated over the state channels.  State and convolution tail are fp32 in the slot pool.
struct Mamba2Mixer final : Sublayer {
    Engine& E;
    int H, P, N, G, NG, taps, inner, Cc, n_in;
    LinearAny in, out;
    float *conv_w = nullptr, *conv_b = nullptr, *dt_bias = nullptr, *a_log = nullptr, *Dw = nullptr, *norm_w = nullptr, *state = nullptr, *tails = nullptr;
    size_t slot_stride = 0, tail_stride = 0;
    int ld = 0, s_off = 0;
    Mamba2Mixer(Engine& e, const Json& mx, const WeightTable& wt, const std::string& p) : E(e) {
        H = mx.integer("heads"); P = mx.integer("vdim"); N = mx.integer("state"); G = mx.integer_or("groups", 1); NG = mx.integer_or("norm_groups", 1);
        AHA_REQUIRE(H >= 1 && P >= 1 && N >= 1 && G >= 1 && H % G == 0 && NG >= 1 && (H * P) % NG == 0, "mamba2: bad sizes");
        inner = H * P; Cc = inner + 2 * G * N; n_in = 2 * inner + 2 * G * N + H;
        const aha_tensor_desc& dc = wt.get(p + "conv");
        AHA_REQUIRE(dc.rank == 2 && dc.shape[0] == Cc, "mamba2: conv must be [channels, taps]");
        taps = (int)dc.shape[1];
        AHA_REQUIRE(taps >= 1 && taps <= kShortConvMaxTaps, "mamba2: between 1 and 16 convolution taps");
        in = E.load_linear(wt, {p + "in"}, {n_in}, E.W, {}, 32);
        out = E.load_linear(wt, {p + "o"}, {E.W}, inner, {});
        conv_w = E.vec(wt, p + "conv", (size_t)Cc * taps);
        conv_b = wt.has(p + "conv.b") ? E.vec(wt, p + "conv.b", (size_t)Cc) : nullptr;
        dt_bias = E.vec(wt, p + "dt_bias", (size_t)H); a_log = E.vec(wt, p + "A_log", (size_t)H); Dw = E.vec(wt, p + "D", (size_t)H);
        norm_w = E.vec(wt, p + "norm", (size_t)inner);
        s_off = in.N; ld = in.N + 3 * H * N;
        slot_stride = (size_t)H * N * P;
        state = E.c.alloc<float>(slot_stride * E.slots);
        AHA_CUDA_CHECK(cudaMemset(state, 0, slot_stride * E.slots * sizeof(float)));
        tail_stride = (size_t)(taps - 1) * Cc;
        tails = E.c.alloc<float>(std::max<size_t>(1, tail_stride * E.slots));
        AHA_CUDA_CHECK(cudaMemset(tails, 0, std::max<size_t>(1, tail_stride * E.slots) * sizeof(float)));
        AHA_REQUIRE((N <= 256 && E.opt.seq_impl != 1) || hgrn2_scan_smem(N, P) <= 200 * 1024, "mamba2: state x vdim does not fit shared memory");
        AHA_CUDA_CHECK(cudaFuncSetAttribute(hgrn2_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    int proj_cols() const override { return ld; }
    int inner_cols() const override { return inner; }
    int q_cols() const override { return Cc; }
    int max_segments() const { return E.Tmax / kSegLen + E.slots; }
    size_t seg_state_floats() const override { return E.Tmax >= kSegMinEntry ? (size_t)max_segments() * slot_stride : 0; }
    size_t seg_decay_floats() const override { return E.Tmax >= kSegMinEntry ? (size_t)max_segments() * H * N : 0; }
    void run(const StepView& v) override {
        const int T = v.rb.T, HN = H * N;
        cudaStream_t st = E.c.stream;
        E.gemm(AEPI_STORE, v.x, E.W, in, E.proj, ld, T);
        E.tic("short convolution", 2.0 * T * Cc * taps, 8.0 * T * Cc);
        ShortConvArgs cv{};
        cv.in = E.proj; cv.ld_in = ld; cv.in_off = inner; cv.C = Cc; cv.taps = taps; cv.w = conv_w; cv.bias = conv_b; cv.tails = tails; cv.tail_slot_stride = tail_stride;
        cv.out = E.qbuf; cv.ld_out = Cc; cv.out_off = 0; cv.silu = 1; cv.rb = v.rb;
        E.c.cnt.kernels += short_conv(st, cv, v.rb.E == T);
        E.toc();
        E.tic("linear recurrence", 4.0 * T * H * N * P, 4.0 * T * (6.0 * HN + 2.0 * inner) + 8.0 * v.rb.E * slot_stride);
        Mamba2GateArgs g{};
        g.dt_raw = E.proj + 2 * inner + 2 * G * N; g.ld_dt = ld; g.bc = E.qbuf; g.ld_bc = Cc; g.b_off = inner; g.c_off = inner + G * N;
        g.dt_bias = dt_bias; g.a_log = a_log; g.out = E.proj; g.ld_out = ld; g.q_off = s_off; g.f_off = s_off + HN; g.k_off = s_off + 2 * HN;
        g.H = H; g.G = G; g.N = N; g.T = T;
        mamba2_gates_kernel<<<(unsigned)(((size_t)T * HN + 255) / 256), 256, 0, st>>>(g);
        E.c.cnt.kernels++;
        Hgrn2Args a{};
        a.qfv = E.proj; a.ld = ld; a.q_off = g.q_off; a.f_off = g.f_off; a.k_off = g.k_off; a.v = E.qbuf; a.ld_v = Cc; a.v_off = 0; a.gates_done = 1;
        a.norm_w = nullptr; a.eps = E.eps; a.state = state; a.slot_stride = slot_stride; a.out = E.inner; a.H = H; a.D = N; a.Dv = P; a.rb = v.rb;
        choose_segments(E, v, a);
        E.c.cnt.kernels += hgrn2_scan(st, a, E.opt.seq_impl);
        // (y + D x) * silu(z), RMS norm in groups, gain: in place
        GroupNormArgs n{};
        n.in = E.inner; n.ld_in = inner; n.gate = E.proj; n.ld_gate = ld; n.skip = E.qbuf; n.ld_skip = Cc; n.skip_w = Dw; n.skip_span = P;
        n.w = norm_w; n.eps = E.eps; n.C = inner; n.groups = NG; n.out = E.inner; n.ld_out = inner;
        group_rmsnorm(st, n, T); E.c.cnt.kernels++;
        E.toc();
        E.gemm(AEPI_STORE, E.inner, inner, out, v.y, E.W, T);
    }
};

// Latent attention (see attention_latent.cuh): the cache holds [latent | rotated key part] per token; a head's query is absorbed through
// W_uk, its output expanded through W_uv; causal, ordinary softmax.  By the layer's config entry and tensors: a rotated part (rot_dim > 0,
// YaRN rotary), queries through a normed latent of their own ('q_rank': q = W_uq norm(W_dq h)) or straight from the input ('.q'), a sliding
// window ('mask.size'), a sigmoid output gate from the mixer's input ('.g'), a learned sink per head in the softmax denominator ('.sink').
struct LatentAttentionMixer final : Sublayer {
    Engine& E;
    int H, D, R, Dv, rank, q_rank = 0, window = 0;
    float scale, rot_mult = 1.f;
    LinearAny in, out, uq, uk_t, uv, ukv;
    bool can_expand = false, has_gate = false;
    int ld = 0, q_off = 0, dkv_off = 0, g_off = 0, n_freq = 0;
    float *c_norm = nullptr, *q_norm = nullptr, *freq = nullptr, *sink = nullptr;
    PagedKV kv;
    LatentAttentionMixer(Engine& e, const Json& mx, const WeightTable& wt, const std::string& p) : E(e) {
        H = mx.integer("heads"); D = mx.integer("dim"); R = mx.integer_or("rot_dim", 0); Dv = mx.integer("vdim"); rank = mx.integer("kv_rank");
        AHA_REQUIRE(H >= 1 && D >= 1 && R >= 0 && Dv >= 1 && rank >= 1, "latent attention: bad sizes");
        scale = (float)mx.number("scale");
        q_rank = mx.integer_or("q_rank", 0);
        window = mx.has("mask") ? mx.at("mask").integer("size") : 0;
        AHA_REQUIRE(q_rank >= 0 && window >= 0, "latent attention: q_rank and mask.size must be positive");
        has_gate = wt.has(p + "g");
        if (wt.has(p + "sink")) sink = E.vec(wt, p + "sink", (size_t)H);
        {   // one product for everything that reads the mixer's input: [q or its latent | dkv | gate]
            const int first = q_rank > 0 ? q_rank : H * (D + R);
            std::vector<std::string> names{p + (q_rank > 0 ? "dq" : "q"), p + "dkv"};
            std::vector<int> rows{first, rank + R};
            dkv_off = first; g_off = dkv_off + rank + R;
            if (has_gate) { names.push_back(p + "g"); rows.push_back(H * Dv); }
            in = E.load_linear(wt, names, rows, E.W, {}, 32);
        }
        ld = in.N;
        if (q_rank > 0) {      // the expanded queries follow in the same rows
            uq = E.load_linear(wt, {p + "uq"}, {H * (D + R)}, q_rank, {}, 32);
            q_norm = E.vec(wt, p + "dq.norm", (size_t)q_rank);
            q_off = in.N; ld = in.N + uq.N;
        }
        out = E.load_linear(wt, {p + "o"}, {E.W}, H * Dv, {});
        c_norm = E.vec(wt, p + "dkv.norm", (size_t)rank);
        // W_uk [H * D, rank] transposed head by head: row h * rank + r holds column r of the head's rows
        {
            wt.expect(p + "uk", {H * D, rank});
            wt.expect(p + "uv", {H * Dv, rank});
            const std::string key = p + "uk^T";
            auto hit = E.lin_cache.find(key);
            if (hit != E.lin_cache.end()) uk_t = hit->second;
            else {
                const aha_tensor_desc& d = wt.get(p + "uk");
                std::vector<float> tr((size_t)H * rank * D);
                for (int h = 0; h < H; ++h)
                    for (int r = 0; r < rank; ++r)
                        for (int k = 0; k < D; ++k) tr[((size_t)h * rank + r) * D + k] = WeightTable::at(d, ((size_t)h * D + k) * rank + r);
                aha_tensor_desc td{};
                td.name = "uk^T"; td.data = tr.data(); td.dtype = AHA_F32; td.rank = 2; td.shape[0] = (int64_t)H * rank; td.shape[1] = D;
                std::vector<std::pair<const aha_tensor_desc*, int>> src;
                for (int n = 0; n < H * rank; ++n) src.push_back({&td, n});
                uk_t = E.load_rows(wt, key, src, D);
            }
            uv = E.load_linear(wt, {p + "uv"}, {H * Dv}, rank, {});
            ukv = E.load_linear(wt, {p + "uk", p + "uv"}, {H * D, H * Dv}, rank, {}, 32);      // the prompt path expands keys and values in one product
        }
        can_expand = E.opt.seq_impl != 1 && E.Tmax >= kLatentExpandMinTokens && latent_flash_supported(D, R, Dv);
        std::vector<float> fr;
        if (R > 0) {
            const Json& rot = mx.at("rot");
            const int dims = rot.integer_or("dims", R);
            AHA_REQUIRE(dims >= 0 && dims <= R && dims % 2 == 0, "latent attention: rot.dims must be even and at most rot_dim");
            if (dims > 0) {
                if (rot.has("scaling")) {
                    const Json& sc = rot.at("scaling");
                    yarn_frequencies(dims, rot.number("base"), sc.number("factor"), sc.number("original"), sc.number("fast"), sc.number("slow"), fr, rot_mult);
                } else yarn_frequencies(dims, rot.number("base"), 0.0, 0.0, 0.0, 0.0, fr, rot_mult);
            }
        }
        n_freq = (int)fr.size();
        if (fr.empty()) fr.push_back(0.f);
        freq = upload(E.c, fr);
        kv.G = 1; kv.D = rank + R; kv.Dv = rank; kv.ldv = rank + R;
        const size_t nk = (size_t)E.num_pages * kPage * kv.D;
        kv.k = E.c.alloc<float>(nk);
        kv.v = kv.k;
        AHA_CUDA_CHECK(cudaMemset(kv.k, 0, nk * sizeof(float)));
    }
    // the most cached rows a prompt portion's expanded form reads: the whole pool, or a step's tokens plus the window before them
    size_t expand_rows() const { const size_t all = (size_t)E.num_pages * kPage; return window > 0 ? std::min(all, (size_t)E.Tmax + window) : all; }
    int proj_cols() const override { return ld; }
    int inner_cols() const override { return H * rank; }
    int q_cols() const override { return std::max(H * (rank + R), H * Dv); }
    size_t attn_part_floats() const override { return window_attn_part_floats(H, rank); }
    uint64_t kv_bytes_per_token() const override { return 4ull * (rank + R); }
    size_t expand_gather_floats() const override { return can_expand ? expand_rows() * (rank + R) : 0; }
    size_t expand_kv_floats() const override { return can_expand ? expand_rows() * ukv.N : 0; }
    size_t expand_out_floats() const override { return (size_t)E.Tmax * H * Dv; }
    bool expand_on_tc() const { return can_expand && !E.fp32 && latent_flash_tc_supported(D, R, Dv); }
    size_t expand_split_halfs() const override {
        if (!can_expand || E.fp32) return 0;
        const size_t smax = expand_rows();
        size_t h = smax * rank;                                               // the expansion product's activations
        if (expand_on_tc()) h = std::max(h, latent_flash_tc_ws_halfs(H, E.Tmax, (int)smax, D, R, Dv) / 2);    // the packed q, k, v^T of the longest entry
        return h;
    }
    void run(const StepView& v) override {
        const int T = v.rb.T, ldq = H * (rank + R);
        cudaStream_t st = E.c.stream;
        E.gemm(AEPI_STORE, v.x, E.W, in, E.proj, ld, T);
        // q = W_uq norm(W_dq h): the query latent is normed in place and the queries land behind the stacked projection.  Without a rotated part
        // the prep kernel has nothing to do on the queries themselves, so it runs first and norms the query latent on the way.
        // Decode-sized steps: the prep kernel leaves the queries alone, and ONE launch absorbs W_uk into them and turns their rotated parts.
        // (One or two tokens of a layer that saves no launch by it stay on the batched product, which is a little faster there.)
        const bool fused_absorb = E.opt.seq_impl != 1 && latent_absorb_supported(T, D) && (T >= 3 || (q_rank > 0 && R > 0));
        const bool norm_in_prep = q_rank > 0 && (R == 0 || fused_absorb);
        if (q_rank > 0 && !norm_in_prep) {
            E.tic("query latent norm", 4.0 * T * q_rank, 8.0 * T * q_rank);
            GroupNormArgs n{};
            n.in = E.proj; n.ld_in = ld; n.w = q_norm; n.eps = E.eps; n.C = q_rank; n.groups = 1; n.out = E.proj; n.ld_out = ld;
            group_rmsnorm(st, n, T); E.c.cnt.kernels++;
            E.toc();
            E.gemm(AEPI_STORE, E.proj, ld, uq, E.proj + q_off, ld, T);
        }
        E.tic("latent norm + rotary + cache write", 8.0 * T * (rank + q_rank + (H + 1) * R), 8.0 * T * (rank + q_rank + (H + 1) * R));
        LatentPrepArgs a{};
        a.proj = E.proj; a.ld = ld; a.q_off = q_off; a.dkv_off = dkv_off; a.H = H; a.D = D; a.R = R; a.rank = rank; a.c_norm = c_norm; a.eps = E.eps;
        a.freq = freq; a.n_freq = n_freq; a.mult = rot_mult; a.q_abs = E.qbuf; a.ld_q = ldq; a.kv = kv; a.rb = v.rb;
        if (norm_in_prep) { a.ql_off = 0; a.ql_rank = q_rank; a.ql_norm = q_norm; }
        a.skip_q = fused_absorb ? 1 : 0;
        latent_prep_kernel<<<T, T <= 8 ? 512 : 128, 0, st>>>(a);
        E.c.cnt.kernels++;
        AHA_CUDA_CHECK(cudaGetLastError());
        E.toc();
        if (norm_in_prep) E.gemm(AEPI_STORE, E.proj, ld, uq, E.proj + q_off, ld, T);
        // which entries are prompt portions (expanded keys / values, below) and which are served by the absorbed form
        bool any_long = false, all_long = can_expand;
        for (int e = 0; e < v.rb.E; ++e) {
            const bool lg = can_expand && v.h_ent_start[e + 1] - v.h_ent_start[e] >= kLatentExpandMinTokens;
            any_long = any_long || lg; all_long = all_long && lg;
        }
        float* attn_out = E.lat_out;      // [T, H * Dv]
        if (fused_absorb) {      // (a decode-sized step has no long entries)
            LatentAbsorbArgs b{};
            b.q = E.proj; b.ld = ld; b.q_off = q_off; b.uk_t = uk_t.w; b.q_abs = E.qbuf; b.ld_q = ldq; b.freq = freq; b.n_freq = n_freq; b.mult = rot_mult;
            b.tok_pos = v.rb.tok_pos; b.T = T; b.H = H; b.D = D; b.R = R; b.rank = rank;
            E.tic("absorbed queries + rotary", 2.0 * T * H * rank * D, (double)H * rank * D * (E.fp32 ? 4 : 2) + 4.0 * T * H * (D + R + rank + R));
            latent_absorb(st, b, E.fp32);
            E.c.cnt.kernels++;
            E.toc();
        } else if (!all_long) {   // q_abs[t][h][:rank] = W_uk(h)^T q_plain[t][h]
            GemmAnyArgs g{};
            g.A = E.proj + q_off; g.lda = ld; g.W = uk_t.w; g.C = E.qbuf; g.ldc = ldq; g.M = T; g.N = rank; g.K = D;
            g.batch = H; g.a_bs = (size_t)(D + R); g.w_bs = (size_t)rank * D; g.c_bs = (size_t)(rank + R);
            E.gemm_batched("per-head latent products", AEPI_STORE, g, 2.0 * T * H * rank * D, (double)H * rank * D * (E.fp32 ? 4 : 2) + 4.0 * T * H * (D + rank));
        }
        if (!all_long) {
            WindowAttnArgs w{};
            w.q = E.qbuf; w.kv = kv; w.slopes = nullptr; w.scale = scale; w.window = window; w.gate = nullptr; w.out = E.inner; w.H = H; w.rb = v.rb;
            w.sink = sink ? 1 : 0; w.sink_logit = sink;
            w.part = E.opt.seq_impl == 1 ? nullptr : E.attn_part;
            w.skip_from_n = any_long ? kLatentExpandMinTokens : 0;
            const int span = window > 0 ? std::min(window, v.span) : v.span;
            E.tic("latent attention (absorbed)", 2.0 * E.prof_pairs(window) * H * (2.0 * rank + R), 4.0 * (T * (double)H * (2.0 * rank + R) + E.prof_unique(window) * (rank + R)));
            if (w.part && !any_long && T <= kWinSplitMaxTokens && latent_decode_supported(kv.D, kv.Dv)) E.c.cnt.kernels += latent_decode_attn(st, w, span, E.c.num_sms);     // all heads share a block's key rows
            else E.c.cnt.kernels += window_attn(st, w, span);
            E.toc();
            // o[t][h] = W_uv(h) o_latent[t][h]  (rows of skipped entries are overwritten below)
            GemmAnyArgs g{};
            g.A = E.inner; g.lda = H * rank; g.W = uv.w; g.C = attn_out; g.ldc = H * Dv; g.M = T; g.N = Dv; g.K = rank;
            g.batch = H; g.a_bs = (size_t)rank; g.w_bs = (size_t)Dv * rank; g.c_bs = (size_t)Dv;
            E.gemm_batched("per-head latent products", AEPI_STORE, g, 2.0 * T * H * rank * Dv, (double)H * rank * Dv * (E.fp32 ? 4 : 2) + 4.0 * T * H * (Dv + rank));
        }
        for (int e = 0; any_long && e < v.rb.E; ++e) {
            const int n = v.h_ent_start[e + 1] - v.h_ent_start[e], pos0 = v.h_ent_pos0[e];
            if (n < kLatentExpandMinTokens) continue;
            // with a window nothing before the first query's first visible key is expanded; positions then count from that key
            const int kv0 = window > 0 ? std::max(0, pos0 - window + 1) : 0, S = pos0 + n - kv0, rel0 = pos0 - kv0;
            E.tic("latent expansion (gather + linear)", 0.0, 8.0 * S * (rank + R));
            latent_gather_kernel<<<S, 128, 0, st>>>(kv, v.rb.page_tables + (size_t)v.h_ent_slot[e] * v.rb.max_pages, E.lat_gather, kv0, S);
            E.c.cnt.kernels++;
            E.toc();
            E.gemm(AEPI_STORE, E.lat_gather, rank + R, ukv, E.lat_kv, ukv.N, S);
            LatentFlashArgs f{};
            f.q_plain = E.proj + q_off; f.ld_qp = ld; f.qp_head_stride = D + R;
            f.q_rot = E.qbuf + rank; f.ld_qr = ldq; f.qr_head_stride = rank + R;
            f.kx = E.lat_kv; f.ld_k = ukv.N; f.k_head_stride = D;
            f.vx = E.lat_kv + (size_t)H * D; f.ld_v = ukv.N; f.v_head_stride = Dv;
            f.k_rot = E.lat_gather + rank; f.ld_kr = rank + R;
            f.out = attn_out; f.ld_o = H * Dv; f.t0 = v.h_ent_start[e]; f.n = n; f.pos0 = rel0; f.D = D; f.R = R; f.Dv = Dv; f.scale = scale; f.window = window; f.sink = sink;
            double pairs = 0;
            for (int k = 0; k < n; ++k) pairs += window > 0 ? std::min(pos0 + k + 1, window) : pos0 + k + 1;
            if (expand_on_tc()) {
                E.tic("latent attention (expanded, tcgen05, split fp16)", 2.0 * pairs * H * (D + R + Dv), 4.0 * ((double)n * H * (D + R + Dv) + (double)S * (H * (D + Dv) + R)));
                E.c.cnt.kernels += latent_flash_tc(st, f, H, E.c.split_buf((latent_flash_tc_ws_halfs(H, n, S, D, R, Dv) + 1) / 2));
            } else {
                E.tic("latent attention (expanded, CUDA cores)", 2.0 * pairs * H * (D + R + Dv), 4.0 * ((double)n * H * (D + R + Dv) + (double)S * (H * (D + Dv) + R)));
                latent_flash(st, f, H);
                E.c.cnt.kernels++;
            }
            E.toc();
        }
        if (has_gate) {
            E.tic("output gate", 4.0 * T * H * Dv, 12.0 * T * H * Dv);
            gate_mul_kernel<<<(unsigned)(((size_t)T * H * Dv + 255) / 256), 256, 0, st>>>(attn_out, H * Dv, E.proj + g_off, ld, H * Dv, (size_t)T * H * Dv, 0);
            E.c.cnt.kernels++;
            E.toc();
        }
        E.gemm(AEPI_STORE, attn_out, H * Dv, out, v.y, E.W, T);
    }
};

// minGRU (see recurrence_elem.cuh): z = sigmoid(W_z h + b_z), candidate from W_x h + b_x, S <- (1 - z) S + z candidate per channel,
// output W_o (S * silu(W_g h)).  The state is one fp32 per channel and sequence in the slot pool.
struct MinGruMixer final : Sublayer {
    Engine& E;
    int n;
    LinearAny in, out;
    float* state = nullptr;
    MinGruMixer(Engine& e, const Json& mx, const WeightTable& wt, const std::string& p) : E(e) {
        n = mx.integer("width");
        AHA_REQUIRE(n >= 1, "mingru: bad width");
        in = E.load_linear(wt, {p + "z", p + "x", p + "g"}, {n, n, n}, E.W, {p + "z.b", p + "x.b", ""}, 32);
        out = E.load_linear(wt, {p + "o"}, {E.W}, n, {});
        state = E.c.alloc<float>((size_t)n * E.slots);
        AHA_CUDA_CHECK(cudaMemset(state, 0, (size_t)n * E.slots * sizeof(float)));
    }
    int proj_cols() const override { return in.N; }
    int inner_cols() const override { return n; }
    void run(const StepView& v) override {
        const int T = v.rb.T;
        E.gemm(AEPI_STORE, v.x, E.W, in, E.proj, in.N, T);
        ElemScanArgs a{};
        a.proj = E.proj; a.ld = in.N; a.z_off = 0; a.c_off = n; a.g_off = 2 * n; a.n = n; a.state = state; a.slot_stride = (size_t)n;
        a.out = E.inner; a.ld_out = n; a.rb = v.rb;
        int longest = 0;
        for (int e = 0; e < v.rb.E; ++e) longest = std::max(longest, v.h_ent_start[e + 1] - v.h_ent_start[e]);
        E.tic("elementwise recurrence", 12.0 * T * n, 16.0 * T * n + 8.0 * v.rb.E * n);
        E.c.cnt.kernels += mingru_scan(E.c.stream, a, longest, E.c.num_sms);
        E.toc();
        E.gemm(AEPI_STORE, E.inner, n, out, v.y, E.W, T);
    }
};

// Mixture of experts chosen by a table: row `token id` of '.table' names the token's `top` experts, each weighted 1 / top.  Expert:
// W_down (silu(W_gate h) * (W_up h)).  The experts' gate and up rows are interleaved into one matrix per expert (the gate / up epilogue),
// all experts stacked, so that the products are batched (decode steps: one row per assignment with its expert's matrix) or grouped
// (assignments ordered by expert on the device, a batch per expert over its rows).
struct TableMoeFF final : Sublayer {
    Engine& E;
    int ff, experts, top, table_ld;
    LinearAny gu, down;     // [experts * 2 ff, W], [experts * W, ff]
    int* table = nullptr;
    int* tok_of_assign = nullptr;   // [kGraphMaxTokens * top]: assignment a belongs to packed token a / top
    int* err = nullptr;
    TableMoeFF(Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) : E(e) {
        ff = cfg.at("expert").integer("ff"); experts = cfg.at("router").integer("experts"); top = cfg.at("router").integer("top");
        AHA_REQUIRE(ff >= 1 && experts >= 1 && top >= 1 && top <= experts, "moe: bad sizes");
        std::vector<std::pair<const aha_tensor_desc*, int>> s1, s2;
        for (int x = 0; x < experts; ++x) {
            const std::string q = p + "e" + std::to_string(x) + ".";
            wt.expect(q + "gate", {ff, E.W}); wt.expect(q + "up", {ff, E.W}); wt.expect(q + "down", {E.W, ff});
            for (int j = 0; j < ff; ++j) { s1.push_back({&wt.get(q + "gate"), j}); s1.push_back({&wt.get(q + "up"), j}); }
            for (int j = 0; j < E.W; ++j) s2.push_back({&wt.get(q + "down"), j});
        }
        gu = E.load_rows(wt, p + "gate/up", s1, E.W);
        down = E.load_rows(wt, p + "down", s2, ff);
        const aha_tensor_desc& dt = wt.get(p + "table");
        AHA_REQUIRE(dt.rank == 2 && dt.shape[0] == E.V && dt.shape[1] >= top, "moe: table must be [vocab, top]");
        table_ld = (int)dt.shape[1];
        const std::string tkey = p + "table";
        auto hit = E.int_cache.find(tkey);
        if (hit != E.int_cache.end()) table = hit->second;
        else {
            std::vector<int> tb((size_t)E.V * table_ld);
            for (size_t i = 0; i < tb.size(); ++i) {
                tb[i] = (int)std::llround(WeightTable::at(dt, i));
                AHA_REQUIRE(tb[i] >= 0 && tb[i] < experts, "moe: a table entry names no expert");
            }
            table = E.int_cache[tkey] = upload(E.c, tb);
        }
        std::vector<int> ta((size_t)kGraphMaxTokens * top);
        for (size_t i = 0; i < ta.size(); ++i) ta[i] = (int)(i / top);
        tok_of_assign = upload(E.c, ta);
        err = E.c.alloc<int>(1);
        AHA_CUDA_CHECK(cudaMemset(err, 0, sizeof(int)));
    }
    int proj_cols() const override { return top * ff; }
    int inner_cols() const override { return top * E.W; }
    size_t route_ints() const override { return 3 * (size_t)E.Tmax * top + experts + 1; }
    void run(const StepView& v) override {
        const int T = v.rb.T, A = T * top, W = E.W;
        cudaStream_t st = E.c.stream;
        int* expert_of = E.route_buf; int* sorted_tok = expert_of + (size_t)E.Tmax * top; int* place_of = sorted_tok + (size_t)E.Tmax * top; int* offsets = place_of + (size_t)E.Tmax * top;
        const bool rows = T <= kGraphMaxTokens && E.opt.seq_impl != 1;      // decode-sized steps: a batch per assignment, no ordering
        if (!rows) {      // (decode-sized steps look the experts up inside the products)
            E.tic("expert routing (table)", 0.0, 16.0 * A);
            MoeRouteArgs r{};
            r.tokens = v.rb.tokens; r.T = T; r.table = table; r.table_ld = table_ld; r.V = E.V; r.top = top; r.experts = experts;
            r.expert_of = expert_of; r.offsets = offsets; r.sorted_tok = sorted_tok; r.place_of = place_of; r.error = err; r.sort = 1;
            moe_table_route(st, r); E.c.cnt.kernels++;
            E.toc();
        }
        const double wb = E.fp32 ? 4.0 : 2.0, used = std::min(A, experts);
        // prompt portions in serving mode, sizes that tile: both products on the tensor cores, ONE grouped launch each over the ordered rows
        if (!rows && !E.fp32 && E.opt.gemm_impl != 1 && T >= kTcMinRows && W % kTcBK == 0 && ff % kTcBK == 0 && W % 32 == 0) {
            __half* hi = E.c.split_buf((size_t)A * std::max(W, ff));
            __half* lo = hi + E.c.split_cap;
            E.tic("expert linear (grouped, tcgen05, bf16 hi+lo)", 6.0 * A * ff * W, used * 3.0 * ff * W * wb + 4.0 * A * (3.0 * W + 3.0 * ff));
            gather_split_f32_to_bf16x2_kernel<<<(unsigned)(((size_t)A * W / 4 + 255) / 256), 256, 0, st>>>(v.x, W, sorted_tok, reinterpret_cast<__nv_bfloat16*>(hi), reinterpret_cast<__nv_bfloat16*>(lo), A, W);
            if (!gu.has_tmap) { gu.tmap = make_tmap_f16(gu.w, (uint64_t)gu.N, (uint64_t)gu.K); gu.has_tmap = true; }
            if (!down.has_tmap) { down.tmap = make_tmap_f16(down.w, (uint64_t)down.N, (uint64_t)down.K); down.has_tmap = true; }
            GemmTcArgs t{};
            t.bias = nullptr; t.resid = nullptr; t.ldr = 0; t.C = E.proj; t.ldc = ff; t.M = A; t.N = 2 * ff; t.K = W; t.act = ACT_NONE; t.bf16 = 1;
            t.grp_offsets = offsets; t.groups = experts;
            gemm_tc_grouped_launch(st, EPI_SWIGLU, hi, lo, gu.tmap, t);
            split_f32_to_bf16x2_kernel<<<(unsigned)(((size_t)A * ff / 4 + 255) / 256), 256, 0, st>>>(E.proj, ff, reinterpret_cast<__nv_bfloat16*>(hi), reinterpret_cast<__nv_bfloat16*>(lo), A, ff);
            t.C = E.inner; t.ldc = W; t.N = W; t.K = ff;
            gemm_tc_grouped_launch(st, EPI_STORE, hi, lo, down.tmap, t);
            E.c.cnt.kernels += 4;
            E.toc();
            E.tic("expert combine", 1.0 * A * W, 4.0 * (A + T) * W);
            moe_combine_kernel<<<(unsigned)(((size_t)T * W + 255) / 256), 256, 0, st>>>(E.inner, place_of, v.y, W, top, 1.0f / (float)top, (size_t)T * W);
            E.c.cnt.kernels++;
            AHA_CUDA_CHECK(cudaGetLastError());
            E.toc();
            return;
        }
        GemmAnyArgs g{};
        g.A = v.x; g.lda = W; g.W = gu.w; g.C = E.proj; g.ldc = ff; g.N = 2 * ff; g.K = W; g.w_bs = (size_t)2 * ff * W;
        if (rows) {
            g.M = 1; g.batch = A; g.a_index = tok_of_assign; g.a_bs = (size_t)W; g.c_bs = (size_t)ff;
            g.w_keys = reinterpret_cast<const int*>(v.rb.tokens); g.w_table = table; g.w_table_ld = table_ld; g.w_div = top;
        }
        else { g.M = A; g.batch = experts; g.row_offsets = offsets; g.a_gather = sorted_tok; }
        E.gemm_batched(rows ? "expert linear (decode rows)" : "expert linear (grouped, CUDA cores)", AEPI_SWIGLU, g, 4.0 * A * ff * W, used * 2.0 * ff * W * wb + 4.0 * A * (W + ff));
        GemmAnyArgs d{};
        d.A = E.proj; d.lda = ff; d.W = down.w; d.C = E.inner; d.ldc = W; d.N = W; d.K = ff; d.w_bs = (size_t)W * ff;
        if (rows) {
            d.M = 1; d.batch = A; d.a_bs = (size_t)ff; d.c_bs = (size_t)W;
            d.w_keys = reinterpret_cast<const int*>(v.rb.tokens); d.w_table = table; d.w_table_ld = table_ld; d.w_div = top;
        }
        else { d.M = A; d.batch = experts; d.row_offsets = offsets; }
        E.gemm_batched(rows ? "expert linear (decode rows)" : "expert linear (grouped, CUDA cores)", AEPI_STORE, d, 2.0 * A * ff * W, used * ff * W * wb + 4.0 * A * (W + ff));
        if (rows && E.sandwich) { E.out_src = E.inner; E.out_rows = top; E.out_scale = 1.0f / (float)top; return; }     // summed by the norm + residual kernel
        E.tic("expert combine", 1.0 * A * W, 4.0 * (A + T) * W);
        moe_combine_kernel<<<(unsigned)(((size_t)T * W + 255) / 256), 256, 0, st>>>(E.inner, rows ? nullptr : place_of, v.y, W, top, 1.0f / (float)top, (size_t)T * W);
        E.c.cnt.kernels++;
        AHA_CUDA_CHECK(cudaGetLastError());
        E.toc();
    }
};

// What differs between the designs' routed feed-forwards; sizes, limits, groups and factors come from the layer's config entry.
struct RoutedFlavor {
    int act = AEPI_RELU2;            // the expert's unit: an activation on W_up h (AEPI_RELU2), or a gated unit of W_gate h and W_up h (AEPI_SWIGLU, AEPI_CLAMP_GLU)
    float glu_slope = 1.f;           // AEPI_CLAMP_GLU: the gate passes through g * sigmoid(glu_slope * g); its limit is the expert's 'limit'
    bool shared_gate = true;         // the shared expert is multiplied by sigmoid(W_sg h) (else added as it is)
    bool correction = false;         // '.correction' is added to the scores for the choice
    bool groups = false;             // router.groups {count, keep}: experts are chosen from the best groups only
    bool renorm = false;             // the chosen scores are divided by their sum (+ floor), then ...
    float floor = 0.f;
    bool scaled = false;             // ... multiplied by router.scale
    bool gated() const { return act == AEPI_SWIGLU || act == AEPI_CLAMP_GLU; }
};

// Mixture of experts chosen by a router (see moe_router.cuh): scores = softmax(W_router h) over all experts, the `top` best (by the flavour's
// rule) weigh their experts' outputs; expert: W_down unit(h) without biases, the unit by the flavour; an optional shared expert of the same form
// runs for every token and is added, times sigmoid(W_sg h) if the flavour has that gate.  The router and the shared gate are ONE fp32 product
// whatever the engine's mode; the experts' matrices are stacked (gate and up rows interleaved for a gated unit) so that the products are batched
// (decode steps: one row per assignment with its expert's matrix) or grouped (assignments ordered by expert on the device, one launch over all
// experts; on the tensor cores where the sizes tile).
struct RoutedMoeFF final : Sublayer {
    Engine& E;
    RoutedFlavor fl;
    int ff, ffs = 0, experts, top, nup;  // nup: rows of an expert's first matrix (ff, or 2 ff interleaved)
    float limit = 0.f, slimit = 0.f;     // clamp of the experts' / the shared expert's unit
    LinearAny up, down, sup, sdown;     // [experts * nup, W], [experts * W, ff]; the shared expert's
    float* router = nullptr;             // [experts (+ 1), W] fp32: the router's rows, then the shared gate's
    RouterRule rule;
    int n_router = 0, ldl = 0;
    int* tok_of_assign = nullptr;
    int* err = nullptr;
    RoutedMoeFF(Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p, RoutedFlavor flavor) : E(e), fl(flavor) {
        const Json& rt = cfg.at("router");
        ff = cfg.at("expert").integer("ff"); experts = rt.integer("experts"); top = rt.integer("top");
        AHA_REQUIRE(ff >= 1 && experts >= 1 && top >= 1 && top <= experts, "moe: bad sizes");
        if (fl.act == AEPI_CLAMP_GLU) limit = (float)cfg.at("expert").number("limit");
        nup = fl.gated() ? 2 * ff : ff;
        std::vector<std::pair<const aha_tensor_desc*, int>> s1, s2;
        for (int x = 0; x < experts; ++x) {
            const std::string q = p + "e" + std::to_string(x) + ".";
            wt.expect(q + "up", {ff, E.W}); wt.expect(q + "down", {E.W, ff});
            if (fl.gated()) wt.expect(q + "gate", {ff, E.W});
            for (int j = 0; j < ff; ++j) {
                if (fl.gated()) s1.push_back({&wt.get(q + "gate"), j});
                s1.push_back({&wt.get(q + "up"), j});
            }
            for (int j = 0; j < E.W; ++j) s2.push_back({&wt.get(q + "down"), j});
        }
        up = E.load_rows(wt, p + (fl.gated() ? "experts.gate/up" : "experts.up"), s1, E.W);
        down = E.load_rows(wt, p + "experts.down", s2, ff);
        const bool shared = cfg.has("shared") && cfg.at("shared").kind == Json::Obj;
        if (shared) {
            ffs = cfg.at("shared").integer("ff");
            AHA_REQUIRE(ffs >= 1, "moe: bad shared expert size");
            if (fl.act == AEPI_CLAMP_GLU) slimit = (float)cfg.at("shared").number("limit");
            if (fl.gated()) {
                wt.expect(p + "shared.gate", {ffs, E.W}); wt.expect(p + "shared.up", {ffs, E.W});
                std::vector<std::pair<const aha_tensor_desc*, int>> s3;
                for (int j = 0; j < ffs; ++j) { s3.push_back({&wt.get(p + "shared.gate"), j}); s3.push_back({&wt.get(p + "shared.up"), j}); }
                sup = E.load_rows(wt, p + "shared.gate/up", s3, E.W);
            } else sup = E.load_linear(wt, {p + "shared.up"}, {ffs}, E.W, {});
            sdown = E.load_linear(wt, {p + "shared.down"}, {E.W}, ffs, {});
        }
        const bool sgate = shared && fl.shared_gate;
        n_router = experts + (sgate ? 1 : 0);
        ldl = n_router + top;      // a token's row: router logits | shared gate | the chosen experts' weights
        {
            const std::string key = p + "router (fp32)";
            auto hit = E.vec_cache.find(key);
            if (hit != E.vec_cache.end()) router = hit->second;
            else {
                std::vector<float> r = wt.vec_f32(p + "router", (size_t)experts * E.W);
                if (sgate) { auto g = wt.vec_f32(p + "shared.sg", (size_t)E.W); r.insert(r.end(), g.begin(), g.end()); }
                router = E.vec_cache[key] = upload(E.c, r);
            }
        }
        if (fl.correction) rule.correction = E.vec(wt, p + "correction", (size_t)experts);
        if (fl.groups && rt.has("groups") && rt.at("groups").kind == Json::Obj) {
            rule.group_count = rt.at("groups").integer("count"); rule.group_keep = rt.at("groups").integer("keep");
            AHA_REQUIRE(rule.group_count >= 1 && experts % rule.group_count == 0 && rule.group_keep >= 1 && rule.group_keep <= rule.group_count,
                        "moe: router.groups.count must divide the experts, keep lie between 1 and count");
            AHA_REQUIRE((int64_t)rule.group_keep * (experts / rule.group_count) >= top, "moe: the kept groups hold fewer than `top` experts");
        }
        rule.renorm = fl.renorm ? 1 : 0; rule.floor = fl.floor;
        if (fl.scaled) rule.scale = (float)rt.number_or("scale", 1.0);
        std::vector<int> ta((size_t)kGraphMaxTokens * top);
        for (size_t i = 0; i < ta.size(); ++i) ta[i] = (int)(i / top);
        tok_of_assign = upload(E.c, ta);
        err = E.c.alloc<int>(1);
        AHA_CUDA_CHECK(cudaMemset(err, 0, sizeof(int)));
    }
    int proj_cols() const override { return top * ff + ffs; }           // the experts' hidden rows [T * top, ff], then the shared expert's [T, ffs]
    int inner_cols() const override { return (top + 1) * E.W; }          // the experts' outputs [T * top, W], then the shared expert's [T, W]
    int q_cols() const override { return ldl; }
    size_t route_ints() const override { return 3 * (size_t)E.Tmax * top + experts + 1; }
    void run(const StepView& v) override {
        const int T = v.rb.T, A = T * top, W = E.W;
        cudaStream_t st = E.c.stream;
        int* expert_of = E.route_buf; int* sorted_tok = expert_of + (size_t)E.Tmax * top; int* place_of = sorted_tok + (size_t)E.Tmax * top; int* offsets = place_of + (size_t)E.Tmax * top;
        float* logits = E.qbuf;
        float* hid = E.proj; float* shid = E.proj + (size_t)E.Tmax * top * ff;
        float* rows_out = E.inner; float* sout = E.inner + (size_t)E.Tmax * top * W;
        // router (+ shared gate): true fp32 on the CUDA cores in both modes
        E.tic("router", 2.0 * T * n_router * W, 4.0 * ((double)n_router * W + (double)T * (W + n_router)));
        if (router_fused_supported(W, n_router, rule.group_count)) {      // product, softmax and choice in one launch
            RouterFusedArgs r{};
            r.x = v.x; r.ldx = W; r.w = router; r.T = T; r.K = W; r.experts = experts; r.n_out = n_router; r.top = top; r.logits = logits; r.ld = ldl; r.expert_of = expert_of;
            r.rule = rule;
            router_fused(st, r);
            E.c.cnt.kernels++;
        } else {
            GemmAnyArgs g{};
            g.A = v.x; g.lda = W; g.W = router; g.C = logits; g.ldc = ldl; g.M = T; g.N = n_router; g.K = W;
            gemm_any(st, AEPI_STORE, true, g, E.c.num_sms);
            RouterArgs r{};
            r.logits = logits; r.ld = ldl; r.T = T; r.experts = experts; r.top = top; r.expert_of = expert_of; r.weights = logits + n_router; r.ld_w = ldl;
            r.rule = rule;
            router_topk(st, r);
            E.c.cnt.kernels += 2;
        }
        E.toc();
        const bool rows = T <= kGraphMaxTokens && E.opt.seq_impl != 1;      // decode-sized steps: a batch per assignment, no ordering
        if (!rows) {
            E.tic("expert routing (order by expert)", 0.0, 16.0 * A);
            MoeRouteArgs r{};
            r.tokens = v.rb.tokens; r.T = T; r.table = nullptr; r.table_ld = 0; r.V = E.V; r.top = top; r.experts = experts;
            r.expert_of = expert_of; r.offsets = offsets; r.sorted_tok = sorted_tok; r.place_of = place_of; r.error = err; r.sort = 1;
            moe_table_route(st, r); E.c.cnt.kernels++;
            E.toc();
        }
        const double wb = E.fp32 ? 4.0 : 2.0, used = std::min(A, experts), mats = fl.gated() ? 3.0 : 2.0;
        if (!rows && !E.fp32 && E.opt.gemm_impl != 1 && T >= kTcMinRows && W % kTcBK == 0 && ff % kTcBK == 0 && W % 32 == 0) {
            // both products on the tensor cores, ONE grouped launch each over the ordered rows
            __half* hi = E.c.split_buf((size_t)A * std::max(W, ff));
            __half* lo = hi + E.c.split_cap;
            E.tic("expert linear (grouped, tcgen05, bf16 hi+lo)", 2.0 * mats * A * ff * W, used * mats * ff * W * wb + 4.0 * A * (2.0 * W + 2.0 * ff));
            gather_split_f32_to_bf16x2_kernel<<<(unsigned)(((size_t)A * W / 4 + 255) / 256), 256, 0, st>>>(v.x, W, sorted_tok, reinterpret_cast<__nv_bfloat16*>(hi), reinterpret_cast<__nv_bfloat16*>(lo), A, W);
            if (!up.has_tmap) { up.tmap = make_tmap_f16(up.w, (uint64_t)up.N, (uint64_t)up.K); up.has_tmap = true; }
            if (!down.has_tmap) { down.tmap = make_tmap_f16(down.w, (uint64_t)down.N, (uint64_t)down.K); down.has_tmap = true; }
            GemmTcArgs t{};
            t.bias = nullptr; t.resid = nullptr; t.ldr = 0; t.C = hid; t.ldc = ff; t.M = A; t.N = nup; t.K = W; t.bf16 = 1;
            t.act = fl.act == AEPI_RELU2 ? ACT_RELU2 : (fl.act == AEPI_CLAMP_GLU ? ACT_CLAMP_GLU : ACT_NONE); t.act_a = limit; t.act_b = fl.glu_slope;
            t.grp_offsets = offsets; t.groups = experts;
            gemm_tc_grouped_launch(st, fl.gated() ? EPI_SWIGLU : EPI_ACT, hi, lo, up.tmap, t);
            split_f32_to_bf16x2_kernel<<<(unsigned)(((size_t)A * ff / 4 + 255) / 256), 256, 0, st>>>(hid, ff, reinterpret_cast<__nv_bfloat16*>(hi), reinterpret_cast<__nv_bfloat16*>(lo), A, ff);
            t.C = rows_out; t.ldc = W; t.N = W; t.K = ff; t.act = ACT_NONE;
            gemm_tc_grouped_launch(st, EPI_STORE, hi, lo, down.tmap, t);
            E.c.cnt.kernels += 4;
            E.toc();
        } else {
            GemmAnyArgs g{};
            g.A = v.x; g.lda = W; g.W = up.w; g.C = hid; g.ldc = ff; g.N = nup; g.K = W; g.w_bs = (size_t)nup * W; g.act_a = limit; g.act_b = fl.glu_slope;
            if (rows) { g.M = 1; g.batch = A; g.a_index = tok_of_assign; g.a_bs = (size_t)W; g.c_bs = (size_t)ff; g.w_index = expert_of; }
            else { g.M = A; g.batch = experts; g.row_offsets = offsets; g.a_gather = sorted_tok; }
            E.gemm_batched(rows ? "expert linear (decode rows)" : "expert linear (grouped, CUDA cores)", fl.act, g, 2.0 * A * nup * W, used * nup * W * wb + 4.0 * A * (W + ff));
            GemmAnyArgs d{};
            d.A = hid; d.lda = ff; d.W = down.w; d.C = rows_out; d.ldc = W; d.N = W; d.K = ff; d.w_bs = (size_t)W * ff;
            if (rows) { d.M = 1; d.batch = A; d.a_bs = (size_t)ff; d.c_bs = (size_t)W; d.w_index = expert_of; }
            else { d.M = A; d.batch = experts; d.row_offsets = offsets; }
            E.gemm_batched(rows ? "expert linear (decode rows)" : "expert linear (grouped, CUDA cores)", AEPI_STORE, d, 2.0 * A * ff * W, used * ff * W * wb + 4.0 * A * (W + ff));
        }
        if (ffs > 0) {
            E.gemm(fl.act, v.x, W, sup, shid, ffs, T, slimit, fl.glu_slope);
            E.gemm(AEPI_STORE, shid, ffs, sdown, sout, W, T);
        }
        WeightedCombineArgs cb{};
        cb.rows = rows_out; cb.place_of = rows ? nullptr : place_of; cb.weights = logits + n_router; cb.ld_w = ldl;
        cb.shared = ffs > 0 ? sout : nullptr; cb.gate = ffs > 0 && fl.shared_gate ? logits + experts : nullptr; cb.ld_gate = ldl; cb.y = v.y; cb.C = W; cb.top = top; cb.total = (size_t)T * W;
        if (rows && E.can_defer_mix(T)) { E.mix = cb; E.mix_pending = true; return; }      // summed by the norm + residual launch that follows
        E.tic("expert combine", 2.0 * (A + T) * W, 4.0 * (A + 2.0 * T) * W);
        moe_weighted_combine_kernel<<<(unsigned)((cb.total + 255) / 256), 256, 0, st>>>(cb);
        E.c.cnt.kernels++;
        AHA_CUDA_CHECK(cudaGetLastError());
        E.toc();
    }
};

using MixerFactory = std::function<std::unique_ptr<Sublayer>(Engine&, const Json&, const WeightTable&, const std::string&, int)>;
const std::map<std::string, MixerFactory>& mixer_registry() {
    static const std::map<std::string, MixerFactory> r = {
        {"hgrn2", [](Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int) { return std::unique_ptr<Sublayer>(new Hgrn2Mixer(e, mx, wt, p)); }},
        {"attention", [](Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int l) { return std::unique_ptr<Sublayer>(new WindowAttentionMixer(e, mx, wt, p, l)); }},
        {"gla", [](Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int) { return std::unique_ptr<Sublayer>(new GlaMixer(e, mx, wt, p)); }},
        {"mamba2", [](Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int) { return std::unique_ptr<Sublayer>(new Mamba2Mixer(e, mx, wt, p)); }},
        {"latent_attention", [](Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int) { return std::unique_ptr<Sublayer>(new LatentAttentionMixer(e, mx, wt, p)); }},
        {"mingru", [](Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int) { return std::unique_ptr<Sublayer>(new MinGruMixer(e, mx, wt, p)); }},
        {"lupolorn:attention", [](Engine& e, const Json& mx, const WeightTable& wt, const std::string& p, int l) {
             AttentionFlavor f;
             f.distance_penalty = false; f.rotary = true; f.unit_qk = true; f.sink = true; f.head_gate = true;
             return std::unique_ptr<Sublayer>(new WindowAttentionMixer(e, mx, wt, p, l, f));
         }},
    };
    return r;
}
// "<design>:<name>" if the design binds the name to a variant of its own, else "<name>"
template <typename M>
typename M::const_iterator find_for_design(const M& reg, const std::string& design, const std::string& name) {
    auto it = reg.find(design + ":" + name);
    return it != reg.end() ? it : reg.find(name);
}
using FFFactory = std::function<std::unique_ptr<Sublayer>(Engine&, const Json&, const WeightTable&, const std::string&)>;
const std::map<std::string, FFFactory>& ff_registry() {
    static const std::map<std::string, FFFactory> r = {
        {"dense", [](Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) { return std::unique_ptr<Sublayer>(new DenseFF(e, cfg, wt, p)); }},
        {"moe", [](Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) { return std::unique_ptr<Sublayer>(new TableMoeFF(e, cfg, wt, p)); }},
        {"lupolorn:dense", [](Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) { return std::unique_ptr<Sublayer>(new DenseFF(e, cfg, wt, p, AEPI_RELU2)); }},
        {"lupolorn:moe", [](Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) { return std::unique_ptr<Sublayer>(new RoutedMoeFF(e, cfg, wt, p, RoutedFlavor())); }},
        {"gomerax:dense", [](Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) { return std::unique_ptr<Sublayer>(new GatedDenseFF(e, cfg, wt, p)); }},
        {"gomerax:moe", [](Engine& e, const Json& cfg, const WeightTable& wt, const std::string& p) {
             RoutedFlavor f;
             f.act = AEPI_CLAMP_GLU; f.glu_slope = 1.702f; f.shared_gate = false; f.correction = true; f.groups = true; f.renorm = true; f.floor = 1e-20f; f.scaled = true;
             return std::unique_ptr<Sublayer>(new RoutedMoeFF(e, cfg, wt, p, f));
         }},
    };
    return r;
}

float* upload_scalar(Engine& E, const WeightTable& wt, const std::string& name) { return upload_vec(E.c, wt, name, 1); }

}  // namespace

SeqEngine* make_layered_engine(Ctx& ctx, const Json& cfg, const WeightTable& wt, const SeqEngineOptions& opt) {
    std::unique_ptr<Engine> E(new Engine(ctx, opt));
    Engine& e = *E;
    const size_t before = ctx.alloc_bytes;
    e.fp32 = opt.fp32;
    e.W = cfg.integer("width"); e.V = cfg.integer("vocab");
    e.eps = (float)cfg.at("norm").number("eps");
    const Json& ls = cfg.at("layers");
    AHA_REQUIRE(ls.kind == Json::Arr && !ls.arr.empty(), "config.json: 'layers' must be a non-empty list");
    // the layer template
    std::string arch = cfg.string_or("architecture", "");
    for (auto& ch : arch) ch = (char)std::tolower((unsigned char)ch);
    e.design = arch;
    e.sandwich = arch == "gatuzen" || arch == "lupolorn";      // (Lupolorn: the same frame without groups, convolution or multiplier)
    e.parallel = arch == "gomerax";
    if (e.parallel) e.gain_offset = 1.f;                       // its norm gains are stored around zero
    // the runs: layers before the loop once, the loop's span `times` times, the rest once
    std::vector<std::pair<int, int>> runs;      // (layer, pass it opens or -1)
    {
        const int nl = (int)ls.arr.size();
        int start = 0, stop = 0, times = 1;
        if (cfg.has("loop")) {
            const Json& lp = cfg.at("loop");
            start = lp.integer("start"); stop = lp.integer("stop"); times = lp.integer("times");
            AHA_REQUIRE(e.sandwich || e.parallel, "config.json: 'loop' is only known to the sandwich and parallel layer templates");
            AHA_REQUIRE(0 <= start && start <= stop && stop <= nl && times >= 1, "config.json: bad 'loop'");
        }
        for (int l = 0; l < start; ++l) runs.push_back({l, -1});
        if (stop > start)
            for (int t = 0; t < times; ++t)
                for (int l = start; l < stop; ++l) runs.push_back({l, l == start ? t : -1});
        for (int l = stop; l < nl; ++l) runs.push_back({l, -1});
        if (stop > start && e.sandwich) e.loop_step = e.vec(wt, "loop.step", (size_t)times * e.W);
    }
    e.L = (int)runs.size();
    if (e.parallel && cfg.has("embedding")) e.embed_scale = (float)cfg.at("embedding").number_or("scale", 1.0);
    if (e.sandwich) {
        e.norm_groups = cfg.at("norm").integer_or("groups", 1);
        AHA_REQUIRE(e.norm_groups >= 1 && e.W % e.norm_groups == 0, "config.json: norm.groups must divide the width");
        e.resid_mult = (float)cfg.number_or("residual_mult", 1.0);
        e.logit_scale = (float)cfg.number_or("logit_scale", 1.0);
        if (cfg.has("embedding")) e.embed_scale = (float)cfg.at("embedding").number_or("scale", 1.0);
        e.conv_taps = cfg.has("canon") ? cfg.at("canon").integer("taps") : 0;
        AHA_REQUIRE(e.conv_taps >= 0 && e.conv_taps <= kShortConvMaxTaps, "config.json: canon.taps must be at most 16");
    }
    e.slots = std::max(1, opt.max_seqs);
    e.num_pages = std::max(1, ceil_div(std::max(1, opt.max_tokens), kPage));
    e.max_pages = e.num_pages;
    e.Tmax = std::max(1, opt.max_step_tokens);
    e.Rmax = std::min(e.Tmax, 128);
    e.embed = e.load_linear(wt, {"embed"}, {e.V}, e.W, {}).w;
    e.head = e.load_linear(wt, {wt.has("head") ? "head" : "embed"}, {e.V}, e.W, {});      // no 'head' tensor: the embedding table is the output projection
    if (e.sandwich || e.parallel) e.final_w = e.gain_vec(wt, "final.norm", (size_t)e.W);
    else e.final_gain = upload_scalar(e, wt, "final.norm");
    if (e.parallel && wt.has("pos")) {      // learned position rows [max_positions, W]
        const aha_tensor_desc& dp = wt.get("pos");
        AHA_REQUIRE(dp.rank == 2 && dp.shape[1] == e.W && dp.shape[0] >= 1, "weight 'pos' must be [positions, width]");
        e.max_positions = (int)dp.shape[0];
        if (cfg.has("max_positions")) AHA_REQUIRE(cfg.integer("max_positions") <= e.max_positions, "config.json: max_positions exceeds the rows of 'pos'");
        e.pos_table = e.vec(wt, "pos", (size_t)e.max_positions * e.W);
    }
    int proj_cols = 1, inner_cols = 1, q_cols = 1;
    size_t route_ints = 0;
    for (int r = 0; r < e.L; ++r) {
        const int l = runs[r].first;
        const Json& ly = ls.arr[l];
        const std::string p = "l" + std::to_string(l) + ".";
        const std::string type = ly.string_or("type", "");
        auto it = find_for_design(mixer_registry(), e.design, type);
        AHA_REQUIRE(it != mixer_registry().end(), "config.json: layer " + std::to_string(l) + " has an unknown mixer type '" + type + "'");
        Engine::LayerRec rec;
        rec.mixer = it->second(e, ly.at("mixer"), wt, p + "mix.", l);
        e.mixer_of_layer.push_back(rec.mixer.get());
        rec.pass = runs[r].second;
        rec.reinject = e.parallel && rec.pass >= 1;
        auto conv_state = [&](const std::string& name, float*& w, float*& tails) {
            if (e.conv_taps < 1 || !wt.has(name)) return;
            w = e.vec(wt, name, (size_t)e.W * e.conv_taps);
            const size_t n = std::max<size_t>(1, (size_t)(e.conv_taps - 1) * e.W * e.slots);
            tails = ctx.alloc<float>(n);
            AHA_CUDA_CHECK(cudaMemset(tails, 0, n * sizeof(float)));
        };
        if (e.sandwich) {
            rec.pre1 = e.vec(wt, p + "norm1", (size_t)e.W); rec.post1 = e.vec(wt, p + "norm1b", (size_t)e.W);
            conv_state(p + "canon1", rec.conv1, rec.tails1);
        } else if (e.parallel) rec.pre1 = e.gain_vec(wt, p + "norm1", (size_t)e.W);
        else rec.gain1 = upload_scalar(e, wt, p + "norm1");
        if (ly.has("mlp") && ly.at("mlp").kind == Json::Obj) {
            const Json& ml = ly.at("mlp");
            const std::string kind = ml.string_or("kind", "");
            auto jt = find_for_design(ff_registry(), e.design, kind);
            AHA_REQUIRE(jt != ff_registry().end(), "config.json: layer " + std::to_string(l) + " has an unknown feed-forward kind '" + kind + "'");
            rec.ff = jt->second(e, ml, wt, p + "mlp.");
            if (e.sandwich) {
                rec.pre2 = e.vec(wt, p + "norm2", (size_t)e.W); rec.post2 = e.vec(wt, p + "norm2b", (size_t)e.W);
                conv_state(p + "canon2", rec.conv2, rec.tails2);
            } else if (!e.parallel) rec.gain2 = upload_scalar(e, wt, p + "norm2");
            route_ints = std::max(route_ints, rec.ff->route_ints());
        }
        for (Sublayer* s : {rec.mixer.get(), rec.ff.get()})
            if (s) { proj_cols = std::max(proj_cols, s->proj_cols()); inner_cols = std::max(inner_cols, s->inner_cols()); q_cols = std::max(q_cols, s->q_cols()); }
        e.layers.push_back(std::move(rec));
    }
    e.wbytes = ctx.alloc_bytes - before;
    // pools and scratch
    for (int p = 0; p < e.num_pages; ++p) e.free_pages.push_back(p);
    e.h_tables.resize(e.slots);
    e.seqs.resize(e.slots);
    e.d_tables = ctx.alloc<int>((size_t)e.slots * e.max_pages);
    AHA_CUDA_CHECK(cudaMemset(e.d_tables, 0, (size_t)e.slots * e.max_pages * sizeof(int)));
    const size_t T = e.Tmax;
    e.x = ctx.alloc<float>(T * e.W); e.y = ctx.alloc<float>(T * e.W);
    if (e.sandwich) { e.hnorm = ctx.alloc<float>(T * e.W); e.hin = ctx.alloc<float>(T * e.W); }
    if (e.parallel) {
        e.hnorm = ctx.alloc<float>(T * e.W); e.y2 = ctx.alloc<float>(T * e.W);
        bool again = false;
        for (auto& ly : e.layers) again = again || ly.reinject;
        if (again) e.x0 = ctx.alloc<float>(T * e.W);
    }
    if (route_ints) e.route_buf = ctx.alloc<int>(route_ints);
    {
        size_t ga = 0, kvf = 0, of = 0, sh = 0;
        for (auto& ly : e.layers) {
            ga = std::max(ga, ly.mixer->expand_gather_floats()); kvf = std::max(kvf, ly.mixer->expand_kv_floats());
            of = std::max(of, ly.mixer->expand_out_floats()); sh = std::max(sh, ly.mixer->expand_split_halfs());
        }
        if (ga) e.lat_gather = ctx.alloc<float>(ga);
        if (kvf) e.lat_kv = ctx.alloc<float>(kvf);
        if (of) e.lat_out = ctx.alloc<float>(of);
        if (sh) ctx.split_buf(sh);
    }
    e.proj = ctx.alloc<float>(T * proj_cols); e.inner = ctx.alloc<float>(T * inner_cols); e.qbuf = ctx.alloc<float>(T * q_cols);
    if (!e.fp32) { gemm_tc_init(); flash_attn_tc_init(); ctx.split_buf(T * (size_t)std::max({e.W, proj_cols, inner_cols})); }
    size_t part = 0;
    for (auto& ly : e.layers) part = std::max(part, ly.mixer->attn_part_floats());
    if (part) e.attn_part = ctx.alloc<float>(part);
    size_t seg_s = 0, seg_d = 0;
    for (auto& ly : e.layers) { seg_s = std::max(seg_s, ly.mixer->seg_state_floats()); seg_d = std::max(seg_d, ly.mixer->seg_decay_floats()); }
    if (seg_s) { e.seg_state = ctx.alloc<float>(seg_s); e.seg_decay = ctx.alloc<float>(seg_d); }
    e.hn = ctx.alloc<float>((size_t)e.Rmax * e.W); e.logits = ctx.alloc<float>((size_t)e.Rmax * e.V);
    e.meta_ints = 4 * T + (e.slots + 1) + 2 * e.slots + (T + e.slots);
    e.d_meta = ctx.alloc<int>(e.meta_ints);
    AHA_CUDA_CHECK(cudaMallocHost(&e.h_meta, e.meta_ints * sizeof(int)));
    std::memset(e.h_meta, 0, e.meta_ints * sizeof(int));
    AHA_CUDA_CHECK(cudaEventCreateWithFlags(&e.ev_meta, cudaEventDisableTiming));
    e.hist_cap = std::max(64, e.num_pages * kPage);
    e.d_states = ctx.alloc<DecodeState>(e.slots);
    AHA_CUDA_CHECK(cudaMemset(e.d_states, 0, e.slots * sizeof(DecodeState)));
    e.d_hist = ctx.alloc<uint32_t>((size_t)e.slots * e.hist_cap);
    e.d_tok = ctx.alloc<uint32_t>(e.slots);
    AHA_CUDA_CHECK(cudaMemset(e.d_tok, 0, e.slots * sizeof(uint32_t)));
    e.pmax = ctx.alloc<float>(e.n_pcand); e.pidx = ctx.alloc<int>(e.n_pcand);
    e.sample_work = ctx.alloc<float>((size_t)e.V);
    e.d_sample_err = ctx.alloc<int>(1);
    AHA_CUDA_CHECK(cudaMemset(e.d_sample_err, 0, sizeof(int)));
    return E.release();
}

}  // namespace aha
