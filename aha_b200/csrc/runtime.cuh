// runtime.cuh -- what every model of the library shares on the host side: the per-handle launch context (stream, device
// allocations, counters), the checkpoint tensor table with its dtype conversions, and upload helpers.
#pragma once
#include <cmath>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/aha_b200.h"
#include "common.cuh"

namespace aha {

// ---------------------------------------------------------------------------------------------------
struct Counters {
    uint64_t kernels = 0, graphs = 0;
};

struct Ctx {  // per-handle launch context
    cudaStream_t stream = nullptr;
    int device = 0;
    int num_sms = 148;
    Counters cnt;
    bool capturing = false;
    std::vector<void*> allocs;
    size_t alloc_bytes = 0;
    int attn_impl = 0;            // 0 = auto (tcgen05 flash attention for head_dim 64, mma.sync for 128), 1 = fp32 SIMT flash attention, 2 = mma.sync everywhere
    int gemm_impl = 0;            // 0 = auto (tcgen05 where the shape tiles), 1 = SIMT fp32, 2 / 3 / 4 = tcgen05 required: 128 x 128 tiles / persistent 128 x 256 / CTA-pair 256 x 256
    bool gemm_wide = true;        // auto: the persistent 128 x 256 kernel where N >= 256 (15-26 % faster than 128 x 128 on every prefill shape, profiles/r02_gemm_sweep.txt; AHA_GEMM_WIDE=0 turns it off)
    bool gemm_pair = true;        // auto: the CTA-pair kernel (cta_group::2, 256 x 256 tile per cluster) for prefill-sized M (>= 1024) and N >= 256: 1-3 % over the
                                  // single-CTA persistent kernel, bit-identical results (profiles/r02_gemm_sweep_pair.txt; AHA_GEMM_PAIR=0 turns it off)
    int gemm_group_m = 8;         // row blocks per band of the persistent kernel's tile walk (AHA_GEMM_GROUP)
    __half* split_ws = nullptr;   // [2][rows*K] hi | lo halves of the activation operand
    size_t split_cap = 0;         // halfs per half-buffer
    __half* split_buf(size_t halfs) {
        if (halfs > split_cap) {
            if (split_ws) { AHA_CUDA_CHECK(cudaStreamSynchronize(stream)); cudaFree(split_ws); }
            AHA_CUDA_CHECK(cudaMalloc(&split_ws, 2 * halfs * sizeof(__half)));
            split_cap = halfs;
        }
        return split_ws;
    }

    // Pre-split activations (two ping-pong buffers): a producer -- norm kernel, attention, GEMM epilogue -- writes the fp16 hi + lo
    // halves the next tensor-core GEMM reads, instead of an fp32 tensor that linear_gemm would have to read back and split.
    bool presplit = true;         // AHA_PRESPLIT=0: every GEMM splits its own fp32 input (the data flow without a shared split pass; results are bit-identical)
    __half* act_ws[2] = {nullptr, nullptr};
    size_t act_cap[2] = {0, 0};
    __half* act_split(int which, size_t halfs) {   // hi at the returned pointer, lo at + act_cap[which]
        if (halfs > act_cap[which]) {
            if (act_ws[which]) { AHA_CUDA_CHECK(cudaStreamSynchronize(stream)); cudaFree(act_ws[which]); }
            AHA_CUDA_CHECK(cudaMalloc(&act_ws[which], 2 * halfs * sizeof(__half)));
            act_cap[which] = halfs;
        }
        return act_ws[which];
    }

    template <typename T>
    T* alloc(size_t n) {
        void* p = nullptr;
        AHA_CUDA_CHECK(cudaMalloc(&p, std::max<size_t>(n, 1) * sizeof(T)));
        allocs.push_back(p);
        alloc_bytes += n * sizeof(T);
        return reinterpret_cast<T*>(p);
    }
    void free_all() {
        for (void* p : allocs) cudaFree(p);
        allocs.clear();
        if (split_ws) { cudaFree(split_ws); split_ws = nullptr; split_cap = 0; }
        for (int i = 0; i < 2; ++i)
            if (act_ws[i]) { cudaFree(act_ws[i]); act_ws[i] = nullptr; act_cap[i] = 0; }
    }
};

// ---------------------------------------------------------------------------------------------------
// Host-side weight table (descs by name) + dtype conversion.
inline float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
    uint32_t f;
    if (exp == 0) {
        if (man == 0) f = sign << 31;
        else {
            int e = -1; uint32_t m = man;
            do { ++e; m <<= 1; } while (!(m & 0x400));
            f = (sign << 31) | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3ff) << 13);
        }
    } else if (exp == 31) f = (sign << 31) | 0x7f800000u | (man << 13);
    else f = (sign << 31) | ((exp + 112) << 23) | (man << 13);
    float r; std::memcpy(&r, &f, 4); return r;
}
inline float bf16_bits_to_float(uint16_t b) { uint32_t f = (uint32_t)b << 16; float r; std::memcpy(&r, &f, 4); return r; }

struct WeightTable {
    std::map<std::string, const aha_tensor_desc*> by_name;
    explicit WeightTable(const aha_tensor_desc* w, size_t n) {
        for (size_t i = 0; i < n; ++i)
            if (w[i].name) by_name[w[i].name] = &w[i];
    }
    bool has(const std::string& n) const { return by_name.count(n) != 0; }
    const aha_tensor_desc& get(const std::string& n) const {
        auto it = by_name.find(n);
        if (it == by_name.end()) throw std::runtime_error("missing weight tensor '" + n + "'");
        return *it->second;
    }
    static size_t numel(const aha_tensor_desc& d) { size_t n = 1; for (int i = 0; i < d.rank; ++i) n *= (size_t)d.shape[i]; return n; }
    // element i as float
    static float at(const aha_tensor_desc& d, size_t i) {
        switch (d.dtype) {
            case AHA_F32: return reinterpret_cast<const float*>(d.data)[i];
            case AHA_F16: return half_bits_to_float(reinterpret_cast<const uint16_t*>(d.data)[i]);
            case AHA_BF16: return bf16_bits_to_float(reinterpret_cast<const uint16_t*>(d.data)[i]);
            default: throw std::runtime_error(std::string("weight '") + (d.name ? d.name : "?") + "': unsupported dtype");
        }
    }
    void expect(const std::string& n, std::initializer_list<int64_t> shape) const {
        const aha_tensor_desc& d = get(n);
        size_t want = 1; for (auto s : shape) want *= (size_t)s;
        if (numel(d) != want) throw std::runtime_error("weight '" + n + "' has " + std::to_string(numel(d)) + " elements, expected " + std::to_string(want));
    }
    // rows [r0, r0+nr) of a [R, C] matrix -> fp16 staging (cols [c0, c0+nc))
    void rows_to_half(const std::string& n, int64_t R, int64_t C, int64_t r0, int64_t nr, int64_t c0, int64_t nc, __half* dst, int64_t dst_ld) const {
        const aha_tensor_desc& d = get(n);
        if ((int64_t)numel(d) != R * C) throw std::runtime_error("weight '" + n + "': unexpected size");
        if (d.dtype == AHA_F16) {
            const uint16_t* s = reinterpret_cast<const uint16_t*>(d.data);
            for (int64_t r = 0; r < nr; ++r) std::memcpy(reinterpret_cast<uint16_t*>(dst) + r * dst_ld, s + (r0 + r) * C + c0, (size_t)nc * 2);
        } else {
            // bf16 / f32 checkpoints are narrowed to fp16 (8 -> 10 mantissa bits for bf16: exact inside fp16's normal range).  A value
            // outside that range would silently become inf (|w| > 65504) or lose bits (|w| < 2^-14): refuse the checkpoint loudly.
            for (int64_t r = 0; r < nr; ++r)
                for (int64_t c = 0; c < nc; ++c) {
                    const float v = at(d, (size_t)((r0 + r) * C + c0 + c));
                    const float av = std::fabs(v);
                    if (!(av <= 65504.0f)) throw std::runtime_error("weight '" + n + "' holds a value outside the fp16 range (|w| > 65504 or not finite): this build stores linear weights as fp16");
                    if (d.dtype == AHA_BF16 && av != 0.0f && av < 6.103515625e-05f) throw std::runtime_error("weight '" + n + "' holds a bf16 value below fp16's normal range (|w| < 2^-14): it would lose bits as fp16");
                    dst[r * dst_ld + c] = __float2half_rn(v);
                }
        }
    }
    std::vector<float> vec_f32(const std::string& n, size_t expect_n) const {
        const aha_tensor_desc& d = get(n);
        if (numel(d) != expect_n) throw std::runtime_error("weight '" + n + "': unexpected size");
        std::vector<float> v(expect_n);
        for (size_t i = 0; i < expect_n; ++i) v[i] = at(d, i);
        return v;
    }
};

template <typename T>
inline T* upload(Ctx& c, const std::vector<T>& h) {
    T* d = c.alloc<T>(h.size());
    AHA_CUDA_CHECK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}
inline float* upload_vec(Ctx& c, const WeightTable& wt, const std::string& name, size_t n) { return upload(c, wt.vec_f32(name, n)); }

}  // namespace aha
