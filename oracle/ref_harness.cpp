// TEST INFRASTRUCTURE ONLY. C entry points around the REFERENCE's own NF4 operator
// (src/ops/Bnb4BitLinear.cpp, compiled unmodified from where it lies, against the stand-in headers
// in ref_shim/): host arrays in, host arrays out. Used by the tests to check the CPU oracle's
// restatement against the code it restates; never by the product.
//
// What this pins: Bnb4BitLinear::init (nested absmax expansion, :453-497), init_fused_rows
// (:499-629), dequantize_weight (:723-757), packed_nf4_gemv_bf16 (:271-410, both branches),
// packed_nf4_gemv_gate_up_swiglu (:142-246), the forward dispatch (:799-949). What it cannot pin:
// the order of sub-group / work-group reductions (unspecified by SYCL; the stand-in uses a balanced
// tree) and the bf16 matmul of the seq_len > 1 route (oneDNN in the reference; a plain fp32 loop in
// the stand-in).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <memory>
#include <numeric>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include <sycl/sycl.hpp>
#include <dnnl.hpp>

// the harness reads two private members (absmax_f32_, dequantize_weight) to expose intermediate
// results; the class layout is the same in both translation units
#define private public
#include "ops/Bnb4BitLinear.hpp"
#undef private

extern "C" {

struct AilaRefWeight {
    const uint8_t* packed;        // [N*K/2]
    const void* absmax;           // u8 codes (nested) or fp32, one per block
    const float* quant_map;       // [16]
    const float* nested_absmax;   // [ceil(blocks / nested_blocksize)] or NULL
    const float* nested_quant_map;  // [256] or NULL
    int64_t nested_absmax_count;
    int64_t out_features, in_features;
    int32_t blocksize, nested, nested_blocksize;
    float nested_offset;
};

}  // extern "C"

namespace {

using bf16 = sycl::ext::oneapi::bfloat16;
using dt = dnnl::memory::data_type;

struct Loaded {
    Tensor packed, absmax, qmap, nabs, nmap, state;
    Bnb4BitWeightRef ref;
    Bnb4BitLinear linear;
};

Context& context() {
    static Context ctx;
    return ctx;
}

void copy_error(const std::string& msg, char* err, int cap) {
    if (err && cap > 0) {
        std::snprintf(err, static_cast<size_t>(cap), "%s", msg.c_str());
    }
}

// Tensors are views of the caller's host arrays ("device" memory is host memory here).
std::unique_ptr<Loaded> load(const AilaRefWeight& w, std::string* error) {
    Context& ctx = context();
    auto L = std::make_unique<Loaded>();
    const int64_t N = w.out_features, K = w.in_features;
    const int64_t blocks = (N * K + w.blocksize - 1) / w.blocksize;
    static uint8_t state_bytes[4] = {'{', '}', 0, 0};
    L->packed = Tensor::view(ctx, const_cast<uint8_t*>(w.packed), {N * K / 2, 1}, dt::u8);
    L->absmax = Tensor::view(ctx, const_cast<void*>(w.absmax), {blocks}, w.nested ? dt::u8 : dt::f32);
    L->qmap = Tensor::view(ctx, const_cast<float*>(w.quant_map), {16}, dt::f32);
    L->state = Tensor::view(ctx, state_bytes, {2}, dt::u8);
    L->ref.name = "w";
    L->ref.packed_weight = &L->packed;
    L->ref.absmax = &L->absmax;
    L->ref.quant_map = &L->qmap;
    L->ref.packed_quant_state = &L->state;
    L->ref.quant_state.quant_type = "nf4";
    L->ref.quant_state.dtype = "bfloat16";
    L->ref.quant_state.shape = {N, K};
    L->ref.quant_state.blocksize = w.blocksize;
    if (w.nested) {
        L->nabs = Tensor::view(ctx, const_cast<float*>(w.nested_absmax), {w.nested_absmax_count}, dt::f32);
        L->nmap = Tensor::view(ctx, const_cast<float*>(w.nested_quant_map), {256}, dt::f32);
        L->ref.nested_absmax = &L->nabs;
        L->ref.nested_quant_map = &L->nmap;
        L->ref.quant_state.nested = true;
        L->ref.quant_state.nested_blocksize = w.nested_blocksize;
        L->ref.quant_state.nested_dtype = "float32";
        L->ref.quant_state.nested_offset = w.nested_offset;
    }
    if (!L->linear.init(ctx, L->ref, error)) return nullptr;
    return L;
}

template <typename F>
int guarded(char* err, int cap, F&& f) {
    try {
        return f();
    } catch (const std::exception& e) {
        copy_error(e.what(), err, cap);
        return -1;
    }
}

}  // namespace

extern "C" {

// y[M][N_total] = forward(x[M][K]) of one linear, or of init_fused_rows over 2..4 linears.
// Returns 0, or -1 with a message.
int aila_ref_forward(const AilaRefWeight* weights, int n_weights, const uint16_t* x, int M, uint16_t* y,
                     const uint16_t* add_residual, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Context& ctx = context();
        std::string msg;
        std::vector<std::unique_ptr<Loaded>> parts;
        for (int i = 0; i < n_weights; ++i) {
            parts.push_back(load(weights[i], &msg));
            if (!parts.back()) throw std::runtime_error(msg);
        }
        Bnb4BitLinear fused;
        Bnb4BitLinear* lin = &parts[0]->linear;
        if (n_weights > 1) {
            bool ok = false;
            if (n_weights == 2) ok = fused.init_fused_rows(ctx, parts[0]->linear, parts[1]->linear, &msg);
            else if (n_weights == 3)
                ok = fused.init_fused_rows(ctx, parts[0]->linear, parts[1]->linear, parts[2]->linear, &msg);
            else if (n_weights == 4)
                ok = fused.init_fused_rows(ctx, parts[0]->linear, parts[1]->linear, parts[2]->linear,
                                           parts[3]->linear, &msg);
            else
                msg = "2 to 4 linears can be fused";
            if (!ok) throw std::runtime_error(msg);
            lin = &fused;
        }
        const int64_t K = lin->in_features(), N = lin->out_features();
        Tensor in = Tensor::view(ctx, const_cast<uint16_t*>(x), {M, K}, dt::bf16);
        Tensor out = Tensor::view(ctx, y, {M, N}, dt::bf16);
        Bnb4BitLinearScratch scratch;
        lin->forward(ctx, scratch, in, out, M, reinterpret_cast<const bf16*>(add_residual));
        ctx.synchronize();
        return 0;
    });
}

// out[ff] = try_forward_decode_gate_up_swiglu on init_fused_rows(gate, up). Returns 1 when the
// fused path ran, 0 when the reference declined it, -1 with a message on an error.
int aila_ref_gate_up_swiglu(const AilaRefWeight* gate, const AilaRefWeight* up, const uint16_t* x, int ff_dim,
                            uint16_t* out, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Context& ctx = context();
        std::string msg;
        auto g = load(*gate, &msg);
        if (!g) throw std::runtime_error(msg);
        auto u = load(*up, &msg);
        if (!u) throw std::runtime_error(msg);
        Bnb4BitLinear fused;
        if (!fused.init_fused_rows(ctx, g->linear, u->linear, &msg)) throw std::runtime_error(msg);
        Tensor in = Tensor::view(ctx, const_cast<uint16_t*>(x), {1, (int64_t)fused.in_features()}, dt::bf16);
        Tensor o = Tensor::view(ctx, out, {1, (int64_t)ff_dim}, dt::bf16);
        const bool ran = Bnb4BitLinear::try_forward_decode_gate_up_swiglu(ctx, fused, in, o, ff_dim);
        ctx.synchronize();
        return ran ? 1 : 0;
    });
}

// The per-block fp32 absmax that init leaves in the linear (:472-494).
int aila_ref_expand_absmax(const AilaRefWeight* w, float* out, char* err, int cap) {
    return guarded(err, cap, [&]() {
        std::string msg;
        auto L = load(*w, &msg);
        if (!L) throw std::runtime_error(msg);
        const int64_t blocks = (w->out_features * w->in_features + w->blocksize - 1) / w->blocksize;
        std::memcpy(out, L->linear.absmax_f32_.data(), static_cast<size_t>(blocks) * sizeof(float));
        return 0;
    });
}

// dequantize_weight: bf16 [K][N] (transposed, as the reference stores it for its matmul).
int aila_ref_dequantize(const AilaRefWeight* w, uint16_t* out_kn, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Context& ctx = context();
        std::string msg;
        auto L = load(*w, &msg);
        if (!L) throw std::runtime_error(msg);
        Tensor view = Tensor::view(ctx, out_kn, {w->in_features, w->out_features}, dt::bf16);
        L->linear.dequantize_weight(ctx, view);
        ctx.synchronize();
        return 0;
    });
}

}  // extern "C"
