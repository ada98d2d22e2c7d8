// TEST INFRASTRUCTURE ONLY. C entry points around the REFERENCE's own operators that sit between
// the NF4 linears of a decode step (src/ops/NormOps.cpp, src/ops/ElementwiseOps.cpp, src/ops/SamplingOps.cpp, src/ops/AttentionOps.cpp, compiled
// unmodified from where they lie against the stand-in headers in ref_shim/): host arrays in, host
// arrays out. Used by the tests to check the CPU oracle's restatement; never by the product.
//
// Pinned through here: ops::rms_norm (NormOps.cpp:14-75), ops::fused_add_rms_norm (:141-275),
// ops::embedding_lookup (ElementwiseOps.cpp:14-27), ops::decode_prepare_qkv (:105-215), ops::swiglu
// (:223-245), ops::fused_gate_up_swiglu (:247-294), ops::argmax (src/ops/SamplingOps.cpp:321-358),
// ops::attention_decode (src/ops/AttentionOps.cpp:499-647 -> attention_decode_baseline :73-166).
// The stand-in fixes what SYCL leaves open: reduce_over_group adds in a balanced tree,
// native::exp/cos/sin are libm's.
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "ops/Ops.hpp"
#include "profile/Profiling.hpp"

// the reference's logger (its own definition lives in a source file that is not part of this build)
namespace aila {
void log(LogLevel, const char*, ...) {}
}  // namespace aila

namespace {

using dt = dnnl::memory::data_type;

Context& context() {
    static Context ctx;
    return ctx;
}

template <typename F>
int guarded(char* err, int cap, F&& f) {
    try {
        f();
        context().synchronize();
        return 0;
    } catch (const std::exception& e) {
        if (err && cap > 0) std::snprintf(err, static_cast<size_t>(cap), "%s", e.what());
        return -1;
    }
}

Tensor bf16_view(void* p, std::initializer_list<int64_t> shape) {
    return Tensor::view(context(), p, std::vector<int64_t>(shape), dt::bf16);
}

}  // namespace

extern "C" {

// out = rms_norm(in) * weight; in [rows][hidden]
int aila_ref_rms_norm(uint16_t* in, uint16_t* weight, float eps, uint16_t* out, int rows, int hidden, char* err,
                      int cap) {
    return guarded(err, cap, [&]() {
        Tensor i = bf16_view(in, {rows, hidden}), w = bf16_view(weight, {hidden}), o = bf16_view(out, {rows, hidden});
        ops::rms_norm(context(), i, w, eps, o, rows, hidden);
    });
}

// in <- bf16(in + residual) (in place, as the reference does); out = rms_norm of the sum * weight
int aila_ref_fused_add_rms_norm(uint16_t* in, uint16_t* residual, uint16_t* weight, float eps, uint16_t* out,
                                int rows, int hidden, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Tensor i = bf16_view(in, {rows, hidden}), r = bf16_view(residual, {rows, hidden}),
               w = bf16_view(weight, {hidden}), o = bf16_view(out, {rows, hidden});
        ops::fused_add_rms_norm(context(), i, r, w, eps, o, rows, hidden);
    });
}

int aila_ref_embedding_lookup(uint16_t* table, int vocab, const int32_t* ids, int seq_len, uint16_t* out, int hidden,
                              char* err, int cap) {
    return guarded(err, cap, [&]() {
        Tensor t = bf16_view(table, {vocab, hidden}), o = bf16_view(out, {seq_len, hidden});
        ops::embedding_lookup(context(), t, ids, seq_len, o, hidden);
    });
}

// q [heads*hd], k and v [kv*hd] are updated in place; caches are [kv][max_seq_len][hd]
int aila_ref_decode_prepare_qkv(uint16_t* q, uint16_t* k, uint16_t* v, float* rope_freq, uint16_t* q_norm,
                                uint16_t* k_norm, uint16_t* k_cache, uint16_t* v_cache, int max_seq_len, int start_pos,
                                int heads, int kv_heads, int head_dim, float eps, float theta, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Context& ctx = context();
        Tensor tq = bf16_view(q, {1, (int64_t)heads * head_dim}), tk = bf16_view(k, {1, (int64_t)kv_heads * head_dim}),
               tv = bf16_view(v, {1, (int64_t)kv_heads * head_dim});
        Tensor tf = Tensor::view(ctx, rope_freq, {(int64_t)head_dim / 2}, dt::f32);
        Tensor qn = bf16_view(q_norm, {head_dim}), kn = bf16_view(k_norm, {head_dim});
        Tensor kc = bf16_view(k_cache, {kv_heads, max_seq_len, head_dim}),
               vc = bf16_view(v_cache, {kv_heads, max_seq_len, head_dim});
        ops::decode_prepare_qkv(ctx, tq, tk, tv, tf, qn, kn, kc, vc, start_pos, heads, kv_heads, head_dim, eps, theta);
    });
}

// single-token attention over the first cached_len cache rows; caches are [kv][max_seq_len][hd]
int aila_ref_attention_decode(uint16_t* q, uint16_t* k_cache, uint16_t* v_cache, uint16_t* out, int max_seq_len,
                              int heads, int kv_heads, int head_dim, int cached_len, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Context& ctx = context();
        Tensor tq = bf16_view(q, {1, (int64_t)heads * head_dim}), to = bf16_view(out, {1, (int64_t)heads * head_dim});
        Tensor kc = bf16_view(k_cache, {kv_heads, max_seq_len, head_dim}),
               vc = bf16_view(v_cache, {kv_heads, max_seq_len, head_dim});
        Tensor scores = Tensor::allocate(ctx, {(int64_t)heads, (int64_t)max_seq_len}, dt::f32);
        ops::attention_decode(ctx, tq, kc, vc, to, scores, heads, kv_heads, head_dim, cached_len, nullptr);
    });
}

// the token ops::argmax chooses over n bf16 logits
int aila_ref_argmax(uint16_t* logits, int n, int32_t* out, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Tensor l = bf16_view(logits, {n});
        int result = -1;
        ops::argmax(context(), l, n, &result);
        *out = result;
    });
}

int aila_ref_swiglu(uint16_t* gate, uint16_t* up, uint16_t* out, int n, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Tensor g = bf16_view(gate, {n}), u = bf16_view(up, {n}), o = bf16_view(out, {n});
        ops::swiglu(context(), g, u, o, n);
    });
}

int aila_ref_fused_gate_up_swiglu(uint16_t* gate_up, uint16_t* out, int ff_dim, char* err, int cap) {
    return guarded(err, cap, [&]() {
        Tensor gu = bf16_view(gate_up, {2 * (int64_t)ff_dim}), o = bf16_view(out, {ff_dim});
        ops::fused_gate_up_swiglu(context(), gu, o, ff_dim);
    });
}

}  // extern "C"
