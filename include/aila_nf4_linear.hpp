// aila_nf4_linear.hpp - header-only C++ adapter that keeps the reference operator's interface
// (class Bnb4BitLinear, struct Bnb4BitLinearScratch; reference src/ops/Bnb4BitLinear.hpp:12-59)
// on top of the C ABI in aila_nf4.h, so the two model backends that call it
// (src/models/Qwen3Bnb4Backend.cpp:339-418, src/models/Qwen35HybridBnb4Backend.cpp:2167-2197)
// compile against it with their call sites unchanged.
//
// What changes for the caller
//   Context      -> aila::nf4::Context {device ordinal, cudaStream_t}: the reference's Context
//                   (src/core/Context.hpp:14-90) owns one in-order SYCL queue; here the caller's
//                   CUDA stream plays that role.
//   Tensor       -> aila::nf4::TensorView {void* data, dims, is_bf16}: the subset of
//                   src/core/Tensor.hpp:15-202 the operator touches (data(), dtype(), ndim()).
//   Bnb4BitWeightRef -> AilaNf4WeightDesc (same tensors as raw pointers, aila_nf4.h).
// Error behaviour is the reference's: init* return bool and fill *error_message, forward throws
// std::runtime_error, try_forward_decode_gate_up_swiglu returns false to mean "fall back".
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "aila_nf4.h"

namespace aila {
namespace nf4 {

struct Context {
    int device = 0;
    void* stream = nullptr;  // cudaStream_t
    // Work space of the calls that take no scratch argument in the reference
    // (try_forward_decode_gate_up_swiglu(ctx, fused, in, out, ff)): one per context, made on first use.
    AilaNf4Scratch* decode_scratch = nullptr;

    Context() = default;
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
    ~Context() { aila_nf4_scratch_destroy(decode_scratch); }
};

struct TensorView {
    void* ptr = nullptr;
    int64_t rows = 0, cols = 0;
    int dims = 2;
    bool bf16 = true;
    void* data() const { return ptr; }
    int ndim() const { return dims; }
    bool is_bf16() const { return bf16; }
};

// Bnb4BitLinearScratch (reference src/ops/Bnb4BitLinear.hpp:12-24): grow-only work space
// shared by all linears of one backend.
struct Bnb4BitLinearScratch {
    AilaNf4Scratch* handle = nullptr;

    Bnb4BitLinearScratch() = default;
    Bnb4BitLinearScratch(const Bnb4BitLinearScratch&) = delete;
    Bnb4BitLinearScratch& operator=(const Bnb4BitLinearScratch&) = delete;
    ~Bnb4BitLinearScratch() { aila_nf4_scratch_destroy(handle); }

    // Bnb4BitLinearScratch::ensure (reference src/ops/Bnb4BitLinear.cpp:414-451).
    void ensure(Context& ctx, int seq_len, int in_features, int out_features, bool need_weight) {
        open(ctx);
        if (aila_nf4_scratch_reserve(handle, seq_len, in_features, out_features,
                                     need_weight ? 1 : 0) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
    }

    void open(Context& ctx) {
        if (!handle && aila_nf4_scratch_create(ctx.device, &handle) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
    }
};

// Dense bf16 linear (reference class Linear, src/ops/Ops.hpp:16-31): weight [out_features,
// in_features] bf16 in host or device memory, copied at init. forward throws like the reference
// operator on a contract violation.
class Linear {
public:
    Linear() = default;
    Linear(const Linear&) = delete;
    Linear& operator=(const Linear&) = delete;
    ~Linear() { aila_dense_linear_destroy(handle_); }

    void init(Context& ctx, const void* weight_bf16, int in_features, int out_features,
              bool weight_on_device = true) {
        AilaDenseLinear* fresh = nullptr;
        if (aila_dense_linear_create(weight_bf16, out_features, in_features, weight_on_device ? 1 : 0,
                                     ctx.device, &fresh) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
        aila_dense_linear_destroy(handle_);
        handle_ = fresh;
    }

    void forward(Context& ctx, Bnb4BitLinearScratch& scratch, TensorView& input, TensorView& output,
                 int seq_len, const void* add_residual = nullptr) {
        if (!input.is_bf16() || !output.is_bf16())
            throw std::runtime_error("Linear expects bf16 input/output tensors");
        scratch.open(ctx);
        if (aila_dense_linear_forward(handle_, scratch.handle, input.data(), output.data(), seq_len,
                                      add_residual, ctx.stream) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
    }

    int in_features() const { return (int)aila_dense_linear_in_features(handle_); }
    int out_features() const { return (int)aila_dense_linear_out_features(handle_); }

private:
    AilaDenseLinear* handle_ = nullptr;
};

// ops::argmax (reference src/ops/SamplingOps.cpp:321-365): greedy token over bf16 logits,
// written to device memory; equal logits resolve as in the reference's reduction.
inline void argmax(Context& ctx, TensorView& logits, int vocab_size, int* d_result) {
    if (aila_argmax_bf16(logits.data(), vocab_size, d_result, ctx.device, ctx.stream) != AILA_NF4_OK)
        throw std::runtime_error(aila_nf4_last_error());
}

// The same over one shard of a vocabulary (no reference counterpart): logits[0] has the global index
// index_offset, ties are resolved on global indices, the result is the LOCAL index.
inline void argmax_shard(Context& ctx, TensorView& logits, int shard_size, int64_t index_offset, int* d_result) {
    if (aila_argmax_bf16_shard(logits.data(), shard_size, index_offset, d_result, ctx.device, ctx.stream) !=
        AILA_NF4_OK)
        throw std::runtime_error(aila_nf4_last_error());
}

// One memory-mapped safetensors file; stands where the reference keeps a ModelWeights
// (src/utils/SafeTensors.hpp:86-121) for the purpose of finding bitsandbytes weights.
struct SafetensorsFile {
    AilaStFile* handle = nullptr;

    SafetensorsFile() = default;
    explicit SafetensorsFile(const std::string& path) {
        if (aila_st_open(path.c_str(), &handle) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
    }
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;
    ~SafetensorsFile() { aila_st_close(handle); }

    bool has(const std::string& name) const {
        AilaStTensorView v;
        return aila_st_find(handle, name.c_str(), &v) == AILA_NF4_OK;
    }
};

// LoadBnb4BitWeightRef (reference src/utils/SafeTensors.hpp:136-140, .cpp:370-489): assembles
// and checks the view of weight `name`; false + message when a rule is violated. The view
// points into the mapped file: keep `weights` alive until Bnb4BitLinear::init has returned.
inline bool LoadBnb4BitWeightRef(Context& ctx, SafetensorsFile& weights, const std::string& name,
                                 AilaNf4WeightDesc& out, std::string* error_message = nullptr) {
    if (aila_st_load_bnb4_weight(weights.handle, name.c_str(), ctx.device, &out) == AILA_NF4_OK)
        return true;
    if (error_message) *error_message = aila_nf4_last_error();
    return false;
}

// A model directory: model.safetensors or the shards of model.safetensors.index.json
// (reference LoadModelWeightsFromDir, src/utils/SafeTensors.cpp:491-535). Throws
// std::runtime_error with the reference's messages, as that function does.
struct ModelWeightsDir {
    AilaStDir* handle = nullptr;

    ModelWeightsDir() = default;
    explicit ModelWeightsDir(const std::string& model_dir) {
        if (aila_st_dir_open(model_dir.c_str(), &handle) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
    }
    ModelWeightsDir(const ModelWeightsDir&) = delete;
    ModelWeightsDir& operator=(const ModelWeightsDir&) = delete;
    ~ModelWeightsDir() { aila_st_dir_close(handle); }

    bool has(const std::string& name) const {
        AilaStTensorView v;
        return aila_st_dir_find(handle, name.c_str(), &v) == AILA_NF4_OK;
    }
};

inline bool LoadBnb4BitWeightRef(Context& ctx, ModelWeightsDir& weights, const std::string& name,
                                 AilaNf4WeightDesc& out, std::string* error_message = nullptr) {
    if (aila_st_dir_load_bnb4_weight(weights.handle, name.c_str(), ctx.device, &out) == AILA_NF4_OK)
        return true;
    if (error_message) *error_message = aila_nf4_last_error();
    return false;
}

class Bnb4BitLinear {
public:
    Bnb4BitLinear() = default;
    Bnb4BitLinear(const Bnb4BitLinear&) = delete;
    Bnb4BitLinear& operator=(const Bnb4BitLinear&) = delete;
    ~Bnb4BitLinear() { aila_nf4_linear_destroy(handle_); }

    // Bnb4BitLinear::init (reference src/ops/Bnb4BitLinear.cpp:453-497).
    bool init(Context& ctx, const AilaNf4WeightDesc& weight, std::string* error_message = nullptr) {
        AilaNf4WeightDesc d = weight;
        d.device = ctx.device;
        return adopt(aila_nf4_linear_create(&d, &fresh_), error_message);
    }

    // Bnb4BitLinear::init_fused_rows, 2..4 sources (reference :499-521).
    bool init_fused_rows(Context&, const Bnb4BitLinear& a, const Bnb4BitLinear& b,
                         std::string* error_message = nullptr) {
        AilaNf4Linear* s[2] = {a.handle_, b.handle_};
        return adopt(aila_nf4_linear_create_fused_rows(s, 2, &fresh_), error_message);
    }
    bool init_fused_rows(Context&, const Bnb4BitLinear& a, const Bnb4BitLinear& b,
                         const Bnb4BitLinear& c, std::string* error_message = nullptr) {
        AilaNf4Linear* s[3] = {a.handle_, b.handle_, c.handle_};
        return adopt(aila_nf4_linear_create_fused_rows(s, 3, &fresh_), error_message);
    }
    bool init_fused_rows(Context&, const Bnb4BitLinear& a, const Bnb4BitLinear& b,
                         const Bnb4BitLinear& c, const Bnb4BitLinear& d,
                         std::string* error_message = nullptr) {
        AilaNf4Linear* s[4] = {a.handle_, b.handle_, c.handle_, d.handle_};
        return adopt(aila_nf4_linear_create_fused_rows(s, 4, &fresh_), error_message);
    }

    // Bnb4BitLinear::forward (reference :799-949). add_residual: bf16 [seq_len][out] or null.
    void forward(Context& ctx, Bnb4BitLinearScratch& scratch, TensorView& input, TensorView& output,
                 int seq_len, const void* add_residual = nullptr) {
        if (!input.is_bf16() || !output.is_bf16())
            throw std::runtime_error("Bnb4BitLinear expects bf16 input/output tensors");
        if (seq_len <= 0)
            throw std::runtime_error("Bnb4BitLinear::forward: seq_len must be positive");
        scratch.open(ctx);
        if (aila_nf4_forward(handle_, scratch.handle, input.data(), output.data(), seq_len,
                             add_residual, ctx.stream) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
    }

    // Bnb4BitLinear::try_forward_decode_gate_up_swiglu (reference :759-797). The reference
    // takes no scratch here; this one needs the split-K work space, hence the extra argument.
    static bool try_forward_decode_gate_up_swiglu(Context& ctx, Bnb4BitLinearScratch& scratch,
                                                  Bnb4BitLinear& fused_gate_up, TensorView& input,
                                                  TensorView& output, int ff_dim, int seq_len = 1) {
        if (!input.is_bf16() || !output.is_bf16()) return false;
        if (input.ndim() != 2) return false;
        scratch.open(ctx);
        const AilaNf4Status st = aila_nf4_forward_gate_up_swiglu(
            fused_gate_up.handle_, scratch.handle, input.data(), output.data(), seq_len, ff_dim,
            ctx.stream);
        if (st == AILA_NF4_NOT_APPLICABLE) return false;
        if (st != AILA_NF4_OK) throw std::runtime_error(aila_nf4_last_error());
        return true;
    }

    // The reference's own signature (src/ops/Bnb4BitLinear.hpp:52-56; called at
    // src/models/Qwen35HybridBnb4Backend.cpp:2172-2173): the work space is the context's.
    static bool try_forward_decode_gate_up_swiglu(Context& ctx, Bnb4BitLinear& fused_gate_up,
                                                  TensorView& input, TensorView& output, int ff_dim) {
        if (!input.is_bf16() || !output.is_bf16()) return false;
        if (input.ndim() != 2 || input.rows != 1) return false;
        if (!ctx.decode_scratch && aila_nf4_scratch_create(ctx.device, &ctx.decode_scratch) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
        const AilaNf4Status st = aila_nf4_forward_gate_up_swiglu(
            fused_gate_up.handle_, ctx.decode_scratch, input.data(), output.data(), 1, ff_dim, ctx.stream);
        if (st == AILA_NF4_NOT_APPLICABLE) return false;
        if (st != AILA_NF4_OK) throw std::runtime_error(aila_nf4_last_error());
        return true;
    }

    int in_features() const { return static_cast<int>(aila_nf4_linear_in_features(handle_)); }
    int out_features() const { return static_cast<int>(aila_nf4_linear_out_features(handle_)); }
    AilaNf4Linear* handle() const { return handle_; }

private:
    bool adopt(AilaNf4Status st, std::string* error_message) {
        if (st != AILA_NF4_OK) {
            if (error_message) *error_message = aila_nf4_last_error();
            fresh_ = nullptr;
            return false;
        }
        aila_nf4_linear_destroy(handle_);
        handle_ = fresh_;
        fresh_ = nullptr;
        return true;
    }
    AilaNf4Linear* handle_ = nullptr;
    AilaNf4Linear* fresh_ = nullptr;
};

// A run of seq_len == 1 linears as ONE launch (aila_nf4_chain_*): what the decode step issues
// back to back (reference src/models/Qwen3Bnb4Backend.cpp:339-418), listed once after load() and
// run per token. add() returns *this so the list reads like the call sites it replaces:
//
//   chain.add(layer.o_proj, attn_out.data(), nullptr)                          // x given, y linked on
//        .add_gate_up(layer.gate_up_proj, ff_dim, nullptr, nullptr, &post_attn_norm)
//        .add(layer.down_proj, nullptr, mlp_out.data());
//   chain.build(ctx, scratch_);   ...   chain.run(ctx);
class DecodeChain {
public:
    DecodeChain() = default;
    DecodeChain(const DecodeChain&) = delete;
    DecodeChain& operator=(const DecodeChain&) = delete;
    ~DecodeChain() { aila_nf4_chain_destroy(handle_); }

    // x == nullptr: the previous operation's output; y == nullptr: only the next operation reads it.
    DecodeChain& add(const Bnb4BitLinear& linear, const void* x, void* y, const void* residual = nullptr,
                     const AilaNf4RmsNorm* norm = nullptr) {
        return push(linear, 0, x, y, residual, norm);
    }
    DecodeChain& add_gate_up(const Bnb4BitLinear& fused_gate_up, int ff_dim, const void* x, void* y,
                             const AilaNf4RmsNorm* norm = nullptr) {
        return push(fused_gate_up, ff_dim, x, y, nullptr, norm);
    }

    bool build(Context& ctx, Bnb4BitLinearScratch& scratch, std::string* error_message = nullptr) {
        scratch.open(ctx);
        for (size_t i = 0; i < ops_.size(); ++i)
            if (has_norm_[i]) ops_[i].norm = &norms_[i];
        AilaNf4Chain* fresh = nullptr;
        if (aila_nf4_chain_create(scratch.handle, ops_.data(), (int)ops_.size(), &fresh) != AILA_NF4_OK) {
            if (error_message) *error_message = aila_nf4_last_error();
            return false;
        }
        aila_nf4_chain_destroy(handle_);
        handle_ = fresh;
        return true;
    }

    void run(Context& ctx) {
        if (aila_nf4_chain_run(handle_, ctx.stream) != AILA_NF4_OK) throw std::runtime_error(aila_nf4_last_error());
    }
    // host x in, host y out, one synchronisation
    void run_host(Context& ctx, const void* x_host_bf16, void* y_host_bf16) {
        if (aila_nf4_chain_run_host(handle_, x_host_bf16, y_host_bf16, ctx.stream) != AILA_NF4_OK)
            throw std::runtime_error(aila_nf4_last_error());
    }
    int length() const { return aila_nf4_chain_length(handle_); }

private:
    DecodeChain& push(const Bnb4BitLinear& l, int ff, const void* x, void* y, const void* res,
                      const AilaNf4RmsNorm* norm) {
        AilaNf4ChainOp op{};
        op.linear = l.handle();
        op.ff_dim = ff;
        op.x_bf16 = x;
        op.y_bf16 = y;
        op.residual_bf16 = res;
        op.norm = nullptr;
        ops_.push_back(op);
        norms_.push_back(norm ? *norm : AilaNf4RmsNorm{});
        has_norm_.push_back(norm != nullptr);
        return *this;
    }
    std::vector<AilaNf4ChainOp> ops_;
    std::vector<AilaNf4RmsNorm> norms_;   // copies: the caller's structs need not outlive add()
    std::vector<bool> has_norm_;
    AilaNf4Chain* handle_ = nullptr;
};

}  // namespace nf4
}  // namespace aila
