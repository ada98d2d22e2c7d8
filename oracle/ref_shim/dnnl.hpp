// TEST INFRASTRUCTURE ONLY. A host stand-in for the few oneDNN types the reference's NF4 operator
// touches (memory descriptors, a bf16 matmul primitive and the SYCL interop constructors), so that
// src/ops/Bnb4BitLinear.cpp compiles and runs without oneDNN. The matmul is a plain loop:
// dst[M,N] = bf16( sum_k fp32(src[M,K]) * fp32(weights[K,N]) ), row-major, fp32 accumulation in
// ascending k - this file's own arithmetic, not oneDNN's (whose blocking and summation order are
// not public); only the operands fed to it are the reference's.
#pragma once

#include <sycl/sycl.hpp>

#include <cstdint>
#include <stdexcept>
#include <unordered_map>
#include <vector>

#define DNNL_ARG_SRC 1
#define DNNL_ARG_WEIGHTS 33
#define DNNL_ARG_DST 17
#define DNNL_ARG_SCRATCHPAD 80
#define DNNL_ARG_BIAS 41

namespace dnnl {

struct engine {};
struct stream {
    void wait() {}
};

enum class scratchpad_mode { library, user };

struct primitive_attr {
    void set_scratchpad_mode(scratchpad_mode) {}
};

class memory {
public:
    enum class data_type { undef, f16, bf16, f32, s32, s8, u8, f64 };
    enum class format_tag { undef, any, a, ab, abc, abcd, abcde, abcdef, ba };
    using dim = int64_t;
    using dims = std::vector<dim>;

    class desc {
    public:
        desc() = default;
        desc(const dims& d, data_type t, format_tag) : dims_(d), type_(t) {}
        desc(const dims& d, data_type t, const dims& strides) : dims_(d), type_(t), strides_(strides) {}
        const dims& get_dims() const { return dims_; }
        data_type get_data_type() const { return type_; }
        size_t get_size() const {
            size_t n = 1;
            for (dim d : dims_) n *= static_cast<size_t>(d);
            size_t e = 1;
            switch (type_) {
                case data_type::f32: case data_type::s32: e = 4; break;
                case data_type::bf16: case data_type::f16: e = 2; break;
                case data_type::f64: e = 8; break;
                default: e = 1; break;
            }
            return dims_.empty() ? 0 : n * e;
        }

    private:
        dims dims_;
        data_type type_ = data_type::undef;
        dims strides_;
    };

    memory() = default;
    memory(const desc& d, void* handle) : desc_(d), handle_(handle) {}
    void* get_data_handle() const { return handle_; }
    void set_data_handle(void* h) { handle_ = h; }
    const desc& get_desc() const { return desc_; }

private:
    desc desc_;
    void* handle_ = nullptr;
};

class matmul {
public:
    struct primitive_desc {
        memory::desc src, weights, dst;
        primitive_desc() = default;
        primitive_desc(const engine&, const memory::desc& s, const memory::desc& w, const memory::desc& d,
                       const primitive_attr& = primitive_attr())
            : src(s), weights(w), dst(d) {}
        memory::desc scratchpad_desc() const { return memory::desc(); }
    };

    matmul() = default;
    explicit matmul(const primitive_desc& pd) : pd_(pd) {}

    void execute(stream&, const std::unordered_map<int, memory>& args) const {
        using bf16 = sycl::ext::oneapi::bfloat16;
        const memory& s = args.at(DNNL_ARG_SRC);
        const memory& w = args.at(DNNL_ARG_WEIGHTS);
        const memory& d = args.at(DNNL_ARG_DST);
        const auto& sd = pd_.src.get_dims();
        const auto& wd = pd_.weights.get_dims();
        if (sd.size() != 2 || wd.size() != 2 || sd[1] != wd[0] ||
            pd_.src.get_data_type() != memory::data_type::bf16 ||
            pd_.weights.get_data_type() != memory::data_type::bf16 ||
            pd_.dst.get_data_type() != memory::data_type::bf16)
            throw std::runtime_error("dnnl shim: only row-major bf16 [M,K] x [K,N] matmuls");
        const int64_t M = sd[0], K = sd[1], N = wd[1];
        const bf16* a = static_cast<const bf16*>(s.get_data_handle());
        const bf16* b = static_cast<const bf16*>(w.get_data_handle());
        bf16* c = static_cast<bf16*>(d.get_data_handle());
        std::vector<float> acc(static_cast<size_t>(N));
        for (int64_t m = 0; m < M; ++m) {
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int64_t k = 0; k < K; ++k) {
                const float av = static_cast<float>(a[m * K + k]);
                const bf16* br = b + k * N;
                for (int64_t n = 0; n < N; ++n) acc[static_cast<size_t>(n)] += av * static_cast<float>(br[n]);
            }
            for (int64_t n = 0; n < N; ++n) c[m * N + n] = bf16(acc[static_cast<size_t>(n)]);
        }
    }

private:
    primitive_desc pd_;
};

namespace sycl_interop {
enum class memory_kind { usm, buffer };
inline engine make_engine(const sycl::device&, const sycl::context&) { return engine{}; }
inline stream make_stream(const engine&, sycl::queue&) { return stream{}; }
inline memory make_memory(const memory::desc& d, const engine&, memory_kind, void* handle) { return memory(d, handle); }
}  // namespace sycl_interop

}  // namespace dnnl
