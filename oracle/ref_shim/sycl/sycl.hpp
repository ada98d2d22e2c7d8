// TEST INFRASTRUCTURE ONLY. A serial CPU stand-in for the part of SYCL 2020 that the reference's
// operators of the NF4 decode path use (src/ops/Bnb4BitLinear.cpp, NormOps.cpp, ElementwiseOps.cpp,
// SamplingOps.cpp, AttentionOps.cpp and the headers they include), so that the reference's own
// kernel source can be compiled with g++ and run on the host as a second opinion on the CPU oracle. Not a SYCL implementation: one device (the host), in-order queues that run
// every command at submission, USM = malloc.
//
// Work-items of a work-group run as cooperatively scheduled fibers (ucontext), so barriers and
// group collectives have their lock-step meaning. Sub-groups are 16 consecutive work-items (the
// only size the reference's kernels ask for). What SYCL leaves unspecified is fixed here:
// reduce_over_group adds in a balanced binary tree (t[i] += t[i + w], w = n/2 .. 1), the usual
// hardware order and the one the CPU oracle assumes; native:: functions are the libm ones.
#pragma once

#include <ucontext.h>

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <stdexcept>
#include <type_traits>
#include <vector>

namespace sycl {

// ---------------------------------------------------------------- index types
template <int D>
struct range {
    size_t v[D > 0 ? D : 1] = {};
    range() = default;
    range(size_t a) { v[0] = a; }
    range(size_t a, size_t b) { v[0] = a; v[1] = b; }
    range(size_t a, size_t b, size_t c) { v[0] = a; v[1] = b; v[2] = c; }
    size_t operator[](int i) const { return v[i]; }
    size_t& operator[](int i) { return v[i]; }
    size_t size() const {
        size_t s = 1;
        for (int i = 0; i < D; ++i) s *= v[i];
        return s;
    }
};

template <int D>
struct id {
    size_t v[D > 0 ? D : 1] = {};
    id() = default;
    id(size_t a) { v[0] = a; }
    size_t operator[](int i) const { return v[i]; }
    size_t& operator[](int i) { return v[i]; }
    size_t get(int i) const { return v[i]; }
    operator size_t() const { return v[0]; }
};

// the argument of a plain parallel_for when the kernel asks for an item instead of an id
template <int D>
struct item {
    id<D> index;
    range<D> extent;
    item(const id<D>& i, const range<D>& r) : index(i), extent(r) {}
    size_t get_id(int i) const { return index[i]; }
    size_t operator[](int i) const { return index[i]; }
    size_t get_range(int i) const { return extent[i]; }
    id<D> get_id() const { return index; }
    size_t get_linear_id() const {
        size_t lin = 0;
        for (int i = 0; i < D; ++i) lin = lin * extent[i] + index[i];
        return lin;
    }
    operator id<D>() const { return index; }
};

template <int D>
struct nd_range {
    range<D> global, local;
    nd_range(range<D> g, range<D> l) : global(g), local(l) {}
};

namespace access {
enum class fence_space { local_space, global_space, global_and_local };
enum class decorated { no, yes, legacy };
enum class address_space { global_space, local_space, private_space, generic_space };
}
enum class aspect { ext_intel_matrix, fp16, fp64, gpu, cpu };
template <access::address_space S, access::decorated D, typename T>
inline T* address_space_cast(T* p) { return p; }

// ---------------------------------------------------------------- bfloat16
namespace ext {
namespace oneapi {
class bfloat16 {
public:
    bfloat16() = default;
    bfloat16(float f) { bits_ = from_float(f); }
    operator float() const {
        uint32_t u = static_cast<uint32_t>(bits_) << 16;
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }
    uint16_t raw() const { return bits_; }

private:
    static uint16_t from_float(float f) {  // round to nearest even; NaN stays NaN
        uint32_t u;
        std::memcpy(&u, &f, 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
        return static_cast<uint16_t>((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
    }
    uint16_t bits_ = 0;
};
// Declarations only for the matrix extension: the stand-in device reports no matrix hardware, so
// the kernels that use it are compiled but never chosen; calling one throws.
namespace experimental {
namespace matrix {
enum class use { a, b, accumulator };
enum class layout { row_major, col_major, dynamic };
enum class matrix_type { bf16, fp16, tf32, fp32, fp64, sint8, uint8, sint32 };
struct combination {
    size_t max_msize = 0, max_nsize = 0, max_ksize = 0, msize = 0, nsize = 0, ksize = 0;
    matrix_type atype = matrix_type::fp32, btype = matrix_type::fp32, ctype = matrix_type::fp32,
                dtype = matrix_type::fp32;
};
template <typename Group, typename T, use U, size_t R, size_t C, layout L = layout::dynamic>
struct joint_matrix {};
template <typename... A>
inline void joint_matrix_fill(A&&...) { throw std::runtime_error("sycl shim: no matrix extension"); }
template <typename... A>
inline void joint_matrix_load(A&&...) { throw std::runtime_error("sycl shim: no matrix extension"); }
template <typename... A>
inline void joint_matrix_mad(A&&...) { throw std::runtime_error("sycl shim: no matrix extension"); }
template <typename... A>
inline void joint_matrix_store(A&&...) { throw std::runtime_error("sycl shim: no matrix extension"); }
}  // namespace matrix
namespace info {
namespace device {
struct matrix_combinations {
    using return_type = std::vector<matrix::combination>;
};
}  // namespace device
}  // namespace info
}  // namespace experimental
}  // namespace oneapi
}  // namespace ext

template <typename T, int N>
struct vec {
    T data[N];
    vec() = default;
    explicit vec(T v) {
        for (int i = 0; i < N; ++i) data[i] = v;
    }
    const T& operator[](int i) const { return data[i]; }
    T& operator[](int i) { return data[i]; }
    friend vec operator*(const vec& a, const vec& b) {
        vec r;
        for (int i = 0; i < N; ++i) r.data[i] = a.data[i] * b.data[i];
        return r;
    }
    friend vec operator+(const vec& a, const vec& b) {
        vec r;
        for (int i = 0; i < N; ++i) r.data[i] = a.data[i] + b.data[i];
        return r;
    }
    vec& operator+=(const vec& b) {
        for (int i = 0; i < N; ++i) data[i] += b.data[i];
        return *this;
    }
};

// ---------------------------------------------------------------- math
inline float fma(float a, float b, float c) { return std::fma(a, b, c); }
inline float sqrt(float a) { return std::sqrt(a); }
inline float rsqrt(float a) { return 1.0f / std::sqrt(a); }
inline float fmax(float a, float b) { return std::fmax(a, b); }
inline float fmin(float a, float b) { return std::fmin(a, b); }
inline float fabs(float a) { return std::fabs(a); }
inline bool isfinite(float a) { return std::isfinite(a); }
inline bool isnan(float a) { return std::isnan(a); }
inline float exp(float a) { return std::exp(a); }
inline float log(float a) { return std::log(a); }
inline float pow(float a, float b) { return std::pow(a, b); }
inline float cos(float a) { return std::cos(a); }
inline float sin(float a) { return std::sin(a); }
inline float tanh(float a) { return std::tanh(a); }
template <typename T>
inline T min(T a, T b) { return b < a ? b : a; }
template <typename T>
inline T max(T a, T b) { return a < b ? b : a; }
namespace native {
inline float exp(float a) { return std::exp(a); }
inline float cos(float a) { return std::cos(a); }
inline float sin(float a) { return std::sin(a); }
}  // namespace native

template <typename T = void>
struct plus {
    template <typename U>
    U operator()(U a, U b) const { return a + b; }
};
template <typename T = void>
struct maximum {
    template <typename U>
    U operator()(U a, U b) const { return a < b ? b : a; }
};

// ---------------------------------------------------------------- work-group execution
namespace shim {

constexpr int kSubGroup = 16;

struct GroupState {
    int n_items = 0;
    int running = 0;              // fibers not finished yet
    // barrier
    int arrived = 0;
    unsigned generation = 0;
    // collectives: one slot per work-item (double, wide enough for every type used), per scope
    std::vector<double> slot;
    std::vector<int> sg_arrived;          // per sub-group
    std::vector<unsigned> sg_generation;
    // scheduling
    ucontext_t scheduler;
    std::vector<ucontext_t> fiber;
    std::vector<char> done;
    int current = 0;
    std::vector<std::unique_ptr<char[]>> local_mem;  // local_accessor storage of this launch
};

inline GroupState*& active() {
    static thread_local GroupState* g = nullptr;
    return g;
}

inline void yield() {
    GroupState* g = active();
    swapcontext(&g->fiber[g->current], &g->scheduler);
}

// every work-item of the group
inline void group_barrier() {
    GroupState* g = active();
    const unsigned gen = g->generation;
    if (++g->arrived == g->running) {
        g->arrived = 0;
        ++g->generation;
        return;
    }
    while (g->generation == gen) yield();
}

inline void sub_group_barrier(int sg, int members) {
    GroupState* g = active();
    const unsigned gen = g->sg_generation[sg];
    if (++g->sg_arrived[sg] == members) {
        g->sg_arrived[sg] = 0;
        ++g->sg_generation[sg];
        return;
    }
    while (g->sg_generation[sg] == gen) yield();
}

template <typename T, typename Op>
inline T tree(const double* v, int n, Op op) {
    // balanced tree over n = 2^k values (n is a sub-group or work-group size here)
    T t[1024];
    int w = 1;
    while (w * 2 <= n) w *= 2;
    if (w != n || n > 1024)
        throw std::runtime_error("sycl shim: reduce_over_group over a size that is not a power of two up to 1024");
    for (int i = 0; i < n; ++i) t[i] = static_cast<T>(v[i]);
    for (w = n / 2; w >= 1; w /= 2)
        for (int i = 0; i < w; ++i) t[i] = op(t[i], t[i + w]);
    return t[0];
}

struct Fiber {
    std::function<void(int)>* body;
    int index;
};

inline void fiber_entry(unsigned lo, unsigned hi) {
    Fiber* f = reinterpret_cast<Fiber*>((static_cast<uintptr_t>(hi) << 32) | static_cast<uintptr_t>(lo));
    (*f->body)(f->index);
    GroupState* g = active();
    g->done[f->index] = 1;
    --g->running;
    // a finished item no longer takes part in barriers: release one that is now complete
    if (g->running > 0 && g->arrived == g->running) {
        g->arrived = 0;
        ++g->generation;
    }
    swapcontext(&g->fiber[f->index], &g->scheduler);
}

// Runs `body(local_linear_id)` for the n_items work-items of one work-group in lock step.
inline void run_group(int n_items, std::function<void(int)> body, GroupState& g) {
    constexpr size_t kStack = 128 * 1024;
    static thread_local std::vector<std::unique_ptr<char[]>> stacks;
    while (static_cast<int>(stacks.size()) < n_items) stacks.emplace_back(new char[kStack]);
    g.n_items = n_items;
    g.running = n_items;
    g.arrived = 0;
    g.generation = 0;
    g.slot.assign(static_cast<size_t>(n_items), 0.0);
    const int n_sg = (n_items + kSubGroup - 1) / kSubGroup;
    g.sg_arrived.assign(static_cast<size_t>(n_sg), 0);
    g.sg_generation.assign(static_cast<size_t>(n_sg), 0u);
    g.fiber.resize(static_cast<size_t>(n_items));
    g.done.assign(static_cast<size_t>(n_items), 0);
    std::vector<Fiber> args(static_cast<size_t>(n_items));
    for (int i = 0; i < n_items; ++i) {
        args[i] = Fiber{&body, i};
        getcontext(&g.fiber[i]);
        g.fiber[i].uc_stack.ss_sp = stacks[i].get();
        g.fiber[i].uc_stack.ss_size = kStack;
        g.fiber[i].uc_link = nullptr;
        const uintptr_t p = reinterpret_cast<uintptr_t>(&args[i]);
        makecontext(&g.fiber[i], reinterpret_cast<void (*)()>(fiber_entry), 2, static_cast<unsigned>(p & 0xffffffffu),
                    static_cast<unsigned>(p >> 32));
    }
    GroupState* prev = active();
    active() = &g;
    while (g.running > 0) {
        bool progressed = false;
        for (int i = 0; i < n_items; ++i) {
            if (g.done[i]) continue;
            g.current = i;
            swapcontext(&g.scheduler, &g.fiber[i]);
            progressed = true;
        }
        if (!progressed) break;
    }
    active() = prev;
}

}  // namespace shim

// ---------------------------------------------------------------- groups and items
struct sub_group {
    int sg_index = 0, lane = 0, members = shim::kSubGroup, first_item = 0;
    size_t get_local_id() const { return static_cast<size_t>(lane); }
    size_t get_local_range() const { return static_cast<size_t>(members); }
    size_t get_group_id() const { return static_cast<size_t>(sg_index); }
};

template <int D>
struct group {
    int n_items = 0, item = 0;
    size_t get_local_range(int = 0) const { return static_cast<size_t>(n_items); }
};

template <int D>
class nd_item {
public:
    range<D> local_range, group_range;
    size_t local_id[D], group_id[D];
    int linear_local = 0, n_local = 0;

    size_t get_local_id(int i) const { return local_id[i]; }
    size_t get_group(int i) const { return group_id[i]; }
    size_t get_local_range(int i) const { return local_range[i]; }
    size_t get_group_range(int i) const { return group_range[i]; }
    size_t get_global_id(int i) const { return group_id[i] * local_range[i] + local_id[i]; }
    size_t get_local_linear_id() const { return static_cast<size_t>(linear_local); }
    group<D> get_group() const { return group<D>{n_local, linear_local}; }
    sub_group get_sub_group() const {
        sub_group s;
        s.sg_index = linear_local / shim::kSubGroup;
        s.lane = linear_local % shim::kSubGroup;
        s.first_item = s.sg_index * shim::kSubGroup;
        s.members = std::min(shim::kSubGroup, n_local - s.first_item);
        return s;
    }
    void barrier(access::fence_space = access::fence_space::global_and_local) const { shim::group_barrier(); }
};

template <typename T, typename Op>
inline T reduce_over_group(const sub_group& sg, T x, Op op) {
    shim::GroupState* g = shim::active();
    g->slot[static_cast<size_t>(sg.first_item + sg.lane)] = static_cast<double>(x);
    shim::sub_group_barrier(sg.sg_index, sg.members);
    const T r = shim::tree<T>(g->slot.data() + sg.first_item, sg.members, op);
    shim::sub_group_barrier(sg.sg_index, sg.members);  // (the slots may be written again after this)
    return r;
}

template <int D, typename T, typename Op>
inline T reduce_over_group(const group<D>& grp, T x, Op op) {
    shim::GroupState* g = shim::active();
    g->slot[static_cast<size_t>(grp.item)] = static_cast<double>(x);
    shim::group_barrier();
    const T r = shim::tree<T>(g->slot.data(), grp.n_items, op);
    shim::group_barrier();
    return r;
}

// ---------------------------------------------------------------- handler, queue, USM
class handler;

template <typename T, int D = 1>
class local_accessor {
public:
    local_accessor() = default;
    local_accessor(range<D> r, handler& h);
    T& operator[](size_t i) const { return ptr_[i]; }
    T* get_pointer() const { return ptr_; }
    template <access::decorated Dec = access::decorated::no>
    T* get_multi_ptr() const { return ptr_; }

private:
    T* ptr_ = nullptr;
};

class handler {
public:
    // storage for local accessors: one copy, reused by the groups (they run one after another)
    std::vector<std::unique_ptr<char[]>> local_mem;

    template <int D, typename K>
    void parallel_for(nd_range<D> r, const K& kernel) {
        range<D> groups;
        size_t n_groups = 1;
        for (int i = 0; i < D; ++i) {
            if (r.local[i] == 0 || r.global[i] % r.local[i] != 0)
                throw std::runtime_error("sycl shim: global range is not a multiple of the local range");
            groups[i] = r.global[i] / r.local[i];
            n_groups *= groups[i];
        }
        const int n_local = static_cast<int>(r.local.size());
        shim::GroupState state;
        for (size_t gidx = 0; gidx < n_groups; ++gidx) {
            size_t gid[D], rem = gidx;
            for (int i = D - 1; i >= 0; --i) {
                gid[i] = rem % groups[i];
                rem /= groups[i];
            }
            shim::run_group(n_local, [&](int lin) {
                nd_item<D> it;
                it.local_range = r.local;
                it.group_range = groups;
                it.linear_local = lin;
                it.n_local = n_local;
                size_t rem2 = static_cast<size_t>(lin);
                for (int i = D - 1; i >= 0; --i) {
                    it.local_id[i] = rem2 % r.local[i];
                    rem2 /= r.local[i];
                    it.group_id[i] = gid[i];
                }
                kernel(it);
            }, state);
        }
    }

    // plain range: work-items in row-major order (the last dimension runs fastest), one after another
    template <int D, typename K>
    void parallel_for(range<D> r, const K& kernel) {
        const size_t total = r.size();
        for (size_t lin = 0; lin < total; ++lin) {
            id<D> idx;
            size_t rem = lin;
            for (int i = D - 1; i >= 0; --i) {
                idx[i] = rem % r[i];
                rem /= r[i];
            }
            if constexpr (std::is_invocable_v<const K&, id<D>>) kernel(idx);
            else kernel(item<D>(idx, r));
        }
    }
};

template <typename T, int D>
local_accessor<T, D>::local_accessor(range<D> r, handler& h) {
    h.local_mem.emplace_back(new char[r.size() * sizeof(T) + 64]());
    ptr_ = reinterpret_cast<T*>(h.local_mem.back().get());
}

struct event {
    void wait() {}
};
struct device {
    bool has(aspect) const { return false; }   // no matrix hardware: the plain kernels are chosen
    template <typename Info>
    typename Info::return_type get_info() const { return typename Info::return_type(); }
};
struct context {
    bool operator==(const context&) const { return true; }
    bool operator!=(const context&) const { return false; }
};
struct default_selector_t {};
inline constexpr default_selector_t default_selector_v{};
namespace property {
namespace queue {
struct in_order {};
}  // namespace queue
}  // namespace property

class queue {
public:
    queue() = default;
    template <typename... A>
    explicit queue(A&&...) {}
    template <typename F>
    event submit(F&& f) {
        handler h;
        f(h);
        return event{};
    }
    template <int D, typename K>
    event parallel_for(range<D> r, const K& k) {
        handler h;
        h.parallel_for(r, k);
        return event{};
    }
    event memcpy(void* dst, const void* src, size_t n) {
        std::memmove(dst, src, n);
        return event{};
    }
    event memset(void* dst, int v, size_t n) {
        std::memset(dst, v, n);
        return event{};
    }
    void wait() {}
    void wait_and_throw() {}
    device get_device() const { return device{}; }
    context get_context() const { return context{}; }
};

inline void* malloc_device(size_t bytes, const queue&) { return std::calloc(bytes ? bytes : 1, 1); }
inline void* malloc_host(size_t bytes, const queue&) { return std::calloc(bytes ? bytes : 1, 1); }
inline void* malloc_shared(size_t bytes, const queue&) { return std::calloc(bytes ? bytes : 1, 1); }
inline void free(void* p, const queue&) { std::free(p); }
inline void free(void* p, const context&) { std::free(p); }
template <typename T>
inline T* malloc_device(size_t count, const queue& q) { return static_cast<T*>(malloc_device(count * sizeof(T), q)); }
template <typename T>
inline T* malloc_host(size_t count, const queue& q) { return static_cast<T*>(malloc_host(count * sizeof(T), q)); }
template <typename T>
inline T* malloc_shared(size_t count, const queue& q) { return static_cast<T*>(malloc_shared(count * sizeof(T), q)); }

}  // namespace sycl
