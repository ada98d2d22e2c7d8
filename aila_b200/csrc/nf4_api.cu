// C ABI of the NF4 linear operator (include/aila_nf4.h): handle management, validation with
// the reference loader's rules, dispatch between the decode and prefill kernels.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "nf4_internal.h"

namespace {

thread_local std::string g_last_error;
int g_gemv_kernel = -1;  // -1 = read AILA_NF4_GEMV_KERNEL on first use

int gemv_kernel_choice() {
    if (g_gemv_kernel < 0) {
        const char* e = std::getenv("AILA_NF4_GEMV_KERNEL");
        int v = e ? std::atoi(e) : 0;
        g_gemv_kernel = (v >= 0 && v <= 3) ? v : 0;
    }
    return g_gemv_kernel;
}

bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }
int ilog2i(int64_t v) {
    int s = 0;
    while (((int64_t)1 << s) < v) ++s;
    return s;
}

// Makes `device` current for the lifetime of the guard.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) {
            err = cudaSetDevice(device);
            switched = (err == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

// Code-book tables (the 16-entry first-level map, the 256-entry second-level map) are the same
// in every layer of a model. One device copy per distinct content and device is shared by all
// linears that use it, so back-to-back launches for different layers find the table in L2
// instead of fetching a private copy from HBM at every kernel start.
struct InternedTable {
    int device = 0;
    std::vector<uint32_t> bits;
    float* ptr = nullptr;
    int refs = 0;
};
std::mutex g_intern_mutex;
std::vector<InternedTable> g_interned;

cudaError_t intern_table(float** dst, const float* src, size_t count, bool src_on_device,
                         int device) {
    std::vector<uint32_t> bits(count);
    cudaError_t e = cudaMemcpy(bits.data(), src, count * 4,
                               src_on_device ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(g_intern_mutex);
    for (auto& t : g_interned)
        if (t.device == device && t.bits == bits) {
            ++t.refs;
            *dst = t.ptr;
            return cudaSuccess;
        }
    InternedTable t;
    t.device = device;
    e = cudaMalloc(reinterpret_cast<void**>(&t.ptr), count * 4 + 16);
    if (e != cudaSuccess) return e;
    e = cudaMemcpy(t.ptr, bits.data(), count * 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(t.ptr);
        return e;
    }
    t.bits = std::move(bits);
    t.refs = 1;
    *dst = t.ptr;
    g_interned.push_back(std::move(t));
    return cudaSuccess;
}

void release_table(float* ptr) {
    if (!ptr) return;
    std::lock_guard<std::mutex> lock(g_intern_mutex);
    for (size_t i = 0; i < g_interned.size(); ++i)
        if (g_interned[i].ptr == ptr) {
            if (--g_interned[i].refs == 0) {
                cudaFree(ptr);
                g_interned.erase(g_interned.begin() + (long)i);
            }
            return;
        }
}

void free_linear(AilaNf4Linear* l) {
    if (!l) return;
    DeviceGuard g(l->device);
    cudaFree(l->d_units);
    release_table(l->d_qmap);
    release_table(l->d_nmap);
    cudaFree(l->d_nabs);
    cudaFree(l->d_cache_bf16);
    cudaFree(l->d_row_scales);
    delete l;
}

template <typename T>
cudaError_t upload(T** dst, const T* src, size_t count, bool src_on_device) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(dst), count * sizeof(T) + 16);
    if (e != cudaSuccess) return e;
    return cudaMemcpy(*dst, src, count * sizeof(T),
                      src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice);
}

// AILA_BNB4_CACHE_DEQUANT=1 (same name and meaning as the reference flag read in
// Bnb4BitLinear::finish_init, src/ops/Bnb4BitLinear.cpp:642-650): keep a bf16 copy of the whole
// weight so seq_len > 1 calls skip the dequantisation pass, at four times the weight memory.
bool cache_dequant_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("AILA_BNB4_CACHE_DEQUANT");
        return e && e[0] != '\0' && e[0] != '0';
    }();
    return on;
}

// Last step of every way a linear comes into being: the per-row second-level scales of the
// chained decode kernel (when no row changes its second-level block twice), and the optional
// bf16 copy.
AilaNf4Status maybe_cache_dequant(AilaNf4Linear* l) {
    if (l->absmax_kind == nf4::kAbsmaxCodes && l->KU <= l->nbs * (l->blocksize / nf4::kUnitK)) {
        cudaError_t e = cudaMalloc(&l->d_row_scales, (size_t)l->N * 16 + 16);
        if (e != cudaSuccess) return nf4::cuda_fail(e, "cudaMalloc(row scales)");
        NF4_CUDA(nf4::launch_row_scales(*l, 0));
        NF4_CUDA(cudaDeviceSynchronize());
        l->device_bytes += (int64_t)l->N * 16;
    }
    if (!cache_dequant_enabled()) return AILA_NF4_OK;
    const size_t bytes = (size_t)l->N * (size_t)l->K * 2;
    cudaError_t e = cudaMalloc(&l->d_cache_bf16, bytes + 256);
    if (e != cudaSuccess) return nf4::cuda_fail(e, "cudaMalloc(bf16 weight cache)");
    NF4_CUDA(nf4::launch_dequant_nk(*l, l->d_cache_bf16, 0));
    NF4_CUDA(cudaDeviceSynchronize());
    l->device_bytes += (int64_t)bytes;
    return AILA_NF4_OK;
}

// Validation shared by create and create_shard: the checks of LoadBnb4BitWeightRef
// (reference src/utils/SafeTensors.cpp:406-487) that can be made on raw pointers, plus the
// constraints of this implementation.
AilaNf4Status validate_desc(const AilaNf4WeightDesc* d) {
    using nf4::fail;
    if (!d) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "weight descriptor is NULL");
    if (d->out_features <= 0 || d->in_features <= 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes logical weight shape is invalid");
    if (!d->packed_weight || !d->absmax || !d->quant_map)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "Missing required bitsandbytes side tensors (packed_weight, absmax, quant_map)");
    if (d->blocksize <= 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "bitsandbytes blocksize must be positive");
    if (d->blocksize % nf4::kUnitK != 0 || !is_pow2(d->blocksize / nf4::kUnitK))
        return fail(AILA_NF4_ERR_UNSUPPORTED, "blocksize must be 64 times a power of two");
    if (d->in_features % d->blocksize != 0)
        return fail(AILA_NF4_ERR_UNSUPPORTED, "in_features must be a multiple of blocksize");
    if (d->nested) {
        if (!d->nested_absmax || !d->nested_quant_map)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes nested quantization tensors are missing");
        if (d->nested_blocksize <= 0)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes nested blocksize must be positive");
        if (!is_pow2(d->nested_blocksize))
            return fail(AILA_NF4_ERR_UNSUPPORTED, "nested blocksize must be a power of two");
        const int64_t blocks = d->out_features * d->in_features / d->blocksize;
        const int64_t want = (blocks + d->nested_blocksize - 1) / d->nested_blocksize;
        if (d->nested_absmax_count != want)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "bitsandbytes nested_absmax length does not match nested block count");
        if (blocks + d->nested_blocksize >= ((int64_t)1 << 31))
            return fail(AILA_NF4_ERR_UNSUPPORTED, "weight has too many absmax blocks");
    }
    if (d->out_features >= ((int64_t)1 << 27) || d->in_features >= ((int64_t)1 << 27))
        return fail(AILA_NF4_ERR_UNSUPPORTED, "weight dimension too large");
    if (d->device < 0) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "device ordinal is negative");
    return AILA_NF4_OK;
}

// Builds the linear for rows [row0, row0+rows) x columns [col0, col0+cols) of the described
// weight (the whole weight for a plain create).
AilaNf4Status create_slice(const AilaNf4WeightDesc* d, int64_t row0, int64_t rows, int64_t col0,
                           int64_t cols, AilaNf4Linear** out) {
    using nf4::fail;
    if (!out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "output handle pointer is NULL");
    *out = nullptr;
    int n_dev = 0;
    NF4_CUDA(cudaGetDeviceCount(&n_dev));
    if (d->device >= n_dev) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "no such CUDA device");
    DeviceGuard guard(d->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");

    AilaNf4Linear* l = new (std::nothrow) AilaNf4Linear();
    if (!l) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    l->device = d->device;
    l->N = rows;
    l->K = cols;
    l->blocksize = d->blocksize;
    l->absmax_kind = d->nested ? nf4::kAbsmaxCodes : nf4::kAbsmaxF32;
    l->unit_stride = d->nested ? nf4::kUnitStrideCodes : nf4::kUnitStrideF32;
    l->RT = (int)((rows + nf4::kTileRows - 1) / nf4::kTileRows);
    l->KU = (int)(cols / nf4::kUnitK);
    l->nbs = d->nested ? d->nested_blocksize : 256;
    const bool dev_src = d->pointers_on_device != 0;
    const int64_t bpr_full = d->in_features / d->blocksize;  // absmax per full source row
    const size_t abs_elem = d->nested ? 1 : 4;

    void* tmp_packed = nullptr;
    void* tmp_abs = nullptr;
    auto cleanup = [&](AilaNf4Status st) {
        cudaFree(tmp_packed);
        cudaFree(tmp_abs);
        if (st != AILA_NF4_OK) free_linear(l);
        return st;
    };
#define NF4_TRY(call)                                                        \
    do {                                                                     \
        cudaError_t e__ = (call);                                            \
        if (e__ != cudaSuccess) return cleanup(nf4::cuda_fail(e__, #call)); \
    } while (0)

    NF4_TRY(cudaMalloc(reinterpret_cast<void**>(&l->d_units), l->units_bytes() + 16));
    NF4_TRY(intern_table(&l->d_qmap, d->quant_map, 16, dev_src, l->device));
    NF4_TRY(cudaMemcpy(l->h_qmap, d->quant_map, 16 * sizeof(float),
                       dev_src ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost));
    if (d->nested) {
        NF4_TRY(intern_table(&l->d_nmap, d->nested_quant_map, 256, dev_src, l->device));
        NF4_TRY(upload(&l->d_nabs, d->nested_absmax, (size_t)d->nested_absmax_count, dev_src));
        l->nabs_count = d->nested_absmax_count;
    }
    l->device_bytes = (int64_t)l->units_bytes() + 16 * 4 + (d->nested ? 256 * 4 + l->nabs_count * 4 : 0);

    nf4::RepackSource src;
    if (dev_src) {
        src.packed = d->packed_weight;
        src.row_stride_bytes = d->in_features / 2;
        src.col_byte0 = col0 / 2;
        src.absmax = d->absmax;
        src.abs_row_stride = bpr_full;
        src.abs_col0 = col0 / d->blocksize;
        src.row0 = row0;
    } else {
        // stage only the kept slice
        const size_t pw = (size_t)cols / 2, aw = (size_t)(cols / d->blocksize) * abs_elem;
        NF4_TRY(cudaMalloc(&tmp_packed, (size_t)rows * pw + 16));
        NF4_TRY(cudaMalloc(&tmp_abs, (size_t)rows * aw + 16));
        NF4_TRY(cudaMemcpy2D(tmp_packed, pw,
                             d->packed_weight + (size_t)row0 * (d->in_features / 2) + col0 / 2,
                             (size_t)d->in_features / 2, pw, (size_t)rows, cudaMemcpyHostToDevice));
        NF4_TRY(cudaMemcpy2D(tmp_abs, aw,
                             static_cast<const uint8_t*>(d->absmax) +
                                 ((size_t)row0 * bpr_full + col0 / d->blocksize) * abs_elem,
                             (size_t)bpr_full * abs_elem, aw, (size_t)rows, cudaMemcpyHostToDevice));
        src.packed = static_cast<const uint8_t*>(tmp_packed);
        src.row_stride_bytes = (int64_t)pw;
        src.col_byte0 = 0;
        src.absmax = tmp_abs;
        src.abs_row_stride = cols / d->blocksize;
        src.abs_col0 = 0;
        src.row0 = 0;
    }
    NF4_TRY(nf4::launch_repack(src, *l, 0));
    NF4_TRY(cudaDeviceSynchronize());

    l->nseg = 1;
    l->seg_row0[0] = 0;
    l->seg_rows[0] = (int)rows;
    l->seg_flat0[0] = row0 * bpr_full + col0 / d->blocksize;
    l->seg_row_stride[0] = bpr_full;
    l->seg_nabs_base[0] = 0;
    l->seg_offset[0] = d->nested ? d->nested_offset : 0.0f;
#undef NF4_TRY
    {
        const AilaNf4Status cst = maybe_cache_dequant(l);
        if (cst != AILA_NF4_OK) return cleanup(cst);
    }
    *out = l;
    return cleanup(AILA_NF4_OK);
}

AilaNf4Status check_forward_args(const AilaNf4Linear* l, AilaNf4Scratch* sc, const void* x,
                                 const void* y, int seq_len) {
    using nf4::fail;
    if (!l) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "linear handle is NULL");
    if (!sc) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch handle is NULL");
    if (!x || !y)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Bnb4BitLinear expects bf16 input/output tensors");
    if (seq_len <= 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Bnb4BitLinear::forward: seq_len must be positive");
    if (sc->device != l->device)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch and linear live on different devices");
    return AILA_NF4_OK;
}

AilaNf4Status ensure_weight(AilaNf4Scratch* sc, size_t bytes) {
    if (sc->weight_bytes >= bytes) return AILA_NF4_OK;
    // grow-only, like Bnb4BitLinearScratch::ensure; allocating synchronises the device
    if (sc->d_weight) NF4_CUDA(cudaFree(sc->d_weight));
    sc->d_weight = nullptr;
    sc->weight_bytes = 0;
    cudaError_t e = cudaMalloc(&sc->d_weight, bytes + 256);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return nf4::fail(AILA_NF4_ERR_OUT_OF_MEMORY, "GPU memory allocation failed: " +
                                                         std::to_string(bytes) + " bytes");
    }
    NF4_CUDA(e);
    sc->weight_bytes = bytes;
    return AILA_NF4_OK;
}

using nf4::ensure_counters;

// Accumulation tiles of the K-sliced small-batch kernel: zero when allocated, and every launch
// leaves them zero. Growing allocates and waits for the device (not capturable).
AilaNf4Status ensure_rows_acc(AilaNf4Scratch* sc, size_t bytes) {
    if (sc->rows_acc_bytes >= bytes) return AILA_NF4_OK;
    if (sc->d_rows_acc) NF4_CUDA(cudaFree(sc->d_rows_acc));
    sc->d_rows_acc = nullptr;
    sc->rows_acc_bytes = 0;
    NF4_CUDA(cudaMalloc(reinterpret_cast<void**>(&sc->d_rows_acc), bytes));
    NF4_CUDA(cudaMemset(sc->d_rows_acc, 0, bytes));
    NF4_CUDA(cudaDeviceSynchronize());
    sc->rows_acc_bytes = bytes;
    return AILA_NF4_OK;
}

AilaNf4Status ensure_io(void** buf, size_t* have, size_t need) {
    if (*have >= need) return AILA_NF4_OK;
    if (*buf) NF4_CUDA(cudaFree(*buf));
    *buf = nullptr;
    *have = 0;
    NF4_CUDA(cudaMalloc(buf, need + 256));
    *have = need;
    return AILA_NF4_OK;
}

// Small batches (2 .. AILA_NF4_DECODE_ROWS_MAX rows, default 48; 0 or 1 turns it off): batched decode
// launches of up to 32 rows each (one pass over the weights per launch) instead of the dequantise +
// GEMM route, when a small-batch kernel takes the shape and no bf16 weight cache exists (with a
// cache the GEMM has nothing to dequantise). A pass of 32 and one of 16 rows still beat the GEMM
// route (measured on the cfg4 stack: 5.0 ms against 5.6 ms per step at 48 rows; two passes of 32
// rows, 5.9 ms, do not).
int decode_rows_max() {
    static const int v = [] {
        const char* e = std::getenv("AILA_NF4_DECODE_ROWS_MAX");
        if (!e || !*e) return 48;
        const int n = std::atoi(e);
        return n < 0 ? 0 : (n > 128 ? 128 : n);
    }();
    return v;
}

// The K-sliced kernel (x slice of all rows in shared memory) serves 9 .. 32 rows where it takes the
// linear: up to eight rows the streaming kernel's batched form is faster (its x fragments from L2
// cost less than the K-sliced kernel's accumulation in global memory).
// AILA_NF4_ROWS_KERNEL=0 turns it off, =1 uses it from two rows on.
bool use_rows_kernel(const AilaNf4Linear* l, int64_t ff_pair, int rows) {
    static const int mode = [] {
        const char* e = std::getenv("AILA_NF4_ROWS_KERNEL");
        return (e && e[0] == '0') ? 0 : ((e && e[0] == '1') ? 1 : 2);
    }();
    if (mode == 0 || rows < 2 || (mode == 2 && rows <= 8)) return false;
    return nf4::gemv_rows_supported(*l, ff_pair);
}

bool use_batched_decode(const AilaNf4Linear* l, const AilaNf4Scratch* sc, const void* x, int seq_len,
                  int64_t ff_pair) {
    if (seq_len < 2 || seq_len > decode_rows_max() || l->d_cache_bf16) return false;
    if (gemv_kernel_choice() == 1) return false;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (l->K * 2) % 16) return false;
    return use_rows_kernel(l, ff_pair, seq_len) || nf4::gemv_stream_supported(*l, ff_pair, sc->sm_count);
}

// Rows one batched launch carries: 32 (four row blocks) where the kernel's shared-memory plan has
// room for the larger accumulation tiles, else 8.
int batched_rows_per_launch(const AilaNf4Linear* l, const AilaNf4Scratch* sc, int64_t ff_pair, int seq_len) {
    if (use_rows_kernel(l, ff_pair, seq_len)) return 32;
    if (ff_pair > 0) return 8;
    return nf4::gemv_stream_supported(*l, 0, sc->sm_count, 4) ? 32 : 8;
}

// Prefill with the weight dequantised inside the GEMM instead of a bf16 copy of W written to and read
// back from HBM: AILA_NF4_FUSED_PREFILL=1 takes the fused kernel wherever it takes the linear. It is
// bit-identical to the two-phase route and slower at every measured size (each 256-row tile of x pays
// the dequantisation arithmetic again, and the w tile is produced in step with the tensor core instead
// of arriving by TMA), so the default is the two-phase route.
bool use_fused_prefill(const AilaNf4Linear* l, int64_t ff_dim, int seq_len) {
    static const bool on = [] {
        const char* e = std::getenv("AILA_NF4_FUSED_PREFILL");
        return e && e[0] == '1';
    }();
    (void)seq_len;
    if (!on || l->d_cache_bf16) return false;
    return nf4::gemm_nf4_fused_supported(*l, ff_dim);
}

// seq_len == 1: decode kernels. ff_pair > 0 selects the gate/up pair kernel.
AilaNf4Status run_decode(const AilaNf4Linear* l, AilaNf4Scratch* sc, const void* x, void* y,
                         const void* residual, int64_t ff_pair, cudaStream_t s, int m_rows = 1,
                         const nf4::NormInput* norm = nullptr) {
    if (m_rows > 1 && !norm && use_rows_kernel(l, ff_pair, m_rows) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        AilaNf4Status st = ensure_counters(sc, (size_t)l->RT);
        if (st != AILA_NF4_OK) return st;
        st = ensure_rows_acc(sc, nf4::gemv_rows_acc_bytes(*l));
        if (st != AILA_NF4_OK) return st;
        NF4_CUDA(nf4::launch_gemv_rows(*l, *sc, x, y, residual, ff_pair, s, m_rows));
        return AILA_NF4_OK;
    }
    const int choice = gemv_kernel_choice();
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    // One operation per launch: the ring kernel starts faster than the chained kernel (which pays
    // for a cooperative launch and builds for a whole list), so it is the first choice here; the
    // chained kernel as a one-operation launch takes what the ring kernel does not.
    const bool chain_ok = m_rows == 1 && (reinterpret_cast<uintptr_t>(x) & 7) == 0 &&
                          nf4::gemv_chain_supported(*l, ff_pair, *sc) && !(norm && l->K > 11520);
    bool stream_ok = aligned && nf4::gemv_stream_supported(*l, ff_pair, sc->sm_count);
    if (choice == 1 || choice == 3) stream_ok = false;
    if (choice == 3 && !chain_ok)
        return nf4::fail(AILA_NF4_ERR_UNSUPPORTED,
                         "chained decode kernel was forced but does not take this call");
    if (choice == 2 && !stream_ok)
        return nf4::fail(AILA_NF4_ERR_UNSUPPORTED,
                         "streaming decode kernel was forced but does not take this shape");
    if (!stream_ok && chain_ok && choice != 1 && choice != 2)
        return nf4::launch_gemv_chain_single(*l, *sc, x, y, residual, ff_pair, norm, s);
    if (stream_ok) {
        const size_t tiles = (size_t)(ff_pair > 0 ? ff_pair / nf4::kTileRows : l->RT);
        AilaNf4Status st = ensure_counters(sc, tiles);
        if (st != AILA_NF4_OK) return st;
        NF4_CUDA(nf4::launch_gemv_stream(*l, *sc, x, y, residual, ff_pair, s, nullptr, m_rows, norm));
    } else {
        if (norm)
            return nf4::fail(AILA_NF4_NOT_APPLICABLE,
                             "the fused RMSNorm input needs the streaming decode kernel");
        if (m_rows != 1)
            return nf4::fail(AILA_NF4_ERR_UNSUPPORTED, "batched decode needs the streaming kernel");
        NF4_CUDA(nf4::launch_gemv_simple(*l, x, y, residual, ff_pair, s));
    }
    return AILA_NF4_OK;
}

}  // namespace

// ---------------------------------------------------------------------------------------
namespace nf4 {

AilaNf4Status ensure_counters(AilaNf4Scratch* sc, size_t tiles) {
    if (sc->counters_ints >= tiles) return AILA_NF4_OK;
    if (sc->d_counters) NF4_CUDA(cudaFree(sc->d_counters));
    sc->d_counters = nullptr;
    sc->counters_ints = 0;
    // Growing inside a forward call (more than 262,144 output rows without an
    // aila_nf4_scratch_reserve before) allocates: not capturable, and it waits for the device so
    // that the zeros are in place whatever stream the kernel runs on.
    NF4_CUDA(cudaMalloc(reinterpret_cast<void**>(&sc->d_counters), tiles * sizeof(int)));
    NF4_CUDA(cudaMemset(sc->d_counters, 0, tiles * sizeof(int)));
    NF4_CUDA(cudaDeviceSynchronize());
    sc->counters_ints = tiles;
    return AILA_NF4_OK;
}

AilaNf4Status fail(AilaNf4Status code, const std::string& message) {
    g_last_error = message;
    return code;
}

AilaNf4Status cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return e == cudaErrorMemoryAllocation ? AILA_NF4_ERR_OUT_OF_MEMORY : AILA_NF4_ERR_CUDA;
}

}  // namespace nf4

nf4::ScaleParams AilaNf4Linear::scale_params() const {
    nf4::ScaleParams sp;
    sp.nmap = d_nmap;
    sp.nabs = d_nabs;
    sp.nseg = nseg;
    sp.nbs_shift = ilog2i(nbs);
    sp.blk_shift = ilog2i(blocksize / nf4::kUnitK);
    for (int i = 0; i < nf4::kMaxSegments; ++i) {
        const int j = i < nseg ? i : 0;
        sp.row0[i] = seg_row0[j];
        sp.flat0[i] = (unsigned)(seg_nabs_base[j] * nbs + seg_flat0[j]);
        sp.row_stride[i] = (unsigned)seg_row_stride[j];
        sp.offset[i] = seg_offset[j];
    }
    return sp;
}

// ---------------------------------------------------------------------------------------
AILA_NF4_API const char* aila_nf4_last_error(void) { return g_last_error.c_str(); }

AILA_NF4_API int aila_nf4_version(void) { return 100; }

AILA_NF4_API AilaNf4Status aila_nf4_linear_create(const AilaNf4WeightDesc* desc,
                                                  AilaNf4Linear** out) {
    AilaNf4Status st = validate_desc(desc);
    if (st != AILA_NF4_OK) return st;
    return create_slice(desc, 0, desc->out_features, 0, desc->in_features, out);
}

AILA_NF4_API AilaNf4Status aila_nf4_linear_create_shard(const AilaNf4WeightDesc* desc,
                                                        AilaNf4ShardMode mode, int rank,
                                                        int world, AilaNf4Linear** out) {
    AilaNf4Status st = validate_desc(desc);
    if (st != AILA_NF4_OK) return st;
    if (world <= 0 || rank < 0 || rank >= world)
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "shard rank/world out of range");
    if (mode == AILA_NF4_SHARD_ROWS) {
        if (desc->out_features % world != 0)
            return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                             "out_features is not divisible by the number of shards");
        const int64_t rows = desc->out_features / world;
        return create_slice(desc, rank * rows, rows, 0, desc->in_features, out);
    }
    if (mode == AILA_NF4_SHARD_COLS) {
        if (desc->in_features % world != 0 || (desc->in_features / world) % desc->blocksize != 0)
            return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                             "in_features / shards must be a multiple of blocksize");
        const int64_t cols = desc->in_features / world;
        return create_slice(desc, 0, desc->out_features, rank * cols, cols, out);
    }
    return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "unknown shard mode");
}

AILA_NF4_API AilaNf4Status aila_nf4_linear_create_fused_rows(AilaNf4Linear* const* sources,
                                                             int n_sources,
                                                             AilaNf4Linear** out) {
    using nf4::fail;
    if (!out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "output handle pointer is NULL");
    *out = nullptr;
    if (!sources || n_sources < 2 || n_sources > 4)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "Bnb4BitLinear::init_fused_rows requires 2 to 4 source linears");
    const AilaNf4Linear* first = sources[0];
    for (int i = 0; i < n_sources; ++i)
        if (!sources[i] || !sources[i]->d_units)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "Bnb4BitLinear::init_fused_rows: source linear is not initialized");
    int64_t total_rows = 0, total_nabs = 0;
    int total_seg = 0;
    for (int i = 0; i < n_sources; ++i) {
        const AilaNf4Linear* s = sources[i];
        if (s->K != first->K || s->blocksize != first->blocksize || s->device != first->device ||
            s->absmax_kind != first->absmax_kind)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "Bnb4BitLinear::init_fused_rows: incompatible quantized linears");
        for (int q = 0; q < 16; ++q)
            if (std::abs(s->h_qmap[q] - first->h_qmap[q]) > 1e-6f)
                return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                            "Bnb4BitLinear::init_fused_rows: quant maps do not match");
        if (s->absmax_kind == nf4::kAbsmaxCodes && s->nbs != first->nbs)
            return fail(AILA_NF4_ERR_UNSUPPORTED, "fused sources use different nested block sizes");
        total_rows += s->N;
        total_nabs += s->nabs_count;
        total_seg += s->nseg;
    }
    if (total_seg > nf4::kMaxSegments)
        return fail(AILA_NF4_ERR_UNSUPPORTED, "fused linear would have more than 4 sources");
    DeviceGuard guard(first->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");

    AilaNf4Linear* l = new (std::nothrow) AilaNf4Linear();
    if (!l) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    l->device = first->device;
    l->N = total_rows;
    l->K = first->K;
    l->blocksize = first->blocksize;
    l->absmax_kind = first->absmax_kind;
    l->unit_stride = first->unit_stride;
    l->RT = (int)((total_rows + nf4::kTileRows - 1) / nf4::kTileRows);
    l->KU = first->KU;
    l->nbs = first->nbs;
    std::memcpy(l->h_qmap, first->h_qmap, sizeof(l->h_qmap));
    auto bail = [&](AilaNf4Status st) {
        free_linear(l);
        return st;
    };
#define NF4_TRY(call)                                                     \
    do {                                                                  \
        cudaError_t e__ = (call);                                         \
        if (e__ != cudaSuccess) return bail(nf4::cuda_fail(e__, #call)); \
    } while (0)
    NF4_TRY(cudaMalloc(reinterpret_cast<void**>(&l->d_units), l->units_bytes() + 16));
    NF4_TRY(intern_table(&l->d_qmap, first->d_qmap, 16, true, l->device));
    if (l->absmax_kind == nf4::kAbsmaxCodes) {
        // the second-level code book must be the same table in every source
        std::vector<float> ref(256), cur(256);
        NF4_TRY(cudaMemcpy(ref.data(), first->d_nmap, 256 * 4, cudaMemcpyDeviceToHost));
        for (int i = 1; i < n_sources; ++i) {
            NF4_TRY(cudaMemcpy(cur.data(), sources[i]->d_nmap, 256 * 4, cudaMemcpyDeviceToHost));
            if (std::memcmp(ref.data(), cur.data(), 256 * 4) != 0)
                return bail(fail(AILA_NF4_ERR_UNSUPPORTED,
                                 "fused sources use different nested quant maps"));
        }
        NF4_TRY(intern_table(&l->d_nmap, first->d_nmap, 256, true, l->device));
        NF4_TRY(cudaMalloc(reinterpret_cast<void**>(&l->d_nabs), (size_t)total_nabs * 4 + 16));
        l->nabs_count = total_nabs;
    }
    nf4::GatherSource gs[nf4::kMaxSegments];
    int seg = 0;
    int64_t row = 0, nabs_off = 0;
    for (int i = 0; i < n_sources; ++i) {
        const AilaNf4Linear* s = sources[i];
        gs[i].units = s->d_units;
        gs[i].KU = s->KU;
        gs[i].unit_stride = s->unit_stride;
        gs[i].src_row0 = 0;
        gs[i].src_kb0 = 0;
        gs[i].dst_row0 = (int)row;
        gs[i].rows = (int)s->N;
        for (int j = 0; j < s->nseg; ++j, ++seg) {
            l->seg_row0[seg] = (int)row + s->seg_row0[j];
            l->seg_rows[seg] = s->seg_rows[j];
            l->seg_flat0[seg] = s->seg_flat0[j];
            l->seg_row_stride[seg] = s->seg_row_stride[j];
            l->seg_nabs_base[seg] = nabs_off + s->seg_nabs_base[j];
            l->seg_offset[seg] = s->seg_offset[j];
        }
        if (l->absmax_kind == nf4::kAbsmaxCodes && s->nabs_count > 0)
            NF4_TRY(cudaMemcpy(l->d_nabs + nabs_off, s->d_nabs, (size_t)s->nabs_count * 4,
                               cudaMemcpyDeviceToDevice));
        row += s->N;
        nabs_off += s->nabs_count;
    }
    l->nseg = seg;
    for (int i = 0; i < seg; ++i)
        if (l->seg_nabs_base[i] * l->nbs + l->seg_flat0[i] +
                (int64_t)l->seg_rows[i] * l->seg_row_stride[i] >= ((int64_t)1 << 32))
            return bail(fail(AILA_NF4_ERR_UNSUPPORTED, "fused weight has too many absmax blocks"));
    NF4_TRY(nf4::launch_gather(gs, n_sources, *l, 0));
    NF4_TRY(cudaDeviceSynchronize());
#undef NF4_TRY
    l->device_bytes = (int64_t)l->units_bytes() + 16 * 4 +
                      (l->absmax_kind == nf4::kAbsmaxCodes ? 256 * 4 + l->nabs_count * 4 : 0);
    {
        const AilaNf4Status cst = maybe_cache_dequant(l);
        if (cst != AILA_NF4_OK) {
            free_linear(l);
            return cst;
        }
    }
    *out = l;
    return AILA_NF4_OK;
}

AILA_NF4_API void aila_nf4_linear_destroy(AilaNf4Linear* linear) { free_linear(linear); }

AILA_NF4_API int64_t aila_nf4_linear_in_features(const AilaNf4Linear* l) { return l ? l->K : 0; }
AILA_NF4_API int64_t aila_nf4_linear_out_features(const AilaNf4Linear* l) { return l ? l->N : 0; }
AILA_NF4_API int64_t aila_nf4_linear_device_bytes(const AilaNf4Linear* l) {
    return l ? l->device_bytes : 0;
}
AILA_NF4_API int aila_nf4_linear_device(const AilaNf4Linear* l) { return l ? l->device : -1; }

// ---------------------------------------------------------------------------------------
AILA_NF4_API AilaNf4Status aila_nf4_scratch_create(int device, AilaNf4Scratch** out) {
    using nf4::fail;
    if (!out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "output handle pointer is NULL");
    *out = nullptr;
    int n_dev = 0;
    NF4_CUDA(cudaGetDeviceCount(&n_dev));
    if (device < 0 || device >= n_dev)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "no such CUDA device");
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    AilaNf4Scratch* sc = new (std::nothrow) AilaNf4Scratch();
    if (!sc) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    sc->device = device;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess && prop.major != 10) {
        delete sc;
        return fail(AILA_NF4_ERR_UNSUPPORTED,
                    "this library is built for sm_100a (B200) only; device is sm_" +
                        std::to_string(prop.major) + std::to_string(prop.minor));
    }
    auto bail = [&](cudaError_t err, const char* what) {
        aila_nf4_scratch_destroy(sc);
        return nf4::cuda_fail(err, what);
    };
    if (e != cudaSuccess) return bail(e, "cudaGetDeviceProperties");
    sc->sm_count = prop.multiProcessorCount;
    sc->partials_floats = nf4::gemv_stream_partials_floats(sc->sm_count);
    if ((e = cudaMalloc(reinterpret_cast<void**>(&sc->d_partials), sc->partials_floats * 4)) != cudaSuccess)
        return bail(e, "cudaMalloc(partials)");
    if ((e = cudaMemset(sc->d_partials, 0, sc->partials_floats * 4)) != cudaSuccess)
        return bail(e, "cudaMemset(partials)");
    if ((e = cudaMalloc(reinterpret_cast<void**>(&sc->d_status), 64)) != cudaSuccess)
        return bail(e, "cudaMalloc(status)");
    if ((e = cudaMemset(sc->d_status, 0, 64)) != cudaSuccess) return bail(e, "cudaMemset(status)");
    AilaNf4Status st = ensure_counters(sc, 1 << 14);
    if (st == AILA_NF4_OK) st = nf4::ensure_chain_scratch(sc);
    if (st != AILA_NF4_OK) {
        aila_nf4_scratch_destroy(sc);
        return st;
    }
    NF4_CUDA(cudaDeviceSynchronize());
    *out = sc;
    return AILA_NF4_OK;
}

AILA_NF4_API void aila_nf4_scratch_destroy(AilaNf4Scratch* sc) {
    if (!sc) return;
    DeviceGuard guard(sc->device);
    cudaFree(sc->d_partials);
    cudaFree(sc->d_rows_acc);
    cudaFree(sc->d_counters);
    cudaFree(sc->d_status);
    cudaFree(sc->d_weight);
    cudaFree(sc->d_io_in);
    cudaFree(sc->d_io_out);
    cudaFree(sc->d_chain_ctrl);
    delete sc;
}

AILA_NF4_API AilaNf4Status aila_nf4_scratch_reserve(AilaNf4Scratch* sc, int seq_len,
                                                    int64_t in_features, int64_t out_features,
                                                    int need_weight) {
    if (!sc) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch handle is NULL");
    if (seq_len <= 0 || in_features <= 0 || out_features <= 0)
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch_reserve: sizes must be positive");
    DeviceGuard guard(sc->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    const size_t tiles = (size_t)((out_features + nf4::kTileRows - 1) / nf4::kTileRows);
    AilaNf4Status st = ensure_counters(sc, tiles);
    if (st != AILA_NF4_OK) return st;
    if (seq_len > 1) {
        // accumulation tiles of the small-batch kernel (16 rows x 32 batch columns of fp32 per row tile)
        st = ensure_rows_acc(sc, tiles * nf4::kTileRows * 32 * sizeof(float));
        if (st != AILA_NF4_OK) return st;
    }
    if (need_weight) {
        st = ensure_weight(sc, (size_t)in_features * (size_t)out_features * 2);
        if (st != AILA_NF4_OK) return st;
    }
    st = ensure_io(&sc->d_io_in, &sc->io_in_bytes, (size_t)seq_len * (size_t)in_features * 2);
    if (st != AILA_NF4_OK) return st;
    return ensure_io(&sc->d_io_out, &sc->io_out_bytes, (size_t)seq_len * (size_t)out_features * 2);
}

AILA_NF4_API AilaNf4Status aila_nf4_scratch_check(AilaNf4Scratch* sc, void* stream) {
    if (!sc) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch handle is NULL");
    DeviceGuard guard(sc->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host = 0;
    NF4_CUDA(cudaMemcpyAsync(&host, sc->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    NF4_CUDA(cudaStreamSynchronize(s));
    if (host != 0) {
        NF4_CUDA(cudaMemsetAsync(sc->d_status, 0, sizeof(int), s));
        // the chained kernel's "somebody gave up" word: later launches start clean
        if (sc->d_chain_ctrl) NF4_CUDA(cudaMemsetAsync(sc->d_chain_ctrl + 2, 0, sizeof(unsigned), s));
        // a launch that gave up may have left row-tile counters and accumulation tiles of the decode
        // kernels half-way; every kernel expects to find them zero
        if (sc->d_counters) NF4_CUDA(cudaMemsetAsync(sc->d_counters, 0, sc->counters_ints * sizeof(int), s));
        if (sc->d_rows_acc) NF4_CUDA(cudaMemsetAsync(sc->d_rows_acc, 0, sc->rows_acc_bytes, s));
        NF4_CUDA(cudaStreamSynchronize(s));
        return nf4::fail(AILA_NF4_ERR_KERNEL_TIMEOUT,
                         "a bounded device-side wait expired (code " + std::to_string(host) + ")");
    }
    return AILA_NF4_OK;
}

// ---------------------------------------------------------------------------------------
AILA_NF4_API AilaNf4Status aila_nf4_forward(const AilaNf4Linear* l, AilaNf4Scratch* sc,
                                            const void* x, void* y, int seq_len,
                                            const void* residual, void* stream) {
    AilaNf4Status st = check_forward_args(l, sc, x, y, seq_len);
    if (st != AILA_NF4_OK) return st;
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (seq_len == 1) return run_decode(l, sc, x, y, residual, 0, s);
    if (use_batched_decode(l, sc, x, seq_len, 0)) {
        // a few rows: the batched decode kernel carries up to 32 rows through the tensor-core
        // tile's batch columns (every decoded weight fragment feeds one operation per block of
        // eight rows) and reads 0.52 B per weight per launch; the dequantise + GEMM route moves
        // 4.5 B per weight whatever the row count
        const char* xb = static_cast<const char*>(x);
        char* yb = static_cast<char*>(y);
        const char* rb = static_cast<const char*>(residual);
        const int step = batched_rows_per_launch(l, sc, 0, seq_len);
        for (int m = 0; m < seq_len; m += step) {
            const int rows = seq_len - m < step ? seq_len - m : step;
            st = run_decode(l, sc, xb + (size_t)m * l->K * 2, yb + (size_t)m * l->N * 2,
                            rb ? rb + (size_t)m * l->N * 2 : nullptr, 0, s, rows);
            if (st != AILA_NF4_OK) return st;
        }
        return AILA_NF4_OK;
    }
    if (use_fused_prefill(l, 0, seq_len))
        return nf4::launch_gemm_nf4_fused(*l, x, y, residual, seq_len, 0, sc->sm_count, sc->d_status, s);
    const void* wsrc = l->d_cache_bf16;
    if (!wsrc) {
        st = ensure_weight(sc, (size_t)l->N * (size_t)l->K * 2);
        if (st != AILA_NF4_OK) return st;
        NF4_CUDA(nf4::launch_dequant_nk(*l, sc->d_weight, s));
        wsrc = sc->d_weight;
    }
    return nf4::launch_gemm_bf16(wsrc, x, y, residual, seq_len, l->N, l->K, 0, l->device,
                                 sc->sm_count, sc->d_status, s);
}

AILA_NF4_API AilaNf4Status aila_nf4_forward_gate_up_swiglu(const AilaNf4Linear* l,
                                                           AilaNf4Scratch* sc, const void* x,
                                                           void* out, int seq_len, int64_t ff_dim,
                                                           void* stream) {
    AilaNf4Status st = check_forward_args(l, sc, x, out, seq_len);
    if (st != AILA_NF4_OK) return st;
    if (ff_dim <= 0 || l->N != 2 * ff_dim)
        return nf4::fail(AILA_NF4_NOT_APPLICABLE, "out_features != 2 * ff_dim");
    if (ff_dim % nf4::kTileRows != 0)
        return nf4::fail(AILA_NF4_NOT_APPLICABLE, "ff_dim is not a multiple of 16");
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (seq_len == 1) return run_decode(l, sc, x, out, nullptr, ff_dim, s);
    if (seq_len > 8 && !use_rows_kernel(l, ff_dim, seq_len) && use_batched_decode(l, sc, x, seq_len, 0) &&
        batched_rows_per_launch(l, sc, 0, seq_len) > 8) {
        // more than eight rows: the unpaired batched kernel over the fused rows (one pass over the
        // weights for up to 32 rows) into a bf16 gate|up buffer, then the row-wise activation -
        // the arithmetic of the reference's seq_len > 1 route (bf16 gate_up, then ops::swiglu)
        st = ensure_weight(sc, (size_t)seq_len * (size_t)l->N * 2);
        if (st != AILA_NF4_OK) return st;
        const char* xb = static_cast<const char*>(x);
        char* gu = static_cast<char*>(sc->d_weight);
        for (int m = 0; m < seq_len; m += 32) {
            const int rows = seq_len - m < 32 ? seq_len - m : 32;
            st = run_decode(l, sc, xb + (size_t)m * l->K * 2, gu + (size_t)m * l->N * 2, nullptr, 0, s, rows);
            if (st != AILA_NF4_OK) return st;
        }
        NF4_CUDA(nf4::launch_swiglu_rows(sc->d_weight, out, seq_len, ff_dim, s));
        return AILA_NF4_OK;
    }
    if (use_batched_decode(l, sc, x, seq_len, ff_dim)) {
        const char* xb = static_cast<const char*>(x);
        char* ob = static_cast<char*>(out);
        const int step = batched_rows_per_launch(l, sc, ff_dim, seq_len);
        for (int m = 0; m < seq_len; m += step) {
            const int rows = seq_len - m < step ? seq_len - m : step;
            st = run_decode(l, sc, xb + (size_t)m * l->K * 2, ob + (size_t)m * ff_dim * 2, nullptr,
                            ff_dim, s, rows);
            if (st != AILA_NF4_OK) return st;
        }
        return AILA_NF4_OK;
    }
    if (use_fused_prefill(l, ff_dim, seq_len))
        return nf4::launch_gemm_nf4_fused(*l, x, out, nullptr, seq_len, ff_dim, sc->sm_count, sc->d_status, s);
    const void* wsrc = l->d_cache_bf16;
    if (!wsrc) {
        st = ensure_weight(sc, (size_t)l->N * (size_t)l->K * 2);
        if (st != AILA_NF4_OK) return st;
        NF4_CUDA(nf4::launch_dequant_nk(*l, sc->d_weight, s));
        wsrc = sc->d_weight;
    }
    return nf4::launch_gemm_bf16(wsrc, x, out, nullptr, seq_len, l->N, l->K, ff_dim, l->device,
                                 sc->sm_count, sc->d_status, s);
}

namespace {
AilaNf4Status check_norm(const AilaNf4Linear* l, const void* x, const AilaNf4RmsNorm* norm,
                         nf4::NormInput* out) {
    if (!norm || !norm->weight_bf16)
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "RMSNorm weight is NULL");
    if (!(norm->eps >= 0.0f)) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "RMSNorm eps must be >= 0");
    if (norm->hidden_out_bf16 && (norm->hidden_out_bf16 == x || norm->hidden_out_bf16 == norm->add_bf16))
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                         "hidden_out must not alias x or the added tensor (every CTA reads them)");
    const uintptr_t bits = reinterpret_cast<uintptr_t>(norm->weight_bf16) |
                           reinterpret_cast<uintptr_t>(norm->add_bf16) |
                           reinterpret_cast<uintptr_t>(norm->hidden_out_bf16);
    if (bits & 7) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "RMSNorm tensors must be 8-byte aligned");
    (void)l;
    out->add = norm->add_bf16;
    out->weight = norm->weight_bf16;
    out->hidden_out = norm->hidden_out_bf16;
    out->eps = norm->eps;
    return AILA_NF4_OK;
}
}  // namespace

AILA_NF4_API AilaNf4Status aila_nf4_forward_rmsnorm(const AilaNf4Linear* l, AilaNf4Scratch* sc,
                                                    const void* x, const AilaNf4RmsNorm* norm,
                                                    void* y, const void* residual, void* stream) {
    AilaNf4Status st = check_forward_args(l, sc, x, y, 1);
    if (st != AILA_NF4_OK) return st;
    nf4::NormInput ni;
    if ((st = check_norm(l, x, norm, &ni)) != AILA_NF4_OK) return st;
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    return run_decode(l, sc, x, y, residual, 0, static_cast<cudaStream_t>(stream), 1, &ni);
}

AILA_NF4_API AilaNf4Status aila_nf4_forward_gate_up_swiglu_rmsnorm(
    const AilaNf4Linear* l, AilaNf4Scratch* sc, const void* x, const AilaNf4RmsNorm* norm, void* out,
    int64_t ff_dim, void* stream) {
    AilaNf4Status st = check_forward_args(l, sc, x, out, 1);
    if (st != AILA_NF4_OK) return st;
    if (ff_dim <= 0 || l->N != 2 * ff_dim)
        return nf4::fail(AILA_NF4_NOT_APPLICABLE, "out_features != 2 * ff_dim");
    if (ff_dim % nf4::kTileRows != 0)
        return nf4::fail(AILA_NF4_NOT_APPLICABLE, "ff_dim is not a multiple of 16");
    nf4::NormInput ni;
    if ((st = check_norm(l, x, norm, &ni)) != AILA_NF4_OK) return st;
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    return run_decode(l, sc, x, out, nullptr, ff_dim, static_cast<cudaStream_t>(stream), 1, &ni);
}

namespace {
// A page-locked host buffer that the GPU can address (cudaHostAlloc / cudaHostRegister memory
// under unified addressing): the kernels then write the result straight into it and the
// device-to-host copy of the host entry points is skipped. NULL for pageable memory.
void* device_view_of_host(const void* host_ptr) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host_ptr) != cudaSuccess) {
        cudaGetLastError();  // pageable memory reports an error on some drivers: not a failure
        return nullptr;
    }
    if (attr.type != cudaMemoryTypeHost || !attr.devicePointer) return nullptr;
    return attr.devicePointer;
}
}  // namespace

AILA_NF4_API AilaNf4Status aila_nf4_forward_host(const AilaNf4Linear* l, AilaNf4Scratch* sc,
                                                 const void* x_host, void* y_host, int seq_len,
                                                 void* stream) {
    AilaNf4Status st = check_forward_args(l, sc, x_host, y_host, seq_len);
    if (st != AILA_NF4_OK) return st;
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t in_b = (size_t)seq_len * (size_t)l->K * 2, out_b = (size_t)seq_len * (size_t)l->N * 2;
    if ((st = ensure_io(&sc->d_io_in, &sc->io_in_bytes, in_b)) != AILA_NF4_OK) return st;
    if ((st = ensure_io(&sc->d_io_out, &sc->io_out_bytes, out_b)) != AILA_NF4_OK) return st;
    NF4_CUDA(cudaMemcpyAsync(sc->d_io_in, x_host, in_b, cudaMemcpyHostToDevice, s));
    // single-row results (tens of KB) go straight into GPU-addressable host memory
    void* y_direct = seq_len == 1 ? device_view_of_host(y_host) : nullptr;
    st = aila_nf4_forward(l, sc, sc->d_io_in, y_direct ? y_direct : sc->d_io_out, seq_len, nullptr, stream);
    if (st != AILA_NF4_OK) return st;
    if (!y_direct) NF4_CUDA(cudaMemcpyAsync(y_host, sc->d_io_out, out_b, cudaMemcpyDeviceToHost, s));
    NF4_CUDA(cudaStreamSynchronize(s));
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_forward_gate_up_swiglu_host(
    const AilaNf4Linear* l, AilaNf4Scratch* sc, const void* x_host, void* out_host, int seq_len,
    int64_t ff_dim, void* stream) {
    AilaNf4Status st = check_forward_args(l, sc, x_host, out_host, seq_len);
    if (st != AILA_NF4_OK) return st;
    if (ff_dim <= 0) return nf4::fail(AILA_NF4_NOT_APPLICABLE, "ff_dim must be positive");
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t in_b = (size_t)seq_len * (size_t)l->K * 2, out_b = (size_t)seq_len * (size_t)ff_dim * 2;
    if ((st = ensure_io(&sc->d_io_in, &sc->io_in_bytes, in_b)) != AILA_NF4_OK) return st;
    if ((st = ensure_io(&sc->d_io_out, &sc->io_out_bytes, out_b)) != AILA_NF4_OK) return st;
    NF4_CUDA(cudaMemcpyAsync(sc->d_io_in, x_host, in_b, cudaMemcpyHostToDevice, s));
    void* out_direct = seq_len == 1 ? device_view_of_host(out_host) : nullptr;
    st = aila_nf4_forward_gate_up_swiglu(l, sc, sc->d_io_in, out_direct ? out_direct : sc->d_io_out,
                                         seq_len, ff_dim, stream);
    if (st != AILA_NF4_OK) return st;
    if (!out_direct) NF4_CUDA(cudaMemcpyAsync(out_host, sc->d_io_out, out_b, cudaMemcpyDeviceToHost, s));
    NF4_CUDA(cudaStreamSynchronize(s));
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_forward_decode_static(const AilaNf4Linear* l, const void* x,
                                                          void* y, const void* residual,
                                                          void* stream) {
    if (!l) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "linear handle is NULL");
    if (!x || !y)
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Bnb4BitLinear expects bf16 input/output tensors");
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    return nf4::launch_gemv_stream_static(*l, x, y, residual, static_cast<cudaStream_t>(stream));
}

AILA_NF4_API AilaNf4Status aila_nf4_static_check(int device, void* stream) {
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    return nf4::check_gemv_stream_static(static_cast<cudaStream_t>(stream));
}

AILA_NF4_API AilaNf4Status aila_nf4_dequantize(const AilaNf4Linear* l, void* out_kn, void* stream) {
    if (!l || !out_kn) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    NF4_CUDA(nf4::launch_dequant_kn(*l, out_kn, static_cast<cudaStream_t>(stream)));
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_dequantize_rowmajor(const AilaNf4Linear* l, void* out_nk,
                                                        void* stream) {
    if (!l || !out_nk) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (reinterpret_cast<uintptr_t>(out_nk) & 15)
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "output must be 16-byte aligned");
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    NF4_CUDA(nf4::launch_dequant_nk(*l, out_nk, static_cast<cudaStream_t>(stream)));
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_expand_absmax(const AilaNf4Linear* l, void* out_f32,
                                                  void* stream) {
    if (!l || !out_f32) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    DeviceGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    NF4_CUDA(nf4::launch_expand_absmax(*l, static_cast<float*>(out_f32),
                                       static_cast<cudaStream_t>(stream)));
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_scratch_set_wait_limit(AilaNf4Scratch* sc, int64_t sm_cycles) {
    if (!sc) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch handle is NULL");
    if (sm_cycles <= 0) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "wait limit must be positive");
    sc->wait_limit_cycles = (long long)sm_cycles;
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_set_gemv_kernel(int which) {
    if (which < 0 || which > 3)
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "gemv kernel selector must be 0, 1, 2 or 3");
    g_gemv_kernel = which;
    return AILA_NF4_OK;
}
