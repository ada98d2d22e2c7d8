// Dense bf16 linear: the unquantised projection that sits next to the NF4 linears in the decode
// stack (the lm_head, 29 % of the bytes of a decode step in the 4B configuration), and a greedy
// argmax over its logits.
//
// Role in the reference: class Linear (src/ops/Ops.hpp:16-31, src/ops/Linear.cpp:172-256), a
// library matmul y = x W^T with W bf16 [out][in], fp32 accumulation, bf16 output; called for the
// last token's hidden state (src/models/Qwen3Bnb4Backend.cpp:432-439); ops::argmax
// (src/ops/SamplingOps.cpp:321-365) picks the token on the device.
//
// seq_len == 1: a streaming GEMV, HBM-bound (2 bytes per weight): every warp owns four
// consecutive rows, reads them with 16-byte non-allocating loads (eight loads in flight per
// lane), x sits in shared memory, fp32 accumulation, one shuffle reduction per row.
// seq_len > 1: the tcgen05 GEMM of the prefill route (the weight already has its [out][in] bf16
// layout).
#include <new>
#include <string>

#include "nf4_internal.h"

struct AilaDenseLinear {
    int device = 0;
    int64_t N = 0, K = 0;
    uint16_t* d_w = nullptr;  // [N][K] bf16
};

namespace nf4 {
namespace {

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w}, xx[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc = fmaf(__uint_as_float(ww[i] << 16), __uint_as_float(xx[i] << 16), acc);
        acc = fmaf(__uint_as_float(ww[i] & 0xffff0000u), __uint_as_float(xx[i] & 0xffff0000u), acc);
    }
    return acc;
}

constexpr int kDenseWarps = 8;
constexpr int kDenseRows = 4;  // rows per warp

// K % 8 == 0, rows 16-byte aligned. Dynamic shared memory: x, K bf16.
__global__ void __launch_bounds__(kDenseWarps * 32)
dense_gemv_kernel(const uint16_t* __restrict__ w, const uint16_t* __restrict__ x,
                  uint16_t* __restrict__ y, const uint16_t* __restrict__ residual, long long N, int K) {
    extern __shared__ __align__(16) uint8_t dense_smem[];
    uint4* xs = reinterpret_cast<uint4*>(dense_smem);
    const int k16 = K >> 3;  // 16-byte pieces per row
    // x may have been written by the previous kernel on the stream: coherent (L2) loads
    for (int i = threadIdx.x; i < k16; i += blockDim.x) xs[i] = __ldcg(reinterpret_cast<const uint4*>(x) + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long r0 = ((long long)blockIdx.x * kDenseWarps + warp) * kDenseRows;
    if (r0 >= N) return;
    const uint4* rows[kDenseRows];
#pragma unroll
    for (int r = 0; r < kDenseRows; ++r) {
        const long long rr = (r0 + r < N) ? r0 + r : N - 1;  // clamp: the tail warp re-reads a row
        rows[r] = reinterpret_cast<const uint4*>(w + rr * K);
    }
    float acc[kDenseRows] = {0.0f, 0.0f, 0.0f, 0.0f};
    int i = lane;
    for (; i + 32 < k16; i += 64) {
        uint4 a[kDenseRows], b[kDenseRows];
#pragma unroll
        for (int r = 0; r < kDenseRows; ++r) {
            a[r] = ldg_stream16(rows[r] + i);
            b[r] = ldg_stream16(rows[r] + i + 32);
        }
        const uint4 xa = xs[i], xb = xs[i + 32];
#pragma unroll
        for (int r = 0; r < kDenseRows; ++r) acc[r] = dot8(b[r], xb, dot8(a[r], xa, acc[r]));
    }
    for (; i < k16; i += 32) {
        const uint4 xa = xs[i];
#pragma unroll
        for (int r = 0; r < kDenseRows; ++r) acc[r] = dot8(ldg_stream16(rows[r] + i), xa, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kDenseRows; ++r)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
    if (lane < kDenseRows && r0 + lane < N) {
        float v = acc[0];
#pragma unroll
        for (int r = 1; r < kDenseRows; ++r)
            if (lane == r) v = acc[r];
        if (residual) v += bf16_bits_to_f32(__ldcg(residual + r0 + lane));
        y[r0 + lane] = f32_to_bf16_bits(v);
    }
}

// Any K (scalar loads): one warp per row. The slow path for shapes the vector kernel does not take.
__global__ void __launch_bounds__(256)
dense_gemv_generic_kernel(const uint16_t* __restrict__ w, const uint16_t* __restrict__ x,
                          uint16_t* __restrict__ y, const uint16_t* __restrict__ residual,
                          long long N, int K) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= N) return;
    float acc = 0.0f;
    for (int k = lane; k < K; k += 32)
        acc = fmaf(bf16_bits_to_f32(w[row * K + k]), bf16_bits_to_f32(__ldcg(x + k)), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        if (residual) acc += bf16_bits_to_f32(__ldcg(residual + row));
        y[row] = f32_to_bf16_bits(acc);
    }
}

// Greedy token choice over bf16 logits with the reference's result on ties (ops::argmax,
// src/ops/SamplingOps.cpp:321-358): a work-group of 256 items, item l scans l, l + 256, ... and keeps
// the first strict maximum above its start value -1e30, then a tree over the items keeps the LEFT
// candidate when two are equal. Two equal candidates meet at the level of the lowest bit in which
// their item numbers differ, and the one with a 0 there is on the left: among equal values the
// winner has the smallest bit-reversed (index % 256), then the smallest index. `offset` is the
// global index of logits[0] (a vocabulary shard orders by global indices and returns a local one).
// NaN and values <= -1e30 never win; if nothing wins the result is 0.
__device__ __forceinline__ unsigned long long argmax_tie_key(long long global_index) {
    return ((unsigned long long)(__brev((unsigned)(global_index & 255)) >> 24) << 32) |
           (unsigned long long)global_index;
}
constexpr unsigned long long kNoCandidate = ~0ull;

__device__ __forceinline__ void argmax_merge(float& best, unsigned long long& best_k, float v,
                                             unsigned long long k) {
    if (k == kNoCandidate) return;
    if (v > best || (v == best && k < best_k)) {
        best = v;
        best_k = k;
    }
}

__global__ void __launch_bounds__(1024)
argmax_bf16_kernel(const uint16_t* __restrict__ logits, long long n, long long offset, int* __restrict__ out) {
    __shared__ float s_val[32];
    __shared__ unsigned long long s_key[32];
    float best = -1e30f;
    unsigned long long best_k = kNoCandidate;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = bf16_bits_to_f32(__ldcg(logits + i));
        if (v > -1e30f) argmax_merge(best, best_k, v, argmax_tie_key(offset + i));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best_k, o);
        argmax_merge(best, best_k, ov, ok);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        s_val[warp] = best;
        s_key[warp] = best_k;
    }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? s_val[lane] : -1e30f;
        best_k = lane < nw ? s_key[lane] : kNoCandidate;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best_k, o);
            argmax_merge(best, best_k, ov, ok);
        }
        if (lane == 0)
            *out = best_k == kNoCandidate ? 0 : (int)((long long)(best_k & 0xffffffffull) - offset);
    }
}

// Residual add + RMSNorm, one block per row (ops::fused_add_rms_norm / rms_norm,
// src/ops/NormOps.cpp:141-275): v = x + add in fp32, hidden_out = bf16(v),
// normed = bf16(vn * rsqrt(mean(v^2) + eps) * w). vn = v, except on the reference's single-row route
// for H != 1024 (:189-240), whose second pass re-reads the sum it has just stored as bf16:
// there (`renorm_from_stored`) vn = float(bf16(v)). hidden_out may alias x (each element is read and
// written by the same thread).
__global__ void __launch_bounds__(256)
add_rms_norm_kernel(const uint16_t* x, const uint16_t* __restrict__ add,
                    const uint16_t* __restrict__ w, float eps, int H, uint16_t* hidden_out,
                    uint16_t* __restrict__ normed, int renorm_from_stored) {
    __shared__ float warp_sum[8];
    const size_t row = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
        const float v = bf16_bits_to_f32(__ldcg(x + row + k)) + (add ? bf16_bits_to_f32(__ldcg(add + row + k)) : 0.0f);
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += warp_sum[i];
    const float inv_rms = rsqrtf(total / (float)H + eps);
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
        const float v = bf16_bits_to_f32(__ldcg(x + row + k)) + (add ? bf16_bits_to_f32(__ldcg(add + row + k)) : 0.0f);
        const uint16_t stored = f32_to_bf16_bits(v);
        if (hidden_out) hidden_out[row + k] = stored;
        const float vn = renorm_from_stored ? bf16_bits_to_f32(stored) : v;
        normed[row + k] = f32_to_bf16_bits(vn * inv_rms * bf16_bits_to_f32(w[k]));
    }
}

}  // namespace
}  // namespace nf4

using nf4::fail;

namespace {
struct DenseDevGuard {
    int prev = -1;
    bool switched = false;
    cudaError_t err = cudaSuccess;
    explicit DenseDevGuard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) {
            err = cudaSetDevice(device);
            switched = (err == cudaSuccess);
        }
    }
    ~DenseDevGuard() {
        if (switched) cudaSetDevice(prev);
    }
};
}  // namespace

extern "C" {

AILA_NF4_API AilaNf4Status aila_dense_linear_create(const void* weight_bf16, int64_t out_features,
                                                    int64_t in_features, int weight_on_device,
                                                    int device, AilaDenseLinear** out) {
    if (!out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "out is NULL");
    *out = nullptr;
    if (!weight_bf16) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "weight pointer is NULL");
    if (out_features <= 0 || in_features <= 0 || in_features > (1 << 30) ||
        out_features > (1ll << 40) / in_features)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Linear: in_features/out_features out of range");
    DenseDevGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    AilaDenseLinear* l = new (std::nothrow) AilaDenseLinear();
    if (!l) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    l->device = device;
    l->N = out_features;
    l->K = in_features;
    const size_t bytes = (size_t)out_features * (size_t)in_features * 2;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&l->d_w), bytes + 256);
    if (e == cudaSuccess)
        e = cudaMemcpy(l->d_w, weight_bf16, bytes,
                       weight_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(l->d_w);
        delete l;
        return nf4::cuda_fail(e, "dense weight upload");
    }
    *out = l;
    return AILA_NF4_OK;
}

AILA_NF4_API void aila_dense_linear_destroy(AilaDenseLinear* l) {
    if (!l) return;
    DenseDevGuard guard(l->device);
    cudaFree(l->d_w);
    delete l;
}

AILA_NF4_API int64_t aila_dense_linear_in_features(const AilaDenseLinear* l) { return l ? l->K : 0; }
AILA_NF4_API int64_t aila_dense_linear_out_features(const AilaDenseLinear* l) { return l ? l->N : 0; }

AILA_NF4_API AilaNf4Status aila_dense_linear_forward(const AilaDenseLinear* l, AilaNf4Scratch* sc,
                                                     const void* x, void* y, int seq_len,
                                                     const void* residual, void* stream) {
    if (!l) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "linear handle is NULL");
    if (!sc) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch handle is NULL");
    if (!x || !y) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Linear expects bf16 input/output tensors");
    if (seq_len <= 0) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "Linear::forward: seq_len must be positive");
    if (sc->device != l->device)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch and linear live on different devices");
    DenseDevGuard guard(l->device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (seq_len > 1)
        return nf4::launch_gemm_bf16(l->d_w, x, y, residual, seq_len, l->N, l->K, 0, l->device,
                                     sc->sm_count, sc->d_status, s);
    const uint16_t* w = l->d_w;
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    uint16_t* yp = static_cast<uint16_t*>(y);
    const uint16_t* rp = static_cast<const uint16_t*>(residual);
    const size_t smem = (size_t)l->K * 2;
    const bool vec = (l->K % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && smem <= 200 * 1024;
    if (vec) {
        if (smem > 48 * 1024) {
            static bool raised[64] = {false};
            if (l->device < 64 && !raised[l->device]) {
                NF4_CUDA(cudaFuncSetAttribute(nf4::dense_gemv_kernel,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                raised[l->device] = true;
            }
        }
        const long long rows_per_block = nf4::kDenseWarps * nf4::kDenseRows;
        const unsigned blocks = (unsigned)((l->N + rows_per_block - 1) / rows_per_block);
        nf4::dense_gemv_kernel<<<blocks, nf4::kDenseWarps * 32, smem, s>>>(w, xp, yp, rp, (long long)l->N, (int)l->K);
    } else {
        const unsigned blocks = (unsigned)((l->N + 7) / 8);
        nf4::dense_gemv_generic_kernel<<<blocks, 256, 0, s>>>(w, xp, yp, rp, (long long)l->N, (int)l->K);
    }
    NF4_CUDA(cudaGetLastError());
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_argmax_bf16_shard(const void* logits_bf16, int64_t n, int64_t index_offset,
                                                  int32_t* d_result, int device, void* stream) {
    if (!logits_bf16 || !d_result) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (n <= 0 || index_offset < 0 || n + index_offset > 0x7fffffffll)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "argmax: vocab size out of range");
    DenseDevGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    nf4::argmax_bf16_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(logits_bf16), (long long)n, (long long)index_offset, d_result);
    NF4_CUDA(cudaGetLastError());
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_argmax_bf16(const void* logits_bf16, int64_t n, int32_t* d_result,
                                            int device, void* stream) {
    return aila_argmax_bf16_shard(logits_bf16, n, 0, d_result, device, stream);
}

AILA_NF4_API AilaNf4Status aila_add_rms_norm(const void* x_bf16, const void* add_bf16,
                                             const void* weight_bf16, float eps, int rows,
                                             int hidden_size, void* hidden_out_bf16,
                                             void* normed_out_bf16, int device, void* stream) {
    if (!x_bf16 || !weight_bf16 || !normed_out_bf16)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (rows <= 0 || hidden_size <= 0) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "rows and hidden_size must be positive");
    if (hidden_out_bf16 && hidden_out_bf16 == add_bf16)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "hidden_out may alias x but not the added tensor");
    DenseDevGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    nf4::add_rms_norm_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x_bf16), static_cast<const uint16_t*>(add_bf16),
        static_cast<const uint16_t*>(weight_bf16), eps, hidden_size,
        static_cast<uint16_t*>(hidden_out_bf16), static_cast<uint16_t*>(normed_out_bf16),
        (add_bf16 != nullptr && rows == 1 && hidden_size != 1024) ? 1 : 0);
    NF4_CUDA(cudaGetLastError());
    return AILA_NF4_OK;
}

}  // extern "C"
