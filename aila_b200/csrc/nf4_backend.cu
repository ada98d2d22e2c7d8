// The kernels a decode step needs between the NF4 linears: token embedding, per-head RMSNorm + RoPE
// + KV-cache append of the new token, and single-token attention over the cache. They follow the
// reference's operators as the Qwen3 NF4 backend calls them (src/models/Qwen3Bnb4Backend.cpp:298-439):
//   ops::embedding_lookup      src/ops/ElementwiseOps.cpp:14-27
//   ops::decode_prepare_qkv    src/ops/ElementwiseOps.cpp:105-215
//   ops::attention_decode      src/ops/AttentionOps.cpp:73-166 (the baseline form: whole window)
// Same arithmetic and the same bf16 roundings (normalised q/k are rounded before the rotation, the
// rotated values again; scores, softmax and the value sum stay fp32), simple kernels: these are
// not on the named hot path, they make the linears' callers runnable end to end.
#include <cstdint>
#include <string>

#include "nf4_common.cuh"
#include "nf4_internal.h"

namespace nf4 {
namespace {

__global__ void embedding_kernel(const uint16_t* __restrict__ table, const int* __restrict__ ids,
                                 int hidden, long long vocab, uint16_t* __restrict__ out) {
    const int s = blockIdx.x;
    long long id = ids[s];
    if (id < 0 || id >= vocab) id = 0;  // (the reference reads out of range; a clamped row is the safe form)
    const uint16_t* row = table + id * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) out[(size_t)s * hidden + h] = row[h];
}

__device__ __forceinline__ float block_sum_128(float v, float* scratch) {
    // fixed-order tree over 128 threads, as the reference's work-group reduction
    scratch[threadIdx.x] = v;
    __syncthreads();
    for (int stride = 64; stride > 0; stride >>= 1) {
        if ((int)threadIdx.x < stride) scratch[threadIdx.x] += scratch[threadIdx.x + stride];
        __syncthreads();
    }
    const float total = scratch[0];
    __syncthreads();
    return total;
}

// One block of 128 threads per query head. Heads below n_kv also handle the key head of the same
// index and append k and v to the cache at position pos.
__global__ void __launch_bounds__(128)
prepare_qkv_kernel(uint16_t* __restrict__ q, uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                   const float* __restrict__ rope_freq, const uint16_t* __restrict__ q_norm_w,
                   const uint16_t* __restrict__ k_norm_w, uint16_t* __restrict__ k_cache,
                   uint16_t* __restrict__ v_cache, int max_seq_len, int pos, const int* __restrict__ pos_dev,
                   int n_kv, int head_dim, float eps) {
    __shared__ float scratch[128];
    if (pos_dev) pos = *pos_dev;
    if (pos < 0 || pos >= max_seq_len) return;  // (the host refuses such a step; nothing is written)
    const int head = blockIdx.x;
    const int half = head_dim / 2;
    auto norm_and_rotate = [&](uint16_t* x, const uint16_t* w) {
        float ss = 0.0f;
        for (int d = threadIdx.x; d < head_dim; d += 128) {
            const float a = bf16_bits_to_f32(x[d]);
            ss += a * a;
        }
        const float rms = sqrtf(block_sum_128(ss, scratch) / (float)head_dim + eps);
        for (int d = threadIdx.x; d < head_dim; d += 128)
            x[d] = f32_to_bf16_bits((bf16_bits_to_f32(x[d]) / rms) * bf16_bits_to_f32(w[d]));
        __syncthreads();
        for (int d = threadIdx.x; d < half; d += 128) {
            const float angle = (float)pos * rope_freq[d];
            const float c = cosf(angle), s = sinf(angle);
            const float a = bf16_bits_to_f32(x[d]), b = bf16_bits_to_f32(x[d + half]);
            x[d] = f32_to_bf16_bits(a * c - b * s);
            x[d + half] = f32_to_bf16_bits(b * c + a * s);
        }
        __syncthreads();
    };
    norm_and_rotate(q + (size_t)head * head_dim, q_norm_w);
    if (head >= n_kv) return;
    uint16_t* kh = k + (size_t)head * head_dim;
    norm_and_rotate(kh, k_norm_w);
    const size_t at = ((size_t)head * max_seq_len + pos) * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += 128) {
        k_cache[at + d] = kh[d];
        v_cache[at + d] = v[(size_t)head * head_dim + d];
    }
}

// One block per query head: scores over the cached positions in shared memory, softmax, value sum.
__global__ void __launch_bounds__(256)
attention_decode_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k_cache,
                        const uint16_t* __restrict__ v_cache, uint16_t* __restrict__ out,
                        int heads_per_kv, int head_dim, int cached_len, const int* __restrict__ pos_dev,
                        int max_seq_len) {
    extern __shared__ float att_smem[];
    if (pos_dev) cached_len = min(*pos_dev + 1, cached_len);  // (the launch holds `cached_len` scores at most)
    if (cached_len <= 0) return;
    float* qf = att_smem;                  // [head_dim]
    float* score = att_smem + head_dim;    // [cached_len]
    __shared__ float red[8];
    const int head = blockIdx.x, kv_head = head / heads_per_kv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int d = tid; d < head_dim; d += 256) qf[d] = bf16_bits_to_f32(q[(size_t)head * head_dim + d]);
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)head_dim);
    const uint16_t* kb = k_cache + (size_t)kv_head * max_seq_len * head_dim;
    const uint16_t* vb = v_cache + (size_t)kv_head * max_seq_len * head_dim;
    float mx = -1e30f;
    for (int t = tid; t < cached_len; t += 256) {
        const uint16_t* row = kb + (size_t)t * head_dim;
        float sum = 0.0f;
        for (int d = 0; d < head_dim; ++d) sum += qf[d] * bf16_bits_to_f32(row[d]);
        sum *= scale;
        score[t] = sum;
        mx = fmaxf(mx, sum);
    }
    auto block_reduce = [&](float v, bool is_max) {
        for (int sh = 16; sh > 0; sh >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, v, sh);
            v = is_max ? fmaxf(v, o) : v + o;
        }
        if (lane == 0) red[warp] = v;
        __syncthreads();
        float r = red[0];
        for (int w = 1; w < 8; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
        __syncthreads();
        return r;
    };
    mx = block_reduce(mx, true);
    float den = 0.0f;
    for (int t = tid; t < cached_len; t += 256) {
        const float e = __expf(score[t] - mx);
        score[t] = e;
        den += e;
    }
    den = block_reduce(den, false);
    for (int t = tid; t < cached_len; t += 256) score[t] = score[t] / den;
    __syncthreads();
    for (int d = tid; d < head_dim; d += 256) {
        float acc = 0.0f;
        for (int t = 0; t < cached_len; ++t) acc += score[t] * bf16_bits_to_f32(vb[(size_t)t * head_dim + d]);
        out[(size_t)head * head_dim + d] = f32_to_bf16_bits(acc);
    }
}

struct BackendDevGuard {
    int prev = -1;
    cudaError_t err = cudaSuccess;
    explicit BackendDevGuard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
    }
    ~BackendDevGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace
}  // namespace nf4

using nf4::fail;

AILA_NF4_API AilaNf4Status aila_embedding_lookup(const void* table_bf16, int64_t vocab_size,
                                                 const int32_t* token_ids_device, int seq_len,
                                                 int hidden_size, void* out_bf16, int device,
                                                 void* stream) {
    if (!table_bf16 || !token_ids_device || !out_bf16) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (seq_len <= 0 || hidden_size <= 0 || vocab_size <= 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "seq_len, hidden_size and vocab_size must be positive");
    nf4::BackendDevGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    nf4::embedding_kernel<<<(unsigned)seq_len, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(table_bf16), token_ids_device, hidden_size, (long long)vocab_size,
        static_cast<uint16_t*>(out_bf16));
    NF4_CUDA(cudaGetLastError());
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_decode_prepare_qkv(void* q_bf16, void* k_bf16, const void* v_bf16,
                                                   const float* rope_freq, const void* q_norm_weight_bf16,
                                                   const void* k_norm_weight_bf16, void* k_cache_bf16,
                                                   void* v_cache_bf16, int max_seq_len, int start_pos,
                                                   const int32_t* position_device, int num_heads_q,
                                                   int num_kv_heads, int head_dim, float eps, int device,
                                                   void* stream) {
    if (!q_bf16 || !k_bf16 || !v_bf16 || !rope_freq || !q_norm_weight_bf16 || !k_norm_weight_bf16 ||
        !k_cache_bf16 || !v_cache_bf16)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (num_heads_q <= 0 || num_kv_heads <= 0 || num_kv_heads > num_heads_q || num_heads_q % num_kv_heads != 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "query heads must be a positive multiple of the key/value heads");
    if (head_dim <= 0 || head_dim % 2 != 0) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "head_dim must be positive and even");
    if (start_pos < 0 || start_pos >= max_seq_len)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "context window exceeded (start_pos=" + std::to_string(start_pos) +
                                                       ", max_seq_len=" + std::to_string(max_seq_len) + ")");
    nf4::BackendDevGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    nf4::prepare_qkv_kernel<<<(unsigned)num_heads_q, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t*>(q_bf16), static_cast<uint16_t*>(k_bf16), static_cast<const uint16_t*>(v_bf16),
        rope_freq, static_cast<const uint16_t*>(q_norm_weight_bf16),
        static_cast<const uint16_t*>(k_norm_weight_bf16), static_cast<uint16_t*>(k_cache_bf16),
        static_cast<uint16_t*>(v_cache_bf16), max_seq_len, start_pos, position_device, num_kv_heads, head_dim, eps);
    NF4_CUDA(cudaGetLastError());
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_attention_decode(const void* q_bf16, const void* k_cache_bf16,
                                                 const void* v_cache_bf16, void* out_bf16, int num_heads,
                                                 int num_kv_heads, int head_dim, int cached_len,
                                                 const int32_t* position_device, int max_seq_len, int device,
                                                 void* stream) {
    if (!q_bf16 || !k_cache_bf16 || !v_cache_bf16 || !out_bf16) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || head_dim <= 0)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "query heads must be a positive multiple of the key/value heads");
    if (cached_len <= 0 || cached_len > max_seq_len)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "cached_len out of range");
    const size_t smem = ((size_t)cached_len + (size_t)head_dim) * sizeof(float);
    if (smem > 200 * 1024)
        return fail(AILA_NF4_ERR_UNSUPPORTED, "attention_decode keeps one score per cached position in shared memory: "
                                              "at most about 51,000 positions");
    nf4::BackendDevGuard guard(device);
    if (guard.err != cudaSuccess) return nf4::cuda_fail(guard.err, "cudaSetDevice");
    static bool raised[64] = {false};
    if (smem > 48 * 1024 && device >= 0 && device < 64 && !raised[device]) {
        NF4_CUDA(cudaFuncSetAttribute(nf4::attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      200 * 1024));
        raised[device] = true;
    }
    nf4::attention_decode_kernel<<<(unsigned)num_heads, 256, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(q_bf16), static_cast<const uint16_t*>(k_cache_bf16),
        static_cast<const uint16_t*>(v_cache_bf16), static_cast<uint16_t*>(out_bf16), num_heads / num_kv_heads,
        head_dim, cached_len, position_device, max_seq_len);
    NF4_CUDA(cudaGetLastError());
    return AILA_NF4_OK;
}
