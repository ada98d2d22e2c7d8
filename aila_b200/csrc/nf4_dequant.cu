// Whole-weight dequantisation kernels (bit-exact) and the row-wise SwiGLU.
//   dequant_kn : Wt[K][N] bf16, the layout and arithmetic of Bnb4BitLinear::dequantize_weight
//                (reference src/ops/Bnb4BitLinear.cpp:723-757)
//   dequant_nk : W[N][K] bf16, same values in the orientation the tcgen05 GEMM reads
//   expand     : fp32 absmax per block, the values Bnb4BitLinear::init computes on the host
//                (:472-488)
//   swiglu     : ops::fused_gate_up_swiglu (reference src/ops/ElementwiseOps.cpp:247-294)
// HBM-bound: dequant_nk reads 0.516 B and writes 2 B per weight.
#include "nf4_internal.h"

namespace nf4 {

namespace {

__device__ __forceinline__ float unit_absmax(const uint8_t* unit, int absmax_kind,
                                             const ScaleParams& sp, int n, int kb, int r) {
    if (absmax_kind == kAbsmaxCodes) return decode_absmax(sp, n, kb, unit[kUnitNibbleBytes + r]);
    return reinterpret_cast<const float*>(unit + kUnitNibbleBytes)[r];
}

// One block per unit, 256 threads: thread (r = tid % 16, c = tid / 16) converts the two
// stored bytes p = 2c, 2c+1 of row r, i.e. k = 16*j + 4*t + {0..3} with t = c / 4, j = c % 4.
// Consecutive threads hold consecutive output columns n, so each k-row of Wt gets one 32-byte
// store per warp half.
__global__ void __launch_bounds__(256)
dequant_kn_kernel(const uint8_t* __restrict__ units, const float* __restrict__ qmap,
                  ScaleParams sp, uint16_t* __restrict__ out, int N, int KU, int unit_stride,
                  int absmax_kind) {
    const long long u = blockIdx.x;
    const int kb = (int)(u % KU);
    const int rt = (int)(u / KU);
    const int r = threadIdx.x & 15;
    const int c = threadIdx.x >> 4;
    const int n = rt * kTileRows + r;
    if (n >= N) return;
    const uint8_t* unit = units + (size_t)u * unit_stride;
    const float am = unit_absmax(unit, absmax_kind, sp, n, kb, r);
    const uint16_t two = *reinterpret_cast<const uint16_t*>(unit + r * 32 + 2 * c);
    const int t = c >> 2, j = c & 3;
    const int k0 = kb * kUnitK + 16 * j + 4 * t;
    const uint32_t b0 = two & 0xff, b1 = two >> 8;
    const float w0 = __fmul_rn(__ldg(qmap + (b0 >> 4)), am);
    const float w1 = __fmul_rn(__ldg(qmap + (b0 & 15)), am);
    const float w2 = __fmul_rn(__ldg(qmap + (b1 >> 4)), am);
    const float w3 = __fmul_rn(__ldg(qmap + (b1 & 15)), am);
    out[(size_t)(k0 + 0) * N + n] = f32_to_bf16_bits(w0);
    out[(size_t)(k0 + 1) * N + n] = f32_to_bf16_bits(w1);
    out[(size_t)(k0 + 2) * N + n] = f32_to_bf16_bits(w2);
    out[(size_t)(k0 + 3) * N + n] = f32_to_bf16_bits(w3);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return f32x2_to_bf16x2_bits(lo, hi);
}

// One thread per (unit, row): reads the row's 32 stored bytes (two 16-byte loads; a warp reads
// two whole units, 1 KB contiguous), undoes the intra-row permutation in registers and puts the
// 64 bf16 weights of the block (128 bytes) into shared memory; the warp then writes its 32 rows
// out four at a time, 8 lanes x 16 bytes per row, so every store instruction fills whole
// 128-byte lines of W[n][64kb .. 64kb+64).
constexpr int kDqRowPitch = 144;  // 128 B of bf16 + 16 B pad: conflict-free 16-byte accesses

__global__ void __launch_bounds__(256)
dequant_nk_kernel(const uint8_t* __restrict__ units, const float* __restrict__ qmap,
                  ScaleParams sp, uint16_t* __restrict__ out, int N, long long K, int KU,
                  long long total_units, int unit_stride, int absmax_kind) {
    __shared__ float q[16];
    __shared__ __align__(16) uint8_t tile[8][32 * kDqRowPitch];
    // the GEMM that consumes this pass may start its set-up now; it waits for our completion
    // before it reads the weights
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x < 16) q[threadIdx.x] = qmap[threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long u = tid >> 4;  // this lane's unit (two units per warp)
    const int r = (int)(tid & 15);
    const bool live = u < total_units;
    // (rt, kb) of the warp's two consecutive units: one 32-bit division per warp side instead of
    // 64-bit divisions per lane and per store (the host guarantees total_units < 2^31)
    const unsigned u_first = (unsigned)((tid - lane) >> 4);
    const int rt_a = (int)(u_first / (unsigned)KU), kb_a = (int)(u_first - (unsigned)rt_a * (unsigned)KU);
    const int kb_b = kb_a + 1 == KU ? 0 : kb_a + 1, rt_b = kb_a + 1 == KU ? rt_a + 1 : rt_a;
    const int kb = (lane >> 4) ? kb_b : kb_a;
    const int rt = (lane >> 4) ? rt_b : rt_a;
    const int n = rt * kTileRows + r;
    uint8_t* mine = tile[warp] + lane * kDqRowPitch;
    if (live && n < N) {
        const uint8_t* unit = units + (size_t)u * unit_stride;
        const uint4 lo = *reinterpret_cast<const uint4*>(unit + r * 32);
        const uint4 hi = *reinterpret_cast<const uint4*>(unit + r * 32 + 16);
        const float am = unit_absmax(unit, absmax_kind, sp, n, kb, r);
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        uint32_t o[32];  // 64 bf16, natural k order
        const uint32_t qa = (uint32_t)__cvta_generic_to_shared(q);
        // code book value of nibble `n` (0 = lowest) of a word: the table offset (nibble * 4) comes
        // out of the word with one shift and one mask
        auto qv = [&](uint32_t word, int n) {
            const uint32_t off = n == 0 ? (word << 2) & 0x3cu : (word >> (4 * n - 2)) & 0x3cu;
            float v;
            asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(qa + off));
            return v;
        };
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int t = 0; t < 4; ++t)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int p = 8 * t + 2 * j + e;  // stored byte
                    const uint32_t word = w[p >> 2];
                    const int bi = p & 3;             // byte of the word: nibbles 2 bi (low), 2 bi + 1 (high)
                    // byte covers k = 16j + 4t + 2e (high nibble) and + 1 (low nibble)
                    o[(16 * j + 4 * t + 2 * e) >> 1] =
                        pack_bf16x2(__fmul_rn(qv(word, 2 * bi + 1), am), __fmul_rn(qv(word, 2 * bi), am));
                }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            reinterpret_cast<uint4*>(mine)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
    }
    __syncwarp();
    // lane -> (row within the group of four, 16-byte piece of the row)
    const int piece = lane & 7, sub = lane >> 3;
    const long long u0 = (tid - lane) >> 4;  // first unit of this warp
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int row = g * 4 + sub;          // 0..31: rows 0-15 unit u0, 16-31 unit u0 + 1
        const long long uu = u0 + (row >> 4);
        if (uu < total_units) {
            const int kbb = (row >> 4) ? kb_b : kb_a;
            const int nn = ((row >> 4) ? rt_b : rt_a) * kTileRows + (row & 15);
            if (nn < N) {
                const uint4 v = *reinterpret_cast<const uint4*>(tile[warp] + row * kDqRowPitch + piece * 16);
                *reinterpret_cast<uint4*>(out + (size_t)nn * K + (size_t)kbb * kUnitK + piece * 8) = v;
            }
        }
    }
}

__global__ void expand_absmax_kernel(const uint8_t* __restrict__ units, ScaleParams sp,
                                     float* __restrict__ out, int N, int KU, int blocks_per_row,
                                     int unit_stride, int absmax_kind) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= (long long)N * blocks_per_row) return;
    const int b = (int)(tid % blocks_per_row);
    const int n = (int)(tid / blocks_per_row);
    const int kb = b << sp.blk_shift;
    const uint8_t* unit = units + ((size_t)(n / kTileRows) * KU + kb) * unit_stride;
    out[tid] = unit_absmax(unit, absmax_kind, sp, n, kb, n % kTileRows);
}

// out[m][i] = bf16( silu(g) * u ), g = gate_up[m][i], u = gate_up[m][ff + i], both read as
// bf16; silu(g) = g / (1 + exp(-g)) in fp32.
__global__ void swiglu_rows_kernel(const uint16_t* __restrict__ gate_up,
                                   uint16_t* __restrict__ out, int M, long long ff) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= (long long)M * ff) return;
    const long long m = tid / ff, i = tid % ff;
    const float g = bf16_bits_to_f32(gate_up[m * 2 * ff + i]);
    const float u = bf16_bits_to_f32(gate_up[m * 2 * ff + ff + i]);
    const float silu = g / (1.0f + __expf(-g));
    out[tid] = f32_to_bf16_bits(silu * u);
}

}  // namespace

cudaError_t launch_dequant_kn(const AilaNf4Linear& w, void* out_kn, cudaStream_t s) {
    const long long units = (long long)w.RT * w.KU;
    if (units == 0) return cudaSuccess;
    dequant_kn_kernel<<<(unsigned)units, 256, 0, s>>>(w.d_units, w.d_qmap, w.scale_params(),
                                                     static_cast<uint16_t*>(out_kn), (int)w.N,
                                                     w.KU, w.unit_stride, w.absmax_kind);
    return cudaGetLastError();
}

cudaError_t launch_dequant_nk(const AilaNf4Linear& w, void* out_nk, cudaStream_t s) {
    const long long units = (long long)w.RT * w.KU;
    if (units == 0) return cudaSuccess;
    if (units >= (1ll << 31)) return cudaErrorInvalidValue;  // (2^41 weights: beyond any linear the loader takes)
    const long long threads = units * 16;
    const long long blocks = (threads + 255) / 256;
    dequant_nk_kernel<<<(unsigned)blocks, 256, 0, s>>>(w.d_units, w.d_qmap, w.scale_params(),
                                                      static_cast<uint16_t*>(out_nk), (int)w.N,
                                                      (long long)w.K, w.KU, units, w.unit_stride,
                                                      w.absmax_kind);
    return cudaGetLastError();
}

cudaError_t launch_expand_absmax(const AilaNf4Linear& w, float* out, cudaStream_t s) {
    const int bpr = (int)(w.K / w.blocksize);
    const long long total = (long long)w.N * bpr;
    if (total == 0) return cudaSuccess;
    expand_absmax_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
        w.d_units, w.scale_params(), out, (int)w.N, w.KU, bpr, w.unit_stride, w.absmax_kind);
    return cudaGetLastError();
}

cudaError_t launch_swiglu_rows(const void* gate_up, void* out, int M, int64_t ff, cudaStream_t s) {
    const long long total = (long long)M * ff;
    if (total == 0) return cudaSuccess;
    swiglu_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
        static_cast<const uint16_t*>(gate_up), static_cast<uint16_t*>(out), M, (long long)ff);
    return cudaGetLastError();
}

}  // namespace nf4
