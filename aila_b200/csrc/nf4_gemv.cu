// Decode (seq_len == 1) kernels: y = W x and out = silu(Wg x) * (Wu x).
// Replace packed_nf4_gemv_bf16 and packed_nf4_gemv_gate_up_swiglu
// (reference src/ops/Bnb4BitLinear.cpp:271-410, :142-246).
//
// Two kernels:
//  * gemv_simple: one warp per output row, fp32 weights q*absmax and fp32 FMA, i.e. the
//    reference's arithmetic with a different summation order. Baseline and fallback for
//    shapes the streaming kernel does not take.
//  * gemv_stream: the HBM-roofline kernel. One persistent CTA per SM owns an equal, contiguous
//    slice of the unit stream (split along rows AND k, so any shape balances over 148 SMs),
//    a producer thread keeps a ring of bulk-async copies in flight, 16 consumer warps turn
//    nibbles into bf16 tensor-core operands through a bank-private shared-memory table and
//    accumulate in fp32 with mma.sync m16n8k16; absmax is applied in fp32 per 64-block.
//    Row tiles cut by a slice boundary are completed through per-CTA partial sums in global
//    scratch, summed in CTA order by whichever CTA arrives last (no spinning, deterministic).
//
// Roofline: HBM. Algorithmic bytes per weight: 0.5 (nibbles) + 1/64 (code) + 4/16384 (scale).
#include <mutex>

#include "nf4_internal.h"

namespace nf4 {

namespace {

// ------------------------------------------------------------------------------------------
// gemv_simple
// ------------------------------------------------------------------------------------------
template <bool PAIRED>
__global__ void __launch_bounds__(256)
gemv_simple_kernel(const uint8_t* __restrict__ units, const float* __restrict__ qmap,
                   ScaleParams sp, const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                   const uint16_t* __restrict__ residual, int n_out, int KU, int unit_stride,
                   int absmax_kind, int pair_rt_offset) {
    __shared__ float q[16];
    if (threadIdx.x < 16) q[threadIdx.x] = qmap[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= n_out) return;
    const int rt = n / kTileRows, r = n % kTileRows;
    const int t = lane & 3;
    float acc[PAIRED ? 2 : 1] = {0.0f};
    for (int kb = lane >> 2; kb < KU; kb += 8) {
        const uint2* xp = reinterpret_cast<const uint2*>(x + (size_t)kb * kUnitK + 4 * t);
#pragma unroll
        for (int h = 0; h < (PAIRED ? 2 : 1); ++h) {
            const int rth = rt + h * pair_rt_offset;
            const uint8_t* unit = units + ((size_t)rth * KU + kb) * unit_stride;
            const int nrow = rth * kTileRows + r;
            float am;
            if (absmax_kind == kAbsmaxCodes)
                am = decode_absmax(sp, nrow, kb, unit[kUnitNibbleBytes + r]);
            else
                am = reinterpret_cast<const float*>(unit + kUnitNibbleBytes)[r];
            const uint2 v = *reinterpret_cast<const uint2*>(unit + r * 32 + 8 * t);
            float a = acc[h];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t two = ((j < 2 ? v.x : v.y) >> (16 * (j & 1))) & 0xffff;
                const uint32_t b0 = two & 0xff, b1 = two >> 8;
                const uint2 xv = __ldg(xp + 4 * j);  // x[64kb + 16j + 4t .. +4)
                a = fmaf(bf16_bits_to_f32(xv.x & 0xffff), q[b0 >> 4] * am, a);
                a = fmaf(bf16_bits_to_f32(xv.x >> 16), q[b0 & 15] * am, a);
                a = fmaf(bf16_bits_to_f32(xv.y & 0xffff), q[b1 >> 4] * am, a);
                a = fmaf(bf16_bits_to_f32(xv.y >> 16), q[b1 & 15] * am, a);
            }
            acc[h] = a;
        }
    }
#pragma unroll
    for (int h = 0; h < (PAIRED ? 2 : 1); ++h)
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], o);
    if (lane == 0) {
        float v;
        if (PAIRED) {
            const float g = acc[0], u = acc[PAIRED ? 1 : 0];
            v = (g / (1.0f + __expf(-g))) * u;
        } else {
            v = acc[0];
            if (residual) v += bf16_bits_to_f32(residual[n]);
        }
        y[n] = f32_to_bf16_bits(v);
    }
}

// ------------------------------------------------------------------------------------------
// gemv_stream
// ------------------------------------------------------------------------------------------
constexpr int kConsumerWarps = 16;
constexpr int kStreamThreads = (kConsumerWarps + 1) * 32;  // + one producer warp
constexpr int kLutBytes = 256 * 256;                       // 256 byte values x 256 B (lane-private word)
constexpr int kMaxStages = 24;
constexpr int kMaxLocalTiles = 16;  // row tiles one CTA slice may touch
constexpr int kMaxGridMult = 8;     // grid <= 8 x SM count

struct StreamParams {
    const uint8_t* units;
    const float* qmap;
    ScaleParams sp;
    const uint16_t* x;
    uint16_t* y;
    const uint16_t* residual;
    float* partials;
    int* counters;
    int* status;
    long long total_items;  // work items (units, or gate/up unit pairs)
    int n_out;              // rows written (ff when paired)
    int K;
    int KU;
    int unit_stride;
    int pair_rt_offset;     // paired: row-tile distance from a gate tile to its up tile
    int stages;
    int x_bytes;            // K*2 rounded up to 16
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

extern __shared__ __align__(1024) uint8_t smem_raw[];

// Bank-private table lookup: entry for byte value b of lane l sits at b*256 + l*4, so the 32
// lanes of a warp always hit 32 different banks. One PRMT builds the address.
template <int BYTE>
__device__ __forceinline__ uint32_t lut_pair(uint32_t word, uint32_t lane4) {
    const uint32_t off = __byte_perm(word, lane4, 0x5504 | (BYTE << 4));
    return *reinterpret_cast<const uint32_t*>(smem_raw + off);
}

__device__ __forceinline__ long long slice_begin(long long total, int c, int G) {
    return (total * c) / G;
}

template <int KIND, bool PAIRED>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const StreamParams p) {
    constexpr int NP = PAIRED ? 2 : 1;
    const int unit_stride = (KIND == kAbsmaxCodes) ? kUnitStrideCodes : kUnitStrideF32;
    const int stage_bytes = kConsumerWarps * unit_stride * NP;

    // shared-memory carve-up
    uint8_t* lut = smem_raw;                               // [0, 64 KB)
    uint8_t* xs = smem_raw + kLutBytes;                    // x in fragment order
    uint8_t* ring = xs + p.x_bytes;                        // stages * stage_bytes
    float* slots = reinterpret_cast<float*>(ring + (size_t)p.stages * stage_bytes);
    // slots[local tile][pair][warp][16]
    uint64_t* full = reinterpret_cast<uint64_t*>(slots + kMaxLocalTiles * NP * kConsumerWarps * 16);
    uint64_t* empty = full + kMaxStages;
    int* abort_flag = reinterpret_cast<int*>(empty + kMaxStages);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int G = gridDim.x;
    const int c = blockIdx.x;
    const long long i0 = slice_begin(p.total_items, c, G);
    const long long i1 = slice_begin(p.total_items, c + 1, G);
    const int n_groups = (int)((i1 - i0 + kConsumerWarps - 1) / kConsumerWarps);
    const int rt_first = (int)(i0 / p.KU);
    const int rt_last = (int)((i1 - 1) / p.KU);
    const int n_local = rt_last - rt_first + 1;

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---------------- producer: one thread keeps the ring full ----------------
        if (lane == 0) {
            int issued = 0;
            for (int g = 0; g < n_groups; ++g) {
                const int s = g % p.stages;
                if (g >= p.stages) {
                    if (*(volatile int*)abort_flag) break;
                    if (!mbar_wait_bounded(&empty[s], ((g / p.stages) - 1) & 1)) {
                        atomicExch(p.status, kStatusTimeoutEmpty);
                        *(volatile int*)abort_flag = 1;
                        break;
                    }
                }
                const long long item = i0 + (long long)g * kConsumerWarps;
                const int cnt = (int)min((long long)kConsumerWarps, i1 - item);
                const uint32_t bytes = (uint32_t)cnt * unit_stride;
                uint8_t* dst = ring + (size_t)s * stage_bytes;
                mbar_expect_tx(&full[s], bytes * NP);
                bulk_g2s(dst, p.units + (size_t)item * unit_stride, bytes, &full[s]);
                if (PAIRED)
                    bulk_g2s(dst + kConsumerWarps * unit_stride,
                             p.units + ((size_t)item + (size_t)p.pair_rt_offset * p.KU) * unit_stride,
                             bytes, &full[s]);
                issued = g + 1;
            }
            // never leave the CTA with copies still landing in its shared memory
            for (int g = max(0, issued - p.stages); g < issued; ++g)
                mbar_wait_bounded(&full[g % p.stages], (g / p.stages) & 1);
        }
    } else {
        // ---------------- consumers ----------------
        // build the byte -> bf16x2 table (lane-private columns) and stage x
        {
            const float qv = __ldg(p.qmap + (lane & 15));
            const uint32_t qb = f32_to_bf16_bits(qv);
            // every lane owns the table column of its own lane index: word (b*64 + lane)
            for (int b = warp; b < 256; b += kConsumerWarps) {
                const uint32_t hi = __shfl_sync(0xffffffffu, qb, b >> 4);
                const uint32_t lo = __shfl_sync(0xffffffffu, qb, b & 15);
                // low half = first weight of the byte (even k, HIGH nibble)
                reinterpret_cast<uint32_t*>(lut)[b * 64 + lane] = hi | (lo << 16);
            }
            // x: element k = 64*kb + 16*j + 4*t + e  ->  fragment order
            const int ctid = tid;  // 0..511
            const int n4 = p.K >> 2;  // groups of 4 elements (8 bytes)
            const uint2* xg = reinterpret_cast<const uint2*>(p.x);
            uint2* xd = reinterpret_cast<uint2*>(xs);
            for (int q4 = ctid; q4 < n4; q4 += kConsumerWarps * 32) {
                const int kb = q4 >> 4, j = (q4 >> 2) & 3, t = q4 & 3;
                xd[((kb * 2 + (j >> 1)) * 4 + t) * 2 + (j & 1)] = __ldg(xg + q4);
            }
            for (int i = ctid; i < kMaxLocalTiles * NP * kConsumerWarps * 16; i += kConsumerWarps * 32)
                slots[i] = 0.0f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");

        const int gq = lane >> 2;  // row inside the tile (and row + 8)
        const int t = lane & 3;
        const uint32_t lane4 = (uint32_t)lane << 2;
        float acc[NP][2];
#pragma unroll
        for (int h = 0; h < NP; ++h) acc[h][0] = acc[h][1] = 0.0f;
        int cur_li = -1;

        long long item = i0 + warp;
        int kb = (int)(item % p.KU);
        int rt = (int)(item / p.KU);
        const int kb_step = kConsumerWarps % p.KU;
        const int rt_step = kConsumerWarps / p.KU;

        for (int g = 0; g < n_groups; ++g) {
            const int s = g % p.stages;
            if (*(volatile int*)abort_flag) break;
            if (!mbar_wait_bounded(&full[s], (g / p.stages) & 1)) {
                atomicExch(p.status, kStatusTimeoutFull);
                *(volatile int*)abort_flag = 1;
                break;
            }
            if (item < i1) {
                const int li = rt - rt_first;
                if (li != cur_li) {
                    if (cur_li >= 0 && t == 0) {
#pragma unroll
                        for (int h = 0; h < NP; ++h) {
                            float* sl = slots + ((cur_li * NP + h) * kConsumerWarps + warp) * 16;
                            sl[gq] = acc[h][0];
                            sl[gq + 8] = acc[h][1];
                        }
                    }
#pragma unroll
                    for (int h = 0; h < NP; ++h) acc[h][0] = acc[h][1] = 0.0f;
                    cur_li = li;
                }
                const uint8_t* stage = ring + (size_t)s * stage_bytes;
                // x fragments for batch column 0 (held by the lanes with gq == 0)
                uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
                if (gq == 0) {
                    const uint4* xf = reinterpret_cast<const uint4*>(xs) + (size_t)kb * 8;
                    xa = xf[t];
                    xb = xf[4 + t];
                }
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    const uint8_t* ub = stage + h * (kConsumerWarps * unit_stride) + warp * unit_stride;
                    const uint2 wl = *reinterpret_cast<const uint2*>(ub + gq * 32 + 8 * t);
                    const uint2 wh = *reinterpret_cast<const uint2*>(ub + (gq + 8) * 32 + 8 * t);
                    float am0, am1;
                    const int rth = rt + h * p.pair_rt_offset;
                    if (KIND == kAbsmaxCodes) {
                        am0 = decode_absmax(p.sp, rth * kTileRows + gq, kb, ub[kUnitNibbleBytes + gq]);
                        am1 = decode_absmax(p.sp, rth * kTileRows + gq + 8, kb,
                                            ub[kUnitNibbleBytes + gq + 8]);
                    } else {
                        const float* af = reinterpret_cast<const float*>(ub + kUnitNibbleBytes);
                        am0 = af[gq];
                        am1 = af[gq + 8];
                    }
                    float cfrag[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    // j = 0: bytes 0,1 of wl.x / wh.x ; j = 1: bytes 2,3 ; j = 2,3: .y
                    mma_bf16_16816(cfrag, lut_pair<0>(wl.x, lane4), lut_pair<0>(wh.x, lane4),
                                   lut_pair<1>(wl.x, lane4), lut_pair<1>(wh.x, lane4), xa.x, xa.y);
                    mma_bf16_16816(cfrag, lut_pair<2>(wl.x, lane4), lut_pair<2>(wh.x, lane4),
                                   lut_pair<3>(wl.x, lane4), lut_pair<3>(wh.x, lane4), xa.z, xa.w);
                    mma_bf16_16816(cfrag, lut_pair<0>(wl.y, lane4), lut_pair<0>(wh.y, lane4),
                                   lut_pair<1>(wl.y, lane4), lut_pair<1>(wh.y, lane4), xb.x, xb.y);
                    mma_bf16_16816(cfrag, lut_pair<2>(wl.y, lane4), lut_pair<2>(wh.y, lane4),
                                   lut_pair<3>(wl.y, lane4), lut_pair<3>(wh.y, lane4), xb.z, xb.w);
                    acc[h][0] = fmaf(am0, cfrag[0], acc[h][0]);
                    acc[h][1] = fmaf(am1, cfrag[2], acc[h][1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            item += kConsumerWarps;
            kb += kb_step;
            rt += rt_step;
            if (kb >= p.KU) {
                kb -= p.KU;
                rt += 1;
            }
        }
        if (cur_li >= 0 && t == 0) {
#pragma unroll
            for (int h = 0; h < NP; ++h) {
                float* sl = slots + ((cur_li * NP + h) * kConsumerWarps + warp) * 16;
                sl[gq] = acc[h][0];
                sl[gq + 8] = acc[h][1];
            }
        }
    }
    __syncthreads();
    if (*(volatile int*)abort_flag) return;

    // ---------------- finish: one 16-lane half-warp per local row tile ----------------
    if (warp < kMaxLocalTiles / 2) {
        const int li = warp * 2 + (lane >> 4);
        const int r = lane & 15;
        const bool active = li < n_local;
        const int rtile = rt_first + li;
        float v[NP];
#pragma unroll
        for (int h = 0; h < NP; ++h) v[h] = 0.0f;
        bool is_full = false;
        if (active) {
#pragma unroll
            for (int h = 0; h < NP; ++h) {
                const float* sl = slots + ((li * NP + h) * kConsumerWarps) * 16 + r;
                float sacc = 0.0f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) sacc += sl[w * 16];
                v[h] = sacc;
            }
            const long long t0 = (long long)rtile * p.KU, t1 = t0 + p.KU;
            is_full = (i0 <= t0) && (i1 >= t1);
        }
        const bool is_partial = active && !is_full;
        bool finalize = active && is_full;
        int c_lo = 0, c_hi = 0;
        if (is_partial) {
            const int hslot = (li == 0) ? 0 : 1;
#pragma unroll
            for (int h = 0; h < NP; ++h)
                p.partials[(((size_t)c * 2 + hslot) * NP + h) * 16 + r] = v[h];
            __threadfence();
        }
        __syncwarp();
        int old = 0;
        if (is_partial) {
            const long long t0 = (long long)rtile * p.KU, t1 = t0 + p.KU;
            c_lo = (int)(((t0 + 1) * G - 1) / p.total_items);
            c_hi = (int)((t1 * G - 1) / p.total_items);
            if (r == 0) old = atomicAdd(p.counters + rtile, 1);
        }
        old = __shfl_sync(0xffffffffu, old, lane & 16);
        if (is_partial && old == (c_hi - c_lo)) {
            // last arriver: sum every contributor's partial in CTA order
            __threadfence();
#pragma unroll
            for (int h = 0; h < NP; ++h) v[h] = 0.0f;
            for (int cc = c_lo; cc <= c_hi; ++cc) {
                const int cc_first = (int)(slice_begin(p.total_items, cc, G) / p.KU);
                const int hslot = (rtile == cc_first) ? 0 : 1;
#pragma unroll
                for (int h = 0; h < NP; ++h)
                    v[h] += __ldcg(p.partials + (((size_t)cc * 2 + hslot) * NP + h) * 16 + r);
            }
            if (r == 0) p.counters[rtile] = 0;
            finalize = true;
        }
        if (finalize) {
            const int n = rtile * kTileRows + r;
            if (n < p.n_out) {
                float o;
                if (PAIRED) {
                    const float gt = v[0], up = v[NP - 1];
                    o = (gt / (1.0f + __expf(-gt))) * up;
                } else {
                    o = v[0];
                    if (p.residual) o += bf16_bits_to_f32(p.residual[n]);
                }
                p.y[n] = f32_to_bf16_bits(o);
            }
        }
    }
}

struct StreamPlan {
    int grid = 0;
    int stages = 0;
    int smem = 0;
    bool ok = false;
};

// Grid and ring depth for one launch. The slice of a CTA may touch at most kMaxLocalTiles row
// tiles; long outputs therefore get a grid that is a multiple of the SM count (CTAs never
// wait on each other, so they need not be co-resident).
StreamPlan stream_plan(const AilaNf4Linear& w, bool paired, int64_t ff_pair, int sm_count) {
    StreamPlan pl;
    const int np = paired ? 2 : 1;
    const int stage_bytes = kConsumerWarps * w.unit_stride * np;
    const int x_bytes = (int)((w.K * 2 + 15) / 16 * 16);
    const int fixed = kLutBytes + x_bytes + kMaxLocalTiles * np * kConsumerWarps * 16 * 4 +
                      2 * kMaxStages * 8 + 16;
    const int budget = 227 * 1024 - fixed;
    if (budget < 3 * stage_bytes) return pl;
    pl.stages = budget / stage_bytes;
    if (pl.stages > kMaxStages) pl.stages = kMaxStages;
    pl.smem = fixed + pl.stages * stage_bytes;
    const long long rt_work = paired ? ff_pair / kTileRows : w.RT;
    const long long total = rt_work * w.KU;
    if (total <= 0 || sm_count <= 0) return pl;
    for (int mult = 1; mult <= kMaxGridMult; ++mult) {
        long long grid = (long long)sm_count * mult;
        if (grid > total) grid = total;
        // a slice holds at most total/grid + 1 items -> touches at most (len-1)/KU + 2 tiles
        const long long len = total / grid + 1;
        if ((len - 1) / w.KU + 2 <= kMaxLocalTiles) {
            pl.grid = (int)grid;
            pl.ok = true;
            return pl;
        }
        if (grid == total) break;
    }
    return pl;
}

template <int KIND, bool PAIRED>
cudaError_t launch_stream_t(const StreamParams& p, int grid, int smem, cudaStream_t s) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, PAIRED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    gemv_stream_kernel<KIND, PAIRED><<<grid, kStreamThreads, smem, s>>>(p);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// Fixed work space for the entry point that never allocates (aila_nf4_forward_decode_static).
// The streaming kernel's split-K partial sums, row-tile counters and status word live in this
// file-scope device array instead of an AilaNf4Scratch. Every GPU that loads the library holds
// the array until the process exits. Limits that follow from its size: at most
// kStaticMaxCtas CTAs per launch and kStaticMaxRowTiles row tiles (262,144 output rows).
// ------------------------------------------------------------------------------------------
constexpr int kStaticMaxCtas = 8 * 160;
constexpr int kStaticMaxRowTiles = 16384;
struct StaticScratchLayout {
    float partials[kStaticMaxCtas * 2 * 2 * 16];  // 327,680 B
    int counters[kStaticMaxRowTiles];             //  65,536 B
    int status[64];
};
static __device__ __align__(256) unsigned char g_gemv_static_scratch[sizeof(StaticScratchLayout)];

struct StaticScratchHost {
    StaticScratchLayout* ptr = nullptr;  // device address of the array on this device
    int sm_count = 0;
};
StaticScratchHost g_static_host[64];
std::mutex g_static_mutex;

}  // namespace

cudaError_t launch_gemv_simple(const AilaNf4Linear& w, const void* x, void* y,
                               const void* residual, int64_t ff_pair, cudaStream_t s) {
    const bool paired = ff_pair > 0;
    const int n_out = paired ? (int)ff_pair : (int)w.N;
    if (n_out == 0) return cudaSuccess;
    const int warps = 8;
    const int blocks = (n_out + warps - 1) / warps;
    if (paired)
        gemv_simple_kernel<true><<<blocks, warps * 32, 0, s>>>(
            w.d_units, w.d_qmap, w.scale_params(), static_cast<const uint16_t*>(x),
            static_cast<uint16_t*>(y), nullptr, n_out, w.KU, w.unit_stride, w.absmax_kind,
            (int)(ff_pair / kTileRows));
    else
        gemv_simple_kernel<false><<<blocks, warps * 32, 0, s>>>(
            w.d_units, w.d_qmap, w.scale_params(), static_cast<const uint16_t*>(x),
            static_cast<uint16_t*>(y), static_cast<const uint16_t*>(residual), n_out, w.KU,
            w.unit_stride, w.absmax_kind, 0);
    return cudaGetLastError();
}

size_t gemv_stream_partials_floats(int sm_count) {
    return (size_t)sm_count * kMaxGridMult * 2 * 2 * 16;
}

bool gemv_stream_supported(const AilaNf4Linear& w, int64_t ff_pair, int sm_count) {
    if (w.K > 65535 * 4) return false;
    return stream_plan(w, ff_pair > 0, ff_pair, sm_count).ok;
}

cudaError_t launch_gemv_stream(const AilaNf4Linear& w, AilaNf4Scratch& scratch, const void* x,
                               void* y, const void* residual, int64_t ff_pair, cudaStream_t s) {
    const bool paired = ff_pair > 0;
    const StreamPlan pl = stream_plan(w, paired, ff_pair, scratch.sm_count);
    if (!pl.ok) return cudaErrorInvalidConfiguration;
    StreamParams p;
    p.units = w.d_units;
    p.qmap = w.d_qmap;
    p.sp = w.scale_params();
    p.x = static_cast<const uint16_t*>(x);
    p.y = static_cast<uint16_t*>(y);
    p.residual = static_cast<const uint16_t*>(residual);
    p.partials = scratch.d_partials;
    p.counters = scratch.d_counters;
    p.status = scratch.d_status;
    const int rt_work = paired ? (int)(ff_pair / kTileRows) : w.RT;
    p.total_items = (long long)rt_work * w.KU;
    p.n_out = paired ? (int)ff_pair : (int)w.N;
    p.K = (int)w.K;
    p.KU = w.KU;
    p.unit_stride = w.unit_stride;
    p.pair_rt_offset = paired ? (int)(ff_pair / kTileRows) : 0;
    p.x_bytes = (int)((w.K * 2 + 15) / 16 * 16);
    p.stages = pl.stages;
    if (w.absmax_kind == kAbsmaxCodes)
        return paired ? launch_stream_t<kAbsmaxCodes, true>(p, pl.grid, pl.smem, s)
                      : launch_stream_t<kAbsmaxCodes, false>(p, pl.grid, pl.smem, s);
    return paired ? launch_stream_t<kAbsmaxF32, true>(p, pl.grid, pl.smem, s)
                  : launch_stream_t<kAbsmaxF32, false>(p, pl.grid, pl.smem, s);
}

// Decode GEMV on the static work space: no allocation of any kind. The first call on a device
// resolves the device address of the array (the array's name is only a host-side stand-in for
// it, so the address comes from cudaGetSymbolAddress with that device current).
AilaNf4Status launch_gemv_stream_static(const AilaNf4Linear& w, const void* x, void* y,
                                        const void* residual, cudaStream_t s) {
    int dev = 0;
    NF4_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(AILA_NF4_ERR_UNSUPPORTED, "device ordinal above 63");
    StaticScratchHost host;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static_host[dev].ptr) {
            void* p = nullptr;
            NF4_CUDA(cudaGetSymbolAddress(&p, g_gemv_static_scratch));
            int sms = 0;
            NF4_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            g_static_host[dev].sm_count = sms;
            g_static_host[dev].ptr = static_cast<StaticScratchLayout*>(p);
        }
        host = g_static_host[dev];
    }
    if (w.RT > kStaticMaxRowTiles)
        return fail(AILA_NF4_ERR_UNSUPPORTED,
                    "aila_nf4_forward_decode_static: out_features " + std::to_string(w.N) +
                        " exceeds the fixed work space (max " +
                        std::to_string(kStaticMaxRowTiles * kTileRows) + " rows)");
    const StreamPlan pl = stream_plan(w, false, 0, host.sm_count);
    if (!pl.ok || pl.grid > kStaticMaxCtas || w.K > 65535 * 4)
        return fail(AILA_NF4_ERR_UNSUPPORTED,
                    "aila_nf4_forward_decode_static: shape not taken by the streaming kernel "
                    "within the fixed work space");
    if (reinterpret_cast<uintptr_t>(x) & 15)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "x must be 16-byte aligned");
    // The array keeps whatever the previous call left: counters must start at zero.
    NF4_CUDA(cudaMemsetAsync(host.ptr->counters, 0, sizeof(int) * (size_t)w.RT, s));
    AilaNf4Scratch view;
    view.device = dev;
    view.d_partials = host.ptr->partials;
    view.d_counters = host.ptr->counters;
    view.d_status = host.ptr->status;
    view.sm_count = host.sm_count;
    NF4_CUDA(launch_gemv_stream(w, view, x, y, residual, 0, s));
    return AILA_NF4_OK;
}

}  // namespace nf4
