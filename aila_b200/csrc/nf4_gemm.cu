// Prefill (seq_len > 1) contraction: y[M][N] = x[M][K] * w[N][K]^T, bf16 operands, fp32
// accumulation in tensor memory, bf16 output. `w` is the NF4 weight already rounded to bf16
// exactly as the reference's dequantize_weight does (src/ops/Bnb4BitLinear.cpp:746,:754), so
// this kernel stands where the reference calls oneDNN's bf16 matmul (:689-721, :944).
//
// Blackwell-native structure (sm_100a):
//   * TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, one copy per CTA) stages 128 x 64 tiles of x
//     and BN x 64 tiles of w in a shared-memory ring of as many stages as fit in 216 KB (at most 8);
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN,
//     K = 16) with both operands K-major in shared memory and the accumulator in TMEM;
//   * two shapes of CTA tile, chosen per problem by a cost model (bytes per flop vs. waves):
//     128 x BN with two TMEM accumulator buffers (2 x 256 columns), so the epilogue warps drain
//     tile i with tcgen05.ld while the tensor core already works on tile i+1; or 256 x BN, two
//     M = 128 MMAs per K step sharing one w tile (a third fewer operand bytes per flop, three or
//     four stages in flight), with both accumulators live and eight epilogue warps;
//   * persistent CTAs, one per SM; BN is a multiple of 16 (<= 256) picked so the tile count
//     fills whole waves of 148 SMs.
// Optional epilogues: + residual, or SwiGLU over a gate|up weight (tile = 128 gate columns'
// worth + the matching up columns), rounding gate and up to bf16 first as the reference's
// forward + ops::fused_gate_up_swiglu pair does (src/ops/ElementwiseOps.cpp:247-294).
//
// A second form of the kernel (FUSED) takes the weight as NF4 units and rebuilds every w tile in
// shared memory itself (sixteen more warps), so no bf16 copy of W goes through HBM. Its output is
// bit-identical to the two-phase route; it is the slower of the two at every measured size and is
// therefore only used on request (AILA_NF4_FUSED_PREFILL=1).
//
// Roofline: tensor pipe. Algorithmic flops 2*M*N*K.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "nf4_internal.h"

namespace nf4 {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kMaxBN = 256;
constexpr int kMaxStages = 8;
constexpr int kABytes = BM * BK * 2;         // 16 KB per 128 rows of x
constexpr int kBBytes = kMaxBN * BK * 2;     // 32 KB
constexpr int kRingBytes = 4 * (kABytes + kBBytes);  // = 3 * (2 * kABytes + kBBytes) = 192 KB
constexpr int kGemmThreads = 320;            // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int kDequantWarps = 16;            // fused form: warps 10-25 write the w tiles from NF4 (one unit each)
constexpr int kFusedThreads = kGemmThreads + kDequantWarps * 32;
constexpr int kFusedTableBytes = 64 + 1024;  // fused form: code book (16 floats), second-level code book (256)
constexpr int kNfSlots = 3;                  // fused form: NF4 units in flight per dequantisation warp
constexpr int kNfSlotBytes = kUnitStrideF32; // one unit (528 or 576 bytes)
constexpr int kFusedExtraBytes = kFusedTableBytes + kDequantWarps * kNfSlots * (kNfSlotBytes + 8);
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kRingBytesLarge = 216 * 1024;  // two-phase form: nothing else needs shared memory
constexpr int kGemmSmem = kRingBytesLarge + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int kGemmSmemFusedBase = kRingBytes + 1024 + 256;

// The NF4 weight of the fused form (the w tiles are produced in shared memory from the unit stream
// instead of being copied from a bf16 matrix).
struct FusedWeight {
    const uint8_t* units;      // unit stream: unit (rt, kb) at (rt * KU + kb) * unit_stride
    const float* qmap;         // [16]
    const float* nmap;         // [256] second-level code book (8-bit absmax codes)
    const float4* row_scales;  // [n_rows] {lo, hi, cross, offset} (8-bit absmax codes)
    int KU, RT, n_rows, unit_stride, kind;
};

struct GemmParams {
    uint16_t* y;
    const uint16_t* residual;
    int* status;
    int M;
    int N;        // rows of w (gate|up: 2*ff)
    int K;
    int n_out;    // row pitch of y in elements (N, or ff with SwiGLU)
    int BN;       // UMMA N (SwiGLU: BN/2 gate + BN/2 up columns)
    int m_tiles;
    int n_tiles;
    int swiglu_ff;  // 0 = plain
    int mtile;      // 1: CTA tile 128 x BN (double-buffered accumulator); 2: 256 x BN
    int stages;     // ring depth: as many stages of (x tile + w tile) as fit, at most kMaxStages
    int b_bytes;    // shared-memory bytes of one w tile (BN rows of 128 bytes, rounded up to 1024)
    uint32_t idesc;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle; rows are 128 B apart,
// 8-row groups 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);       // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
    d |= (uint64_t)1 << 46;                        // version
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}

// tcgen05.mma with the two shared-memory descriptors given as their low words (start address field)
// plus the high word both share (layout fields): the issuing thread keeps 32-bit arithmetic in its loop.
__device__ __forceinline__ void umma_bf16_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    return f32x2_to_bf16x2_bits(lo, hi);
}

extern __shared__ __align__(1024) uint8_t gemm_smem[];

// FUSED: the B operand is not a bf16 matrix in global memory. Eight more warps read the NF4 units of
// the tile's rows (the same 512-byte-per-unit pattern as the decode kernels), rebuild
// bf16(code_book[nibble] * absmax) - bit-equal to dequantize_weight - and store it into the stage's
// w tile in the K-major 128-byte-swizzle layout the tensor core expects; a proxy fence and one
// arrival per warp on the stage's `full` barrier stand where the TMA completion stood.
template <bool FUSED>
__global__ void __launch_bounds__(FUSED ? kFusedThreads : kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                         const __grid_constant__ CUtensorMap map_w, const GemmParams p,
                         const FusedWeight fw) {
    // 1024-byte aligned ring (the swizzle pattern is a function of the absolute address)
    uint8_t* base = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(gemm_smem) + 1023) & ~(uintptr_t)1023);
    constexpr int kRing = FUSED ? kRingBytes : kRingBytesLarge;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + kRing);
    uint64_t* full = bars;                      // [kMaxStages]
    uint64_t* empty = bars + kMaxStages;        // [kMaxStages]
    uint64_t* acc_full = bars + 2 * kMaxStages; // [kAccStages]
    uint64_t* acc_empty = acc_full + kAccStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kAccStages);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_qmap = reinterpret_cast<float*>(base + kRingBytes + 256);  // fused form only
    float* s_nmap = s_qmap + 16;
    uint64_t* nf_full = reinterpret_cast<uint64_t*>(base + kRingBytes + 256 + kFusedTableBytes);  // [warp][slot]
    uint8_t* nf_ring = reinterpret_cast<uint8_t*>(nf_full + kDequantWarps * kNfSlots);           // [warp][slot][unit]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_blocks = p.K / BK;
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int kStages = p.stages;
    const int a_bytes = kABytes * p.mtile;
    const int kStageBytes = a_bytes + p.b_bytes;
    const int acc_stages = p.mtile == 1 ? kAccStages : 1;  // 256-row tiles keep both halves live

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], FUSED ? 1 + kDequantWarps : 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < kAccStages; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4 * p.mtile);
        }
        *abort_flag = 0;
        if (FUSED)
            for (int i = 0; i < kDequantWarps * kNfSlots; ++i) mbar_init(&nf_full[i], 1);
        mbar_fence_init();
    }
    if (FUSED) {
        if (threadIdx.x >= 64 && threadIdx.x < 80) s_qmap[threadIdx.x - 64] = __ldg(fw.qmap + (threadIdx.x - 64));
        if (fw.kind == kAbsmaxCodes && threadIdx.x >= 320 && threadIdx.x < 576)
            s_nmap[threadIdx.x - 320] = __ldg(fw.nmap + (threadIdx.x - 320));
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Launched with programmatic stream serialisation: everything above overlapped the tail of
    // the kernel that produces w (the dequantisation pass); from here on its output is needed.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            const uint32_t b_bytes = (uint32_t)p.BN * BK * 2;
            const uint32_t tx_bytes = FUSED ? (uint32_t)a_bytes : a_bytes + b_bytes;
            const int half = p.BN / 2;
            int it = 0;
            int s = 0;            // stage of step `it`
            uint32_t ph = 0;      // parity its `empty` barrier shows when the stage is free again (from round 1 on)
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
                const int m0 = mt * BM * p.mtile;
                const int n0 = p.swiglu_ff == 0 ? nt * p.BN : nt * half;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    if (it >= kStages && !mbar_try_wait(&empty[s], ph)) {
                        if (*abort_flag || !mbar_wait_bounded(&empty[s], ph)) {
                            if (!*abort_flag) atomicExch(p.status, kStatusTimeoutEmpty);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                    }
                    uint8_t* sa = base + s * kStageBytes;
                    uint8_t* sb = sa + a_bytes;
                    mbar_expect_tx(&full[s], tx_bytes);
                    tma_load_2d(sa, &map_x, kb * BK, m0, &full[s]);
                    if (FUSED) {
                        // the dequantisation warps fill the w tile
                    } else if (p.swiglu_ff == 0) {
                        tma_load_2d(sb, &map_w, kb * BK, n0, &full[s]);
                    } else {
                        tma_load_2d(sb, &map_w, kb * BK, n0, &full[s]);
                        tma_load_2d(sb + half * BK * 2, &map_w, kb * BK, p.swiglu_ff + n0, &full[s]);
                    }
                    if (++s == kStages) {
                        s = 0;
                        if (it >= kStages) ph ^= 1u;
                    }
                }
            }
            // drain: copies issued by this thread must have landed before the CTA exits
            for (int g = max(0, it - kStages); g < it; ++g)
                mbar_wait_bounded(&full[g % kStages], (g / kStages) & 1);
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            // One thread issues every MMA of the CTA, and its own instruction latencies are what a
            // K step costs when the tiles are small: the loop keeps the stage index, the barrier
            // parity and the descriptors' address fields as running 32-bit values (no division, no
            // 64-bit arithmetic) and looks at the abort flag only when a wait is not satisfied at once.
            int it = 0, tcount = 0;
            int s = 0;
            uint32_t ph = 0;  // parity of full[s] for the current round
            int as = 0;
            uint32_t aph = 0;  // parity of acc_empty[as] once the accumulators are reused
            const uint64_t d0 = make_smem_desc(smem_u32(base));
            const uint32_t desc_hi = (uint32_t)(d0 >> 32);
            const uint32_t a_lo0 = (uint32_t)d0;                     // stage 0, x tile rows 0..127
            const uint32_t stage_inc = (uint32_t)kStageBytes >> 4;   // address field counts 16-byte units
            const uint32_t a2_inc = (uint32_t)kABytes >> 4;          // rows 128..255 of x
            const uint32_t b_inc = (uint32_t)a_bytes >> 4;           // the w tile
            uint32_t a_cur = a_lo0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
                if (tcount >= acc_stages && !mbar_try_wait(&acc_empty[as], aph)) {
                    if (*abort_flag || !mbar_wait_bounded(&acc_empty[as], aph)) {
                        if (!*abort_flag) atomicExch(p.status, kStatusTimeoutTmem);
                        *abort_flag = 1;
                        break;
                    }
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tacc = tmem_base + (uint32_t)(as * kMaxBN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    if (!mbar_try_wait(&full[s], ph)) {
                        if (*abort_flag || !mbar_wait_bounded(&full[s], ph)) {
                            if (!*abort_flag) atomicExch(p.status, kStatusTimeoutFull);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                    }
                    // (the operands were made visible by the copies' / the producer warps' own
                    // completion on `full`: no fence between the wait and the MMAs)
                    const uint32_t b_cur = a_cur + b_inc;
                    const uint32_t first = kb > 0 ? 1u : 0u;  // the tile's first MMA overwrites the accumulator
                    if (p.mtile == 2) {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) {
                            // advance 16 elements (32 bytes = 2 address units) along K inside the swizzled row
                            umma_bf16_lo(tacc, a_cur + 2 * k, b_cur + 2 * k, desc_hi, p.idesc, k > 0 ? 1u : first);
                            umma_bf16_lo(tacc + kMaxBN, a_cur + a2_inc + 2 * k, b_cur + 2 * k, desc_hi, p.idesc,
                                         k > 0 ? 1u : first);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_bf16_lo(tacc, a_cur + 2 * k, b_cur + 2 * k, desc_hi, p.idesc, k > 0 ? 1u : first);
                    }
                    umma_commit(&empty[s]);  // frees the stage when these MMAs have read it
                    a_cur += stage_inc;
                    if (++s == kStages) {
                        s = 0;
                        a_cur = a_lo0;
                        ph ^= 1u;
                    }
                }
                if (ok) umma_commit(&acc_full[as]);
                if (++as == acc_stages) {
                    as = 0;
                    if (tcount >= acc_stages) aph ^= 1u;
                }
            }
        }
    } else if (FUSED && warp >= kGemmThreads / 32) {
        // ------------------------------ w tiles from NF4 (warps 10..25) ------------------------------
        // Unit iu of a tile = its rows 16 iu .. 16 iu + 15 (gate rows first, then the matching up
        // rows, with SwiGLU); warp dw takes unit dw. Lane (gq, t) holds, as in the decode kernels,
        // 8 bytes of row gq and 8 bytes of row gq + 8: byte 2j + e covers k = 16 j + 4 t + 2 e (high
        // nibble) and + 1 (low nibble).
        const int dw = warp - kGemmThreads / 32;
        const int gq = lane >> 2, t = lane & 3;
        const int n_units = p.BN / 16;
        const int half_units = p.swiglu_ff > 0 ? n_units / 2 : n_units;
        const int ST = fw.unit_stride;
        const uint32_t w_off = (uint32_t)(gq * 32 + 8 * t);
        const uint32_t a_q = smem_u32(s_qmap);
        // The warp's units arrive through a private ring of kNfSlots bulk-async copies, issued
        // kNfSlots steps ahead, so that memory latency never meets the arithmetic. A step whose unit
        // does not exist (rows past the weight, or this warp has no unit in the tile) copies nothing
        // and writes zeros; the j-th copy that IS issued uses slot j % kNfSlots on both sides.
        uint64_t* my_full = nf_full + dw * kNfSlots;
        uint8_t* my_ring = nf_ring + (size_t)dw * kNfSlots * kNfSlotBytes;
        // row tile of unit iu of n-tile nt (>= fw.RT: rows past the weight)
        auto unit_rt = [&](int nt, int iu) {
            if (p.swiglu_ff > 0)
                return iu < half_units ? nt * half_units + iu : p.swiglu_ff / 16 + nt * half_units + (iu - half_units);
            return nt * n_units + iu;
        };
        auto step_rt = [&](int tile) {  // this warp's row tile in `tile`, or -1
            if (dw >= n_units) return -1;
            const int rt = unit_rt(tile / p.m_tiles, dw);
            return rt < fw.RT ? rt : -1;
        };
        int p_tile = blockIdx.x, p_kb = 0, p_j = 0;  // the next step to issue; copies issued so far
        int c_j = 0;                                 // copies consumed so far
        auto issue_next = [&]() {  // one lane
            if (p_tile >= total_tiles) return;
            const int rt = step_rt(p_tile);
            if (rt >= 0) {
                const int slot = p_j % kNfSlots;
                mbar_expect_tx(&my_full[slot], (uint32_t)ST);
                bulk_g2s(my_ring + slot * kNfSlotBytes, fw.units + ((size_t)rt * fw.KU + p_kb) * (size_t)ST,
                         (uint32_t)ST, &my_full[slot]);
                ++p_j;
            }
            if (++p_kb == k_blocks) {
                p_kb = 0;
                p_tile += gridDim.x;
            }
        };
        if (lane == 0)
            for (int i = 0; i < kNfSlots; ++i) issue_next();
        // code book value of nibble `k` (0 = lowest) of `word`; the table never changes after set-up,
        // so the load is free to move (not volatile, no memory clobber)
        auto qv = [&](uint32_t word, int k) {
            const uint32_t off = k == 0 ? (word << 2) & 0x3cu : (word >> (4 * k - 2)) & 0x3cu;
            float v;
            asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a_q + off));
            return v;
        };
        // one row's 8 bytes -> eight packed pairs (k ascending), then four 8-byte stores
        auto emit_row = [&](uint32_t row_base, uint2 w, float am) {
            uint32_t pk[8];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t word = h == 0 ? w.x : w.y;
#pragma unroll
                for (int b = 0; b < 4; ++b)  // byte b: high nibble first
                    pk[4 * h + b] = pack2(__fmul_rn(qv(word, 2 * b + 1), am), __fmul_rn(qv(word, 2 * b), am));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t a = row_base + ((((uint32_t)(2 * j + (t >> 1))) ^ (uint32_t)gq) << 4) + ((uint32_t)(t & 1) << 3);
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a), "r"(pk[2 * j]), "r"(pk[2 * j + 1]));
            }
        };
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int rt = step_rt(tile);
            float4 e0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), e1 = e0;
            if (rt >= 0 && fw.kind == kAbsmaxCodes) {
                e0 = __ldg(fw.row_scales + min(rt * 16 + gq, fw.n_rows - 1));
                e1 = __ldg(fw.row_scales + min(rt * 16 + gq + 8, fw.n_rows - 1));
            }
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % kStages;
                bool good = true;
                if (lane == 0) {
                    if (it >= kStages &&
                        (*abort_flag || !mbar_wait_bounded(&empty[s], ((it / kStages) - 1) & 1))) {
                        if (!*abort_flag) atomicExch(p.status, kStatusTimeoutEmpty);
                        *abort_flag = 1;
                        good = false;
                    }
                    if (good && rt >= 0 &&
                        (*abort_flag || !mbar_wait_bounded(&my_full[c_j % kNfSlots], (c_j / kNfSlots) & 1))) {
                        if (!*abort_flag) atomicExch(p.status, kStatusTimeoutFull);
                        *abort_flag = 1;
                        good = false;
                    }
                }
                good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;
                if (!good) {
                    ok = false;
                    break;
                }
                if (dw < n_units) {
                    uint2 l = make_uint2(0x77777777u, 0x77777777u), u = l;
                    float am0 = 0.0f, am1 = 0.0f;
                    if (rt >= 0) {
                        const uint32_t ua = smem_u32(my_ring + (c_j % kNfSlots) * kNfSlotBytes);
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(l.x), "=r"(l.y) : "r"(ua + w_off));
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(u.x), "=r"(u.y) : "r"(ua + w_off + 256u));
                        if (fw.kind == kAbsmaxCodes) {
                            uint32_t c0, c1;
                            asm volatile("ld.shared.u8 %0, [%1];" : "=r"(c0) : "r"(ua + kUnitNibbleBytes + gq));
                            asm volatile("ld.shared.u8 %0, [%1];" : "=r"(c1) : "r"(ua + kUnitNibbleBytes + gq + 8));
                            // absmax = second-level code book value * the row's second-level scale + offset
                            am0 = __fadd_rn(__fmul_rn(s_nmap[c0], kb >= __float_as_int(e0.z) ? e0.y : e0.x), e0.w);
                            am1 = __fadd_rn(__fmul_rn(s_nmap[c1], kb >= __float_as_int(e1.z) ? e1.y : e1.x), e1.w);
                        } else {
                            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(am0) : "r"(ua + kUnitNibbleBytes + 4u * gq));
                            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(am1) : "r"(ua + kUnitNibbleBytes + 4u * (gq + 8)));
                        }
                    }
                    const uint32_t rb = smem_u32(base + s * kStageBytes + a_bytes) + (uint32_t)dw * 2048u + (uint32_t)gq * 128u;
                    emit_row(rb, l, am0);
                    emit_row(rb + 1024u, u, am1);
                }
                // generic-proxy stores -> visible to the tensor core's (async proxy) reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full[s]);
                    issue_next();  // the unit's slot is free: every lane's loads fed the stores above
                }
                if (rt >= 0) ++c_j;
            }
        }
        // copies issued for steps that were never reached (after a failure) must land before exit
        if (!ok && lane == 0) {
            for (int j = c_j; j < p_j; ++j) mbar_wait_bounded(&my_full[j % kNfSlots], (j / kNfSlots) & 1, 2000000LL);
        }
    } else {
        // ------------------------------ epilogue (warps 2..9) ------------------------------
        const int quarter = warp & 3;      // TMEM lanes [32*quarter, +32)
        const int mhalf = (warp - 2) >> 2;  // which 128-row half of a 256-row tile
        int tcount = 0;
        const bool vec_ok = (p.n_out % 8) == 0;
        // 128-row tiles use four epilogue warps; the other four have nothing to drain
        for (int tile = (mhalf < p.mtile ? (int)blockIdx.x : total_tiles); tile < total_tiles;
             tile += gridDim.x, ++tcount) {
            const int as = tcount % acc_stages;
            const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
            bool ok = true;
            if (lane == 0) {
                if (*abort_flag || !mbar_wait_bounded(&acc_full[as], (tcount / acc_stages) & 1)) {
                    if (!*abort_flag) atomicExch(p.status, kStatusTimeoutTmem);
                    *abort_flag = 1;
                    ok = false;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m = (mt * p.mtile + mhalf) * BM + quarter * 32 + lane;
            const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                  (uint32_t)((as + mhalf) * kMaxBN);
            if (p.swiglu_ff == 0) {
                const int n0 = nt * p.BN;
                for (int c = 0; c < p.BN; c += 16) {
                    uint32_t r[16];
                    tmem_ld16(trow + c, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int n = n0 + c;
                    if (m < p.M && n < p.N) {
                        uint16_t* yp = p.y + (size_t)m * p.n_out + n;
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
                        if (vec_ok && n + 16 <= p.N) {
                            if (p.residual) {
                                const uint4* rp = reinterpret_cast<const uint4*>(
                                    p.residual + (size_t)m * p.n_out + n);
                                const uint4 r0 = rp[0], r1 = rp[1];
                                const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    v[2 * i] += bf16_bits_to_f32(rw[i] & 0xffff);
                                    v[2 * i + 1] += bf16_bits_to_f32(rw[i] >> 16);
                                }
                            }
                            uint4 o0, o1;
                            o0.x = pack2(v[0], v[1]);   o0.y = pack2(v[2], v[3]);
                            o0.z = pack2(v[4], v[5]);   o0.w = pack2(v[6], v[7]);
                            o1.x = pack2(v[8], v[9]);   o1.y = pack2(v[10], v[11]);
                            o1.z = pack2(v[12], v[13]); o1.w = pack2(v[14], v[15]);
                            reinterpret_cast<uint4*>(yp)[0] = o0;
                            reinterpret_cast<uint4*>(yp)[1] = o1;
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                if (n + i < p.N) {
                                    float o = v[i];
                                    if (p.residual)
                                        o += bf16_bits_to_f32(p.residual[(size_t)m * p.n_out + n + i]);
                                    yp[i] = f32_to_bf16_bits(o);
                                }
                            }
                        }
                    }
                }
            } else {
                const int half = p.BN / 2;
                const int n0 = nt * half;
                for (int c = 0; c < half; c += 16) {
                    uint32_t rg[16], ru[16];
                    tmem_ld16(trow + c, rg);
                    tmem_ld16(trow + half + c, ru);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int n = n0 + c;
                    if (m < p.M && n < p.swiglu_ff) {
                        uint16_t* yp = p.y + (size_t)m * p.n_out + n;
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            // gate and up pass through bf16 first, like a bf16 gate_up buffer
                            const float g = bf16_bits_to_f32(f32_to_bf16_bits(__uint_as_float(rg[i])));
                            const float u = bf16_bits_to_f32(f32_to_bf16_bits(__uint_as_float(ru[i])));
                            v[i] = __fdividef(g, 1.0f + __expf(-g)) * u;
                        }
                        if (vec_ok && n + 16 <= p.swiglu_ff) {
                            uint4 o0, o1;
                            o0.x = pack2(v[0], v[1]);   o0.y = pack2(v[2], v[3]);
                            o0.z = pack2(v[4], v[5]);   o0.w = pack2(v[6], v[7]);
                            o1.x = pack2(v[8], v[9]);   o1.y = pack2(v[10], v[11]);
                            o1.z = pack2(v[12], v[13]); o1.w = pack2(v[14], v[15]);
                            reinterpret_cast<uint4*>(yp)[0] = o0;
                            reinterpret_cast<uint4*>(yp)[1] = o1;
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (n + i < p.swiglu_ff) yp[i] = f32_to_bf16_bits(v[i]);
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
    }

    // teardown: everyone done with TMEM before it is released
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(kTmemCols)
                     : "memory");
    }
}

// cuTensorMapEncodeTiled, fetched through the runtime so the library has no link-time
// dependency on the driver library.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D bf16 row-major [rows][K] tensor, box = 64 columns x box_rows rows, 128-byte swizzle,
// out-of-bounds elements read as zero.
bool encode_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t K, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tile shape for this problem. For each candidate (rows 128 or 256, width a multiple of `step`)
// the cost is waves x (K steps x max(tensor-pipe cycles, operand bytes / L2-to-SM rate) +
// exposed epilogue). The 128-row shape hides its epilogue behind the next tile; the 256-row
// shape moves a third fewer bytes per flop and keeps more K steps in flight.
struct TileChoice {
    int mtile;
    int bn;  // accumulator columns per 128-row half
};

// Measurement overrides, read once: AILA_NF4_GEMM_MTILE=1|2 (rows of x per CTA tile / 128) and
// AILA_NF4_GEMM_BN=<multiple of 16> (UMMA N; with SwiGLU gate + up columns together).
int env_tile_override(const char* name) {
    const char* e = std::getenv(name);
    return (e && *e) ? std::atoi(e) : 0;
}

TileChoice choose_tile(int M, int64_t n_cols, int step, int max_bn, int width_scale, int k_blocks,
                       int sm_count) {
    static const int force_mtile = env_tile_override("AILA_NF4_GEMM_MTILE");
    static const int force_bn = env_tile_override("AILA_NF4_GEMM_BN");
    constexpr double kL2BytesPerClk = 70.0;  // sustained L2 -> SM operand rate per SM (measured)
    TileChoice best = {1, step};
    double best_cost = 1e300;
    for (int mtile = 1; mtile <= 2; ++mtile) {
        if (mtile == 2 && M <= BM) continue;
        if ((force_mtile == 1 || force_mtile == 2) && mtile != force_mtile && !(force_mtile == 2 && M <= BM)) continue;
        const int m_tiles = (M + BM * mtile - 1) / (BM * mtile);
        for (int bn = step; bn <= max_bn; bn += step) {
            const int umma_n = bn * width_scale;
            if (force_bn > 0 && force_bn % 16 == 0 && umma_n != force_bn && force_bn <= max_bn * width_scale &&
                force_bn % (step * width_scale) == 0)
                continue;
            const int64_t n_tiles = (n_cols + bn - 1) / bn;
            const int64_t waves = (n_tiles * m_tiles + sm_count - 1) / sm_count;
            const double mma = 2.0 * umma_n * mtile;                       // cycles per K step
            const double mem = (kABytes * mtile + umma_n * BK * 2) / kL2BytesPerClk;
            const double epi = mtile == 2 ? 6.0 * umma_n : 0.0;            // exposed drain
            const double cost = (double)waves * (k_blocks * (mma > mem ? mma : mem) + epi + 400.0);
            if (cost < best_cost * 0.999 || (cost <= best_cost * 1.001 && bn > best.bn)) {
                best_cost = cost;
                best = {mtile, bn};
            }
        }
    }
    return best;
}

}  // namespace

namespace {
// w_nk: the bf16 weight [N][K], or nullptr with `fw` describing the NF4 weight (fused form)
AilaNf4Status launch_gemm_common(const void* w_nk, const FusedWeight* fw, const void* x, void* y,
                                 const void* residual, int M, int64_t N, int64_t K, int64_t swiglu_ff,
                                 int sm_count, int* d_status, cudaStream_t s) {
    if (K % BK != 0) return fail(AILA_NF4_ERR_UNSUPPORTED, "prefill GEMM needs in_features % 64 == 0");
    if ((reinterpret_cast<uintptr_t>(w_nk) | reinterpret_cast<uintptr_t>(x)) & 15)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "prefill GEMM operands must be 16-byte aligned");
    GemmParams p;
    p.y = static_cast<uint16_t*>(y);
    p.residual = static_cast<const uint16_t*>(residual);
    p.status = d_status;
    p.M = M;
    p.N = (int)N;
    p.K = (int)K;
    p.swiglu_ff = (int)swiglu_ff;
    const int k_blocks = (int)(K / BK);
    if (swiglu_ff > 0) {
        // a tile holds `half` gate columns and the matching `half` up columns
        const TileChoice tc = choose_tile(M, swiglu_ff, 16, kMaxBN / 2, 2, k_blocks, sm_count);
        p.mtile = tc.mtile;
        p.BN = 2 * tc.bn;
        p.n_tiles = (int)((swiglu_ff + tc.bn - 1) / tc.bn);
        p.n_out = (int)swiglu_ff;
    } else {
        const TileChoice tc = choose_tile(M, N, 16, kMaxBN, 1, k_blocks, sm_count);
        p.mtile = tc.mtile;
        p.BN = tc.bn;
        p.n_tiles = (int)((N + p.BN - 1) / p.BN);
        p.n_out = (int)N;
    }
    p.m_tiles = (M + BM * p.mtile - 1) / (BM * p.mtile);
    p.b_bytes = (p.BN * BK * 2 + 1023) / 1024 * 1024;
    p.stages = (fw ? kRingBytes : kRingBytesLarge) / (kABytes * p.mtile + p.b_bytes);
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    // instruction descriptor: D = f32, A = B = bf16, both K-major, N >> 3, M >> 4
    p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.BN >> 3) << 17) |
              ((uint32_t)(BM >> 4) << 24);
    CUtensorMap map_x, map_w;
    if (!encode_map(&map_x, x, (uint64_t)M, (uint64_t)K, (uint32_t)(BM * p.mtile)))
        return fail(AILA_NF4_ERR_CUDA, "cuTensorMapEncodeTiled failed for the activation tensor");
    const uint32_t w_box = (uint32_t)(swiglu_ff > 0 ? p.BN / 2 : p.BN);
    if (fw) {
        map_w = map_x;  // unused by the fused form
    } else if (!encode_map(&map_w, w_nk, (uint64_t)N, (uint64_t)K, w_box)) {
        return fail(AILA_NF4_ERR_CUDA, "cuTensorMapEncodeTiled failed for the weight tensor");
    }

    static std::once_flag attr_once[64];
    int dev = 0;
    cudaGetDevice(&dev);
    cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<false>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            kGemmSmemFusedBase + kFusedExtraBytes);
    });
    if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(gemm)");
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int grid = total_tiles < sm_count ? total_tiles : sm_count;
    if (grid <= 0) return AILA_NF4_OK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(fw ? kFusedThreads : kGemmThreads);
    cfg.dynamicSmemBytes = fw ? kGemmSmemFusedBase + kFusedExtraBytes : kGemmSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const FusedWeight none = {};
    cudaError_t e = fw ? cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<true>, map_x, map_w, p, *fw)
                       : cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<false>, map_x, map_w, p, none);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_bf16_tcgen05_kernel launch");
    return AILA_NF4_OK;
}
}  // namespace

AilaNf4Status launch_gemm_bf16(const void* w_nk, const void* x, void* y, const void* residual,
                               int M, int64_t N, int64_t K, int64_t swiglu_ff, int device,
                               int sm_count, int* d_status, cudaStream_t s) {
    (void)device;
    return launch_gemm_common(w_nk, nullptr, x, y, residual, M, N, K, swiglu_ff, sm_count, d_status, s);
}

// The fused form takes the weight as it is stored (NF4 units): no bf16 copy of W goes through HBM.
bool gemm_nf4_fused_supported(const AilaNf4Linear& w, int64_t swiglu_ff) {
    if (w.K % BK != 0 || w.N % kTileRows != 0) return false;
    if (w.absmax_kind == kAbsmaxCodes && !w.d_row_scales) return false;
    if (swiglu_ff > 0 && (swiglu_ff % kTileRows != 0 || w.N != 2 * swiglu_ff)) return false;
    return true;
}

AilaNf4Status launch_gemm_nf4_fused(const AilaNf4Linear& w, const void* x, void* y, const void* residual,
                                    int M, int64_t swiglu_ff, int sm_count, int* d_status, cudaStream_t s) {
    if (!gemm_nf4_fused_supported(w, swiglu_ff))
        return fail(AILA_NF4_ERR_UNSUPPORTED, "fused prefill does not take this linear");
    FusedWeight fw;
    fw.units = w.d_units;
    fw.qmap = w.d_qmap;
    const ScaleParams sp = w.scale_params();
    fw.nmap = sp.nmap;
    fw.row_scales = static_cast<const float4*>(w.d_row_scales);
    fw.KU = w.KU;
    fw.RT = w.RT;
    fw.n_rows = (int)w.N;
    fw.unit_stride = w.unit_stride;
    fw.kind = w.absmax_kind;
    return launch_gemm_common(nullptr, &fw, x, y, residual, M, w.N, w.K, swiglu_ff, sm_count, d_status, s);
}

}  // namespace nf4
