// Shared definitions for the NF4 linear library (sm_100a only).
//
// HBM layout of one quantised weight W[N][K] ("unit stream")
// ----------------------------------------------------------
// The checkpoint layout is row-major nibbles [N][K/2] (high nibble = even k) plus one absmax
// per 64 weights (reference: src/ops/Bnb4BitLinear.cpp:738-746). At load time the library
// regroups it into UNITS. A unit covers 16 consecutive output rows x one 64-wide absmax
// block of k:
//
//   bytes [0,512)   nibbles, 16 rows x 32 B. Inside a row the 32 bytes are permuted so that
//                   the 8-byte chunk t (t = 0..3) holds, for j = 0..3, the two source bytes
//                   covering k = 16*j + 4*t + {0,1,2,3}; stored byte p = 8*t + 2*j + e is
//                   source byte o = 8*j + 2*t + e. A lane of a warp therefore reads the 16
//                   weights it feeds to four m16n8k16 tensor-core tiles with one 8-byte load,
//                   and a warp reads a whole unit with two conflict-free 256-byte loads.
//   bytes [512,..)  the 16 rows' absmax for this block: 16 u8 second-level codes (unit
//                   stride 528 B) or 16 fp32 absmax (unit stride 576 B).
//
// Units are stored row-tile major: unit index u = (n/16) * (K/64) + k/64. Every unit starts
// on a 16-byte boundary, so any contiguous range of units is one bulk-async copy. Rows past N
// in the last row tile are zero nibbles with code 0 and are never written back.
//
// Block sizes that are larger multiples of 64 are stored with the block's code repeated in
// every 64-wide unit it covers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nf4 {

constexpr int kTileRows = 16;
constexpr int kUnitK = 64;
constexpr int kUnitNibbleBytes = kTileRows * kUnitK / 2;  // 512
constexpr int kUnitStrideCodes = kUnitNibbleBytes + kTileRows;      // 528
constexpr int kUnitStrideF32 = kUnitNibbleBytes + kTileRows * 4;    // 576
constexpr int kMaxSegments = 4;

enum AbsmaxKind : int { kAbsmaxCodes = 0, kAbsmaxF32 = 1 };

// Everything a kernel needs to turn (row, 64-block, code) into the fp32 absmax.
// Second-level index of block (n, kblk): the block's flat index in the ORIGINAL tensor it was
// quantised in, divided by the nested block size (Bnb4BitLinear.cpp:482-487). Row fusion
// (Bnb4BitLinear.cpp:604-615) and sharding keep the original numbering per source, so each
// source ("segment") carries the flat index of its first block, the flat distance between
// rows, the offset of its nested_absmax inside the concatenated array, and its own offset.
struct ScaleParams {
    const float* nmap;   // [256] second-level code book
    const float* nabs;   // concatenated nested_absmax
    int nseg;
    int nbs_shift;       // log2(nested block size)
    int blk_shift;       // log2(blocksize / 64): units per absmax block
    int row0[kMaxSegments];            // first row of the segment in this linear
    unsigned flat0[kMaxSegments];      // nabs_base * nbs + flat index of the segment's (row0, k=0) block
    unsigned row_stride[kMaxSegments]; // flat distance between consecutive rows
    float offset[kMaxSegments];
};

// Constants of the segment that owns row n, selected with static indices only (no dynamically
// indexed copy of the parameter block in local memory).
struct SegmentRow {
    unsigned flat;  // flat index of the row's first block (second-level numbering base included)
    float offset;
};

__device__ __forceinline__ SegmentRow segment_row(const ScaleParams& sp, int n) {
    int row0 = sp.row0[0];
    unsigned flat0 = sp.flat0[0], stride = sp.row_stride[0];
    float off = sp.offset[0];
#pragma unroll
    for (int i = 1; i < kMaxSegments; ++i) {
        if (i < sp.nseg && n >= sp.row0[i]) {
            row0 = sp.row0[i];
            flat0 = sp.flat0[i];
            stride = sp.row_stride[i];
            off = sp.offset[i];
        }
    }
    SegmentRow r;
    r.flat = flat0 + (unsigned)(n - row0) * stride;
    r.offset = off;
    return r;
}

// fp32 absmax of (row n, unit column kb) from its 8-bit code: two separately rounded fp32
// operations, never a fused multiply-add (Bnb4BitLinear.cpp:485-487 writes mul then add).
__device__ __forceinline__ float decode_absmax(const ScaleParams& sp, int n, int kb, unsigned code) {
    const SegmentRow sr = segment_row(sp, n);
    const unsigned flat = sr.flat + ((unsigned)kb >> sp.blk_shift);
    const float scale = __ldg(sp.nabs + (flat >> sp.nbs_shift));
    return __fadd_rn(__fmul_rn(__ldg(sp.nmap + code), scale), sr.offset);
}

// Source byte offset (0..31) inside a row's 32-byte segment for stored byte p.
__host__ __device__ __forceinline__ int stored_to_source_byte(int p) {
    const int t = p >> 3, j = (p >> 1) & 3, e = p & 1;
    return 8 * j + 2 * t + e;
}

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// Two floats to a bf16 pair (round to nearest even each, `lo` in the low half): one conversion
// instruction instead of two conversions and a merge.
__device__ __forceinline__ uint32_t f32x2_to_bf16x2_bits(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) {
    return __uint_as_float(((uint32_t)h) << 16);
}

// ---------------------------------------------------------------------------------------
// Bounded waits. Every spin in this library gives up after a limit of SM cycles (this default,
// or the scratch's setting: aila_nf4_scratch_set_wait_limit)
// (about a second), records a code in a global status word and lets the kernel drain.
// ---------------------------------------------------------------------------------------
constexpr long long kSpinLimitCycles = 2000000000LL;

enum KernelStatus : int {
    kStatusOk = 0,
    kStatusTimeoutFull = 1,   // consumer gave up waiting for data
    kStatusTimeoutEmpty = 2,  // producer gave up waiting for a free stage
    kStatusTimeoutTmem = 3,   // epilogue / MMA gave up waiting on a TMEM barrier
    kStatusBadArgument = 4,
    kStatusTimeoutPeer = 5,   // a rank gave up waiting for another rank's rows
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Returns false after the cycle limit; the caller records a status and stops using the pipe.
// A waiting thread backs off with nanosleep so that it does not take issue slots from the warps
// of its scheduler that have work.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  long long limit = kSpinLimitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            __nanosleep(100);
        }
        if (clock64() - t0 > limit) return false;
    }
}

// Untiled bulk-async copy global -> shared of `bytes` (multiple of 16, both sides 16-byte
// aligned), completion counted on `bar`. Every CTA fetches its own copy.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

}  // namespace nf4
