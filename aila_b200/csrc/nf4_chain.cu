// Decode (seq_len == 1) NF4 linears as ONE persistent launch over a list of operations.
// Replaces packed_nf4_gemv_bf16 and packed_nf4_gemv_gate_up_swiglu
// (reference src/ops/Bnb4BitLinear.cpp:271-410, :142-246) for a whole run of linears as the
// reference's decode step issues them (src/models/Qwen3Bnb4Backend.cpp:339-418): the launch walks
// the list; an operation may take the previous operation's output as its input.
//
// Shape of the kernel
//  * One CTA per SM, launched cooperatively (all CTAs resident: CTAs wait on one another inside
//    the launch, every wait is bounded). 16 warps: 15 CONSUMER warps stream and decode weights,
//    one FINALIZER warp turns their sums into outputs and feeds them x, an operation behind.
//  * Work items are UNIT PAIRS: unit (row tile a, 64-block kb) together with unit (row tile b, kb).
//    For a fused gate|up linear a/b are the gate tile and its up tile; for a plain linear two row
//    tiles half the matrix apart ride together. Both halves need the same slice of x.
//  * The item stream (pair-major, then kb) is cut into equal contiguous slices, one per CTA, and
//    each slice into contiguous ranges for the consumer warps (all 15, or fewer when the slice is
//    small: a warp pays a fixed price per operation). A warp walks its range in STEPS of up to
//    four consecutive 64-blocks of one pair.
//  * Weights go global memory -> registers directly (two 8-byte loads per lane and unit; a lane's
//    bytes are exactly its tensor-core fragments, see nf4_common.cuh). While unit u of a step is
//    being decoded, the registers it frees are re-loaded with unit u of the NEXT step - of the next
//    operation, when the range ends - so a full step of loads per warp is always in flight and
//    the pipeline does not drain between operations. No shared-memory staging of weights.
//  * byte -> bf16 pair through a bank-private shared-memory table: one PRMT + one LDS per two
//    weights; the pairs are the A fragments of mma.sync m16n8k16 (bf16 x bf16 -> fp32).
//  * The four blocks of a step put their slice of x into four different columns of the B
//    fragment (lanes g = 0, 2, 4, 6 hold x of block 0..3), so lane (g, t) ends up with the raw
//    sums of rows g and g+8 for block t: every lane decodes and applies exactly the absmax values
//    of its own block, no shuffles. absmax = nmap[code] * second_level + offset in two rounded
//    fp32 operations (Bnb4BitLinear.cpp:485-487). The second-level scale of a row changes at most
//    once along the row; a table built with the linear gives, per row, the value before and after
//    that column and the offset (one 16-byte load per row and pair). The second-level code book
//    sits bank-private in the unused half rows of the byte table.
//  * x of an operation sits in shared memory (up to two buffers, so the next operation's x is in
//    place before the consumers get there). A plain tensor is fetched by the finalizer warp with
//    asynchronous copies that arrive on an mbarrier; the previous operation's output, or an input
//    with a fused RMSNorm, is staged by the consumers themselves.
//  * Row sums: a warp reduces over t when it leaves a pair and writes 32 floats to one of its two
//    slots (tagged with the pair). There are four sets of slots, so the consumers run up to four
//    operations ahead of the finalizer, which adds the slots of a pair in slot order. A pair whose
//    items span several CTAs is finished by the CTA that holds its first item: the others publish
//    their partial sums as 8-byte words {value, tag}, which the owner reads (bounded wait) and adds
//    in CTA order. Every sum is added in a fixed order: results do not depend on timing.
//  * Output: bf16 to y and/or, when the next operation consumes it, as 8-byte words
//    {two bf16, tag} that every CTA polls while it stages the next x into shared memory. A word
//    carries its own validity (a naturally aligned 8-byte access is single-copy atomic), so there
//    is no fence and no flag on the path from one operation to the next.
//  * Exchange words (outputs, partial sums) live in eight slots used round-robin by operation.
//    Every CTA leaves a token when it is through with an operation; a slot is written only when
//    all tokens show that its words of eight operations ago have been read.
//  * Tags are epoch + operation index; the epoch lives in device memory and is advanced by the
//    CTA that finishes last, so launches can be captured in a CUDA graph and replayed.
//
// Numerics are those of the streaming kernel in nf4_gemv.cu: code-book values rounded to bf16
// before the product, fp32 accumulation, fp32 absmax, one rounding of the result.
// Roofline: HBM. Algorithmic bytes per weight: 0.5 + 1/64 + 4/16384.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "nf4_internal.h"

namespace nf4 {

namespace {

constexpr int kChainWarps = 16;            // 15 consumer warps and the finalizer warp
constexpr int kChainThreads = kChainWarps * 32;
constexpr int kConsumerWarps = kChainWarps - 1;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kItemsPerWarp = 8;           // work items a consumer warp should get from an operation, at least
constexpr int kMinWarps = 6;               // consumer warps an operation uses, at least
constexpr int kStepUnits = 4;
constexpr int kXBatch = 6;                 // 8-byte chunks of x one thread has in flight
constexpr uint32_t kLutAddr = 65536u;      // shared-window address of the 64 KB table block
constexpr uint32_t kXAddr = 131072u;       // x in fragment order
constexpr int kDescBytes = 256;
constexpr int kChainMaxGrid = 256;         // CTAs a launch may have (one per SM)
constexpr int kChainMaxOps = 160;          // operations of one launch (their descriptors sit in shared memory)

// One operation of a chain as the kernel sees it (kDescBytes each, copied to shared memory).
// Second-level scales of one output row (8-bit absmax codes): the row's blocks use `lo` up to unit
// column `cross` and `hi` from there on (a row of at most 256 blocks changes its second-level
// block at most once); absmax = code_book[code] * scale + offset.
struct RowScales {
    float lo, hi;
    int cross;
    float offset;
};
static_assert(sizeof(RowScales) == 16, "one 16-byte load per row");

struct ChainOpDev {
    const uint8_t* units;
    ScaleParams sp;
    const uint16_t* x_ext;        // bf16 [K], or NULL: the previous operation's output
    uint16_t* y;                  // bf16 [n_out], or NULL
    const uint16_t* residual;     // bf16 [n_out] added before rounding, or NULL
    const uint16_t* norm_add;     // RMSNorm in front of the linear: see NormInput
    const uint16_t* norm_w;
    uint16_t* norm_hidden_out;
    float norm_eps;
    int K, KB;
    int n_warps;                  // consumer warps that share a CTA's slice of this operation
    uint32_t div_w_m;             // x / n_warps as (x * div_w_m) >> div_w_s
    int n_rows, n_tiles;          // rows / row tiles of the linear
    int swiglu;                   // 1: halves are gate and up, output silu(gate) * up
    int pair_offset;              // row-tile distance from half 0 to half 1
    int n_out;                    // outputs (ff for swiglu, else n_rows)
    int total;                    // work items = pairs * KB
    int slice_q, slice_r;         // total = slice_q * grid + slice_r
    uint32_t div_g_m;
    int div_g_s;
    uint32_t div_kb_m;
    int div_kb_s;
    int publish;                  // 1: the next operation reads this output (exchange words)
    const RowScales* row_scales;  // [n_rows], 8-bit absmax codes only
    long long half1_bytes;        // from a unit of half 0 to the same unit of half 1
    int clamp_pair;               // pairs from here on have no half 1 of their own (it reads the last row tile)
    int x_copy;                   // 1: x is a plain, 16-byte aligned tensor that asynchronous copies can fetch
    int div_w_s;
    int peer;                     // 1: the sums go to the row-parallel exchange instead of y
};
static_assert(sizeof(ChainOpDev) == kDescBytes, "descriptor size");

struct ChainParams {
    const ChainOpDev* ops;        // device array of n_ops descriptors (kDescBytes apart), or NULL
    int n_ops;
    const float* qmap;            // [16]
    const float* nmap;            // [256] or NULL
    unsigned long long* xbuf;     // [8][xwords] exchange words {bf16 pair, tag}, slot = tag & 7
    long long xwords;
    unsigned long long* pbuf;     // [8][grid][32] partial sums {f32, tag}, slot = tag & 7
    unsigned long long* tokens;   // [kChainMaxGrid] {0, tag of the last operation whose finalize phase the CTA left}
    unsigned* ctrl;               // {epoch, CTAs done, abort}
    int* status;
    long long spin_limit;         // SM cycles a wait may take
    int smem_bytes;
    int x_buffers;                // 1 or 2 buffers of x_pitch bytes for x in shared memory (2 when they fit)
    int x_pitch;
    // Row-parallel exchange after the LAST operation (peer_world > 0): its fp32 row sums go, as
    // 8-byte words {value, tag = peer epoch + 1}, into every rank's exchange buffer (plain stores
    // to peer memory); then every CTA adds up a share of the rows over the ranks, in rank order.
    int peer_world, peer_rank;
    long long peer_max_rows;
    unsigned long long* peer_part[8];  // rank d's row area (both parities, all source ranks)
    unsigned* peer_ctrl;               // this rank's {epoch, ...}
    uint16_t* peer_y;                  // bf16 [n_out of the last operation]
    const uint16_t* peer_residual;     // added to the sum, or NULL
    ChainOpDev inline_op;         // the operation of a one-operation launch (ops == NULL)
};

extern __shared__ __align__(1024) uint8_t chain_smem[];

__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_u32(uint32_t a, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_v2(uint32_t a, uint2 v) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a), "r"(v.x), "r"(v.y) : "memory");
}
// streaming weight load: read-only path, no L1 allocation, 256-byte L2 prefetch granularity
__device__ __forceinline__ uint2 ldg_stream_v2(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v2.u32 {%0, %1}, [%2];"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}
// streaming load at a constant distance from the pointer (the distance goes into the instruction)
template <int OFF>
__device__ __forceinline__ uint32_t ldg_stream_u32_at(const uint8_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1+%2];" : "=r"(v) : "l"(p), "n"(OFF));
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_16816_init(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Bank-private table lookup: the table block sits on a 64 KB boundary of the shared window; row
// b (256 bytes) holds, for lane l, the bf16 pair of byte value b at b*256 + l*4 and the
// second-level code-book entry b at b*256 + 128 + l*4. ONE PRMT splices the byte into bits
// [8,16) of the lane's base address.
template <int BYTE>
__device__ __forceinline__ uint32_t lut_pair(uint32_t word, uint32_t lane_base) {
    return lds_u32(__byte_perm(word, lane_base, 0x7604 | (BYTE << 4)));
}

// n / d for 0 <= n < 2^31 as (n * m) >> s (s = 31 + ceil(log2 d), m = ceil(2^s / d))
__host__ __device__ __forceinline__ int fast_div(int n, uint32_t m, int s) {
    return (int)(((unsigned long long)(unsigned)n * m) >> s);
}
void make_fast_div(uint32_t d, uint32_t* m, int* s) {
    int l = 0;
    while ((1ull << l) < d) ++l;
    *s = 31 + l;
    *m = (uint32_t)(((1ull << *s) + d - 1) / d);
}

// First work item of CTA c: floor(total * c / grid) in 32-bit arithmetic, with total = q*grid + r.
__device__ __forceinline__ int slice_begin(const ChainOpDev& op, int c) {
    return op.slice_q * c + fast_div(op.slice_r * c, op.div_g_m, op.div_g_s);
}

constexpr long long kTightLimit = 4096;  // wait limits below this are checked on every polling round

// Waits until the word carries `tag` (exact match) or, with at_least, a tag not older than it.
// Gives up after `limit` SM cycles or when another thread of the grid has given up.
__device__ __forceinline__ bool poll_word(const unsigned long long* w, unsigned tag, bool at_least,
                                          long long limit, const unsigned* g_abort,
                                          unsigned long long& out) {
    unsigned long long q = ld_relaxed_u64(w);
    auto hit = [&](unsigned long long v) {
        const unsigned got = (unsigned)(v >> 32);
        return at_least ? ((int)(got - tag) >= 0) : (got == tag);
    };
    if (hit(q)) {
        out = q;
        return true;
    }
    const long long t0 = clock64();
    unsigned it = 0;
    while (true) {
        q = ld_relaxed_u64(w);
        if (hit(q)) {
            out = q;
            return true;
        }
        // (the clock is read every 16th round; a limit below kTightLimit is looked at every round)
        if ((++it & 15u) == 0u || limit < kTightLimit) {
            if (clock64() - t0 > limit || *(volatile const unsigned*)g_abort != 0u) return false;
            __nanosleep(64);
        }
    }
}

// named barriers (0 is __syncthreads)
constexpr int kRing = 4;                   // operations whose slots exist at once in shared memory
constexpr int kBarConsumers = 1;           // the consumer warps among themselves
constexpr int kBarDone = 2;                // + oi % kRing: consumers arrive when an operation's sums are in the slots
constexpr int kBarGo = kBarDone + kRing;   // + oi % kRing: the finalizer arrives when these slots may be reused
constexpr int kXBlockPitch = 160;          // bytes from one 64-element block of x to the next in shared memory
__device__ __forceinline__ void bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// KIND: how the absmax values are stored in the unit stream (the same for every operation of a
// launch): it fixes the distance between units, so every weight load is base + constant.
template <int KIND>
__global__ void __launch_bounds__(kChainThreads, 1) gemv_chain_kernel(const ChainParams p) {
    constexpr int ST = KIND == kAbsmaxCodes ? kUnitStrideCodes : kUnitStrideF32;
    constexpr bool codes = KIND == kAbsmaxCodes;
    const uint32_t base = smem_u32(chain_smem);
    uint8_t* gen = chain_smem - base;  // generic pointer to shared-window address 0
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int G = gridDim.x;
    const int c = blockIdx.x;

    // ---- shared-memory map (absolute shared-window addresses) ----
    // [base, 64 KB): control words, pair table, second-level table, warp slots, descriptors;
    // [64 KB, 128 KB): bank-private lookup tables; [128 KB, ...): x in fragment order, one or two
    // buffers of x_pitch bytes
    const uint32_t a_ctl = (base + 15u) & ~15u;    // +0 abort flag, +64 [16] warp sums of the RMSNorm
    const uint32_t a_ptab = a_ctl + 128;           // [256] byte value -> bf16 pair
    const uint32_t a_nmap = a_ptab + 1024;         // [256] second-level code book
    const uint32_t a_slots = a_nmap + 1024;        // [kRing][warp][2][32] floats
    const uint32_t a_seg = a_slots + kRing * kChainWarps * 2 * 32 * 4;  // [kRing][warp][2] pair whose sums the slot holds, or -1
    const uint32_t a_xbar = a_seg + kRing * kChainWarps * 2 * 4;        // [2] mbarriers: x buffer granted / filled
    const uint32_t a_rflag = a_xbar + 16;               // [8] tag of the operation that may write exchange slot tag & 7
    const uint32_t a_slice = a_rflag + 32;              // [n_ops] first work item of this CTA and of the next one
    const uint32_t a_desc = a_slice + 8u * kChainMaxOps;
    const int n_ops = p.n_ops;
    const int xbufs = p.x_buffers;
    if (base > 2048u || a_desc + (uint32_t)n_ops * kDescBytes > kLutAddr ||
        base + (uint32_t)p.smem_bytes < kXAddr + (uint32_t)p.x_buffers * (uint32_t)p.x_pitch || G > kChainMaxGrid) {
        if (tid == 0) atomicExch(p.status, kStatusBadArgument);
        return;  // every CTA takes this exit
    }
    int* abort_flag = reinterpret_cast<int*>(gen + a_ctl);
    const unsigned* g_abort = p.ctrl + 2;

    // ---- prologue: tables and descriptors ----
    {
        float q_hi = 0.0f, q_lo = 0.0f, nm = 0.0f;
        if (tid < 256) {
            q_hi = __ldg(p.qmap + (tid >> 4));
            q_lo = __ldg(p.qmap + (tid & 15));
            if (p.nmap) nm = __ldg(p.nmap + tid);
        }
        if (p.ops) {
            const uint4* src = reinterpret_cast<const uint4*>(p.ops);
            for (int i = tid; i < n_ops * (kDescBytes / 16); i += kChainThreads) {
                const uint4 v = __ldg(src + i);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a_desc + 16u * i), "r"(v.x),
                             "r"(v.y), "r"(v.z), "r"(v.w)
                             : "memory");
            }
        } else if (tid == 0) {
            *reinterpret_cast<ChainOpDev*>(gen + a_desc) = p.inline_op;
        }
        if (tid < 256) {
            // low half = first weight (HIGH nibble)
            sts_u32(a_ptab + 4u * tid,
                    (uint32_t)f32_to_bf16_bits(q_hi) | ((uint32_t)f32_to_bf16_bits(q_lo) << 16));
            sts_f32(a_nmap + 4u * tid, nm);
        }
        if (tid < 8) sts_u32(a_rflag + 4u * tid, 0u);
        if (tid == 0) {
            *abort_flag = 0;
            mbar_init(reinterpret_cast<uint64_t*>(gen + a_xbar), 32);  // every lane of the granting warp arrives
            mbar_init(reinterpret_cast<uint64_t*>(gen + a_xbar + 8), 32);
            mbar_fence_init();
        }
        __syncthreads();
        // Table rows are 256 bytes: [0,128) the pair, [128,256) the second-level entry, one word
        // per lane. One 16-byte store per lane fills a quarter of a half row.
#pragma unroll
        for (int bq = warp; bq < 64; bq += kChainWarps) {
            const int b = bq * 4 + (lane >> 3);
            const uint32_t pv = lds_u32(a_ptab + 4u * b);
            const uint32_t nv = lds_u32(a_nmap + 4u * b);
            const uint32_t row = kLutAddr + (uint32_t)b * 256u + (uint32_t)(lane & 7) * 16u;
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(row), "r"(pv) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(row + 128u), "r"(nv) : "memory");
        }
    }
    for (int oj = tid; oj < n_ops; oj += kChainThreads) {
        const ChainOpDev& o = *reinterpret_cast<const ChainOpDev*>(gen + a_desc + (uint32_t)oj * kDescBytes);
        sts_u32(a_slice + 8u * oj, (uint32_t)slice_begin(o, c));
        sts_u32(a_slice + 8u * oj + 4u, (uint32_t)slice_begin(o, c + 1));
    }
    const unsigned epoch0 = *(volatile unsigned*)p.ctrl;
    __syncthreads();

    auto desc = [&](int oj) -> const ChainOpDev& {
        return *reinterpret_cast<const ChainOpDev*>(gen + a_desc + (uint32_t)oj * kDescBytes);
    };
    auto tag_of = [&](int oj) { return epoch0 + (unsigned)oj + 1u; };
    // work items [i0, i1) of this CTA in operation oj
    auto my_slice = [&](int oj, int& i0, int& i1) {
        uint32_t lo, hi;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(a_slice + 8u * (uint32_t)oj));
        i0 = (int)lo;
        i1 = (int)hi;
    };
    auto give_up = [&](int code) {
        atomicExch(p.status, code);
        atomicExch(p.ctrl + 2, 1u);
        *(volatile int*)abort_flag = 1;
    };
    auto is_aborted = [&]() { return *(volatile int*)abort_flag != 0; };
    // x of operation oj lives in buffer oj % xbufs, in natural order with a padded pitch per
    // 64-element block (the four blocks of a step then sit in different banks): element k at
    // (k / 64) * kXBlockPitch + (k % 64) * 2
    auto x_buf = [&](int oj) { return xbufs == 2 ? (oj & 1) : 0; };
    auto x_addr = [&](int oj) { return kXAddr + (uint32_t)x_buf(oj) * (uint32_t)p.x_pitch; };
    auto chunk_off = [&](int q4) {  // 8-byte chunk q4 = k / 4
        return (uint32_t)((q4 >> 4) * kXBlockPitch + (q4 & 15) * 8);
    };
    // An operation whose input is its own plain tensor gets it copied into the x buffer by the
    // copy engine (one bulk copy per block), with no work for the consumers (x_ext is stable:
    // operations of a chain never read through a pointer what an earlier one writes).
    auto prestaged = [&](int oj) { return desc(oj).x_copy != 0; };
    auto x_phase = [&](int oj) { return (uint32_t)((xbufs == 2 ? (oj >> 1) : oj) & 1); };
    auto x_bar = [&](int oj) { return reinterpret_cast<uint64_t*>(gen + a_xbar + 8u * (uint32_t)x_buf(oj)); };
    // The x buffer of operation oj is free (every consumer is through with its previous user):
    // fill it if the input can be copied, and tell the consumers. Called by one warp.
    auto x_grant = [&](int oj, bool skip_copy) {
        const uint32_t bar = a_xbar + 8u * (uint32_t)x_buf(oj);
        if (!skip_copy && prestaged(oj)) {
            const ChainOpDev& o = desc(oj);
            const uint8_t* xg = reinterpret_cast<const uint8_t*>(o.x_ext);
            const uint32_t xa = x_addr(oj);
            const int n16 = o.K >> 3;  // 16-byte pieces of eight elements
            for (int q = lane; q < n16; q += 32)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(xa + (uint32_t)((q >> 3) * kXBlockPitch + (q & 7) * 16)),
                             "l"(xg + 16 * (size_t)q)
                             : "memory");
            // arrives once this lane's copies have landed
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
        } else {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
        }
    };
    auto x_wait = [&](int oj) {  // false: the wait ran out
        uint64_t* bar = x_bar(oj);
        const uint32_t ph = x_phase(oj);
        if (mbar_try_wait(bar, ph)) return true;
        const long long t0 = clock64();
        for (unsigned it = 0;; ++it) {
            if (mbar_try_wait(bar, ph)) return true;
            if (((it & 63u) == 63u || p.spin_limit < kTightLimit) && (clock64() - t0 > p.spin_limit || is_aborted()))
                return false;
            __nanosleep(32);
        }
    };

    // row-parallel exchange: this launch's tag and half of the buffers
    const unsigned peer_epoch = p.peer_world > 0 ? *(volatile unsigned*)p.peer_ctrl : 0u;
    auto peer_store = [&](int n, bool valid, float sum) {
        const size_t at = ((size_t)(peer_epoch & 1u) * p.peer_world + p.peer_rank) * (size_t)p.peer_max_rows + n;
        const unsigned long long word =
            ((unsigned long long)(peer_epoch + 1u) << 32) | (unsigned long long)__float_as_uint(sum);
        if (valid)
            for (int d = 0; d < p.peer_world; ++d)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.peer_part[d] + at), "l"(word) : "memory");
    };

    // ---- the output of one pair of operation o: lane = half * 16 + row holds the finished sum ----
    auto epilogue = [&](const ChainOpDev& o, unsigned tg, int pr, float v) {
        const int row = lane & 15;
        const bool hl = lane < 16;
        int n;
        bool valid;
        float out;
        if (o.swiglu) {
            const float up = __shfl_down_sync(0xffffffffu, v, 16);
            n = pr * kTileRows + row;
            valid = hl && n < o.n_out;
            out = __fdividef(v, 1.0f + __expf(-v)) * up;
        } else {
            const int tile = pr + (hl ? 0 : o.pair_offset);
            n = tile * kTileRows + row;
            valid = tile < o.n_tiles && n < o.n_out;
            out = v;
            if (valid && o.residual) out += bf16_bits_to_f32(__ldcg(o.residual + n));
        }
        if (o.peer) {
            peer_store(n, valid, out);
            return;
        }
        const uint32_t bits = f32_to_bf16_bits(out);
        if (valid && o.y) o.y[n] = (uint16_t)bits;
        if (o.publish) {
            const uint32_t hi = __shfl_down_sync(0xffffffffu, bits, 1);
            if (valid && !(row & 1))
                st_relaxed_u64(p.xbuf + (size_t)(tg & 7u) * (size_t)p.xwords + (n >> 1),
                               ((unsigned long long)tg << 32) | (unsigned long long)(bits | (hi << 16)));
        }
    };
    // Exchange slots (x words, partial sums) are used round-robin over eight operations. Before a
    // warp writes slot tag & 7 every CTA must have left the finalize phase of the operation seven
    // back (it has then read all words of the one eight back). Tokens only grow. The finalizer
    // warp checks ahead of time and leaves the operation's tag in a shared-memory flag; a warp
    // that does not find it there reads the tokens itself.
    auto ring_ok = [&](int oj) {
        if (oj < 7) return true;
        if (lds_u32(a_rflag + 4u * (uint32_t)(oj & 7)) == tag_of(oj)) return true;
        const unsigned need = tag_of(oj) - 7u;
        unsigned long long tk[kChainMaxGrid / 32];
#pragma unroll
        for (int i = 0; i < kChainMaxGrid / 32; ++i) {
            tk[i] = (unsigned long long)need << 32;
            if (lane + 32 * i < G) tk[i] = ld_relaxed_u64(p.tokens + lane + 32 * i);
        }
        bool fine = true;
#pragma unroll
        for (int i = 0; i < kChainMaxGrid / 32; ++i)
            if ((int)((unsigned)(tk[i] >> 32) - need) < 0)
                if (!poll_word(p.tokens + lane + 32 * i, need, true, p.spin_limit, g_abort, tk[i])) fine = false;
        return __all_sync(0xffffffffu, fine) != 0;
    };
    // first item of consumer warp w in a slice of len items from i0: i0 + len * w / n_warps
    auto warp_begin = [&](const ChainOpDev& o, int i0, int len, int w) {
        return i0 + fast_div(len * min(w, o.n_warps), o.div_w_m, o.div_w_s);
    };

    if (warp == kConsumerWarps) {
        // =====================================================================================
        // finalizer warp: finishes the pairs of each operation while the consumers run ahead
        // =====================================================================================
        for (int oj = 0; oj < min(xbufs, n_ops); ++oj) x_grant(oj, false);  // the first buffers are free
        int flag_next = 7;  // first operation whose exchange slot has not been cleared for writing yet
        for (int oi = 0; oi < n_ops; ++oi) {
            const ChainOpDev& op = desc(oi);
            const unsigned tag = tag_of(oi);
            const int r = oi & (kRing - 1);
            // exchange slots that may be written by now: operation oj needs every token >= tag(oj) - 7
            if (flag_next < n_ops && flag_next <= oi + 3) {
                int behind = 0x7fffffff;  // tokens relative to the first operation of this launch
                unsigned long long tk[kChainMaxGrid / 32];  // (all loads in flight together)
#pragma unroll
                for (int i = 0; i < kChainMaxGrid / 32; ++i) {
                    tk[i] = ~0ull >> 1;
                    if (lane + 32 * i < G) tk[i] = ld_relaxed_u64(p.tokens + lane + 32 * i);
                }
#pragma unroll
                for (int i = 0; i < kChainMaxGrid / 32; ++i)
                    if (lane + 32 * i < G) behind = min(behind, (int)((unsigned)(tk[i] >> 32) - tag_of(0)));
#pragma unroll
                for (int sh = 16; sh > 0; sh >>= 1) behind = min(behind, __shfl_xor_sync(0xffffffffu, behind, sh));
                while (flag_next < n_ops && behind >= flag_next - 7) {
                    if (lane == 0) sts_u32(a_rflag + 4u * (uint32_t)(flag_next & 7), tag_of(flag_next));
                    ++flag_next;
                }
            }
            bar_sync(kBarDone + r, kChainThreads);
            const bool aborted = is_aborted();
            // every consumer is through with operation oi: its x buffer goes to operation oi + xbufs
            if (oi + xbufs < n_ops) x_grant(oi + xbufs, aborted);
            // Add up the consumers' slots pair by pair, in slot order (warp 0 slot 0, warp 0 slot 1,
            // warp 1 slot 0, ...; the pairs in them never decrease), and finish every pair.
            int i0, i1;
            my_slice(oi, i0, i1);
            if (!aborted && i1 > i0) {
                const int KB = op.KB;
                const uint32_t slots = a_slots + (uint32_t)r * (kChainWarps * 256u);
                const uint32_t segs = a_seg + (uint32_t)r * (kChainWarps * 8u);
                constexpr int NQ = kConsumerWarps * 2;
                // lane q holds the tag of slot q: which slots hold sums, and which of them start a pair
                // (the valid tags never decrease)
                const int tq = lane < NQ ? (int)lds_u32(segs + 4u * (uint32_t)lane) : -1;
                const unsigned valid = __ballot_sync(0xffffffffu, tq >= 0);
                unsigned first;
                {
                    const unsigned before = valid & ((1u << lane) - 1u);
                    const int prev = 31 - __clz((int)before);  // the valid slot before this one, or -1
                    const int ptag = __shfl_sync(0xffffffffu, tq, prev & 31);
                    first = __ballot_sync(0xffffffffu, tq >= 0 && (before == 0u || ptag != tq));
                }
                // what the epilogue needs, read from the descriptor once
                const int e_swiglu = op.swiglu, e_n_out = op.n_out, e_pair_offset = op.pair_offset;
                const int e_n_tiles = op.n_tiles, e_publish = op.publish, e_peer = op.peer;
                uint16_t* const e_y = op.y;
                const uint16_t* const e_res = op.residual;
                unsigned long long* const e_xw = p.xbuf + (size_t)(tag & 7u) * (size_t)p.xwords;
                const int row = lane & 15;
                const bool hl = lane < 16;
                auto finish = [&](int pr, float val) {
                    int n;
                    bool ok_row;
                    float out;
                    if (e_swiglu) {
                        const float up = __shfl_down_sync(0xffffffffu, val, 16);
                        n = pr * kTileRows + row;
                        ok_row = hl && n < e_n_out;
                        out = __fdividef(val, 1.0f + __expf(-val)) * up;
                    } else {
                        const int tile = pr + (hl ? 0 : e_pair_offset);
                        n = tile * kTileRows + row;
                        ok_row = tile < e_n_tiles && n < e_n_out;
                        out = val;
                        if (ok_row && e_res) out += bf16_bits_to_f32(__ldcg(e_res + n));
                    }
                    if (e_peer) {
                        peer_store(n, ok_row, out);
                        return;
                    }
                    const uint32_t bits = f32_to_bf16_bits(out);
                    if (ok_row && e_y) e_y[n] = (uint16_t)bits;
                    if (e_publish) {
                        const uint32_t hi16 = __shfl_down_sync(0xffffffffu, bits, 1);
                        if (ok_row && !(row & 1))
                            st_relaxed_u64(e_xw + (n >> 1),
                                           ((unsigned long long)tag << 32) | (unsigned long long)(bits | (hi16 << 16)));
                    }
                };
                // The sums of the pair whose first slot is the lowest bit of `rest`, added in slot order
                // (eight independent loads at a time); takes that pair out of `rest`.
                auto gather = [&](unsigned& rest, int& pr, float& sum) {
                    const int q0 = __ffs((int)rest) - 1;
                    rest &= rest - 1u;
                    const unsigned upto = rest != 0u ? ((1u << (__ffs((int)rest) - 1)) - 1u) : 0xffffffffu;
                    unsigned run = (valid & upto) >> q0;  // bit 0 is set
                    pr = __shfl_sync(0xffffffffu, tq, q0);
                    uint32_t at = slots + (uint32_t)q0 * 128u + 4u * lane;
                    sum = 0.0f;
                    do {
                        float part[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            part[k] = 0.0f;
                            if (run & (1u << k)) part[k] = lds_f32(at + 128u * k);
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k) sum += part[k];  // (absent slots add +0)
                        run >>= 8;
                        at += 1024u;
                    } while (run != 0u);
                };
                int checked = 0;  // 1: the exchange slots of this operation may be written
                int pr_next = 0;
                float sum_next = 0.0f;
                bool more = first != 0u;
                if (more) gather(first, pr_next, sum_next);
                while (more && checked >= 0) {
                    const int pr = pr_next;
                    float sum = sum_next;
                    more = first != 0u;
                    if (more) gather(first, pr_next, sum_next);  // (its loads overlap this pair's epilogue)
                    const int t0 = pr * KB, t1 = t0 + KB;
                    const int lo = max(i0, t0), hi = min(i1, t1);
                    const bool writes_ring = e_publish || hi - lo != KB;
                    if (writes_ring && checked == 0) checked = ring_ok(oi) ? 1 : -1;
                    if (writes_ring && checked < 0) break;
                    if (hi - lo == KB) {
                        finish(pr, sum);
                    } else if (lo == t0) {
                        // this CTA holds the pair's first item: add the later CTAs' sums in CTA order
                        int cover = hi - lo;
                        bool got = true;
                        for (int cc = c + 1; cc < G && cover < KB && got; ++cc) {
                            const int j0 = slice_begin(op, cc), j1 = slice_begin(op, cc + 1);
                            const int s1 = min(j1, t1);
                            if (s1 <= j0) continue;
                            unsigned long long q;
                            got = poll_word(p.pbuf + ((size_t)(tag & 7u) * G + cc) * 32 + lane, tag, false,
                                            p.spin_limit, g_abort, q);
                            sum += __uint_as_float((unsigned)q);
                            cover += s1 - j0;
                        }
                        if (__all_sync(0xffffffffu, got))
                            finish(pr, sum);
                        else
                            checked = -1;
                    } else {
                        st_relaxed_u64(p.pbuf + ((size_t)(tag & 7u) * G + c) * 32 + lane,
                                       ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(sum));
                    }
                }
                if (checked < 0 && lane == 0) give_up(kStatusTimeoutFull);
            }
            // this CTA has left the finalize phase of operation oi
            __syncwarp();
            if (lane == 0) st_relaxed_u64(p.tokens + c, (unsigned long long)tag << 32);
            // the slots of this ring position are free for operation oi + kRing
            if (oi + kRing < n_ops) bar_arrive(kBarGo + r, kChainThreads);
        }
        // ---- row-parallel exchange: this CTA's share of the rows, summed over the ranks ----
        if (p.peer_world > 0 && !is_aborted()) {
            const int n_out = desc(n_ops - 1).n_out;
            const int per = (n_out + G - 1) / G;
            const int r0 = c * per, r1 = min(n_out, r0 + per);
            const unsigned long long* part =
                p.peer_part[p.peer_rank] + (size_t)(peer_epoch & 1u) * p.peer_world * (size_t)p.peer_max_rows;
            bool ok = true;
            for (int row = r0 + lane; row < r1 && ok; row += 32) {
                float acc = 0.0f;
                for (int src = 0; src < p.peer_world && ok; ++src) {
                    const unsigned long long* word = part + (size_t)src * (size_t)p.peer_max_rows + row;
                    unsigned long long q;
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(q) : "l"(word) : "memory");
                    if ((unsigned)(q >> 32) != peer_epoch + 1u) {
                        const long long t0 = clock64();
                        do {
                            __nanosleep(40);
                            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(q) : "l"(word) : "memory");
                            if (clock64() - t0 > p.spin_limit || *(volatile const unsigned*)g_abort != 0u) {
                                ok = false;
                                break;
                            }
                        } while ((unsigned)(q >> 32) != peer_epoch + 1u);
                    }
                    acc += __uint_as_float((unsigned)q);
                }
                if (ok) {
                    if (p.peer_residual) acc += bf16_bits_to_f32(p.peer_residual[row]);
                    p.peer_y[row] = f32_to_bf16_bits(acc);
                }
            }
            if (!ok) {
                atomicExch(p.status, kStatusTimeoutPeer);
                atomicExch(p.ctrl + 2, 1u);
            }
        }
        // ---- the CTA that finishes last advances the epoch (every CTA has read it by then) ----
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            const unsigned done = atomicAdd(p.ctrl + 1, 1u);
            if (done == (unsigned)G - 1u) {
                p.ctrl[1] = 0u;
                __threadfence();
                *(volatile unsigned*)p.ctrl = epoch0 + (unsigned)n_ops;
                if (p.peer_world > 0) *(volatile unsigned*)p.peer_ctrl = peer_epoch + 1u;
            }
        }
        return;
    }

    // =========================================================================================
    // consumer warps
    // =========================================================================================
    const int ctid = tid;  // 0 .. kConsumerThreads - 1
    const int g = lane >> 2;  // row inside the tile (and row + 8)
    const int t = lane & 3;   // block of the step this lane scales
    const uint32_t lane_base = kLutAddr + ((uint32_t)lane << 2);
    const uint32_t nmap_base = lane_base + 128u;
    const uint32_t lane_off = (uint32_t)(g * 32 + 8 * t);
    // lanes g = 0, 2, 4, 6 carry the x slice of block 0..3 of a step in the B fragment
    const bool x_lane = (g & 1) == 0;
    const int x_unit = g >> 1;

    // ---- per-warp pipeline state; it crosses operation boundaries ----
    uint2 W[2][kStepUnits][2];   // packed weights of the step about to run (loads in flight)
    uint32_t raw[2][2];          // absmax codes (or fp32 absmax) of this lane's block of that step
    float slo[2][2], shi[2][2];  // second-level scales of those rows: before / from column scross
    int scross[2][2];
    float rowoff[2][2];
    int prep_op = -1, prep_pair = -1;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            raw[h][r] = 0u;
            slo[h][r] = shi[h][r] = 0.0f;
            scross[h][r] = 0;
            rowoff[h][r] = 0.0f;
#pragma unroll
            for (int u = 0; u < kStepUnits; ++u) W[h][u][r] = make_uint2(0u, 0u);
        }
    // the step about to run: items [pos, pos + n) of this warp's range [.., w1), pair / first block,
    // where each half's units start (this lane's bytes), distance between units
    int pos = 0, w1 = 0, pair = 0, kb0 = 0, n = 0;
    const uint8_t* ph0 = nullptr;
    const uint8_t* ph1 = nullptr;
    bool loaded = false;  // W / raw / sc already hold the first step of the operation that starts next
    int next_n = 0;       // ... and that step has this many units

    auto half_ptr = [&](const ChainOpDev& o, int h, int pr, int kb) {
        const int tile = min(pr + h * o.pair_offset, o.n_tiles - 1);
        return o.units + ((size_t)tile * o.KB + kb) * (size_t)ST + lane_off;
    };
    auto load_half = [&](int h, int u, const uint8_t* q) {
        W[h][u][0] = ldg_stream_v2(q + u * ST);
        W[h][u][1] = ldg_stream_v2(q + u * ST + 256);
    };
    // Scale inputs of a step, fetched one step ahead: the absmax codes (or fp32 absmax) of this
    // lane's block t, rows g and g+8 of both halves, and for codes the second-level scale
    // nabs[flat / 256] of each; rowflat / rowoff follow the step's pair.
    // (this lane's block t of a step: its absmax entries sit scale_off bytes after the pointer the
    // weight loads use)
    const int scale_off = t * ST + kUnitNibbleBytes - (int)lane_off + (codes ? (g >> 2) * 4 : 4 * g);
    const uint32_t code_sel = 0x7604u | ((uint32_t)(g & 3) << 4);  // PRMT: byte g % 4 of a code word into bits [8,16)
    auto prepare_scales = [&](const ChainOpDev& o, int oj, int pr, int kb, int nn, const uint8_t* q0,
                              const uint8_t* q1) {
        if (codes && (pr != prep_pair || oj != prep_op)) {
            prep_pair = pr;
            prep_op = oj;
            const float4* table = reinterpret_cast<const float4*>(o.row_scales);
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int tile = min(pr + h * o.pair_offset, o.n_tiles - 1);
                    const int row = min(tile * kTileRows + g + 8 * r, o.n_rows - 1);
                    const float4 e = __ldg(table + row);
                    slo[h][r] = e.x;
                    shi[h][r] = e.y;
                    scross[h][r] = __float_as_int(e.z);
                    rowoff[h][r] = e.w;
                }
        }
        if (t < nn) {
            if (codes) {
                // the four-byte words that hold the codes of rows g and g + 8
                raw[0][0] = ldg_stream_u32_at<0>(q0 + scale_off);
                raw[0][1] = ldg_stream_u32_at<8>(q0 + scale_off);
                raw[1][0] = ldg_stream_u32_at<0>(q1 + scale_off);
                raw[1][1] = ldg_stream_u32_at<8>(q1 + scale_off);
            } else {
                raw[0][0] = ldg_stream_u32_at<0>(q0 + scale_off);
                raw[0][1] = ldg_stream_u32_at<32>(q0 + scale_off);
                raw[1][0] = ldg_stream_u32_at<0>(q1 + scale_off);
                raw[1][1] = ldg_stream_u32_at<32>(q1 + scale_off);
            }
        }
    };
    // first step of this warp in operation o (arithmetic only)
    struct First {
        int pos, w1, pair, kb0, n;
        const uint8_t* p0;
        const uint8_t* p1;
    };
    auto first_step = [&](const ChainOpDev& o, int oj) {
        First f;
        int i0, i1;
        my_slice(oj, i0, i1);
        f.pos = warp_begin(o, i0, i1 - i0, warp);
        f.w1 = warp_begin(o, i0, i1 - i0, warp + 1);
        f.pair = 0;
        f.kb0 = 0;
        f.n = 0;
        f.p0 = f.p1 = o.units;
        if (f.pos < f.w1) {
            f.pair = fast_div(f.pos, o.div_kb_m, o.div_kb_s);
            f.kb0 = f.pos - f.pair * o.KB;
            f.n = min(min(kStepUnits, f.w1 - f.pos), o.KB - f.kb0);
            // (half 0: the unit of work item i is unit i of the stream)
            f.p0 = o.units + (size_t)f.pos * (size_t)ST + lane_off;
            f.p1 = f.pair < o.clamp_pair ? f.p0 + o.half1_bytes : half_ptr(o, 1, f.pair, f.kb0);
        }
        return f;
    };
    auto issue_first = [&](const ChainOpDev& o, int oj) {  // this warp's first step of operation oj
        const First f = first_step(o, oj);
        pos = f.pos; w1 = f.w1; pair = f.pair; kb0 = f.kb0; n = f.n; ph0 = f.p0; ph1 = f.p1;
        if (n > 0) {
#pragma unroll
            for (int u = 0; u < kStepUnits; ++u)
                if (u < n) {
                    load_half(0, u, ph0);
                    load_half(1, u, ph1);
                }
            prepare_scales(o, oj, pair, kb0, n, ph0, ph1);
        }
    };

    // ---- the consumers stage x of operation oj themselves (linked input, RMSNorm, one x buffer) ----
    // With skip (a wait ran out somewhere) nothing is read, but the barrier count stays the same.
    auto stage_x = [&](int oj, bool skip) {  // returns false when a wait ran out
        const ChainOpDev& o = desc(oj);
        const unsigned tg = tag_of(oj);
        bool ok = true;
        int j0, j1;
        my_slice(oj, j0, j1);
        const int len = j1 - j0;
        // CTA 0 stages x even without work when it has the residual stream to write
        const bool stage = !skip && (len > 0 || (c == 0 && o.norm_w != nullptr && o.norm_hidden_out != nullptr));
        const uint32_t xa = x_addr(oj);
        if (stage) {
            const int n8 = o.K >> 2;  // 8-byte chunks of four elements
            const unsigned want = tg - 1u;  // the previous operation's words
            const unsigned long long* xw = p.xbuf + (size_t)(want & 7u) * (size_t)p.xwords;
            const uint2* xg = reinterpret_cast<const uint2*>(o.x_ext);
            // fetches up to kXBatch chunks of this thread, all loads issued before the first wait
            auto fetch = [&](int q_first, uint2 (&xv)[kXBatch]) {
                if (xg) {
#pragma unroll
                    for (int b = 0; b < kXBatch; ++b) {
                        const int q4 = q_first + b * kConsumerThreads;
                        xv[b] = make_uint2(0u, 0u);
                        if (q4 < n8) xv[b] = __ldcg(xg + q4);
                    }
                } else {
                    // every word that does not carry the tag yet is read again, all of them in one
                    // go (one round trip per round, not per word), until the batch is complete
                    unsigned long long wq[kXBatch][2];
#pragma unroll
                    for (int b = 0; b < kXBatch; ++b) {
                        const int q4 = q_first + b * kConsumerThreads;
                        wq[b][0] = wq[b][1] = (unsigned long long)want << 32;
                        if (q4 < n8) {
                            wq[b][0] = ld_relaxed_u64(xw + 2 * q4);
                            wq[b][1] = ld_relaxed_u64(xw + 2 * q4 + 1);
                        }
                    }
                    long long t_start = 0;
                    for (unsigned round = 0; ok; ++round) {
                        bool all = true;
#pragma unroll
                        for (int b = 0; b < kXBatch; ++b)
                            all = all && (unsigned)(wq[b][0] >> 32) == want && (unsigned)(wq[b][1] >> 32) == want;
                        if (all) break;
                        if (round == 0) t_start = clock64();
                        if (((round & 7u) == 7u || p.spin_limit < kTightLimit) &&
                            (clock64() - t_start > p.spin_limit || *(volatile const unsigned*)g_abort != 0u)) {
                            ok = false;
                            break;
                        }
                        __nanosleep(20);
#pragma unroll
                        for (int b = 0; b < kXBatch; ++b) {
                            const int q4 = q_first + b * kConsumerThreads;
                            if ((unsigned)(wq[b][0] >> 32) != want) wq[b][0] = ld_relaxed_u64(xw + 2 * q4);
                            if ((unsigned)(wq[b][1] >> 32) != want) wq[b][1] = ld_relaxed_u64(xw + 2 * q4 + 1);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < kXBatch; ++b) xv[b] = make_uint2((uint32_t)wq[b][0], (uint32_t)wq[b][1]);
                }
            };
            if (o.norm_w == nullptr) {
                for (int q0 = ctid; q0 < n8; q0 += kConsumerThreads * kXBatch) {
                    uint2 xv[kXBatch];
                    fetch(q0, xv);
#pragma unroll
                    for (int b = 0; b < kXBatch; ++b) {
                        const int q4 = q0 + b * kConsumerThreads;
                        if (q4 < n8) sts_v2(xa + chunk_off(q4), xv[b]);
                    }
                }
            } else {
                // ---- residual add + RMSNorm while staging x (K <= 4 * kXBatch * consumer threads) ----
                // v = x + add in fp32; input = bf16(v * rsqrt(mean(v^2) + eps) * w); CTA 0 writes
                // bf16(v) to hidden_out. The same fixed reduction order in every CTA.
                const uint2* ag = reinterpret_cast<const uint2*>(o.norm_add);
                const uint2* wg = reinterpret_cast<const uint2*>(o.norm_w);
                uint2 xv[kXBatch];
                fetch(ctid, xv);
                float ss = 0.0f;
                float vv[kXBatch][4];
#pragma unroll
                for (int b = 0; b < kXBatch; ++b) {
                    const int q4 = ctid + b * kConsumerThreads;
                    uint2 ad = make_uint2(0u, 0u);
                    if (ag && q4 < n8) ad = __ldcg(ag + q4);
                    vv[b][0] = __uint_as_float(xv[b].x << 16) + __uint_as_float(ad.x << 16);
                    vv[b][1] = __uint_as_float(xv[b].x & 0xffff0000u) + __uint_as_float(ad.x & 0xffff0000u);
                    vv[b][2] = __uint_as_float(xv[b].y << 16) + __uint_as_float(ad.y << 16);
                    vv[b][3] = __uint_as_float(xv[b].y & 0xffff0000u) + __uint_as_float(ad.y & 0xffff0000u);
                    if (q4 < n8)
                        ss += vv[b][0] * vv[b][0] + vv[b][1] * vv[b][1] + vv[b][2] * vv[b][2] + vv[b][3] * vv[b][3];
                }
#pragma unroll
                for (int sh = 16; sh > 0; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
                if (lane == 0) sts_f32(a_ctl + 64u + 4u * warp, ss);
                bar_sync(kBarConsumers, kConsumerThreads);
                float total = 0.0f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) total += lds_f32(a_ctl + 64u + 4u * w);
                const float inv_rms = rsqrtf(total / (float)o.K + o.norm_eps);
                const bool renorm_from_stored = ag != nullptr && o.K != 1024;
#pragma unroll
                for (int b = 0; b < kXBatch; ++b) {
                    const int q4 = ctid + b * kConsumerThreads;
                    if (q4 < n8) {
                        const uint2 wq = __ldg(wg + q4);
                        const float w0f = __uint_as_float(wq.x << 16), w1f = __uint_as_float(wq.x & 0xffff0000u);
                        const float w2f = __uint_as_float(wq.y << 16), w3f = __uint_as_float(wq.y & 0xffff0000u);
                        uint2 hq;  // the updated residual stream bf16(v)
                        hq.x = (uint32_t)f32_to_bf16_bits(vv[b][0]) | ((uint32_t)f32_to_bf16_bits(vv[b][1]) << 16);
                        hq.y = (uint32_t)f32_to_bf16_bits(vv[b][2]) | ((uint32_t)f32_to_bf16_bits(vv[b][3]) << 16);
                        // the reference's single-row add+RMSNorm normalises what it stored (bf16) unless
                        // H == 1024 (src/ops/NormOps.cpp:189-240 against :152-187)
                        const float n0 = renorm_from_stored ? __uint_as_float(hq.x << 16) : vv[b][0];
                        const float n1 = renorm_from_stored ? __uint_as_float(hq.x & 0xffff0000u) : vv[b][1];
                        const float n2 = renorm_from_stored ? __uint_as_float(hq.y << 16) : vv[b][2];
                        const float n3 = renorm_from_stored ? __uint_as_float(hq.y & 0xffff0000u) : vv[b][3];
                        uint2 ov;
                        ov.x = (uint32_t)f32_to_bf16_bits(n0 * inv_rms * w0f) |
                               ((uint32_t)f32_to_bf16_bits(n1 * inv_rms * w1f) << 16);
                        ov.y = (uint32_t)f32_to_bf16_bits(n2 * inv_rms * w2f) |
                               ((uint32_t)f32_to_bf16_bits(n3 * inv_rms * w3f) << 16);
                        sts_v2(xa + chunk_off(q4), ov);
                        if (c == 0 && o.norm_hidden_out) reinterpret_cast<uint2*>(o.norm_hidden_out)[q4] = hq;
                    }
                }
            }
        } else if (o.norm_w != nullptr) {
            bar_sync(kBarConsumers, kConsumerThreads);  // keeps the barrier count of the RMSNorm path
        }
        return ok;
    };

    // ---- before the first operation: the loads of its first step ----
    issue_first(desc(0), 0);
    loaded = true;
    next_n = n;

    for (int oi = 0; oi < n_ops; ++oi) {
        const ChainOpDev& op = desc(oi);
        const unsigned tag = tag_of(oi);
        const int KB = op.KB;
        const bool has_next = oi + 1 < n_ops;
        // the finalizer is through with operation oi - kRing: its slots are ours
        if (oi >= kRing) bar_sync(kBarGo + (oi & (kRing - 1)), kChainThreads);
        // the x buffer is ours (and already filled when the input could be copied)
        if (!x_wait(oi)) give_up(kStatusTimeoutFull);
        if (!prestaged(oi)) {
            if (!stage_x(oi, is_aborted())) give_up(kStatusTimeoutFull);
            bar_sync(kBarConsumers, kConsumerThreads);
        }
        const bool aborted = is_aborted();
        if (loaded) {
            n = next_n;
        } else {  // (only warps that had nothing to do in the previous operation get here)
            issue_first(op, oi);
        }
        loaded = false;
        const uint32_t my_slots = a_slots + (uint32_t)(oi & (kRing - 1)) * (kChainWarps * 256u) + (uint32_t)warp * 256u;
        const uint32_t my_seg = a_seg + (uint32_t)(oi & (kRing - 1)) * (kChainWarps * 8u) + (uint32_t)warp * 8u;
        if (lane < 2) sts_u32(my_seg + 4u * lane, 0xffffffffu);  // no sums in the slots yet
        const uint32_t xs = x_addr(oi);

        // ---- main loop over the steps of this warp ----
        float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
        int cur_pair = -1, seg_kb_start = 0;
        const int first_pair = pair;
        uint4 xq0 = make_uint4(0u, 0u, 0u, 0u), xq1 = make_uint4(0u, 0u, 0u, 0u);
        if (aborted) n = 0;
        while (n > 0) {
            // the step after this one: in this operation, or the first step of the next one
            const int pos_n = pos + n;
            int kb0_n = kb0 + n, pair_n = pair, n_n = 0;
            if (kb0_n == KB) {
                kb0_n = 0;
                pair_n = pair + 1;
            }
            // what the freed registers are re-loaded with
            int ld_n = 0, ld_pair = pair_n, ld_kb0 = kb0_n, ld_pos = pos_n, ld_w1 = w1;
            const uint8_t* pl0 = ph0;
            const uint8_t* pl1 = ph1;
            bool cross = false;
            if (pos_n < w1) {
                n_n = min(min(kStepUnits, w1 - pos_n), KB - kb0_n);
                ld_n = n_n;
                // the units follow one another in memory, across pairs too; only a pair without a
                // half 1 of its own needs its pointer worked out
                pl0 = ph0 + n * ST;
                pl1 = ph1 + n * ST;
                if (kb0_n == 0 && pair_n >= op.clamp_pair) pl1 = half_ptr(op, 1, pair_n, 0);
            } else if (has_next) {
                const ChainOpDev& nx = desc(oi + 1);
                const First f = first_step(nx, oi + 1);
                cross = true;
                ld_n = f.n; ld_pair = f.pair; ld_kb0 = f.kb0; ld_pos = f.pos; ld_w1 = f.w1;
                pl0 = f.p0; pl1 = f.p1;
            }
            if (pair != cur_pair) {
                cur_pair = pair;
                seg_kb_start = kb0;
            }
            // absmax of this lane's block (kb0 + t), rows g and g+8, both halves: two rounded fp32
            // operations; lanes without a block get a finite value that is never used
            float am[2][2];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    if (codes) {
                        const float nm = __uint_as_float(lds_u32(__byte_perm(raw[h][r], nmap_base, code_sel)));
                        const float second = kb0 + t >= scross[h][r] ? shi[h][r] : slo[h][r];
                        am[h][r] = __fadd_rn(__fmul_rn(nm, second), rowoff[h][r]);
                    } else {
                        am[h][r] = __uint_as_float(raw[h][r]);
                    }
                }
            // x of this lane's block: tile j wants k = 16 j + 4 t + {0..3}, i.e. 8 bytes at 32 j + 8 t;
            // tiles j = 0,1 in xq0, j = 2,3 in xq1
            {
                const uint32_t xa = xs + (uint32_t)(kb0 + x_unit) * (uint32_t)kXBlockPitch + 8u * t;
                const uint32_t pred = (x_lane && x_unit < n) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred q;\n\t"
                    "setp.ne.u32 q, %9, 0;\n\t"
                    "@q ld.shared.v2.u32 {%0,%1}, [%8];\n\t"
                    "@q ld.shared.v2.u32 {%2,%3}, [%8+32];\n\t"
                    "@q ld.shared.v2.u32 {%4,%5}, [%8+64];\n\t"
                    "@q ld.shared.v2.u32 {%6,%7}, [%8+96];\n\t}"
                    : "+r"(xq0.x), "+r"(xq0.y), "+r"(xq0.z), "+r"(xq0.w), "+r"(xq1.x), "+r"(xq1.y),
                      "+r"(xq1.z), "+r"(xq1.w)
                    : "r"(xa), "r"(pred));
            }
#pragma unroll
            for (int u = 0; u < kStepUnits; ++u) {
                if (u < n) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // all sixteen table addresses first (one PRMT each: the byte goes into bits
                        // [8,16) of the lane's base address), then the sixteen loads
                        uint32_t a[16];
                        const uint2 l = W[h][u][0], up = W[h][u][1];
                        a[0] = __byte_perm(l.x, lane_base, 0x7604);   a[1] = __byte_perm(up.x, lane_base, 0x7604);
                        a[2] = __byte_perm(l.x, lane_base, 0x7614);   a[3] = __byte_perm(up.x, lane_base, 0x7614);
                        a[4] = __byte_perm(l.x, lane_base, 0x7624);   a[5] = __byte_perm(up.x, lane_base, 0x7624);
                        a[6] = __byte_perm(l.x, lane_base, 0x7634);   a[7] = __byte_perm(up.x, lane_base, 0x7634);
                        a[8] = __byte_perm(l.y, lane_base, 0x7604);   a[9] = __byte_perm(up.y, lane_base, 0x7604);
                        a[10] = __byte_perm(l.y, lane_base, 0x7614);  a[11] = __byte_perm(up.y, lane_base, 0x7614);
                        a[12] = __byte_perm(l.y, lane_base, 0x7624);  a[13] = __byte_perm(up.y, lane_base, 0x7624);
                        a[14] = __byte_perm(l.y, lane_base, 0x7634);  a[15] = __byte_perm(up.y, lane_base, 0x7634);
#pragma unroll
                        for (int i = 0; i < 16; ++i) a[i] = lds_u32(a[i]);
                        // the registers of this unit are free: fetch the same unit of the next step
                        if (u < ld_n) load_half(h, u, h == 0 ? pl0 : pl1);
                        float d[4];
                        mma_16816_init(d, a[0], a[1], a[2], a[3], xq0.x, xq0.y);
                        mma_16816(d, a[4], a[5], a[6], a[7], xq0.z, xq0.w);
                        mma_16816(d, a[8], a[9], a[10], a[11], xq1.x, xq1.y);
                        mma_16816(d, a[12], a[13], a[14], a[15], xq1.z, xq1.w);
                        // column 2u of the tile = block u: lanes t == u hold it in d[0] / d[2]
                        acc[h][0] = fmaf((t == u) ? am[h][0] : 0.0f, d[0], acc[h][0]);
                        acc[h][1] = fmaf((t == u) ? am[h][1] : 0.0f, d[2], acc[h][1]);
                    }
                } else if (u < ld_n) {
                    load_half(0, u, pl0);
                    load_half(1, u, pl1);
                }
            }
            if (ld_n > 0) prepare_scales(cross ? desc(oi + 1) : op, cross ? oi + 1 : oi, ld_pair, ld_kb0, ld_n, pl0, pl1);
            // leaving the pair: reduce over t, hand the 32 row sums over
            if (n_n == 0 || pair_n != pair) {

                float v[2][2];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        float sum = acc[h][r];
                        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                        v[h][r] = sum;
                        acc[h][r] = 0.0f;
                    }
                const bool whole = seg_kb_start == 0 && kb0 + n == KB;
                const uint32_t which = (whole || pair != first_pair) ? 1u : 0u;
                const uint32_t sl = my_slots + which * 128u;
                if (!whole && lane == 0) sts_u32(my_seg + which * 4u, (uint32_t)pair);
                if (t == 0) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        sts_f32(sl + 4u * (uint32_t)(h * 16 + g), v[h][0]);
                        sts_f32(sl + 4u * (uint32_t)(h * 16 + g + 8), v[h][1]);
                    }
                }
                if (whole) {  // this warp saw every block of the pair: finish it here
                    __syncwarp();
                    const float vs = lds_f32(sl + 4u * lane);
                    // (rare: a whole pair inside one warp's range means in_features <= 640)
                    if (!op.publish || ring_ok(oi))
                        epilogue(op, tag, pair, vs);
                    else if (lane == 0)
                        give_up(kStatusTimeoutFull);
                    __syncwarp();
                }
            }
            // the registers now hold the step that runs next (possibly the next operation's first)
            pos = ld_pos;
            w1 = ld_w1;
            pair = ld_pair;
            kb0 = ld_kb0;
            ph0 = pl0;
            ph1 = pl1;
            if (cross) {
                loaded = true;  // leaves the loop; the registers belong to the next operation
                next_n = ld_n;
                n = 0;
            } else {
                n = n_n;
            }
        }
        // this warp's sums of operation oi are in its slots
        bar_arrive(kBarDone + (oi & (kRing - 1)), kChainThreads);
    }
}


// Shared memory the system keeps at the bottom of every block's window: the dynamic allocation
// of a kernel without static shared memory starts right after it.
int chain_window_base() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1024;
    if (cached[dev] == 0) {
        int r = 0;
        if (cudaDeviceGetAttribute(&r, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess || r < 0)
            r = 1024;
        cached[dev] = r + 1;
    }
    return cached[dev] - 1;
}

constexpr int kChainSmemMax = 227 * 1024;

// bytes between two x buffers for a launch whose largest in_features is k_max
int chain_x_pitch(int64_t k_max) { return (int)(k_max / kUnitK) * kXBlockPitch; }
// bytes of dynamic shared memory with `buffers` x buffers (0: too large)
int chain_smem_bytes(int64_t k_max, int buffers = 1) {
    const long long need = (long long)kXAddr - chain_window_base() + (long long)buffers * chain_x_pitch(k_max) + 256;
    return need <= kChainSmemMax ? (int)need : 0;
}
// fills the shared-memory fields of the launch parameters
void chain_plan_smem(ChainParams* p, int64_t k_max, int n_ops) {
    p->x_pitch = chain_x_pitch(k_max);
    p->x_buffers = (n_ops > 1 && chain_smem_bytes(k_max, 2) != 0) ? 2 : 1;
    p->smem_bytes = chain_smem_bytes(k_max, p->x_buffers);
}

cudaError_t chain_prepare_kernel(int device, int smem) {
    static int have[64] = {0};
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (have[device] >= smem) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(gemv_chain_kernel<kAbsmaxCodes>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kChainSmemMax);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemv_chain_kernel<kAbsmaxF32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kChainSmemMax);
    if (e != cudaSuccess) return e;
    have[device] = kChainSmemMax;
    return cudaSuccess;
}

// Fills the part of a descriptor that depends only on the linear and the grid.
__global__ void row_scales_kernel(ScaleParams sp, int n_rows, int KB, RowScales* out) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= n_rows) return;
    const SegmentRow sr = segment_row(sp, n);
    const unsigned nbs = 1u << sp.nbs_shift;
    const unsigned first = sr.flat >> sp.nbs_shift;
    const long long cross = (long long)(nbs - (sr.flat & (nbs - 1u))) << sp.blk_shift;
    RowScales e;
    e.lo = __ldg(sp.nabs + first);
    e.hi = cross < KB ? __ldg(sp.nabs + first + 1) : e.lo;
    e.cross = (int)(cross < 0x7fffffffll ? cross : 0x7fffffffll);
    e.offset = sr.offset;
    out[n] = e;
}

bool chain_fill_op(ChainOpDev* d, const AilaNf4Linear& w, int64_t ff_pair, int grid) {
    std::memset(d, 0, sizeof(*d));
    const bool paired = ff_pair > 0;
    if (paired && (ff_pair % kTileRows != 0 || w.N != 2 * ff_pair)) return false;
    if (w.absmax_kind == kAbsmaxCodes && !w.d_row_scales) return false;
    d->units = w.d_units;
    d->row_scales = static_cast<const RowScales*>(w.d_row_scales);
    d->sp = w.scale_params();
    d->K = (int)w.K;
    d->KB = w.KU;
    d->n_rows = (int)w.N;
    d->n_tiles = w.RT;
    d->swiglu = paired ? 1 : 0;
    const long long pairs = paired ? ff_pair / kTileRows : (w.RT + 1) / 2;
    d->pair_offset = (int)pairs;
    d->n_out = paired ? (int)ff_pair : (int)w.N;
    const long long total = pairs * w.KU;
    if (total <= 0 || total >= (1ll << 31) || w.KU <= 0) return false;
    d->total = (int)total;
    d->slice_q = (int)(total / grid);
    d->slice_r = (int)(total % grid);
    make_fast_div((uint32_t)grid, &d->div_g_m, &d->div_g_s);
    make_fast_div((uint32_t)w.KU, &d->div_kb_m, &d->div_kb_s);
    d->half1_bytes = (long long)pairs * w.KU * w.unit_stride;
    // A warp pays a fixed price per operation: a small slice goes to fewer warps, about
    // kItemsPerWarp work items each.
    const long long per_cta = (total + grid - 1) / grid;
    long long nw = (per_cta + kItemsPerWarp - 1) / kItemsPerWarp;
    nw = nw < kMinWarps ? kMinWarps : nw > kConsumerWarps ? kConsumerWarps : nw;
    d->n_warps = (int)nw;
    make_fast_div((uint32_t)nw, &d->div_w_m, &d->div_w_s);
    d->clamp_pair = w.RT - (int)pairs;
    return true;
}

// After the tensors of an operation are known.
void chain_seal_op(ChainOpDev* d) {
    d->x_copy = d->x_ext != nullptr && d->norm_w == nullptr && (reinterpret_cast<uintptr_t>(d->x_ext) & 15) == 0;
}

cudaError_t chain_launch(const ChainParams& p, int kind, int grid, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kChainThreads);
    cfg.dynamicSmemBytes = (size_t)p.smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident at once: CTAs wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return kind == kAbsmaxCodes ? cudaLaunchKernelEx(&cfg, gemv_chain_kernel<kAbsmaxCodes>, p)
                                : cudaLaunchKernelEx(&cfg, gemv_chain_kernel<kAbsmaxF32>, p);
}

void chain_params_from_scratch(ChainParams* p, const AilaNf4Scratch& sc) {
    p->xbuf = sc.d_chain_x;
    p->xwords = sc.chain_xwords;
    p->pbuf = sc.d_chain_p;
    p->tokens = sc.d_chain_tok;
    p->ctrl = sc.d_chain_ctrl;
    p->status = sc.d_status;
    p->spin_limit = sc.wait_limit_cycles;

}

}  // namespace

cudaError_t launch_row_scales(const AilaNf4Linear& l, cudaStream_t s) {
    const int threads = 256;
    row_scales_kernel<<<(unsigned)((l.N + threads - 1) / threads), threads, 0, s>>>(
        l.scale_params(), (int)l.N, l.KU, static_cast<RowScales*>(l.d_row_scales));
    return cudaGetLastError();
}

bool gemv_chain_supported(const AilaNf4Linear& w, int64_t ff_pair, const AilaNf4Scratch& sc) {
    if (!sc.d_chain_x || sc.sm_count <= 0 || sc.sm_count > kChainThreads || sc.sm_count > kChainMaxGrid)
        return false;
    if (chain_smem_bytes(w.K) == 0 || w.K / 2 > sc.chain_xwords) return false;
    ChainOpDev d;
    return chain_fill_op(&d, w, ff_pair, sc.sm_count);
}

AilaNf4Status launch_gemv_chain_single(const AilaNf4Linear& w, AilaNf4Scratch& sc, const void* x, void* y,
                                       const void* residual, int64_t ff_pair, const NormInput* norm,
                                       cudaStream_t s) {
    ChainParams p;
    std::memset(&p, 0, sizeof(p));
    if (!chain_fill_op(&p.inline_op, w, ff_pair, sc.sm_count))
        return fail(AILA_NF4_ERR_UNSUPPORTED, "decode kernel does not take this shape");
    if (norm && w.K > 4 * kXBatch * kConsumerThreads)
        return fail(AILA_NF4_NOT_APPLICABLE, "the fused RMSNorm input takes in_features <= 11520");
    p.inline_op.x_ext = static_cast<const uint16_t*>(x);
    p.inline_op.y = static_cast<uint16_t*>(y);
    p.inline_op.residual = ff_pair > 0 ? nullptr : static_cast<const uint16_t*>(residual);
    if (norm) {
        p.inline_op.norm_add = static_cast<const uint16_t*>(norm->add);
        p.inline_op.norm_w = static_cast<const uint16_t*>(norm->weight);
        p.inline_op.norm_hidden_out = static_cast<uint16_t*>(norm->hidden_out);
        p.inline_op.norm_eps = norm->eps;
    }
    chain_seal_op(&p.inline_op);
    p.ops = nullptr;
    p.n_ops = 1;
    p.qmap = w.d_qmap;
    p.nmap = w.d_nmap;
    chain_params_from_scratch(&p, sc);
    chain_plan_smem(&p, w.K, 1);
    NF4_CUDA(chain_prepare_kernel(sc.device, p.smem_bytes));
    NF4_CUDA(chain_launch(p, w.absmax_kind, sc.sm_count, s));
    return AILA_NF4_OK;
}

AilaNf4Status ensure_chain_scratch(AilaNf4Scratch* sc) {
    if (sc->d_chain_x) return AILA_NF4_OK;
    const size_t xwords = 32768;  // in_features up to 65536
    const size_t ctrl_b = 256, tok_b = (size_t)kChainMaxGrid * 8, p_b = (size_t)8 * kChainMaxGrid * 32 * 8;
    const size_t x_b = 8 * xwords * 8;
    uint8_t* base = nullptr;
    NF4_CUDA(cudaMalloc(reinterpret_cast<void**>(&base), ctrl_b + tok_b + p_b + x_b));
    NF4_CUDA(cudaMemset(base, 0, ctrl_b + tok_b + p_b + x_b));

    sc->d_chain_ctrl = reinterpret_cast<unsigned*>(base);
    sc->d_chain_tok = reinterpret_cast<unsigned long long*>(base + ctrl_b);
    sc->d_chain_p = reinterpret_cast<unsigned long long*>(base + ctrl_b + tok_b);
    sc->d_chain_x = reinterpret_cast<unsigned long long*>(base + ctrl_b + tok_b + p_b);
    sc->chain_xwords = (long long)xwords;
    return AILA_NF4_OK;
}

}  // namespace nf4

// ---------------------------------------------------------------------------------------------
// C ABI: a chain of decode linears run by one launch (include/aila_nf4.h)
// ---------------------------------------------------------------------------------------------
struct AilaNf4Chain {
    int device = 0;
    int n_ops = 0;
    int kind = nf4::kAbsmaxCodes;  // how every linear of the chain stores its absmax
    AilaNf4Scratch* scratch = nullptr;
    nf4::ChainOpDev* d_ops = nullptr;
    nf4::ChainParams params;
    int64_t first_in = 0, last_out = 0;
    void* first_x = nullptr;       // where the first operation reads x (device)
    void* last_y = nullptr;        // where the last operation writes y (device)
};

namespace {
AilaNf4Status chain_create(AilaNf4Scratch* scratch, const AilaNf4ChainOp* ops, int n_ops,
                           const AilaNf4PeerBuf* peers, AilaNf4Chain** out);
}

AILA_NF4_API AilaNf4Status aila_nf4_chain_create(AilaNf4Scratch* scratch, const AilaNf4ChainOp* ops,
                                                 int n_ops, AilaNf4Chain** out) {
    return chain_create(scratch, ops, n_ops, nullptr, out);
}

AILA_NF4_API AilaNf4Status aila_nf4_chain_create_allreduce(AilaNf4Scratch* scratch,
                                                           const AilaNf4ChainOp* ops, int n_ops,
                                                           AilaNf4PeerBuf* peers, AilaNf4Chain** out) {
    if (!peers) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "peer buffer is NULL");
    return chain_create(scratch, ops, n_ops, peers, out);
}

namespace {
AilaNf4Status chain_create(AilaNf4Scratch* scratch, const AilaNf4ChainOp* ops, int n_ops,
                           const AilaNf4PeerBuf* peers, AilaNf4Chain** out) {
    using nf4::fail;
    if (!out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "output handle pointer is NULL");
    *out = nullptr;
    if (!scratch || !ops) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "scratch or operation list is NULL");
    if (n_ops < 1 || n_ops > nf4::kChainMaxOps)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "a chain holds 1 to " + std::to_string(nf4::kChainMaxOps) + " operations");
    std::vector<nf4::ChainOpDev> h((size_t)n_ops);
    int64_t k_max = 0;
    const AilaNf4Linear* first = ops[0].linear;
    for (int i = 0; i < n_ops; ++i) {
        const AilaNf4ChainOp& o = ops[i];
        const std::string at = "chain operation " + std::to_string(i) + ": ";
        if (!o.linear) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "linear handle is NULL");
        const AilaNf4Linear& w = *o.linear;
        if (w.device != scratch->device)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "scratch and linear live on different devices");
        if (w.d_qmap != first->d_qmap || w.d_nmap != first->d_nmap || w.absmax_kind != first->absmax_kind)
            return fail(AILA_NF4_ERR_UNSUPPORTED,
                        at + "all linears of a chain must share their code books and absmax storage");
        if (o.ff_dim < 0 || (o.ff_dim > 0 && (w.N != 2 * o.ff_dim || o.ff_dim % nf4::kTileRows != 0)))
            return fail(AILA_NF4_NOT_APPLICABLE, at + "out_features != 2 * ff_dim or ff_dim not a multiple of 16");
        if (o.ff_dim > 0 && o.residual_bf16)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "the gate|up operation takes no residual");
        if (!nf4::gemv_chain_supported(w, o.ff_dim, *scratch))
            return fail(AILA_NF4_ERR_UNSUPPORTED, at + "shape not taken by the decode kernel");
        nf4::chain_fill_op(&h[(size_t)i], w, o.ff_dim, scratch->sm_count);
        nf4::ChainOpDev& d = h[(size_t)i];
        const void* x = o.x_bf16;
        if (i > 0 && x && x == ops[i - 1].y_bf16) x = nullptr;  // reads the previous output: take the link
        if (i == 0 && !x) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "the first operation needs an input");
        if (x && (reinterpret_cast<uintptr_t>(x) & 7))
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "x must be 8-byte aligned");
        if (i > 0) {
            if (!x) {
                if (h[(size_t)i - 1].n_out != d.K)
                    return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                                at + "in_features differs from the previous operation's output size");
                h[(size_t)i - 1].publish = 1;
            }
        }
        if (!x && !o.y_bf16 && i == n_ops - 1)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "the last operation needs an output");
        d.x_ext = static_cast<const uint16_t*>(x);
        d.y = static_cast<uint16_t*>(o.y_bf16);
        d.residual = static_cast<const uint16_t*>(o.residual_bf16);
        if (o.norm) {
            if (!o.norm->weight_bf16) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "RMSNorm weight is NULL");
            if (!(o.norm->eps >= 0.0f)) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "RMSNorm eps must be >= 0");
            if (w.K > 4 * nf4::kXBatch * nf4::kConsumerThreads)
                return fail(AILA_NF4_NOT_APPLICABLE, at + "the fused RMSNorm input takes in_features <= 11520");
            const uintptr_t bits = reinterpret_cast<uintptr_t>(o.norm->weight_bf16) |
                                   reinterpret_cast<uintptr_t>(o.norm->add_bf16) |
                                   reinterpret_cast<uintptr_t>(o.norm->hidden_out_bf16);
            if (bits & 7) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "RMSNorm tensors must be 8-byte aligned");
            if (o.norm->hidden_out_bf16 && (o.norm->hidden_out_bf16 == x || o.norm->hidden_out_bf16 == o.norm->add_bf16))
                return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "hidden_out must not alias x or the added tensor");
            d.norm_add = static_cast<const uint16_t*>(o.norm->add_bf16);
            d.norm_w = static_cast<const uint16_t*>(o.norm->weight_bf16);
            d.norm_hidden_out = static_cast<uint16_t*>(o.norm->hidden_out_bf16);
            d.norm_eps = o.norm->eps;
        }
        if (!d.y && i == n_ops - 1) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, at + "the last operation needs an output");
        nf4::chain_seal_op(&d);
        k_max = w.K > k_max ? w.K : k_max;
    }
    // row-parallel exchange after the last operation: its sums go to the ranks, y is written from
    // the sum over the ranks
    nf4::PeerTargets pt;
    uint16_t* peer_y = nullptr;
    const uint16_t* peer_residual = nullptr;
    if (peers) {
        nf4::ChainOpDev& last = h.back();
        if (ops[n_ops - 1].ff_dim > 0)
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "the row-parallel operation cannot be a gate|up operation");
        const AilaNf4Status st = nf4::peer_targets_of(peers, scratch->device, last.n_out, &pt);
        if (st != AILA_NF4_OK) return st;
        peer_y = last.y;
        peer_residual = last.residual;
        last.y = nullptr;
        last.residual = nullptr;
        last.peer = 1;
    }
    int prev = -1;
    NF4_CUDA(cudaGetDevice(&prev));
    if (prev != scratch->device) NF4_CUDA(cudaSetDevice(scratch->device));
    AilaNf4Chain* ch = new (std::nothrow) AilaNf4Chain();
    if (!ch) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    auto restore = [&]() {
        if (prev != scratch->device) cudaSetDevice(prev);
    };
    ch->device = scratch->device;
    ch->n_ops = n_ops;
    ch->kind = first->absmax_kind;
    ch->scratch = scratch;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ch->d_ops), (size_t)n_ops * nf4::kDescBytes);
    if (e == cudaSuccess)
        e = cudaMemcpy(ch->d_ops, h.data(), (size_t)n_ops * nf4::kDescBytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = nf4::chain_prepare_kernel(ch->device, nf4::chain_smem_bytes(k_max));
    if (e != cudaSuccess) {
        cudaFree(ch->d_ops);
        delete ch;
        restore();
        return nf4::cuda_fail(e, "aila_nf4_chain_create");
    }
    std::memset(&ch->params, 0, sizeof(ch->params));
    ch->params.ops = ch->d_ops;
    ch->params.n_ops = n_ops;
    ch->params.qmap = first->d_qmap;
    ch->params.nmap = first->d_nmap;
    nf4::chain_plan_smem(&ch->params, k_max, n_ops);
    if (peers) {
        ch->params.peer_world = pt.world;
        ch->params.peer_rank = pt.rank;
        ch->params.peer_max_rows = pt.max_rows;
        for (int d = 0; d < 8; ++d) ch->params.peer_part[d] = pt.part_base[d];
        ch->params.peer_ctrl = pt.ctrl;
        ch->params.peer_y = peer_y;
        ch->params.peer_residual = peer_residual;
    }
    ch->first_in = ops[0].linear->K;
    ch->last_out = h[(size_t)n_ops - 1].n_out;
    ch->first_x = const_cast<void*>(ops[0].x_bf16);
    ch->last_y = ops[n_ops - 1].y_bf16;
    restore();
    *out = ch;
    return AILA_NF4_OK;
}
}  // namespace

AILA_NF4_API void aila_nf4_chain_destroy(AilaNf4Chain* chain) {
    if (!chain) return;
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != chain->device) cudaSetDevice(chain->device);
    cudaFree(chain->d_ops);
    if (prev != chain->device) cudaSetDevice(prev);
    delete chain;
}

AILA_NF4_API int aila_nf4_chain_length(const AilaNf4Chain* chain) { return chain ? chain->n_ops : 0; }

AILA_NF4_API AilaNf4Status aila_nf4_chain_run(AilaNf4Chain* chain, void* stream) {
    if (!chain) return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "chain handle is NULL");
    int prev = -1;
    NF4_CUDA(cudaGetDevice(&prev));
    if (prev != chain->device) NF4_CUDA(cudaSetDevice(chain->device));
    nf4::chain_params_from_scratch(&chain->params, *chain->scratch);
    const cudaError_t e = nf4::chain_launch(chain->params, chain->kind, chain->scratch->sm_count,
                                            static_cast<cudaStream_t>(stream));
    if (prev != chain->device) cudaSetDevice(prev);
    NF4_CUDA(e);
    return AILA_NF4_OK;
}

// Host-buffer form of a chain: x of the first operation comes from host memory, y of the last
// goes back to host memory, one stream synchronisation for the whole chain.
AILA_NF4_API AilaNf4Status aila_nf4_chain_run_host(AilaNf4Chain* chain, const void* x_host_bf16,
                                                   void* y_host_bf16, void* stream) {
    if (!chain || !x_host_bf16 || !y_host_bf16)
        return nf4::fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    int prev = -1;
    NF4_CUDA(cudaGetDevice(&prev));
    if (prev != chain->device) NF4_CUDA(cudaSetDevice(chain->device));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(chain->first_x, x_host_bf16, (size_t)chain->first_in * 2,
                                    cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        nf4::chain_params_from_scratch(&chain->params, *chain->scratch);
        e = nf4::chain_launch(chain->params, chain->kind, chain->scratch->sm_count, s);
    }
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(y_host_bf16, chain->last_y, (size_t)chain->last_out * 2, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (prev != chain->device) cudaSetDevice(prev);
    NF4_CUDA(e);
    return AILA_NF4_OK;
}
