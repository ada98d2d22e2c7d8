// Decode (seq_len == 1) kernels: y = W x and out = silu(Wg x) * (Wu x).
// Replace packed_nf4_gemv_bf16 and packed_nf4_gemv_gate_up_swiglu
// (reference src/ops/Bnb4BitLinear.cpp:271-410, :142-246).
//
// Two kernels:
//  * gemv_simple: one warp per output row, fp32 weights q*absmax and fp32 FMA, i.e. the
//    reference's arithmetic with a different summation order. Baseline and fallback for
//    shapes the streaming kernel does not take.
//  * gemv_stream: the streaming kernel. One persistent CTA per SM owns an equal, contiguous
//    slice of the unit stream (split along rows AND k, so any shape balances over 148 SMs).
//    A producer thread keeps a ring of bulk-async (TMA) copies in flight; 16 consumer warps turn
//    nibbles into bf16 tensor-core operands through a bank-private shared-memory table (one PRMT
//    plus one LDS per two weights) and accumulate in fp32 with mma.sync m16n8k16; absmax is
//    decoded from its 8-bit code in fp32 (two rounded operations) and applied per 64-block.
//    A CTA walks its slice starting with its LAST row tile, so the two tiles it may share with
//    neighbouring CTAs complete first: their per-CTA partial sums go to global scratch and
//    whichever CTA arrives last at the tile's counter sums them in CTA order (no spinning,
//    deterministic) while everybody streams on. Row tiles are completed as soon as every warp
//    has signed them off, so there is no end-of-kernel reduction phase.
//    The kernel is launched with programmatic stream serialisation: it issues
//    griddepcontrol.launch_dependents at once and waits (griddepcontrol.wait) only before it
//    fetches x, so its table build and first weight copies overlap the previous kernel's tail.
//
// Roofline: HBM. Algorithmic bytes per weight: 0.5 (nibbles) + 1/64 (code) + 4/16384 (scale).
#include <cstdlib>
#include <cstring>
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
constexpr int kStreamThreads = (kConsumerWarps + 2) * 32;  // + producer warp + finalizer warp
constexpr int kItemsPerWarp = 2;   // work items a consumer warp takes from one stage
constexpr int kStageItems = kConsumerWarps * kItemsPerWarp;
constexpr int kMaxStages = 24;
constexpr int kMaxLocalTiles = 8;  // row tiles one CTA slice may touch
constexpr int kMaxGridMult = 8;     // grid <= 8 x SM count
constexpr int kNabsWindow = 256;    // second-level scales kept in shared memory per half
constexpr int kEarlyBytes = 68 * 1024;  // ring bytes requested before x has been asked for
constexpr int kMaxPeerWorld = 8;
constexpr int kPairSkewBytes = 64;  // shared-memory distance added between a stage's gate and up units

struct StreamParams {
    const uint8_t* units;
    const float* qmap;      // [16] first-level code book
    ScaleParams sp;
    const uint16_t* x;
    uint16_t* y;
    const uint16_t* residual;
    float* partials;
    int* counters;
    int* status;
    long long spin_limit;   // SM cycles a wait may take
    int total_items;        // work items (units, or gate/up unit pairs), < 2^31
    int slice_q, slice_r;   // total_items = slice_q * grid + slice_r
    uint32_t div_g_m, div_ku_m;  // multiply-shift division by the grid size and by KU
    int div_g_s, div_ku_s;
    int kb_step, rt_step;   // consumer warp count mod / div KU (a warp's items are that far apart)
    int n_out;              // rows written (ff when paired)
    int K;
    int KU;
    int unit_stride;
    int pair_rt_offset;     // paired: row-tile distance from a gate tile to its up tile
    int stages;             // ring depth = stages_b + stages_a
    int stages_b;           // stages above the table (used first), the rest sit below it
    int x_bytes;            // K*2 rounded up to 16
    int x_in_b;             // 1: x lives above the table (large K), 0: below it
    int smem_bytes;         // dynamic shared memory of the launch
    int n_rows;             // rows of the linear (for clamping the padded rows of the last tile)
    int m_rows;             // batch rows of x / y handled by this launch (1; 2..8 in the batched kernel)
    // residual add + RMSNorm folded into the staging of x (single-row kernel, norm_w != NULL):
    // v = x + norm_add (fp32), the linear's input is bf16(v * rsqrt(mean(v^2) + eps) * norm_w),
    // CTA 0 writes bf16(v) to norm_hidden_out
    const uint16_t* norm_add;
    const uint16_t* norm_w;
    uint16_t* norm_hidden_out;
    float norm_eps;
    // row-parallel exchange (peer_world > 0): the epilogue stores the fp32 row sums of this
    // rank into every rank's exchange buffer as 8-byte words {value, tag = epoch + 1}; a reader
    // that finds the call's tag in a word has the value (one naturally aligned 64-bit access)
    int peer_world;
    int peer_rank;
    long long peer_max_rows;
    unsigned long long* peer_part[kMaxPeerWorld];  // rank d's row area (all parities and source ranks)
    unsigned* peer_ctrl;                  // this rank's {epoch, unused, CTAs / reducer blocks done}
    int n_row_tiles;                      // row tiles of the launch (all CTAs)
    int peer_inline;                      // 1: the CTAs also sum the ranks' rows and write y
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// first tile of a chain: accumulator operands are the constant zero (no register initialisation)
__device__ __forceinline__ void mma_bf16_16816_init(float (&c)[4], uint32_t a0, uint32_t a1,
                                                    uint32_t a2, uint32_t a3, uint32_t b0,
                                                    uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

extern __shared__ __align__(1024) uint8_t smem_raw[];

// ---- shared-memory access by 32-bit shared-window address (keeps address arithmetic 32-bit) ----
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
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}

// Bank-private table lookup. The 64 KB table sits on a 64 KB boundary of the shared window and
// holds, for byte value b and lane l, the bf16 pair of b's two nibbles at b*256 + l*4: the 32
// lanes of a warp always hit 32 different banks. `lane_base` = table address + l*4; ONE PRMT
// splices the byte into bits [8,16) of it and the result is the load address.
template <int BYTE>
__device__ __forceinline__ uint32_t lut_pair(uint32_t word, uint32_t lane_base) {
    return lds_u32(__byte_perm(word, lane_base, 0x7604 | (BYTE << 4)));
}

// n / d for 0 <= n < 2^31 as (n * m) >> s, with s = 31 + ceil(log2 d) and m = ceil(2^s / d) < 2^32:
// n*m / 2^s exceeds n/d by less than 2^31 / 2^s <= 1/d, which cannot carry into the next integer.
__host__ __device__ __forceinline__ int fast_div(int n, uint32_t m, int s) {
    return (int)(((unsigned long long)(unsigned)n * m) >> s);
}
void make_fast_div(uint32_t d, uint32_t* m, int* s) {
    int l = 0;
    while ((1ull << l) < d) ++l;
    *s = 31 + l;
    *m = (uint32_t)(((1ull << *s) + d - 1) / d);
}

// First work item of CTA c: floor(total * c / G) in 32-bit arithmetic, with total = q*G + r.
__device__ __forceinline__ int slice_begin(const StreamParams& p, int c) {
    return p.slice_q * c + fast_div(p.slice_r * c, p.div_g_m, p.div_g_s);
}


// Bytes of the per-(row tile, half) accumulation slot: one 16-float row per consumer warp in the
// single-row kernel, `row_blocks` tiles of 16 rows x 8 batch columns in the batched one.
__host__ __device__ constexpr int stream_slot_bytes(int row_blocks) {
    return kConsumerWarps * 64 > row_blocks * 512 ? kConsumerWarps * 64 : row_blocks * 512;
}

// BATCH = number of 8-row blocks of x (0: the single-row kernel; 1, 2 or 4: up to 8, 16 or 32 rows).
// The rows of a block ride in the eight batch columns of the tensor-core tile, and every decoded
// weight fragment feeds one tensor-core operation per block, so the weights are read and
// dequantised once for all rows. Differences from the single-row kernel: x fragments come straight
// from global memory (L2) per work item, every lane keeps 2x2 accumulators per half and block,
// warps add their tile sums into shared fp32 tiles with shared-memory atomics (the order of these
// additions is not fixed: last-bit differences between runs), and the epilogue writes [rows][out]
// outputs. More than one block only without the gate/up pairing (register budget).
template <int KIND, bool PAIRED, int BATCH>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const StreamParams p) {
    constexpr int NP = PAIRED ? 2 : 1;
    constexpr int RB = BATCH > 0 ? BATCH : 1;  // 8-row blocks of x
    static_assert(BATCH == 0 || BATCH == 1 || BATCH == 2 || BATCH == 4, "row blocks");
    static_assert(!(PAIRED && RB > 1), "the paired kernel takes one row block");
    constexpr int kSlotBytes = stream_slot_bytes(RB);
    constexpr int W = kConsumerWarps;
    constexpr int IPW = kItemsPerWarp;
    constexpr int unit_stride = (KIND == kAbsmaxCodes) ? kUnitStrideCodes : kUnitStrideF32;
    // one stage of gate (or plain) units; the up units follow 64 bytes (16 banks) further so that
    // the two halves' absmax bytes never meet in one bank
    constexpr int half_bytes = kStageItems * unit_stride + (PAIRED ? kPairSkewBytes : 0);
    constexpr int stage_bytes = kStageItems * unit_stride * NP + (PAIRED ? kPairSkewBytes : 0);

    // ---- shared-memory map (absolute shared-window addresses) ----
    // region A = [base, 64 KB): barriers, tile counters, code book, per-warp slots, x (if small)
    // table    = [64 KB, 128 KB)
    // region B = [128 KB, ...): x (if large), ring of stages
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t a_bar = (base + 15u) & ~15u;                 // full[kMaxStages], empty[], abort flag
    const uint32_t a_tile = a_bar + 400;                         // tile_bar[kMaxLocalTiles]
    static_assert((2 * kMaxStages + 1) * 8 <= 400, "barrier block");
    static_assert(kMaxLocalTiles * 8 <= 64, "tile barrier block");
    const uint32_t a_info = a_tile + 64;                         // per half: window base, window valid
    const uint32_t a_red = a_info + 16;                          // [W] per-warp sums of the RMSNorm
    const uint32_t a_nmap = a_red + 64;
    const uint32_t a_nabsw = a_nmap + 1024;                      // [2][kNabsWindow] second-level scales
    const uint32_t a_ptab = a_nabsw + 2 * kNabsWindow * 4;       // [256] byte value -> bf16 pair
    const uint32_t a_tinfo = a_ptab + 1024;                      // [tile][lane] absmax row base, offset
    const uint32_t a_slots = a_tinfo + kMaxLocalTiles * 32 * 8;  // [tile][pair][warp][16] floats
    const uint32_t a_xs_small = a_slots + kMaxLocalTiles * NP * kSlotBytes;
    const uint32_t a_lut = 65536u;
    const uint32_t a_xs = p.x_in_b ? 131072u : a_xs_small;
    const uint32_t a_ring_b = 131072u + (p.x_in_b ? (uint32_t)p.x_bytes : 0u);
    const uint32_t a_ring_a = (a_xs_small + (p.x_in_b ? 0u : (uint32_t)p.x_bytes) + 127u) & ~127u;
    auto stage_addr = [&](int st) {
        return st < p.stages_b ? a_ring_b + (uint32_t)st * stage_bytes
                               : a_ring_a + (uint32_t)(st - p.stages_b) * stage_bytes;
    };
    uint8_t* gen = smem_raw - base;  // generic pointer to shared-window address 0
    uint64_t* full = reinterpret_cast<uint64_t*>(gen + a_bar);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tile_bar = reinterpret_cast<uint64_t*>(gen + a_tile);
    int* abort_flag = reinterpret_cast<int*>(empty + kMaxStages);
    uint64_t* x_ready = reinterpret_cast<uint64_t*>(gen + a_bar + 392);  // x is in shared memory

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    // static tables (shared by every launch that uses the same code books): requested before
    // anything else, consumed after the set-up arithmetic
    float nmap_reg = 0.0f, q_hi = 0.0f, q_lo = 0.0f;
    if (tid < 256) {
        if (KIND == kAbsmaxCodes) nmap_reg = __ldg(p.sp.nmap + tid);
        q_hi = __ldg(p.qmap + (tid >> 4));
        q_lo = __ldg(p.qmap + (tid & 15));
    }
    const int G = gridDim.x;
    const int c = blockIdx.x;
    const int i0 = slice_begin(p, c);
    const int i1 = slice_begin(p, c + 1);
    const int len = i1 - i0;
    const int n_groups = (len + kStageItems - 1) / kStageItems;
    const int rt_first = fast_div(i0, p.div_ku_m, p.div_ku_s);
    const int rt_last = fast_div(i1 - 1, p.div_ku_m, p.div_ku_s);
    const int n_local = rt_last - rt_first + 1;
    // Traversal order: the slice's LAST row tile first, then the rest from the front. Both row
    // tiles that may be shared with a neighbouring CTA are then finished early, and their
    // cross-CTA completion overlaps the streaming of the tiles this CTA owns alone.
    const int tail0 = max(i0, rt_last * p.KU);
    const int tail_len = i1 - tail0;
    // virtual index v in [0, len): item = v < tail_len ? tail0 + v : i0 + (v - tail_len)

    if (base > 2048u || base + (uint32_t)p.smem_bytes < a_ring_b + (uint32_t)p.stages_b * stage_bytes ||
        a_ring_a + (uint32_t)(p.stages - p.stages_b) * stage_bytes > 65536u) {
        if (tid == 0) atomicExch(p.status, kStatusBadArgument);
        return;
    }
    // let a dependent launch begin its own set-up; it waits for our completion before reading
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- completing a row tile (finalizer warp) ----
    // write_rows: the epilogue of 16 output rows (lanes 0..15 hold one row each)
    int peer_parity = -1;  // exchange half of this launch, read on first use
    unsigned peer_epoch = 0;
    auto peer_read_epoch = [&]() {
        if (peer_parity < 0) {
            peer_epoch = *(volatile unsigned*)p.peer_ctrl;
            peer_parity = (int)(peer_epoch & 1u);
        }
    };
    // One launch does the whole exchange when every CTA of the grid is resident at once (grid <=
    // SM count): each CTA's finalizer warp sums the ranks' rows of its share of the output in rank
    // order as soon as every rank's word carries the call's tag (bounded wait per word), adds the
    // residual and writes y. The CTA that finishes last advances the epoch. A CTA only waits
    // after it has published its own rows, and this rank's words need nothing but the resident
    // CTAs of this grid.
    auto peer_reduce_inline = [&]() {
        peer_read_epoch();
        const unsigned tag = peer_epoch + 1u;
        const int per = (p.n_out + G - 1) / G;
        const int r0 = c * per, r1 = min(p.n_out, r0 + per);
        const unsigned long long* part =
            p.peer_part[p.peer_rank] + (size_t)peer_parity * p.peer_world * (size_t)p.peer_max_rows;
        bool ok = true;
        for (int r = r0 + lane; r < r1 && ok; r += 32) {
            float acc = 0.0f;
            for (int src = 0; src < p.peer_world && ok; ++src) {
                const unsigned long long* word = part + (size_t)src * (size_t)p.peer_max_rows + r;
                unsigned long long q;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(q) : "l"(word) : "memory");
                if ((unsigned)(q >> 32) != tag) {
                    const long long t0 = clock64();
                    do {
                        __nanosleep(40);
                        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(q) : "l"(word) : "memory");
                        if (*(volatile int*)abort_flag || clock64() - t0 > p.spin_limit) {
                            atomicExch(p.status, kStatusTimeoutPeer);
                            ok = false;
                            break;
                        }
                    } while ((unsigned)(q >> 32) != tag);
                }
                acc += __uint_as_float((unsigned)q);
            }
            if (ok) {
                if (p.residual) acc += bf16_bits_to_f32(__ldcg(p.residual + r));
                p.y[r] = f32_to_bf16_bits(acc);
            }
        }
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            const unsigned done = atomicAdd(p.peer_ctrl + 2, 1u);
            if (done == (unsigned)G - 1u) {
                p.peer_ctrl[2] = 0u;
                __threadfence();
                *(volatile unsigned*)p.peer_ctrl = peer_epoch + 1u;
            }
        }
    };
    auto write_rows = [&](int rtile, const float (&v)[NP]) {
        if (!PAIRED && p.peer_world > 0) {
            // Row-parallel exchange: one 8-byte store {value, tag} per row into every rank's
            // memory (this rank's own included). No fence and no counter: the tag arrives with
            // the value. The exchange alternates between two halves of the buffers (parity of
            // the epoch, which this rank advances when the call's sums have been written).
            peer_read_epoch();
            const size_t slice = ((size_t)peer_parity * p.peer_world + p.peer_rank) * (size_t)p.peer_max_rows;
            const int n = rtile * kTileRows + lane;
            if (lane < 16 && n < p.n_out) {
                const unsigned long long word =
                    ((unsigned long long)(peer_epoch + 1u) << 32) | (unsigned long long)__float_as_uint(v[0]);
                for (int d = 0; d < p.peer_world; ++d)
                    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.peer_part[d] + slice + n), "l"(word) : "memory");
            }
            return;
        }
        if (lane < 16) {
            const int n = rtile * kTileRows + lane;
            if (n < p.n_out) {
                float o;
                if (PAIRED) {
                    const float gt = v[0], up = v[NP - 1];
                    o = __fdividef(gt, 1.0f + __expf(-gt)) * up;
                } else {
                    o = v[0];
                    if (p.residual) o += bf16_bits_to_f32(__ldcg(p.residual + n));
                }
                p.y[n] = f32_to_bf16_bits(o);
            }
        }
    };
    // A tile shared with neighbouring CTAs: every contributor publishes its partial sums and adds
    // its item count to the tile's counter; the contributor that completes the count sums all
    // partial sums in CTA order (deterministic, nobody waits). The counter's old value is not
    // looked at before the next tile has been waited for, so the round trip of the atomic stays
    // off the finalizer's path.
    int pend_li0 = -1, pend_li1 = -1;  // slot 0: the slice's first tile, slot 1: its last tile
    int pend_old0 = 0, pend_old1 = 0;
    auto tile_items = [&](int li) {  // this CTA's items in local tile li
        const int t0 = (rt_first + li) * p.KU;
        return min(i1, t0 + p.KU) - max(i0, t0);
    };
    auto resolve = [&](int& pend_li, int pend_old) {
        const int li = pend_li;
        if (li < 0) return;
        pend_li = -1;
        const int old = __shfl_sync(0xffffffffu, pend_old, 0);
        if (old + tile_items(li) != p.KU) return;  // somebody else completes the tile
        const int rtile = rt_first + li;
        const int t0 = rtile * p.KU, t1 = t0 + p.KU;
        int c_lo = c, c_hi = c;
        while (c_lo > 0 && slice_begin(p, c_lo) > t0) --c_lo;
        while (c_hi + 1 < G && slice_begin(p, c_hi + 1) < t1) ++c_hi;
        float v[NP];
#pragma unroll
        for (int h = 0; h < NP; ++h) v[h] = 0.0f;
        for (int cc = c_lo; cc <= c_hi; ++cc) {
            const int cc_first = fast_div(slice_begin(p, cc), p.div_ku_m, p.div_ku_s);
            const int hs = (rtile == cc_first) ? 0 : 1;
#pragma unroll
            for (int h = 0; h < NP; ++h)
                v[h] += __ldcg(p.partials + (((size_t)cc * 2 + hs) * NP + h) * 16 + (lane & 15));
        }
        if (lane == 0) p.counters[rtile] = 0;
        write_rows(rtile, v);
    };
    // ---- batched variants: a tile is 16 rows x 8 batch columns, lane l holds the four entries
    // 4l .. 4l+3 of its row-major order ----
    auto write_rows_b = [&](int rtile, const float (&v)[NP][4], int rb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = lane * 4 + e, r = idx >> 3, m = (idx & 7) + 8 * rb;
            const int n = rtile * kTileRows + r;
            if (m < p.m_rows && n < p.n_out) {
                float o;
                if (PAIRED) {
                    const float gt = v[0][e], up = v[NP - 1][e];
                    o = __fdividef(gt, 1.0f + __expf(-gt)) * up;
                } else {
                    o = v[0][e];
                    if (p.residual) o += bf16_bits_to_f32(__ldcg(p.residual + (size_t)m * p.n_out + n));
                }
                p.y[(size_t)m * p.n_out + n] = f32_to_bf16_bits(o);
            }
        }
    };
    auto resolve_b = [&](int& pend_li, int pend_old) {
        const int li = pend_li;
        if (li < 0) return;
        pend_li = -1;
        const int old = __shfl_sync(0xffffffffu, pend_old, 0);
        if (old + tile_items(li) != p.KU) return;
        const int rtile = rt_first + li;
        const int t0 = rtile * p.KU, t1 = t0 + p.KU;
        int c_lo = c, c_hi = c;
        while (c_lo > 0 && slice_begin(p, c_lo) > t0) --c_lo;
        while (c_hi + 1 < G && slice_begin(p, c_hi + 1) < t1) ++c_hi;
#pragma unroll 1
        for (int rb = 0; rb < RB; ++rb) {
            float v[NP][4];
#pragma unroll
            for (int h = 0; h < NP; ++h)
#pragma unroll
                for (int e = 0; e < 4; ++e) v[h][e] = 0.0f;
            for (int cc = c_lo; cc <= c_hi; ++cc) {
                const int cc_first = fast_div(slice_begin(p, cc), p.div_ku_m, p.div_ku_s);
                const int hs = (rtile == cc_first) ? 0 : 1;
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    const float4 q = __ldcg(reinterpret_cast<const float4*>(
                        p.partials + ((((size_t)cc * 2 + hs) * NP + h) * RB + rb) * 128) + lane);
                    v[h][0] += q.x; v[h][1] += q.y; v[h][2] += q.z; v[h][3] += q.w;
                }
            }
            write_rows_b(rtile, v, rb);
        }
        if (lane == 0) p.counters[rtile] = 0;
    };
    auto finalize_tile_b = [&](int li) {
        const int rtile = rt_first + li;
        const int items = tile_items(li);
        const int hslot = (li == 0) ? 0 : 1;
#pragma unroll 1
        for (int rb = 0; rb < RB; ++rb) {
            float v[NP][4];
#pragma unroll
            for (int h = 0; h < NP; ++h) {
                uint4 q;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                             : "r"(a_slots + (uint32_t)((li * NP + h) * kSlotBytes + rb * 512 + lane * 16)));
                v[h][0] = __uint_as_float(q.x); v[h][1] = __uint_as_float(q.y);
                v[h][2] = __uint_as_float(q.z); v[h][3] = __uint_as_float(q.w);
            }
            if (items == p.KU) {
                write_rows_b(rtile, v, rb);
                continue;
            }
#pragma unroll
            for (int h = 0; h < NP; ++h)
                reinterpret_cast<float4*>(p.partials + ((((size_t)c * 2 + hslot) * NP + h) * RB + rb) * 128)[lane] =
                    make_float4(v[h][0], v[h][1], v[h][2], v[h][3]);
        }
        if (items == p.KU) return;
        __syncwarp();
        int old = 0;
        if (lane == 0)
            asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;"
                         : "=r"(old) : "l"(p.counters + rtile), "r"(items) : "memory");
        if (hslot == 0) {
            pend_li0 = li;
            pend_old0 = old;
        } else {
            pend_li1 = li;
            pend_old1 = old;
        }
    };
    auto finalize_tile = [&](int li) {
        const int r = lane & 15;
        const int rtile = rt_first + li;
        float v[NP];
#pragma unroll
        for (int h = 0; h < NP; ++h) {
            const uint32_t sl = a_slots + (uint32_t)(((li * NP + h) * W) * 16 + r) * 4u;
            float part[W];
#pragma unroll
            for (int w = 0; w < W; ++w) part[w] = lds_f32(sl + w * 64);
            float sacc = 0.0f;
#pragma unroll
            for (int w = 0; w < W; ++w) sacc += part[w];
            v[h] = sacc;
        }
        const int items = tile_items(li);
        if (items == p.KU) {
            write_rows(rtile, v);
            return;
        }
        const int hslot = (li == 0) ? 0 : 1;
        if (lane < 16) {
#pragma unroll
            for (int h = 0; h < NP; ++h)
                p.partials[(((size_t)c * 2 + hslot) * NP + h) * 16 + r] = v[h];
        }
        __syncwarp();
        int old = 0;
        if (lane == 0)
            asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;"
                         : "=r"(old) : "l"(p.counters + rtile), "r"(items) : "memory");
        if (hslot == 0) {
            pend_li0 = li;
            pend_old0 = old;
        } else {
            pend_li1 = li;
            pend_old1 = old;
        }
    };

    if (warp == W) {
        // ---------------- producer: sets up the barriers, then one thread keeps the ring full ----
        if (lane < p.stages) {
            mbar_init(&full[lane], 1);
            mbar_init(&empty[lane], W);
        }
        if (lane < kMaxLocalTiles) mbar_init(&tile_bar[lane], W);
        if (lane == 0) mbar_init(x_ready, 1);
        if (lane == 0) *abort_flag = 0;
        mbar_fence_init();
        __syncwarp();
        // the other warps pick the initialised barriers up at their first CTA-wide barrier; the
        // producer does not wait for them
        asm volatile("bar.arrive 2, %0;" ::"n"(kStreamThreads) : "memory");
        if (lane == 0) {
            int issued = 0;
            int s = 0;
            uint32_t ph = 0;  // (g / stages) & 1
            const int early_stages = max(1, min(p.stages, kEarlyBytes / stage_bytes));
            for (int g = 0; g < n_groups; ++g) {
                // Only the first stages are requested before x has arrived: the load of x slows
                // down under the copies' traffic (measured), and it is the one load every
                // consumer waits for once the previous kernel has finished.
                if (g == early_stages && !mbar_wait_bounded(x_ready, 0, p.spin_limit)) break;
                if (g >= p.stages) {
                    if (*(volatile int*)abort_flag) break;
                    if (!mbar_wait_bounded(&empty[s], ph ^ 1u, p.spin_limit)) {
                        atomicExch(p.status, kStatusTimeoutEmpty);
                        *(volatile int*)abort_flag = 1;
                        break;
                    }
                }
                const int v0 = g * kStageItems;
                const int cnt = min(kStageItems, len - v0);
                uint8_t* dst = gen + stage_addr(s);
                mbar_expect_tx(&full[s], (uint32_t)cnt * unit_stride * NP);
                // up to two contiguous pieces (the traversal wraps from the tail tile to the front)
                const int n1 = v0 < tail_len ? min(cnt, tail_len - v0) : 0;
                if (n1 > 0) {
                    const size_t it = (size_t)(tail0 + v0);
                    bulk_g2s(dst, p.units + it * unit_stride, (uint32_t)n1 * unit_stride, &full[s]);
                    if (PAIRED)
                        bulk_g2s(dst + half_bytes,
                                 p.units + (it + (size_t)p.pair_rt_offset * p.KU) * unit_stride,
                                 (uint32_t)n1 * unit_stride, &full[s]);
                }
                if (cnt > n1) {
                    const size_t it = (size_t)(i0 + (v0 + n1 - tail_len));
                    bulk_g2s(dst + n1 * unit_stride, p.units + it * unit_stride,
                             (uint32_t)(cnt - n1) * unit_stride, &full[s]);
                    if (PAIRED)
                        bulk_g2s(dst + half_bytes + n1 * unit_stride,
                                 p.units + (it + (size_t)p.pair_rt_offset * p.KU) * unit_stride,
                                 (uint32_t)(cnt - n1) * unit_stride, &full[s]);
                }
                issued = g + 1;
                if (++s == p.stages) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            // never leave the CTA with copies still landing in its shared memory
            // (walk back from the last issued group: s, ph describe group `issued`)
            for (int g = issued - 1; g >= max(0, issued - p.stages); --g) {
                if (--s < 0) {
                    s = p.stages - 1;
                    ph ^= 1u;
                }
                mbar_wait_bounded(&full[s], ph, p.spin_limit);
            }
        }
        return;
    }

    if (warp == W + 1) {
        // ---------------- finalizer: completes row tiles off the consumers' critical path -------
        asm volatile("bar.sync 2, %0;" ::"n"(kStreamThreads) : "memory");
        // the exchange's epoch is advanced by the previous kernel on the stream
        if (!PAIRED && p.peer_world > 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        // tiles complete in traversal order: the slice's last tile, then the others from the front
        for (int q = 0; q < n_local; ++q) {
            const int li = (q == 0) ? n_local - 1 : q - 1;
            bool ok = mbar_try_wait(&tile_bar[li], 0);
            if (!ok) {
                const long long t0 = clock64();
                while (!ok) {
#pragma unroll 1
                    for (int i = 0; i < 64 && !ok; ++i) {
                        __nanosleep(40);
                        ok = mbar_try_wait(&tile_bar[li], 0);
                    }
                    if (ok) break;
                    if (*(volatile int*)abort_flag) break;
                    if (clock64() - t0 > p.spin_limit) {
                        atomicExch(p.status, kStatusTimeoutFull);
                        break;
                    }
                }
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            // counters added to before the wait above have answered by now
            if (BATCH) {
                resolve_b(pend_li0, pend_old0);
                resolve_b(pend_li1, pend_old1);
                finalize_tile_b(li);
            } else {
                resolve(pend_li0, pend_old0);
                resolve(pend_li1, pend_old1);
                finalize_tile(li);
            }
        }
        if (BATCH) {
            resolve_b(pend_li0, pend_old0);
            resolve_b(pend_li1, pend_old1);
        } else {
            resolve(pend_li0, pend_old0);
            resolve(pend_li1, pend_old1);
        }
        if (!PAIRED && !BATCH && p.peer_world > 0 && p.peer_inline) peer_reduce_inline();
        return;
    }

    // ---------------- consumers ----------------
    // Second-level scales this CTA can need: one window of consecutive nested_absmax entries per
    // half (gate/plain rows, up rows), copied to shared memory so the absmax chain has no global
    // load in it. A window that does not fit is read from global memory instead. Warp 8 + h
    // prepares the window of half h and publishes its base and validity.
    static_assert(W >= 8 + NP, "window warps");
    static_assert(kNabsWindow == 256, "eight window entries per lane");
    float win_reg[8];
    unsigned wwin_lo = 0;
    bool wwin_ok = false;
    const int wh = warp - 8;  // the half this warp prepares, if in [0, NP)
    if (KIND == kAbsmaxCodes && wh >= 0 && wh < NP) {
        const int n_a = min((rt_first + wh * p.pair_rt_offset) * kTileRows, p.n_rows - 1);
        const int n_b = min((rt_last + wh * p.pair_rt_offset) * kTileRows + kTileRows - 1, p.n_rows - 1);
        const unsigned f_lo = segment_row(p.sp, n_a).flat;
        const unsigned f_hi = segment_row(p.sp, n_b).flat + ((unsigned)(p.KU - 1) >> p.sp.blk_shift);
        wwin_lo = f_lo >> p.sp.nbs_shift;
        const unsigned cnt = (f_hi >> p.sp.nbs_shift) - wwin_lo + 1;
        wwin_ok = cnt <= (unsigned)kNabsWindow;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            win_reg[i] = 0.0f;
            if (wwin_ok && (unsigned)(lane + 32 * i) < cnt) win_reg[i] = __ldg(p.sp.nabs + wwin_lo + lane + 32 * i);
        }
    }
    auto zero_slots = [&]() {
        constexpr int kSlotVecs = kMaxLocalTiles * NP * kSlotBytes / 16;
#pragma unroll
        for (int i = 0; i < (kSlotVecs + W * 32 - 1) / (W * 32); ++i) {
            const int q = tid + i * W * 32;
            if (q < kSlotVecs)
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(a_slots + 16u * q), "r"(0u) : "memory");
        }
    };

    const int gq = lane >> 2;  // row inside the tile (and row + 8)
    const int t = lane & 3;
    const uint32_t lane_base = a_lut + ((uint32_t)lane << 2);
    const uint32_t w_off = (uint32_t)(gq * 32 + 8 * t);  // this lane's 8 bytes inside a unit
    // absmax decode: the four lanes of a quad (same gq) decode the four scales that the quad's
    // lane t = 0 applies: lane t owns row gq + 8*(t & 1) of the gate/plain unit (t < 2) or of the
    // up unit (t >= 2); an unpaired launch uses t = 0, 1 only
    const int dhalf = PAIRED ? (t >> 1) : 0;
    const int drow = gq + 8 * (t & 1);
    const uint32_t code_off = (uint32_t)(dhalf * half_bytes + kUnitNibbleBytes + drow);
    const uint32_t my_win = a_nabsw + (uint32_t)(dhalf * kNabsWindow) * 4u;

    // single row: [h][row gq / gq + 8] in lanes t = 0; batched: [h][2 * (row) + (column 2t / 2t+1)]
    constexpr int NACC = BATCH ? 4 * RB : 2;  // batched: [4 * block + e]
    float acc[NP][NACC];
#pragma unroll
    for (int h = 0; h < NP; ++h)
#pragma unroll
        for (int e = 0; e < NACC; ++e) acc[h][e] = 0.0f;
    int cur_li = -1;
    unsigned done_mask = 0;  // local tiles this warp has signed off

    // The items of a CTA are dealt to the warps round-robin: this warp takes the traversal
    // positions v = warp, warp + W, warp + 2W, ... (IPW of them in every stage), so the warps'
    // item counts differ by at most one.
    int v = warp;
    int kb = 0, rt = rt_first;
    unsigned d_flat = 0;
    float d_off = 0.0f;
    auto locate = [&](int vv) {  // (kb, rt) of traversal position vv
        const int it = vv < tail_len ? tail0 + vv : i0 + (vv - tail_len);
        rt = fast_div(it, p.div_ku_m, p.div_ku_s);
        kb = it - rt * p.KU;
    };
    // Set-up that nothing needs before the first work item: it runs after the loads of x have been
    // issued, under their latency (x can only be asked for once the previous kernel is done).
    // absmax row base and offset of this lane's row in every local tile: warp li prepares tile li
    auto tile_tables = [&]() {
      if (KIND == kAbsmaxCodes && warp < n_local) {
        // rows past the end of the linear (padding of the last tile) borrow the last row's scale
        const int n = min((rt_first + warp + dhalf * p.pair_rt_offset) * kTileRows + drow, p.n_rows - 1);
        const SegmentRow sr = segment_row(p.sp, n);
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a_tinfo + (uint32_t)(warp * 32 + lane) * 8u),
                     "r"(sr.flat), "r"(__float_as_uint(sr.offset)) : "memory");
      }
    };
    auto refresh = [&]() {  // absmax row base of this lane for row tile rt
        if (KIND == kAbsmaxCodes) {
            const uint2 ti = lds_v2(a_tinfo + (uint32_t)((rt - rt_first) * 32 + lane) * 8u);
            d_flat = ti.x;
            d_off = __uint_as_float(ti.y);
        }
    };
    auto late_setup = [&]() {
        zero_slots();
        tile_tables();
        if (v < len) locate(v);
    };
    const int kb_step = p.kb_step;  // from one item of this warp to its next
    const int rt_step = p.rt_step;

    // the static tables go to shared memory; after the CTA-wide barrier the lookup table is built
    if (tid < 256) {
        // byte value tid -> bf16 pair of its two nibbles; low half = first weight (HIGH nibble)
        const uint32_t ptab_reg = (uint32_t)f32_to_bf16_bits(q_hi) | ((uint32_t)f32_to_bf16_bits(q_lo) << 16);
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(a_ptab + 4u * tid), "r"(ptab_reg) : "memory");
        if (KIND == kAbsmaxCodes) sts_f32(a_nmap + 4u * tid, nmap_reg);
    }
    if (KIND == kAbsmaxCodes && wh >= 0 && wh < NP && lane == 0)
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a_info + 8u * wh), "r"(wwin_lo), "r"(wwin_ok ? 1u : 0u) : "memory");
    asm volatile("bar.sync 2, %0;" ::"n"(kStreamThreads) : "memory");
    unsigned my_win_lo = 0;
    bool my_win_ok = false;
    if (KIND == kAbsmaxCodes) {
        const uint2 info = lds_v2(a_info + 8u * dhalf);
        my_win_lo = info.x;
        my_win_ok = info.y != 0u;
    }
    {
        // Table rows are 128 bytes (one word per lane) on a 256-byte pitch. One 16-byte store per
        // lane fills four rows: lane l writes piece l % 8 of row 4*r4 + l / 8.
        static_assert(64 % W == 0, "table rows per warp");
        uint32_t pv[64 / W];
#pragma unroll
        for (int i = 0; i < 64 / W; ++i)
            pv[i] = lds_u32(a_ptab + 4u * (uint32_t)((warp + i * W) * 4 + (lane >> 3)));
#pragma unroll
        for (int i = 0; i < 64 / W; ++i) {
            const int b = (warp + i * W) * 4 + (lane >> 3);
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(a_lut + (uint32_t)b * 256u +
                                                                         (uint32_t)(lane & 7) * 16u),
                         "r"(pv[i])
                         : "memory");
        }
    }
    if (KIND == kAbsmaxCodes && wh >= 0 && wh < NP && wwin_ok) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            sts_f32(a_nabsw + (uint32_t)(wh * kNabsWindow + lane + 32 * i) * 4u, win_reg[i]);
    }
    // x is the only input that may come from the previous kernel on the stream: everything above
    // (and the producer's weight copies) ran without waiting for it
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // element k = 64*kb + 16*j + 4*t + e goes to fragment order: 16-byte slot (kb*2 + j/2)*4 + t
    // holds tiles j = 2*(j/2) and +1 for lane column t
    const int n8 = p.x_bytes >> 3;
    const uint2* xg = reinterpret_cast<const uint2*>(p.x);
    auto slot_of = [&](int q4) {
        const int kbx = q4 >> 4, j = (q4 >> 2) & 3, tt = q4 & 3;
        return a_xs + (uint32_t)((((kbx * 2 + (j >> 1)) * 4 + tt) * 2 + (j & 1)) * 8);
    };
    auto sts_x = [&](int q4, uint2 xv) {
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(slot_of(q4)), "r"(xv.x), "r"(xv.y) : "memory");
    };
    if (BATCH || p.norm_w != nullptr) late_setup();
    if (!BATCH && p.norm_w != nullptr) {
        // ---- residual add + RMSNorm while staging x ----
        static_assert(W <= 16, "per-warp sums");
        const uint2* ag = reinterpret_cast<const uint2*>(p.norm_add);
        const uint2* wg = reinterpret_cast<const uint2*>(p.norm_w);
        auto load_v = [&](int q4, float (&vv)[4]) {
            const uint2 a = __ldcg(xg + q4);
            uint2 b = make_uint2(0u, 0u);
            if (ag) b = __ldcg(ag + q4);
            vv[0] = __uint_as_float(a.x << 16) + __uint_as_float(b.x << 16);
            vv[1] = __uint_as_float(a.x & 0xffff0000u) + __uint_as_float(b.x & 0xffff0000u);
            vv[2] = __uint_as_float(a.y << 16) + __uint_as_float(b.y << 16);
            vv[3] = __uint_as_float(a.y & 0xffff0000u) + __uint_as_float(b.y & 0xffff0000u);
        };
        auto sq = [](const float (&vv)[4]) { return vv[0] * vv[0] + vv[1] * vv[1] + vv[2] * vv[2] + vv[3] * vv[3]; };
        float v0[4] = {0.f, 0.f, 0.f, 0.f}, v1[4] = {0.f, 0.f, 0.f, 0.f};
        float ss = 0.0f;
        if (tid < n8) {
            load_v(tid, v0);
            ss += sq(v0);
        }
        if (tid + W * 32 < n8) {
            load_v(tid + W * 32, v1);
            ss += sq(v1);
        }
        for (int q4 = tid + 2 * W * 32; q4 < n8; q4 += W * 32) {
            float vv[4];
            load_v(q4, vv);
            ss += sq(vv);
        }
        // the same fixed reduction order in every CTA: shuffle tree, then the warp sums in order
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) sts_f32(a_red + 4u * warp, ss);
        asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < W; ++w) total += lds_f32(a_red + 4u * w);
        const float inv_rms = rsqrtf(total / (float)p.K + p.norm_eps);
        const bool renorm_from_stored = p.norm_add != nullptr && p.K != 1024;
        auto emit = [&](int q4, const float (&vv)[4]) {
            const uint2 wq = __ldg(wg + q4);
            const float w0 = __uint_as_float(wq.x << 16), w1 = __uint_as_float(wq.x & 0xffff0000u);
            const float w2 = __uint_as_float(wq.y << 16), w3 = __uint_as_float(wq.y & 0xffff0000u);
            uint2 hq;  // the updated residual stream bf16(v)
            hq.x = (uint32_t)f32_to_bf16_bits(vv[0]) | ((uint32_t)f32_to_bf16_bits(vv[1]) << 16);
            hq.y = (uint32_t)f32_to_bf16_bits(vv[2]) | ((uint32_t)f32_to_bf16_bits(vv[3]) << 16);
            // the reference's single-row add+RMSNorm normalises what it stored (bf16) unless H == 1024
            // (src/ops/NormOps.cpp:189-240 against :152-187); without an added tensor v is bf16 already
            const float n0 = renorm_from_stored ? __uint_as_float(hq.x << 16) : vv[0];
            const float n1 = renorm_from_stored ? __uint_as_float(hq.x & 0xffff0000u) : vv[1];
            const float n2 = renorm_from_stored ? __uint_as_float(hq.y << 16) : vv[2];
            const float n3 = renorm_from_stored ? __uint_as_float(hq.y & 0xffff0000u) : vv[3];
            uint2 o;
            o.x = (uint32_t)f32_to_bf16_bits(n0 * inv_rms * w0) | ((uint32_t)f32_to_bf16_bits(n1 * inv_rms * w1) << 16);
            o.y = (uint32_t)f32_to_bf16_bits(n2 * inv_rms * w2) | ((uint32_t)f32_to_bf16_bits(n3 * inv_rms * w3) << 16);
            sts_x(q4, o);
            if (c == 0 && p.norm_hidden_out) reinterpret_cast<uint2*>(p.norm_hidden_out)[q4] = hq;
        };
        if (tid < n8) emit(tid, v0);
        if (tid + W * 32 < n8) emit(tid + W * 32, v1);
        for (int q4 = tid + 2 * W * 32; q4 < n8; q4 += W * 32) {
            float vv[4];
            load_v(q4, vv);
            emit(q4, vv);
        }
    }
    const bool plain_x = !BATCH && p.norm_w == nullptr;
    uint2 xv0 = make_uint2(0u, 0u), xv1 = make_uint2(0u, 0u);
    if (plain_x && tid < n8) xv0 = __ldcg(xg + tid);
    if (plain_x && tid + W * 32 < n8) xv1 = __ldcg(xg + tid + W * 32);
    if (plain_x) late_setup();

    if (plain_x && tid < n8) sts_x(tid, xv0);
    if (plain_x && tid + W * 32 < n8) sts_x(tid + W * 32, xv1);
    for (int q4 = tid + 2 * W * 32; plain_x && q4 < n8; q4 += 2 * W * 32) {
        const int q5 = q4 + W * 32;
        const uint2 v0 = __ldcg(xg + q4);
        uint2 v1 = make_uint2(0u, 0u);
        if (q5 < n8) v1 = __ldcg(xg + q5);
        sts_x(q4, v0);
        if (q5 < n8) sts_x(q5, v1);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(W * 32) : "memory");
    if (tid == 0) mbar_arrive(x_ready);  // the producer may now fill the rest of the ring
    if (v < len) refresh();

    // every warp signs off every local tile exactly once, after its last contribution to it
    auto sign_off = [&](int li) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&tile_bar[li]);
        done_mask |= 1u << li;
    };
    auto flush_current = [&]() {
        if (cur_li >= 0) {
            if constexpr (BATCH != 0) {
                // every warp adds its share of the tile into one fp32 tile [16 rows][8 columns] per block
#pragma unroll
                for (int h = 0; h < NP; ++h) {
#pragma unroll
                    for (int rb = 0; rb < RB; ++rb) {
                        const uint32_t tb = a_slots + (uint32_t)((cur_li * NP + h) * kSlotBytes + rb * 512);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t idx = (uint32_t)((gq + 8 * (e >> 1)) * 8 + 2 * t + (e & 1));
                            asm volatile("red.shared.add.f32 [%0], %1;" ::"r"(tb + 4u * idx), "f"(acc[h][4 * rb + e])
                                         : "memory");
                        }
                    }
                }
            } else if (t == 0) {
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    const uint32_t sl = a_slots + (uint32_t)(((cur_li * NP + h) * W + warp) * 16) * 4u;
                    sts_f32(sl + 4u * gq, acc[h][0]);
                    sts_f32(sl + 4u * (gq + 8), acc[h][1]);
                }
            }
            sign_off(cur_li);
        }
#pragma unroll
        for (int h = 0; h < NP; ++h)
#pragma unroll
            for (int e = 0; e < NACC; ++e) acc[h][e] = 0.0f;
    };

    uint4 xq0 = make_uint4(0u, 0u, 0u, 0u), xq1 = make_uint4(0u, 0u, 0u, 0u);
    const uint32_t x_lane = (gq == 0) ? 1u : 0u;
    bool failed = false;
    int s = 0;
    uint32_t ph = 0;  // (g / stages) & 1
    for (int g = 0; g < n_groups; ++g) {
        if (!mbar_wait_bounded(&full[s], ph, p.spin_limit)) {
            atomicExch(p.status, kStatusTimeoutFull);
            *(volatile int*)abort_flag = 1;
            failed = true;
            break;
        }
        const uint32_t ua0 = stage_addr(s) + (uint32_t)warp * unit_stride;
#pragma unroll
        for (int i = 0; i < IPW; ++i) {
            if (v < len) {
                const uint32_t ua = ua0 + (uint32_t)(i * W) * unit_stride;
                // ---- one work item: unit (rt, kb) [and its up partner] ----
                // x fragments: two 16-byte loads (tiles j = 0,1 and j = 2,3) in the four lanes
                // that hold batch column 0 of the tile; the other columns stay zero and are never
                // read back. A 16-byte load is served a quarter warp at a time, so the
                // predicated pair costs two shared-memory wavefronts instead of eight.
                uint4 xr0[RB > 1 ? RB - 1 : 1], xr1[RB > 1 ? RB - 1 : 1];  // blocks 1 .. RB-1
                if (BATCH) {
                    // batch row gq (+ 8 per block) of x, straight from L2 (coherent loads: x may be
                    // the previous kernel's output): tile j wants k = 64 kb + 16 j + 4 t + {0..3}
                    auto load_block = [&](int rb, uint4& q0, uint4& q1) {
                        const int row = gq + 8 * rb;
                        const uint2* xr =
                            reinterpret_cast<const uint2*>(p.x + (size_t)row * p.K + (size_t)kb * 64 + 4 * t);
                        uint2 xb0 = make_uint2(0u, 0u), xb1 = xb0, xb2 = xb0, xb3 = xb0;
                        if (row < p.m_rows) {
                            xb0 = __ldcg(xr);
                            xb1 = __ldcg(xr + 4);
                            xb2 = __ldcg(xr + 8);
                            xb3 = __ldcg(xr + 12);
                        }
                        q0 = make_uint4(xb0.x, xb0.y, xb1.x, xb1.y);
                        q1 = make_uint4(xb2.x, xb2.y, xb3.x, xb3.y);
                    };
                    load_block(0, xq0, xq1);
#pragma unroll
                    for (int rb = 1; rb < RB; ++rb) load_block(rb, xr0[rb - 1], xr1[rb - 1]);
                } else {
                const uint32_t xa = a_xs + (uint32_t)kb * 128u + 16u * t;
                    asm volatile(
                        "{\n\t.reg .pred q;\n\t"
                        "setp.ne.u32 q, %9, 0;\n\t"
                        "@q ld.shared.v4.u32 {%0,%1,%2,%3}, [%8];\n\t"
                        "@q ld.shared.v4.u32 {%4,%5,%6,%7}, [%8+64];\n\t}"
                        : "+r"(xq0.x), "+r"(xq0.y), "+r"(xq0.z), "+r"(xq0.w), "+r"(xq1.x), "+r"(xq1.y),
                          "+r"(xq1.z), "+r"(xq1.w)
                        : "r"(xa), "r"(x_lane));
                }
                float am0[NP], am1[NP];
                if (KIND == kAbsmaxCodes) {
                    const unsigned code = lds_u8(ua + code_off);
                    const unsigned flat = d_flat + ((unsigned)kb >> p.sp.blk_shift);
                    const unsigned sidx = flat >> p.sp.nbs_shift;
                    const float scale = my_win_ok ? lds_f32(my_win + (sidx - my_win_lo) * 4u)
                                                  : __ldg(p.sp.nabs + sidx);
                    const float am = __fadd_rn(__fmul_rn(lds_f32(a_nmap + 4u * code), scale), d_off);
                    // lane t = 0 of each quad collects the quad's scales (the other lanes get
                    // values they never use)
#pragma unroll
                    for (int h = 0; h < NP; ++h) {
                        if (BATCH) {  // every lane of the quad uses all four scales
                            am0[h] = __shfl_sync(0xffffffffu, am, (lane & ~3) | (2 * h));
                            am1[h] = __shfl_sync(0xffffffffu, am, (lane & ~3) | (2 * h + 1));
                        } else {
                            am0[h] = (h == 0) ? am : __shfl_down_sync(0xffffffffu, am, 2 * h);
                            am1[h] = __shfl_down_sync(0xffffffffu, am, 2 * h + 1);
                        }
                    }
                } else {
#pragma unroll
                    for (int h = 0; h < NP; ++h) {
                        am0[h] = lds_f32(ua + h * half_bytes + kUnitNibbleBytes + 4u * gq);
                        am1[h] = lds_f32(ua + h * half_bytes + kUnitNibbleBytes + 4u * (gq + 8));
                    }
                }
                float c0[NP][4], c1[NP][4];
                // both halves' packed weights first, then all table lookups (independent loads),
                // then the tiles: j = 0: bytes 0,1 of .x ; j = 1: bytes 2,3 of .x ; j = 2,3: .y
                uint2 wl[NP], wu[NP];
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    wl[h] = lds_v2(ua + h * half_bytes + w_off);
                    wu[h] = lds_v2(ua + h * half_bytes + w_off + 256u);
                }
                uint32_t a[NP][16];
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    const uint2 l = wl[h], u = wu[h];
                    a[h][0] = lut_pair<0>(l.x, lane_base);  a[h][1] = lut_pair<0>(u.x, lane_base);
                    a[h][2] = lut_pair<1>(l.x, lane_base);  a[h][3] = lut_pair<1>(u.x, lane_base);
                    a[h][4] = lut_pair<2>(l.x, lane_base);  a[h][5] = lut_pair<2>(u.x, lane_base);
                    a[h][6] = lut_pair<3>(l.x, lane_base);  a[h][7] = lut_pair<3>(u.x, lane_base);
                    a[h][8] = lut_pair<0>(l.y, lane_base);  a[h][9] = lut_pair<0>(u.y, lane_base);
                    a[h][10] = lut_pair<1>(l.y, lane_base); a[h][11] = lut_pair<1>(u.y, lane_base);
                    a[h][12] = lut_pair<2>(l.y, lane_base); a[h][13] = lut_pair<2>(u.y, lane_base);
                    a[h][14] = lut_pair<3>(l.y, lane_base); a[h][15] = lut_pair<3>(u.y, lane_base);
                }
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    mma_bf16_16816_init(c0[h], a[h][0], a[h][1], a[h][2], a[h][3], xq0.x, xq0.y);
                    mma_bf16_16816_init(c1[h], a[h][4], a[h][5], a[h][6], a[h][7], xq0.z, xq0.w);
                }
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    mma_bf16_16816(c0[h], a[h][8], a[h][9], a[h][10], a[h][11], xq1.x, xq1.y);
                    mma_bf16_16816(c1[h], a[h][12], a[h][13], a[h][14], a[h][15], xq1.z, xq1.w);
                }
                // ---- accumulate into the current row tile (switching tiles is rare) ----
                const int li = rt - rt_first;
                if (li != cur_li) {
                    flush_current();
                    if (v >= tail_len) {
                        // the front part runs through the tiles in order and never returns to
                        // the slice's last tile: sign off what this warp will not touch again
                        for (int q = 0; q < li; ++q)
                            if (!((done_mask >> q) & 1u)) sign_off(q);
                        if (!((done_mask >> (n_local - 1)) & 1u)) sign_off(n_local - 1);
                    }
                    cur_li = li;
                }
#pragma unroll
                for (int h = 0; h < NP; ++h) {
                    if constexpr (BATCH != 0) {
                        acc[h][0] = fmaf(am0[h], c0[h][0] + c1[h][0], acc[h][0]);
                        acc[h][1] = fmaf(am0[h], c0[h][1] + c1[h][1], acc[h][1]);
                        acc[h][2] = fmaf(am1[h], c0[h][2] + c1[h][2], acc[h][2]);
                        acc[h][3] = fmaf(am1[h], c0[h][3] + c1[h][3], acc[h][3]);
                    } else {
                        acc[h][0] = fmaf(am0[h], c0[h][0] + c1[h][0], acc[h][0]);
                        acc[h][1] = fmaf(am1[h], c0[h][2] + c1[h][2], acc[h][1]);
                    }
                }
                if constexpr (RB > 1) {
                    // the other row blocks against the same decoded fragments
#pragma unroll
                    for (int rb = 1; rb < RB; ++rb) {
                        const uint4 q0 = xr0[rb - 1], q1 = xr1[rb - 1];
#pragma unroll
                        for (int h = 0; h < NP; ++h) {
                            mma_bf16_16816_init(c0[h], a[h][0], a[h][1], a[h][2], a[h][3], q0.x, q0.y);
                            mma_bf16_16816_init(c1[h], a[h][4], a[h][5], a[h][6], a[h][7], q0.z, q0.w);
                            mma_bf16_16816(c0[h], a[h][8], a[h][9], a[h][10], a[h][11], q1.x, q1.y);
                            mma_bf16_16816(c1[h], a[h][12], a[h][13], a[h][14], a[h][15], q1.z, q1.w);
                            acc[h][4 * rb + 0] = fmaf(am0[h], c0[h][0] + c1[h][0], acc[h][4 * rb + 0]);
                            acc[h][4 * rb + 1] = fmaf(am0[h], c0[h][1] + c1[h][1], acc[h][4 * rb + 1]);
                            acc[h][4 * rb + 2] = fmaf(am1[h], c0[h][2] + c1[h][2], acc[h][4 * rb + 2]);
                            acc[h][4 * rb + 3] = fmaf(am1[h], c0[h][3] + c1[h][3], acc[h][4 * rb + 3]);
                        }
                    }
                }
                // ---- this warp's next item: W positions further along the traversal ----
                const int vn = v + W;
                if (vn < len) {
                    const int rt_old = rt;
                    if (v < tail_len && vn >= tail_len) {
                        locate(vn);  // wrapped from the tail tile to the front of the slice
                    } else {
                        kb += kb_step;
                        rt += rt_step;
                        if (kb >= p.KU) {
                            kb -= p.KU;
                            ++rt;
                        }
                    }
                    if (rt != rt_old) refresh();
                }
                v = vn;
            }
        }
        // the stage's shared memory is no longer needed by this warp
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (++s == p.stages) {
            s = 0;
            ph ^= 1u;
        }
    }
    if (failed) return;
    // last contribution of this warp, then sign off whatever it never touched
    flush_current();
    cur_li = -1;
    for (int q = 0; q < n_local; ++q)
        if (!((done_mask >> q) & 1u)) sign_off(q);
}

struct StreamPlan {
    int grid = 0;
    int stages = 0;
    int stages_b = 0;
    int smem = 0;
    int x_in_b = 0;
    bool ok = false;
};

// Grid and ring depth for one launch. The slice of a CTA may touch at most kMaxLocalTiles row
// tiles; long outputs therefore get a grid that is a multiple of the SM count (CTAs never
// wait on each other, so they need not be co-resident).
// Shared memory the system keeps at the bottom of every block's window: the dynamic allocation
// of a kernel without static shared memory starts right after it.
int smem_window_base() {
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

constexpr int kStreamSmemBytes = 227 * 1024;  // every launch asks for the whole budget

StreamPlan stream_plan(const AilaNf4Linear& w, bool paired, int64_t ff_pair, int sm_count, int row_blocks = 1) {
    StreamPlan pl;
    const int np = paired ? 2 : 1;
    const int stage_bytes = kStageItems * w.unit_stride * np + (paired ? kPairSkewBytes : 0);
    const int x_bytes = (int)((w.K * 2 + 15) / 16 * 16);
    // Shared-window map: region A = [base, 64 KB): barriers, code books, tile tables, slots, x if
    // it fits, then ring stages in what is left; table = [64 KB, 128 KB); region B = [128 KB,
    // base + budget): x otherwise, then ring stages.
    const int base = (smem_window_base() + 15) / 16 * 16;
    const int a_fixed = base + 400 + 64 + 16 + 64 + 1024 + 2 * kNabsWindow * 4 + 1024 +
                        kMaxLocalTiles * 32 * 8 + kMaxLocalTiles * np * stream_slot_bytes(row_blocks);
    pl.x_in_b = (a_fixed + x_bytes > 65536) ? 1 : 0;
    const int ring_a = (a_fixed + (pl.x_in_b ? 0 : x_bytes) + 127) / 128 * 128;
    const int stages_a = ring_a < 65536 ? (65536 - ring_a) / stage_bytes : 0;
    const int ring_b = 131072 + (pl.x_in_b ? x_bytes : 0);
    const int end_b = smem_window_base() + kStreamSmemBytes;
    pl.stages_b = end_b > ring_b ? (end_b - ring_b) / stage_bytes : 0;
    if (pl.stages_b > kMaxStages) pl.stages_b = kMaxStages;
    pl.stages = pl.stages_b + stages_a;
    if (pl.stages > kMaxStages) pl.stages = kMaxStages;
    if (pl.stages < 2) return pl;
    pl.smem = kStreamSmemBytes;
    const long long rt_work = paired ? ff_pair / kTileRows : w.RT;
    const long long total = rt_work * w.KU;
    if (total <= 0 || total >= (1ll << 31) || sm_count <= 0) return pl;
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

template <int KIND, bool PAIRED, int BATCH>
cudaError_t launch_stream_t(const StreamParams& p, int grid, int smem, cudaStream_t s) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, PAIRED, BATCH>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    // Programmatic dependent launch: the next kernel on the stream may start its set-up (table
    // build, first weight copies) while this one drains; it waits for our completion before it
    // reads x. Disabled with AILA_NF4_PDL=0.
    static const bool use_pdl = [] {
        const char* e = std::getenv("AILA_NF4_PDL");
        return !(e && e[0] == '0');
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<KIND, PAIRED, BATCH>, p);
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


// ------------------------------------------------------------------------------------------
// Small batches (2 .. 32 rows of x) with the x slice in shared memory: gemv_rows_kernel.
//
// The streaming kernel's batched form fetches the x fragments of every work item from L2, 8 bytes
// of L2 traffic per weight byte at 32 rows. Here the work is cut along K instead: a work item is
// (K slice s of 512 columns, row tile rt), the items are ordered slice-major, every CTA takes a
// contiguous range of them and keeps the x slice of ALL rows (8 * RB rows x 1 KB) in shared memory
// while its warps run through the row tiles of that slice. Each warp owns its items (round-robin
// inside the CTA's part of a slice), fetches their units itself with bulk-async copies into a
// private ring of three 4-unit chunks, and adds the finished 16 x (8 RB) partial tile into an fp32
// accumulation tile in global memory with vector reductions. A counter per row tile (per gate/up
// pair) counts the finished items; the warp that completes the count reads the tile back,
// applies the epilogue (residual, or SiLU(gate) * up on the bf16-rounded halves as the reference's
// seq_len > 1 route does), writes y and leaves tile and counter zero for the next launch. Nothing
// waits on another CTA. Column order of the accumulation tile: batch row m sits in column m; the
// x row fed to tensor-core column g of block rb is m = (g/2) * 2RB + 2 rb + g%2, so that a lane's
// 2 RB results are adjacent in memory.
// ------------------------------------------------------------------------------------------
constexpr int kRowsWarps = 16;
constexpr int kRowsThreads = kRowsWarps * 32;
constexpr int kRowsSliceUnits = 8;   // 512 columns of K per slice
constexpr int kRowsChunkUnits = 4;   // units per bulk copy
constexpr int kRowsSlots = 3;        // chunks in flight per warp
constexpr int kRowsSmemBytes = 227 * 1024;

struct RowsParams {
    const uint8_t* units;
    const float* qmap;
    const float* nmap;         // [256] second-level code book (8-bit absmax codes)
    const float4* row_scales;  // [n_rows] {lo, hi, cross, offset} (8-bit absmax codes)
    const uint16_t* x;         // [m_rows][K]
    uint16_t* y;               // [m_rows][n_out]
    const uint16_t* residual;  // [m_rows][n_out] or null (unpaired only)
    float* acc;                // [n_tiles * 16][8 * RB], zero on entry and on exit
    int* counters;             // [n_tiles], zero on entry and on exit
    int* status;
    long long spin_limit;
    int K, KU, n_slices, n_tiles, n_rows, n_out, m_rows;
    int pair_offset;           // row tiles between a gate tile and its up tile; 0 = unpaired
    int total_items, slice_q, slice_r;
    uint32_t div_g_m;
    int div_g_s;
    int smem_bytes;
};

__device__ __forceinline__ int rows_slice_begin(const RowsParams& p, int c) {
    return p.slice_q * c + fast_div(p.slice_r * c, p.div_g_m, p.div_g_s);
}

template <int N>
__device__ __forceinline__ void red_add_f32(float* dst, const float* v);
template <>
__device__ __forceinline__ void red_add_f32<2>(float* dst, const float* v) {
    asm volatile("red.global.add.v2.f32 [%0], {%1,%2};" ::"l"(dst), "f"(v[0]), "f"(v[1]) : "memory");
}
template <>
__device__ __forceinline__ void red_add_f32<4>(float* dst, const float* v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3])
                 : "memory");
}
template <>
__device__ __forceinline__ void red_add_f32<8>(float* dst, const float* v) {
    red_add_f32<4>(dst, v);
    red_add_f32<4>(dst + 4, v + 4);
}

template <int KIND, int RB>
__global__ void __launch_bounds__(kRowsThreads, 1) gemv_rows_kernel(const RowsParams p) {
    constexpr int W = kRowsWarps;
    constexpr int ST = (KIND == kAbsmaxCodes) ? kUnitStrideCodes : kUnitStrideF32;
    constexpr int CH = kRowsChunkUnits * ST;
    constexpr int COLS = 8 * RB;          // batch columns of the accumulation tile
    constexpr int XS_BYTES = COLS * 1024; // x slice: COLS rows of 512 bf16

    // ---- shared-memory map (absolute shared-window addresses) ----
    // [base, 64 KB): barriers, code books, x slice, ring chunks; [64 KB, 128 KB): lookup table;
    // [128 KB, ...): ring chunks
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t a_bar = (base + 15u) & ~15u;  // full[W * kRowsSlots]
    static_assert(W * kRowsSlots * 8 <= 400, "barrier block");
    const uint32_t a_nmap = a_bar + 400;
    const uint32_t a_ptab = a_nmap + 1024;
    const uint32_t a_xs = (a_ptab + 1024 + 1023u) & ~1023u;
    const uint32_t a_ring_a = a_xs + XS_BYTES;
    const uint32_t a_lut = 65536u;
    const uint32_t a_ring_b = 131072u;
    const int n_b = (int)((base + (uint32_t)p.smem_bytes - a_ring_b) / CH);  // chunks behind the table
    auto chunk_addr = [&](int j) {
        return j < n_b ? a_ring_b + (uint32_t)j * CH : a_ring_a + (uint32_t)(j - n_b) * CH;
    };
    uint8_t* gen = smem_raw - base;  // generic pointer to shared-window address 0
    uint64_t* full = reinterpret_cast<uint64_t*>(gen + a_bar);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int gq = lane >> 2;
    const int t = lane & 3;
    const int G = gridDim.x;
    const int c = blockIdx.x;
    const int RT = p.n_tiles;
    const int I0 = rows_slice_begin(p, c);
    const int I1 = rows_slice_begin(p, c + 1);

    {
        const int need_a = W * kRowsSlots - n_b;  // chunks that must fit below the table
        if (base > 2048u || p.smem_bytes < 131072 || (need_a > 0 && a_ring_a + (uint32_t)need_a * CH > 65536u) ||
            a_ring_a > 65536u || I1 <= I0 || G <= 0) {
            if (tid == 0 && I1 > I0) atomicExch(p.status, kStatusBadArgument);
            return;
        }
    }

    // let a dependent launch begin its own set-up; it waits for our completion before it reads x
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- tables: byte value -> bf16 pair, second-level code book; barriers ----
    if (tid < 256) {
        const float q_hi = __ldg(p.qmap + (tid >> 4)), q_lo = __ldg(p.qmap + (tid & 15));
        const uint32_t pr = (uint32_t)f32_to_bf16_bits(q_hi) | ((uint32_t)f32_to_bf16_bits(q_lo) << 16);
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(a_ptab + 4u * tid), "r"(pr) : "memory");
        if (KIND == kAbsmaxCodes) sts_f32(a_nmap + 4u * tid, __ldg(p.nmap + tid));
    }
    if (tid < W * kRowsSlots) mbar_init(&full[tid], 1);
    mbar_fence_init();
    __syncthreads();
    {
        // the bank-private table: rows of 128 bytes (one word per lane) on a 256-byte pitch
        static_assert(64 % W == 0, "table rows per warp");
#pragma unroll
        for (int i = 0; i < 64 / W; ++i) {
            const int b = (warp + i * W) * 4 + (lane >> 3);
            const uint32_t pv = lds_u32(a_ptab + 4u * (uint32_t)b);
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(a_lut + (uint32_t)b * 256u +
                                                                         (uint32_t)(lane & 7) * 16u),
                         "r"(pv)
                         : "memory");
        }
    }
    // (the table is first read after the CTA-wide barrier that follows the first x slice)

    // ---- this warp's sequence of chunks: its items slice by slice, two chunks per item ----
    const int s_first = I0 / RT;  // (host guarantees the quotient is small: plain division)
    const int s_last = (I1 - 1) / RT;
    struct It {
        int s, I, h;
    };
    auto seg_lo = [&](int s) { return max(I0, s * RT); };
    auto seg_hi = [&](int s) { return min(I1, (s + 1) * RT); };
    auto normalize = [&](It& it) {
        while (it.s <= s_last && it.I >= seg_hi(it.s)) {
            ++it.s;
            if (it.s <= s_last) it.I = seg_lo(it.s) + warp;
        }
    };
    auto slice_units = [&](int s) { return min(kRowsSliceUnits, p.KU - s * kRowsSliceUnits); };
    auto advance = [&](It& it) {
        if (it.h == 0 && slice_units(it.s) > kRowsChunkUnits) {
            it.h = 1;
        } else {
            it.h = 0;
            it.I += W;
            normalize(it);
        }
    };
    auto chunk_units = [&](const It& it) { return min(kRowsChunkUnits, slice_units(it.s) - it.h * kRowsChunkUnits); };
    auto issue = [&](const It& it, int k) {  // one lane
        const int rt = it.I - it.s * RT;
        const size_t unit0 = (size_t)rt * p.KU + (size_t)(it.s * kRowsSliceUnits + it.h * kRowsChunkUnits);
        const uint32_t bytes = (uint32_t)chunk_units(it) * ST;
        const int j = warp * kRowsSlots + (k % kRowsSlots);
        mbar_expect_tx(&full[j], bytes);
        bulk_g2s(gen + chunk_addr(j), p.units + unit0 * ST, bytes, &full[j]);
    };
    It prod, cons;
    prod.s = s_first;
    prod.I = seg_lo(s_first) + warp;
    prod.h = 0;
    normalize(prod);
    cons = prod;
    int kp = 0, kc = 0;
    for (; kp < kRowsSlots && prod.s <= s_last; ++kp) {
        if (lane == 0) issue(prod, kp);
        advance(prod);
    }

    const uint32_t lane_base = a_lut + ((uint32_t)lane << 2);
    const uint32_t w_off = (uint32_t)(gq * 32 + 8 * t);
    const int drow = gq + 8 * (t & 1);  // the row whose absmax this lane decodes (8-bit codes)
    // x rows of this lane's tensor-core column in every block, and the swizzle of their 32-byte chunks
    // (a 64-bit shared load is served half a warp at a time: the four rows a half-warp touches must
    // fall into four different 32-byte bank groups, hence the swizzle by gq % 4)
    const uint32_t x_swz = (uint32_t)(gq & 3);
    const uint32_t x_row0 = a_xs + (uint32_t)((gq >> 1) * 2 * RB + (gq & 1)) * 1024u + 8u * (uint32_t)t;

    float acc[RB][4];
    float4 rs = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    bool failed = false;
    int pending_ctr = -1;  // row tile whose count this warp still owes (its additions are in flight)

    // ---- epilogue of one row tile (or gate/up pair of tiles) by the warp that completed it ----
    auto finalize = [&](int ctr) {
        __threadfence();
        constexpr int GR = 32 / COLS;  // lane groups: 1, 2, 4
        constexpr int R = 16 / GR;     // rows of the tile per lane: 16, 8, 4
        const int m = lane % COLS, grp = lane / COLS;
        const int n0 = ctr * kTileRows + grp * R;
        float* tg = p.acc + ((size_t)ctr * kTileRows + grp * R) * COLS + m;
        float* tu = tg + (size_t)p.pair_offset * kTileRows * COLS;
        float vg[R], vu[R];
#pragma unroll
        for (int i = 0; i < R; ++i) vg[i] = __ldcg(tg + i * COLS);
        if (p.pair_offset > 0) {
#pragma unroll
            for (int i = 0; i < R; ++i) vu[i] = __ldcg(tu + i * COLS);
        }
#pragma unroll
        for (int i = 0; i < R; ++i) __stcg(tg + i * COLS, 0.0f);
        if (p.pair_offset > 0) {
#pragma unroll
            for (int i = 0; i < R; ++i) __stcg(tu + i * COLS, 0.0f);
        }
        if (lane == 0) p.counters[ctr] = 0;
        if (m >= p.m_rows) return;
        uint16_t o[R];
        const bool whole = (p.n_out % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);  // tile inside the output and rows aligned for vector access
        const size_t yo = (size_t)m * p.n_out + n0;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            float v = vg[i];
            if (p.pair_offset > 0) {
                const float gt = bf16_bits_to_f32(f32_to_bf16_bits(vg[i]));
                const float up = bf16_bits_to_f32(f32_to_bf16_bits(vu[i]));
                v = __fdividef(gt, 1.0f + __expf(-gt)) * up;
            } else if (p.residual && n0 + i < p.n_out) {
                v += bf16_bits_to_f32(__ldcg(p.residual + yo + i));
            }
            o[i] = f32_to_bf16_bits(v);
        }
        if (whole) {
            if constexpr (R == 4) {
                *reinterpret_cast<uint2*>(p.y + yo) =
                    make_uint2((uint32_t)o[0] | ((uint32_t)o[1] << 16), (uint32_t)o[2] | ((uint32_t)o[3] << 16));
            } else {
#pragma unroll
                for (int q = 0; q < R / 8; ++q)
                    *reinterpret_cast<uint4*>(p.y + yo + 8 * q) =
                        make_uint4((uint32_t)o[8 * q] | ((uint32_t)o[8 * q + 1] << 16),
                                   (uint32_t)o[8 * q + 2] | ((uint32_t)o[8 * q + 3] << 16),
                                   (uint32_t)o[8 * q + 4] | ((uint32_t)o[8 * q + 5] << 16),
                                   (uint32_t)o[8 * q + 6] | ((uint32_t)o[8 * q + 7] << 16));
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i)
                if (n0 + i < p.n_out) p.y[yo + i] = o[i];
        }
    };

    // Everything above touched only this launch's shared memory and data that no kernel writes
    // (weights, code books, row scales). x, the accumulation tiles and the counters belong to the
    // stream's order: wait for the kernels before this one.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // Publishes the owed count: every lane's additions are ordered before it (fence, then the warp
    // barrier, then one release/acquire increment); the warp that completes a tile finishes it.
    auto count_pending = [&]() {
        if (pending_ctr < 0) return;
        const int ctr = pending_ctr;
        pending_ctr = -1;
        __threadfence();
        __syncwarp();
        const int target = p.n_slices * (p.pair_offset > 0 ? 2 : 1);
        int old = 0;
        if (lane == 0)
            asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;"
                         : "=r"(old) : "l"(p.counters + ctr), "r"(1) : "memory");
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == target - 1) finalize(ctr);
    };

    for (int s = s_first; s <= s_last; ++s) {
        // ---- the x slice of every row: 16-byte pieces, 32-byte chunks swizzled by the row group ----
        if (s != s_first) __syncthreads();  // every warp is done with the previous slice
        {
            const int k0 = s * kRowsSliceUnits * kUnitK;
#pragma unroll
            for (int i = 0; i < COLS * 64 / kRowsThreads; ++i) {
                const int piece = tid + i * kRowsThreads;
                const int m = piece >> 6, q = piece & 63;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (m < p.m_rows && k0 + q * 8 < p.K)
                    v = __ldcg(reinterpret_cast<const uint4*>(p.x + (size_t)m * p.K + k0 + q * 8));
                const uint32_t swz = ((((uint32_t)(m / (2 * RB))) & 1u) << 1) | ((uint32_t)m & 1u);
                const uint32_t dst = a_xs + (uint32_t)m * 1024u + ((((uint32_t)q >> 1) ^ swz) << 5) + (((uint32_t)q & 1u) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                             : "memory");
            }
        }
        __syncthreads();

        while (cons.s == s) {
            const int rt = cons.I - s * RT;
            if (cons.h == 0) {
#pragma unroll
                for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[rb][e] = 0.0f;
                if (KIND == kAbsmaxCodes) rs = __ldg(p.row_scales + min(rt * kTileRows + drow, p.n_rows - 1));
            }
            const int j = warp * kRowsSlots + (kc % kRowsSlots);
            if (!mbar_wait_bounded(&full[j], (uint32_t)((kc / kRowsSlots) & 1), failed ? 1000000LL : p.spin_limit)) {
                if (!failed) atomicExch(p.status, kStatusTimeoutFull);
                failed = true;
            }
            const int nu = chunk_units(cons);
            const uint32_t ca = chunk_addr(j);
            if (!failed) {
                // (two units in flight per warp where the registers allow it)
#pragma unroll(RB <= 2 ? 2 : 1)
                for (int u = 0; u < nu; ++u) {
                    const uint32_t ua = ca + (uint32_t)u * ST;
                    const int ul = cons.h * kRowsChunkUnits + u;  // unit inside the slice
                    const int kb = s * kRowsSliceUnits + ul;
                    // x fragments of every block: k = 64 kb + 16 i + 4 t + {0..3}, i = 0..3
                    uint2 xb[RB][4];
#pragma unroll
                    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            xb[rb][i] = lds_v2(x_row0 + (uint32_t)rb * 2048u + ((((uint32_t)(ul * 4 + i)) ^ x_swz) << 5));
                    float am0, am1;
                    if (KIND == kAbsmaxCodes) {
                        const unsigned code = lds_u8(ua + kUnitNibbleBytes + drow);
                        const float scale = kb >= __float_as_int(rs.z) ? rs.y : rs.x;
                        const float am = __fadd_rn(__fmul_rn(lds_f32(a_nmap + 4u * code), scale), rs.w);
                        am0 = __shfl_sync(0xffffffffu, am, lane & ~3);
                        am1 = __shfl_sync(0xffffffffu, am, (lane & ~3) | 1);
                    } else {
                        am0 = lds_f32(ua + kUnitNibbleBytes + 4u * gq);
                        am1 = lds_f32(ua + kUnitNibbleBytes + 4u * (gq + 8));
                    }
                    const uint2 l = lds_v2(ua + w_off), uu = lds_v2(ua + w_off + 256u);
                    uint32_t a[16];
                    a[0] = lut_pair<0>(l.x, lane_base);  a[1] = lut_pair<0>(uu.x, lane_base);
                    a[2] = lut_pair<1>(l.x, lane_base);  a[3] = lut_pair<1>(uu.x, lane_base);
                    a[4] = lut_pair<2>(l.x, lane_base);  a[5] = lut_pair<2>(uu.x, lane_base);
                    a[6] = lut_pair<3>(l.x, lane_base);  a[7] = lut_pair<3>(uu.x, lane_base);
                    a[8] = lut_pair<0>(l.y, lane_base);  a[9] = lut_pair<0>(uu.y, lane_base);
                    a[10] = lut_pair<1>(l.y, lane_base); a[11] = lut_pair<1>(uu.y, lane_base);
                    a[12] = lut_pair<2>(l.y, lane_base); a[13] = lut_pair<2>(uu.y, lane_base);
                    a[14] = lut_pair<3>(l.y, lane_base); a[15] = lut_pair<3>(uu.y, lane_base);
#pragma unroll
                    for (int rb = 0; rb < RB; ++rb) {
                        float c0[4], c1[4];
                        mma_bf16_16816_init(c0, a[0], a[1], a[2], a[3], xb[rb][0].x, xb[rb][0].y);
                        mma_bf16_16816_init(c1, a[4], a[5], a[6], a[7], xb[rb][1].x, xb[rb][1].y);
                        mma_bf16_16816(c0, a[8], a[9], a[10], a[11], xb[rb][2].x, xb[rb][2].y);
                        mma_bf16_16816(c1, a[12], a[13], a[14], a[15], xb[rb][3].x, xb[rb][3].y);
                        acc[rb][0] = fmaf(am0, c0[0] + c1[0], acc[rb][0]);
                        acc[rb][1] = fmaf(am0, c0[1] + c1[1], acc[rb][1]);
                        acc[rb][2] = fmaf(am1, c0[2] + c1[2], acc[rb][2]);
                        acc[rb][3] = fmaf(am1, c0[3] + c1[3], acc[rb][3]);
                    }
                }
            }
            // the chunk's shared memory is free (every lane's loads have fed the arithmetic above):
            // refill the slot with this warp's next chunk
            __syncwarp();
            if (prod.s <= s_last) {
                if (lane == 0 && !failed) issue(prod, kp);
                if (failed) prod.s = s_last + 1;  // stop issuing
                else {
                    ++kp;
                    advance(prod);
                }
            }
            ++kc;
            const bool last_chunk = !(cons.h == 0 && slice_units(s) > kRowsChunkUnits);
            if (last_chunk && !failed) {
                // ---- the item's partial tile into the accumulation tile, then the count ----
                float lo[2 * RB], hi[2 * RB];
#pragma unroll
                for (int rb = 0; rb < RB; ++rb) {
                    lo[2 * rb] = acc[rb][0];
                    lo[2 * rb + 1] = acc[rb][1];
                    hi[2 * rb] = acc[rb][2];
                    hi[2 * rb + 1] = acc[rb][3];
                }
                // The count of an item is published one item late: by then its additions have long
                // been acknowledged, so the fence in front of the count does not wait for them.
                count_pending();
                float* dst = p.acc + ((size_t)rt * kTileRows + gq) * COLS + t * 2 * RB;
                red_add_f32<2 * RB>(dst, lo);
                red_add_f32<2 * RB>(dst + 8 * COLS, hi);
                pending_ctr = (p.pair_offset > 0 && rt >= p.pair_offset) ? rt - p.pair_offset : rt;
            }
            advance(cons);
        }
    }
    count_pending();
    // never leave with copies still landing in this CTA's shared memory (only after a failure can
    // issued chunks be unconsumed here)
    if (failed) {
        for (; kc < kp; ++kc)
            mbar_wait_bounded(&full[warp * kRowsSlots + (kc % kRowsSlots)], (uint32_t)((kc / kRowsSlots) & 1), 1000000LL);
    }
}

template <int KIND, int RB>
cudaError_t launch_rows_t(const RowsParams& p, int grid, cudaStream_t s) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_rows_kernel<KIND, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kRowsSmemBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    // Programmatic dependent launch, as for the streaming kernel: table build, barrier set-up and the
    // first weight copies overlap the previous kernel's tail. Disabled with AILA_NF4_PDL=0.
    static const bool use_pdl = [] {
        const char* e = std::getenv("AILA_NF4_PDL");
        return !(e && e[0] == '0');
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kRowsThreads);
    cfg.dynamicSmemBytes = (size_t)kRowsSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_rows_kernel<KIND, RB>, p);
}

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
    // per CTA: two shared tiles x (two halves of one row block, or one half of up to four row blocks)
    // x (16 rows x 8 batch columns)
    return (size_t)sm_count * kMaxGridMult * 2 * 4 * 128;
}

int gemv_stream_grid(const AilaNf4Linear& w, int64_t ff_pair, int sm_count) {
    const StreamPlan pl = stream_plan(w, ff_pair > 0, ff_pair, sm_count);
    return pl.ok ? pl.grid : 0;
}

bool gemv_stream_supported(const AilaNf4Linear& w, int64_t ff_pair, int sm_count, int row_blocks) {
    if (w.K > 65535 * 4) return false;
    if (ff_pair > 0 && row_blocks > 1) return false;
    return stream_plan(w, ff_pair > 0, ff_pair, sm_count, row_blocks).ok;
}

cudaError_t launch_gemv_stream(const AilaNf4Linear& w, AilaNf4Scratch& scratch, const void* x,
                               void* y, const void* residual, int64_t ff_pair, cudaStream_t s,
                               const PeerTargets* peers, int m_rows, const NormInput* norm) {
    const bool paired = ff_pair > 0;
    if (m_rows < 1 || m_rows > (paired ? 8 : 32) || (m_rows > 1 && (peers || norm))) return cudaErrorInvalidValue;
    const int row_blocks = m_rows <= 8 ? 1 : (m_rows <= 16 ? 2 : 4);
    const StreamPlan pl = stream_plan(w, paired, ff_pair, scratch.sm_count, row_blocks);
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
    p.spin_limit = scratch.wait_limit_cycles;
    const int rt_work = paired ? (int)(ff_pair / kTileRows) : w.RT;
    p.total_items = rt_work * w.KU;
    p.slice_q = p.total_items / pl.grid;
    p.slice_r = p.total_items % pl.grid;
    make_fast_div((uint32_t)pl.grid, &p.div_g_m, &p.div_g_s);
    make_fast_div((uint32_t)w.KU, &p.div_ku_m, &p.div_ku_s);
    p.kb_step = kConsumerWarps % w.KU;
    p.rt_step = kConsumerWarps / w.KU;
    p.n_out = paired ? (int)ff_pair : (int)w.N;
    p.K = (int)w.K;
    p.KU = w.KU;
    p.unit_stride = w.unit_stride;
    p.pair_rt_offset = paired ? (int)(ff_pair / kTileRows) : 0;
    p.x_bytes = (int)((w.K * 2 + 15) / 16 * 16);
    p.stages = pl.stages;
    p.stages_b = pl.stages_b;
    p.x_in_b = pl.x_in_b;
    p.smem_bytes = pl.smem;
    p.n_rows = (int)w.N;
    p.m_rows = m_rows;
    p.norm_add = norm ? static_cast<const uint16_t*>(norm->add) : nullptr;
    p.norm_w = norm ? static_cast<const uint16_t*>(norm->weight) : nullptr;
    p.norm_hidden_out = norm ? static_cast<uint16_t*>(norm->hidden_out) : nullptr;
    p.norm_eps = norm ? norm->eps : 0.0f;
    p.peer_world = 0;
    p.peer_rank = 0;
    p.peer_max_rows = 0;
    p.peer_ctrl = nullptr;
    p.peer_inline = 0;
    p.n_row_tiles = rt_work;
    for (int d = 0; d < kMaxPeerWorld; ++d) {
        p.peer_part[d] = nullptr;
    }
    if (peers) {
        if (paired || peers->world < 1 || peers->world > kMaxPeerWorld) return cudaErrorInvalidValue;
        p.peer_world = peers->world;
        p.peer_rank = peers->rank;
        p.peer_max_rows = peers->max_rows;
        p.peer_ctrl = peers->ctrl;
        p.peer_inline = peers->inline_reduce ? 1 : 0;
        for (int d = 0; d < peers->world; ++d) {
            p.peer_part[d] = peers->part_base[d];
        }
    }
    const bool batch = m_rows > 1;
    if (w.absmax_kind == kAbsmaxCodes) {
        if (batch && row_blocks == 4) return launch_stream_t<kAbsmaxCodes, false, 4>(p, pl.grid, pl.smem, s);
        if (batch && row_blocks == 2) return launch_stream_t<kAbsmaxCodes, false, 2>(p, pl.grid, pl.smem, s);
        if (batch)
            return paired ? launch_stream_t<kAbsmaxCodes, true, 1>(p, pl.grid, pl.smem, s)
                          : launch_stream_t<kAbsmaxCodes, false, 1>(p, pl.grid, pl.smem, s);
        return paired ? launch_stream_t<kAbsmaxCodes, true, 0>(p, pl.grid, pl.smem, s)
                      : launch_stream_t<kAbsmaxCodes, false, 0>(p, pl.grid, pl.smem, s);
    }
    if (batch && row_blocks == 4) return launch_stream_t<kAbsmaxF32, false, 4>(p, pl.grid, pl.smem, s);
    if (batch && row_blocks == 2) return launch_stream_t<kAbsmaxF32, false, 2>(p, pl.grid, pl.smem, s);
    if (batch)
        return paired ? launch_stream_t<kAbsmaxF32, true, 1>(p, pl.grid, pl.smem, s)
                      : launch_stream_t<kAbsmaxF32, false, 1>(p, pl.grid, pl.smem, s);
    return paired ? launch_stream_t<kAbsmaxF32, true, 0>(p, pl.grid, pl.smem, s)
                  : launch_stream_t<kAbsmaxF32, false, 0>(p, pl.grid, pl.smem, s);
}

bool gemv_rows_supported(const AilaNf4Linear& w, int64_t ff_pair) {
    if (w.absmax_kind == kAbsmaxCodes && !w.d_row_scales) return false;
    if (ff_pair > 0 && (ff_pair % kTileRows != 0 || w.N != 2 * ff_pair)) return false;
    const long long total = (long long)((w.KU + kRowsSliceUnits - 1) / kRowsSliceUnits) * w.RT;
    return total > 0 && total < (1ll << 30);
}

size_t gemv_rows_acc_bytes(const AilaNf4Linear& w) { return (size_t)w.RT * kTileRows * 32 * sizeof(float); }

// 2 .. 32 rows of x through the K-sliced kernel. scratch.d_rows_acc (gemv_rows_acc_bytes, zero) and
// scratch.d_counters (one per row tile, zero) must be in place; both are zero again afterwards.
cudaError_t launch_gemv_rows(const AilaNf4Linear& w, AilaNf4Scratch& scratch, const void* x, void* y,
                             const void* residual, int64_t ff_pair, cudaStream_t s, int m_rows) {
    if (m_rows < 1 || m_rows > 32 || !gemv_rows_supported(w, ff_pair) || (ff_pair > 0 && residual))
        return cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(x) & 15) return cudaErrorInvalidValue;
    RowsParams p;
    p.units = w.d_units;
    p.qmap = w.d_qmap;
    const ScaleParams sp = w.scale_params();
    p.nmap = sp.nmap;
    p.row_scales = static_cast<const float4*>(w.d_row_scales);
    p.x = static_cast<const uint16_t*>(x);
    p.y = static_cast<uint16_t*>(y);
    p.residual = static_cast<const uint16_t*>(residual);
    p.acc = scratch.d_rows_acc;
    p.counters = scratch.d_counters;
    p.status = scratch.d_status;
    p.spin_limit = scratch.wait_limit_cycles;
    p.K = (int)w.K;
    p.KU = w.KU;
    p.n_slices = (w.KU + kRowsSliceUnits - 1) / kRowsSliceUnits;
    p.n_tiles = w.RT;
    p.n_rows = (int)w.N;
    p.n_out = ff_pair > 0 ? (int)ff_pair : (int)w.N;
    p.m_rows = m_rows;
    p.pair_offset = ff_pair > 0 ? (int)(ff_pair / kTileRows) : 0;
    p.total_items = p.n_slices * p.n_tiles;
    const int grid = p.total_items < scratch.sm_count ? p.total_items : scratch.sm_count;
    p.slice_q = p.total_items / grid;
    p.slice_r = p.total_items % grid;
    make_fast_div((uint32_t)grid, &p.div_g_m, &p.div_g_s);
    p.smem_bytes = kRowsSmemBytes;
    const int rb = m_rows <= 8 ? 1 : (m_rows <= 16 ? 2 : 4);
    if (w.absmax_kind == kAbsmaxCodes) {
        if (rb == 1) return launch_rows_t<kAbsmaxCodes, 1>(p, grid, s);
        if (rb == 2) return launch_rows_t<kAbsmaxCodes, 2>(p, grid, s);
        return launch_rows_t<kAbsmaxCodes, 4>(p, grid, s);
    }
    if (rb == 1) return launch_rows_t<kAbsmaxF32, 1>(p, grid, s);
    if (rb == 2) return launch_rows_t<kAbsmaxF32, 2>(p, grid, s);
    return launch_rows_t<kAbsmaxF32, 4>(p, grid, s);
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

// Reads (and clears) the status word of the static work space on the current device: what
// aila_nf4_scratch_check does for a scratch object. Allocates nothing.
AilaNf4Status check_gemv_stream_static(cudaStream_t s) {
    int dev = 0;
    NF4_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(AILA_NF4_ERR_UNSUPPORTED, "device ordinal above 63");
    StaticScratchHost host;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        host = g_static_host[dev];
    }
    if (!host.ptr) return AILA_NF4_OK;  // no call on this device yet
    int code = 0;
    NF4_CUDA(cudaMemcpyAsync(&code, host.ptr->status, sizeof(int), cudaMemcpyDeviceToHost, s));
    NF4_CUDA(cudaStreamSynchronize(s));
    if (code != 0) {
        NF4_CUDA(cudaMemsetAsync(host.ptr->status, 0, sizeof(int), s));
        NF4_CUDA(cudaStreamSynchronize(s));
        return fail(AILA_NF4_ERR_KERNEL_TIMEOUT,
                    "aila_nf4_forward_decode_static: a bounded device-side wait expired (code " +
                        std::to_string(code) + ")");
    }
    return AILA_NF4_OK;
}

}  // namespace nf4

