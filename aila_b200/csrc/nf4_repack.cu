// Load-time regrouping of checkpoint-layout NF4 tensors into the unit stream, and
// unit-stream -> unit-stream gathers (row fusion, re-slicing). Replaces the host loop and
// device-to-device copies of Bnb4BitLinear::init / init_fused_rows_impl
// (reference src/ops/Bnb4BitLinear.cpp:470-494, :604-615).
#include "nf4_internal.h"

namespace nf4 {

namespace {

// One thread per (unit, row): reads the row's 32 source bytes for this 64-wide block and
// stores them permuted; copies the block's absmax (u8 code or fp32).
__global__ void repack_kernel(RepackSource src, uint8_t* __restrict__ units, int N, int RT,
                              int KU, int unit_stride, int absmax_kind, int blk_shift) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)RT * KU * kTileRows;
    if (tid >= total) return;
    const int r = (int)(tid % kTileRows);
    const long long u = tid / kTileRows;
    const int kb = (int)(u % KU);
    const int rt = (int)(u / KU);
    const int n = rt * kTileRows + r;
    uint8_t* unit = units + (size_t)u * unit_stride;

    uint32_t words[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) words[i] = 0;
    if (n < N) {
        const uint8_t* srow = src.packed + (size_t)(src.row0 + n) * src.row_stride_bytes +
                              src.col_byte0 + (size_t)kb * 32;
#pragma unroll
        for (int p = 0; p < 32; ++p) {
            const uint32_t b = srow[stored_to_source_byte(p)];
            words[p >> 2] |= b << (8 * (p & 3));
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(unit + r * 32);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);

    const long long aidx = (long long)(src.row0 + n) * src.abs_row_stride + src.abs_col0 +
                           (kb >> blk_shift);
    if (absmax_kind == kAbsmaxCodes) {
        unit[kUnitNibbleBytes + r] =
            (n < N) ? static_cast<const uint8_t*>(src.absmax)[aidx] : (uint8_t)0;
    } else {
        reinterpret_cast<float*>(unit + kUnitNibbleBytes)[r] =
            (n < N) ? static_cast<const float*>(src.absmax)[aidx] : 0.0f;
    }
}

struct GatherParams {
    GatherSource src[kMaxSegments];
    int n_src;
};

// One thread per (destination unit, row): finds the source that owns the row and copies its
// 32 nibble bytes and its absmax entry. Both sides use the unit layout, so the intra-row
// permutation carries over unchanged.
__global__ void gather_kernel(GatherParams gp, uint8_t* __restrict__ units, int N, int RT, int KU,
                              int unit_stride, int absmax_kind) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)RT * KU * kTileRows;
    if (tid >= total) return;
    const int r = (int)(tid % kTileRows);
    const long long u = tid / kTileRows;
    const int kb = (int)(u % KU);
    const int rt = (int)(u / KU);
    const int n = rt * kTileRows + r;
    uint8_t* unit = units + (size_t)u * unit_stride;

    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
    uint32_t code = 0;
    float amf = 0.0f;
    if (n < N) {
        int s = 0;
        for (int i = 1; i < gp.n_src; ++i)
            if (n >= gp.src[i].dst_row0) s = i;
        const GatherSource& g = gp.src[s];
        const int sn = n - g.dst_row0 + g.src_row0;
        const size_t su = (size_t)(sn / kTileRows) * g.KU + (size_t)(kb + g.src_kb0);
        const uint8_t* sunit = g.units + su * g.unit_stride;
        const uint4* sp = reinterpret_cast<const uint4*>(sunit + (sn % kTileRows) * 32);
        lo = sp[0];
        hi = sp[1];
        if (absmax_kind == kAbsmaxCodes)
            code = sunit[kUnitNibbleBytes + (sn % kTileRows)];
        else
            amf = reinterpret_cast<const float*>(sunit + kUnitNibbleBytes)[sn % kTileRows];
    }
    uint4* dst = reinterpret_cast<uint4*>(unit + r * 32);
    dst[0] = lo;
    dst[1] = hi;
    if (absmax_kind == kAbsmaxCodes)
        unit[kUnitNibbleBytes + r] = (uint8_t)code;
    else
        reinterpret_cast<float*>(unit + kUnitNibbleBytes)[r] = amf;
}

int ilog2(int v) {
    int s = 0;
    while ((1 << s) < v) ++s;
    return s;
}

}  // namespace

cudaError_t launch_repack(const RepackSource& src, const AilaNf4Linear& dst, cudaStream_t s) {
    const long long total = (long long)dst.RT * dst.KU * kTileRows;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    repack_kernel<<<(unsigned)blocks, threads, 0, s>>>(src, dst.d_units, (int)dst.N, dst.RT, dst.KU,
                                                       dst.unit_stride, dst.absmax_kind,
                                                       ilog2(dst.blocksize / kUnitK));
    return cudaGetLastError();
}

cudaError_t launch_gather(const GatherSource* srcs, int n_src, const AilaNf4Linear& dst,
                          cudaStream_t s) {
    GatherParams gp;
    gp.n_src = n_src;
    for (int i = 0; i < n_src; ++i) gp.src[i] = srcs[i];
    for (int i = n_src; i < kMaxSegments; ++i) gp.src[i] = srcs[0];
    const long long total = (long long)dst.RT * dst.KU * kTileRows;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    gather_kernel<<<(unsigned)blocks, threads, 0, s>>>(gp, dst.d_units, (int)dst.N, dst.RT, dst.KU,
                                                       dst.unit_stride, dst.absmax_kind);
    return cudaGetLastError();
}

}  // namespace nf4
