// Host-side objects behind the opaque C handles, and the launchers each .cu file exports.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/aila_nf4.h"
#include "nf4_common.cuh"

struct AilaNf4Linear {
    int device = 0;
    int64_t N = 0, K = 0;
    int blocksize = 64;
    int absmax_kind = nf4::kAbsmaxCodes;
    int RT = 0, KU = 0;      // row tiles (16 rows), units per row tile (64 k)
    int unit_stride = nf4::kUnitStrideCodes;
    uint8_t* d_units = nullptr;  // RT*KU*unit_stride bytes
    float* d_qmap = nullptr;     // [16]
    float* d_nmap = nullptr;     // [256]
    float* d_nabs = nullptr;     // concatenated nested_absmax
    void* d_cache_bf16 = nullptr;  // optional bf16 [N][K] copy (AILA_BNB4_CACHE_DEQUANT=1)
    // Per output row, for 8-bit absmax codes: the second-level scale of the row's first block, the
    // scale after the row's (single) change of second-level block, the unit column of that change
    // and the second-level offset (nf4::RowScales). Null when a row could change twice.
    void* d_row_scales = nullptr;
    int64_t nabs_count = 0;
    float h_qmap[16] = {0};
    int nbs = 256;
    // segments (sources of a fused linear); a plain linear has one
    int nseg = 1;
    int seg_row0[nf4::kMaxSegments] = {0, 0, 0, 0};
    int seg_rows[nf4::kMaxSegments] = {0, 0, 0, 0};
    int64_t seg_flat0[nf4::kMaxSegments] = {0, 0, 0, 0};   // flat index of (row0, k = 0) block, source numbering
    int64_t seg_row_stride[nf4::kMaxSegments] = {0, 0, 0, 0};
    int64_t seg_nabs_base[nf4::kMaxSegments] = {0, 0, 0, 0};
    float seg_offset[nf4::kMaxSegments] = {0, 0, 0, 0};
    int64_t device_bytes = 0;

    nf4::ScaleParams scale_params() const;
    size_t units_bytes() const { return (size_t)RT * (size_t)KU * (size_t)unit_stride; }
};

struct AilaNf4Scratch {
    int device = 0;
    // split-K fix-up space of the streaming GEMV: per-CTA partial sums and per-row-tile
    // arrival counters (counters are zero between launches; the last arriver resets them).
    float* d_partials = nullptr;
    size_t partials_floats = 0;
    float* d_rows_acc = nullptr;  // accumulation tiles of the K-sliced small-batch kernel (kept zero)
    size_t rows_acc_bytes = 0;
    int* d_counters = nullptr;
    size_t counters_ints = 0;
    int* d_status = nullptr;  // device status word written by bounded waits
    // bf16 [N][K] weight of the seq_len > 1 route
    void* d_weight = nullptr;
    size_t weight_bytes = 0;
    // staging for the host-buffer entry points
    void* d_io_in = nullptr;
    size_t io_in_bytes = 0;
    void* d_io_out = nullptr;
    size_t io_out_bytes = 0;
    int sm_count = 0;
    // exchange space of the chained decode kernel (one allocation, d_chain_ctrl is its base):
    // control words {epoch, CTAs done, abort}, one token per CTA, partial-sum words, x words
    unsigned* d_chain_ctrl = nullptr;
    unsigned long long* d_chain_tok = nullptr;
    unsigned long long* d_chain_p = nullptr;
    unsigned long long* d_chain_x = nullptr;
    long long chain_xwords = 0;
    long long wait_limit_cycles = 2000000000LL;  // bound of every device-side wait of the decode kernels
};

struct AilaNf4PeerBuf;

namespace nf4 {

// error plumbing (nf4_api.cu)
AilaNf4Status fail(AilaNf4Status code, const std::string& message);
AilaNf4Status cuda_fail(cudaError_t e, const char* what);
#define NF4_CUDA(call)                                         \
    do {                                                       \
        cudaError_t e__ = (call);                              \
        if (e__ != cudaSuccess) return nf4::cuda_fail(e__, #call); \
    } while (0)

// nf4_repack.cu -------------------------------------------------------------------------
struct RepackSource {
    const uint8_t* packed;     // device, row-major nibbles of the source tensor
    int64_t row_stride_bytes;  // bytes between source rows (K_src / 2)
    int64_t col_byte0;         // first byte of the kept column range inside a row
    const void* absmax;        // device u8 codes or f32, [rows][abs_row_stride]
    int64_t abs_row_stride;    // elements between source rows (K_src / blocksize)
    int64_t abs_col0;          // first kept absmax column
    int64_t row0;              // first kept source row
};
cudaError_t launch_repack(const RepackSource& src, const AilaNf4Linear& dst, cudaStream_t s);

struct GatherSource {
    const uint8_t* units;
    int KU;          // units per row tile in the source
    int unit_stride;
    int src_row0;    // source row that lands on dst_row0
    int src_kb0;     // source unit column that lands on unit column 0
    int dst_row0;
    int rows;
};
cudaError_t launch_gather(const GatherSource* srcs, int n_src, const AilaNf4Linear& dst,
                          cudaStream_t s);

// nf4_dequant.cu ------------------------------------------------------------------------
cudaError_t launch_dequant_kn(const AilaNf4Linear& w, void* out_kn, cudaStream_t s);
cudaError_t launch_dequant_nk(const AilaNf4Linear& w, void* out_nk, cudaStream_t s);
cudaError_t launch_expand_absmax(const AilaNf4Linear& w, float* out, cudaStream_t s);
cudaError_t launch_swiglu_rows(const void* gate_up, void* out, int M, int64_t ff,
                               cudaStream_t s);

// nf4_gemv.cu ---------------------------------------------------------------------------
cudaError_t launch_gemv_simple(const AilaNf4Linear& w, const void* x, void* y,
                               const void* residual, int64_t ff_pair, cudaStream_t s);
size_t gemv_stream_partials_floats(int sm_count);
// Row-parallel exchange of one launch: where this rank's fp32 row sums go on every rank (its
// own included), as 8-byte words {value, tag}. part_base[d] is rank d's row area as mapped in
// this process; the word of (parity, source rank, row) sits at
// part_base + (parity * world + rank) * max_rows + row. ctrl is this rank's own control block
// {epoch, unused, CTAs or reducer blocks done}.
struct PeerTargets {
    int world;
    int rank;
    long long max_rows;
    unsigned long long* part_base[8];
    unsigned* ctrl;
    bool inline_reduce;  // the GEMV's CTAs also sum the ranks' rows (grid <= SM count only)
};
// Residual add + RMSNorm folded into the staging of x (single-row launches): weight != NULL.
struct NormInput {
    const void* add;     // bf16 [K] added to x first, or NULL
    const void* weight;  // bf16 [K]
    void* hidden_out;    // bf16 [K] receives bf16(x + add), or NULL; must not alias x or add
    float eps;
};
cudaError_t launch_gemv_stream(const AilaNf4Linear& w, AilaNf4Scratch& scratch, const void* x,
                               void* y, const void* residual, int64_t ff_pair, cudaStream_t s,
                               const PeerTargets* peers = nullptr, int m_rows = 1,
                               const NormInput* norm = nullptr);
// row_blocks: 8-row blocks of x one launch carries (1 for a single row; 2 or 4 only unpaired)
bool gemv_stream_supported(const AilaNf4Linear& w, int64_t ff_pair, int sm_count, int row_blocks = 1);
int gemv_stream_grid(const AilaNf4Linear& w, int64_t ff_pair, int sm_count);  // 0: shape not taken
AilaNf4Status launch_gemv_stream_static(const AilaNf4Linear& w, const void* x, void* y,
                                        const void* residual, cudaStream_t s);
AilaNf4Status check_gemv_stream_static(cudaStream_t s);
// K-sliced small-batch decode kernel (2 .. 32 rows, x slice in shared memory)
bool gemv_rows_supported(const AilaNf4Linear& w, int64_t ff_pair);
size_t gemv_rows_acc_bytes(const AilaNf4Linear& w);
cudaError_t launch_gemv_rows(const AilaNf4Linear& w, AilaNf4Scratch& scratch, const void* x, void* y,
                             const void* residual, int64_t ff_pair, cudaStream_t s, int m_rows);

// Fills l.d_row_scales (N entries of 16 bytes, allocated by the caller).
cudaError_t launch_row_scales(const AilaNf4Linear& l, cudaStream_t s);

// nf4_chain.cu --------------------------------------------------------------------------
// The chained decode kernel: one cooperative launch walks a list of linears. A one-operation
// launch serves aila_nf4_forward and its siblings.
bool gemv_chain_supported(const AilaNf4Linear& w, int64_t ff_pair, const AilaNf4Scratch& sc);
AilaNf4Status launch_gemv_chain_single(const AilaNf4Linear& w, AilaNf4Scratch& sc, const void* x,
                                       void* y, const void* residual, int64_t ff_pair,
                                       const NormInput* norm, cudaStream_t s);
AilaNf4Status ensure_chain_scratch(AilaNf4Scratch* sc);

// nf4_peer.cu ---------------------------------------------------------------------------
// y[n] = bf16(sum over ranks of the tagged words [parity][rank][n] (+ residual[n])), each word
// waited for (bounded, kStatusTimeoutPeer) until it carries the call's tag. The last block
// advances the epoch.
cudaError_t launch_peer_reduce(const unsigned long long* part_base, unsigned* ctrl, int world,
                               int64_t max_rows, int64_t n, const void* residual, void* y,
                               int* d_status, long long spin_limit, cudaStream_t s);
AilaNf4Status ensure_counters(AilaNf4Scratch* sc, size_t tiles);
// The exchange addresses of a peer buffer whose peers have all been imported, for `rows` rows.
AilaNf4Status peer_targets_of(const ::AilaNf4PeerBuf* b, int device, int64_t rows, PeerTargets* out);

// nf4_gemm.cu ---------------------------------------------------------------------------
// y[M][N_out] = x[M][K] * w_nk[N][K]^T on tcgen05. swiglu_ff > 0: N == 2*ff and the output
// is [M][ff] = silu(bf16(gate)) * bf16(up).
// Prefill with the weight dequantised inside the GEMM (no bf16 copy of W through HBM).
bool gemm_nf4_fused_supported(const AilaNf4Linear& w, int64_t swiglu_ff);
AilaNf4Status launch_gemm_nf4_fused(const AilaNf4Linear& w, const void* x, void* y, const void* residual,
                                    int M, int64_t swiglu_ff, int sm_count, int* d_status, cudaStream_t s);
AilaNf4Status launch_gemm_bf16(const void* w_nk, const void* x, void* y, const void* residual,
                               int M, int64_t N, int64_t K, int64_t swiglu_ff, int device,
                               int sm_count, int* d_status, cudaStream_t s);

}  // namespace nf4
