// Row-parallel decode over NVLink peer memory (net-new: the reference is single-device).
//
// A column-sharded linear (o_proj, down) gives every rank a partial y[N]; the ranks need their
// sum. For M = 1 the message is tens of KB and a library all-reduce is latency-bound, so the
// exchange is folded into the GEMV: the kernel's epilogue stores this rank's fp32 row sums
// straight into EVERY rank's exchange buffer (plain peer stores through NVLink, its own buffer
// included) as 8-byte words {value, tag}, tag = epoch + 1. A naturally aligned 64-bit store is
// seen whole or not at all, so a reader that finds the call's tag in a word has its value: no
// fence, no counter, one NVLink store latency. The rank sum (rank order, + residual, one bf16
// rounding: every rank gets the bit-identical result) is done by the GEMV's own CTAs when the
// whole grid is resident at once, otherwise by a small second kernel; readers wait per word,
// bounded.
//
// Exchange buffer of one rank (one cudaMalloc, shared with the other processes through CUDA
// IPC): [2 parities][world][max_rows] 8-byte words, then this rank's control block {epoch,
// unused, CTAs / reducer blocks done}. Calls alternate between the two parities (parity = epoch
// & 1): a rank can run ahead of a peer by less than one call (its next sum needs that peer's
// next rows, which the peer sends only after it has finished reading the current ones), so two
// halves are enough; the tag tells the halves' successive uses apart. The last CTA (or reducer
// block) of a call advances the epoch. All state lives on the device: the call sequence can be
// captured in a CUDA graph and replayed. All ranks must issue the same calls in the same order.
//
// No load in this file or in the GEMV touches another GPU's memory: remote memory is only
// written. No multicast object is created.
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "nf4_internal.h"

struct AilaNf4PeerBuf {
    int device = 0;
    int rank = 0;
    int world = 0;
    int64_t max_rows = 0;
    void* local = nullptr;      // this rank's buffer (cudaMalloc)
    void* base[8] = {nullptr};  // every rank's buffer as mapped here (base[rank] == local)
    bool imported[8] = {false};
    bool by_ipc[8] = {false};   // mapped with cudaIpcOpenMemHandle (closed on destroy)
    size_t bytes = 0;
};

namespace nf4 {

namespace {

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// One thread per output row: wait (bounded) for every rank's word of the row, sum in rank order.
// The last block to finish advances the epoch (every block has read it by then).
__global__ void __launch_bounds__(256)
peer_reduce_kernel(const unsigned long long* __restrict__ part_base, unsigned* ctrl, int world,
                   long long max_rows, long long n, const uint16_t* __restrict__ residual,
                   uint16_t* __restrict__ y, int* status, long long spin_limit) {
    const unsigned epoch = *(volatile unsigned*)ctrl;
    const unsigned parity = epoch & 1u;
    const unsigned tag = epoch + 1u;
    const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (row < n) {
        const unsigned long long* part = part_base + (size_t)parity * world * (size_t)max_rows;
        float acc = 0.0f;
        bool ok = true;
        for (int r = 0; r < world && ok; ++r) {
            const unsigned long long* word = part + (size_t)r * (size_t)max_rows + row;
            unsigned long long q = ld_relaxed_sys_u64(word);
            if ((unsigned)(q >> 32) != tag) {
                const long long t0 = clock64();
                do {
                    __nanosleep(40);
                    q = ld_relaxed_sys_u64(word);
                    if (clock64() - t0 > spin_limit) {
                        atomicExch(status, kStatusTimeoutPeer);
                        ok = false;
                        break;
                    }
                } while ((unsigned)(q >> 32) != tag);
            }
            acc += __uint_as_float((unsigned)q);
        }
        if (ok) {
            if (residual) acc += bf16_bits_to_f32(residual[row]);
            y[row] = f32_to_bf16_bits(acc);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned done = atomicAdd(ctrl + 2, 1u);
        if (done == gridDim.x - 1) {
            ctrl[2] = 0u;
            __threadfence();
            *(volatile unsigned*)ctrl = epoch + 1u;
        }
    }
}

size_t rows_words(int world, int64_t max_rows) { return (size_t)2 * world * (size_t)max_rows; }

size_t peerbuf_bytes(int world, int64_t max_rows) { return rows_words(world, max_rows) * 8 + 64 + 256; }

unsigned long long* part_base_of(void* base) { return static_cast<unsigned long long*>(base); }

unsigned* ctrl_of(void* base, int world, int64_t max_rows) {
    return reinterpret_cast<unsigned*>(static_cast<unsigned long long*>(base) + rows_words(world, max_rows));
}

}  // namespace

cudaError_t launch_peer_reduce(const unsigned long long* part_base, unsigned* ctrl, int world,
                               int64_t max_rows, int64_t n, const void* residual, void* y,
                               int* d_status, long long spin_limit, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    peer_reduce_kernel<<<blocks, 256, 0, s>>>(part_base, ctrl, world, (long long)max_rows,
                                              (long long)n, static_cast<const uint16_t*>(residual),
                                              static_cast<uint16_t*>(y), d_status, spin_limit);
    return cudaGetLastError();
}

}  // namespace nf4

using nf4::fail;

namespace nf4 {
AilaNf4Status peer_targets_of(const AilaNf4PeerBuf* b, int device, int64_t rows, PeerTargets* pt) {
    if (!b) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "peer buffer is NULL");
    if (device != b->device)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "linear, scratch and peer buffer must share a device");
    if (rows > b->max_rows)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "out_features " + std::to_string(rows) +
                                                       " exceeds the peer buffer's " + std::to_string(b->max_rows) + " rows");
    for (int r = 0; r < b->world; ++r)
        if (!b->imported[r])
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "peer buffer of rank " + std::to_string(r) + " has not been imported");
    pt->world = b->world;
    pt->rank = b->rank;
    pt->max_rows = b->max_rows;
    pt->ctrl = ctrl_of(b->local, b->world, b->max_rows);
    for (int d = 0; d < 8; ++d) pt->part_base[d] = nullptr;
    for (int d = 0; d < b->world; ++d) pt->part_base[d] = part_base_of(b->base[d]);
    pt->inline_reduce = false;
    return AILA_NF4_OK;
}
}  // namespace nf4

namespace {
struct DevGuard {
    int prev = -1;
    bool switched = false;
    explicit DevGuard(int device) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != device)
            switched = (cudaSetDevice(device) == cudaSuccess);
    }
    ~DevGuard() {
        if (switched) cudaSetDevice(prev);
    }
};
}  // namespace

extern "C" {

AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_create(int device, int rank, int world,
                                                   int64_t max_rows, AilaNf4PeerBuf** out) {
    if (!out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "out is NULL");
    *out = nullptr;
    if (world < 1 || world > 8 || rank < 0 || rank >= world)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "rank/world out of range (world <= 8)");
    if (max_rows <= 0 || max_rows > (1ll << 28))
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "max_rows out of range");
    DevGuard guard(device);
    AilaNf4PeerBuf* b = new (std::nothrow) AilaNf4PeerBuf();
    if (!b) return fail(AILA_NF4_ERR_OUT_OF_MEMORY, "host allocation failed");
    b->device = device;
    b->rank = rank;
    b->world = world;
    b->max_rows = (max_rows + 15) / 16 * 16;
    b->bytes = nf4::peerbuf_bytes(world, b->max_rows);
    cudaError_t e = cudaMalloc(&b->local, b->bytes);
    if (e == cudaSuccess) e = cudaMemset(b->local, 0, b->bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(b->local);
        delete b;
        return nf4::cuda_fail(e, "peer buffer allocation");
    }
    b->base[rank] = b->local;
    b->imported[rank] = true;
    *out = b;
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_export(const AilaNf4PeerBuf* b, void* handle_out) {
    if (!b || !handle_out) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == AILA_NF4_IPC_HANDLE_BYTES, "IPC handle size");
    DevGuard guard(b->device);
    cudaIpcMemHandle_t h;
    NF4_CUDA(cudaIpcGetMemHandle(&h, b->local));
    std::memcpy(handle_out, &h, sizeof(h));
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_import(AilaNf4PeerBuf* b, int peer_rank,
                                                   const void* handle) {
    if (!b || !handle) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (peer_rank < 0 || peer_rank >= b->world || peer_rank == b->rank)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "peer_rank must name another rank of the group");
    if (b->imported[peer_rank])
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "this peer's buffer is already mapped");
    DevGuard guard(b->device);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    NF4_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    b->base[peer_rank] = p;
    b->imported[peer_rank] = true;
    b->by_ipc[peer_rank] = true;
    return AILA_NF4_OK;
}

AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_import_local(AilaNf4PeerBuf* b, int peer_rank,
                                                         const AilaNf4PeerBuf* peer) {
    if (!b || !peer) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (peer_rank < 0 || peer_rank >= b->world || peer_rank == b->rank)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "peer_rank must name another rank of the group");
    if (peer->rank != peer_rank || peer->world != b->world || peer->max_rows != b->max_rows)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "the peer's buffer belongs to another rank, group size or row count");
    if (b->imported[peer_rank])
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "this peer's buffer is already mapped");
    if (peer->device != b->device) {
        DevGuard guard(b->device);
        int can = 0;
        NF4_CUDA(cudaDeviceCanAccessPeer(&can, b->device, peer->device));
        if (!can) return fail(AILA_NF4_ERR_UNSUPPORTED, "no peer access between the two devices");
        const cudaError_t e = cudaDeviceEnablePeerAccess(peer->device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return nf4::cuda_fail(e, "cudaDeviceEnablePeerAccess");
        (void)cudaGetLastError();
    }
    b->base[peer_rank] = peer->local;
    b->imported[peer_rank] = true;
    b->by_ipc[peer_rank] = false;
    return AILA_NF4_OK;
}

AILA_NF4_API void aila_nf4_peerbuf_destroy(AilaNf4PeerBuf* b) {
    if (!b) return;
    DevGuard guard(b->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < b->world; ++r)
        if (r != b->rank && b->imported[r] && b->by_ipc[r] && b->base[r]) cudaIpcCloseMemHandle(b->base[r]);
    cudaFree(b->local);
    delete b;
}

AILA_NF4_API AilaNf4Status aila_nf4_forward_decode_allreduce(const AilaNf4Linear* l,
                                                             AilaNf4Scratch* sc,
                                                             AilaNf4PeerBuf* b, const void* x,
                                                             void* y, const void* residual,
                                                             void* stream) {
    if (!l || !sc || !b || !x || !y) return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "NULL argument");
    if (l->device != b->device || sc->device != b->device)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "linear, scratch and peer buffer must share a device");
    if (l->N > b->max_rows)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                    "out_features " + std::to_string(l->N) + " exceeds the peer buffer's " +
                        std::to_string(b->max_rows) + " rows");
    for (int r = 0; r < b->world; ++r)
        if (!b->imported[r])
            return fail(AILA_NF4_ERR_INVALID_ARGUMENT,
                        "peer buffer of rank " + std::to_string(r) + " has not been imported");
    if (reinterpret_cast<uintptr_t>(x) & 15)
        return fail(AILA_NF4_ERR_INVALID_ARGUMENT, "x must be 16-byte aligned");
    if (!nf4::gemv_stream_supported(*l, 0, sc->sm_count))
        return fail(AILA_NF4_ERR_UNSUPPORTED, "shape not taken by the streaming decode kernel");
    DevGuard guard(l->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    AilaNf4Status st = nf4::ensure_counters(sc, (size_t)l->RT);
    if (st != AILA_NF4_OK) return st;
    nf4::PeerTargets pt;
    st = nf4::peer_targets_of(b, l->device, l->N, &pt);
    if (st != AILA_NF4_OK) return st;
    // One launch when all CTAs of the grid are resident together (they wait for each other's
    // rows through the arrival counters); otherwise the GEMV publishes and a second kernel sums.
    const int grid = nf4::gemv_stream_grid(*l, 0, sc->sm_count);
    pt.inline_reduce = grid > 0 && grid <= sc->sm_count;
    if (pt.inline_reduce) {
        NF4_CUDA(nf4::launch_gemv_stream(*l, *sc, x, y, residual, 0, s, &pt));
        return AILA_NF4_OK;
    }
    NF4_CUDA(nf4::launch_gemv_stream(*l, *sc, x, nullptr, nullptr, 0, s, &pt));
    NF4_CUDA(nf4::launch_peer_reduce(nf4::part_base_of(b->local), pt.ctrl, b->world, b->max_rows,
                                     l->N, residual, y, sc->d_status, sc->wait_limit_cycles, s));
    return AILA_NF4_OK;
}

}  // extern "C"
