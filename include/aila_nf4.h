/*
 * aila_nf4.h - C ABI of the B200 (sm_100a) bitsandbytes-NF4 linear operator.
 *
 * This is the drop-in boundary for the NF4 linear path of the Aila inference engine: the
 * C++ operator class `Bnb4BitLinear` (reference src/ops/Bnb4BitLinear.hpp:26-59) keeps its
 * signatures in include/aila_nf4_linear.hpp and forwards to the functions below. Each entry
 * point names the reference interface it replaces.
 *
 * Conventions
 *  - plain C, `extern "C"`, default visibility (same export convention as the reference's
 *    include/aila_api.h:19-35); no C++ or framework types cross the boundary;
 *  - every function returns an AilaNf4Status; nothing throws. A message for the last failure
 *    on the calling thread is available from aila_nf4_last_error();
 *  - all device work is enqueued on the caller's stream (`stream` is a cudaStream_t passed as
 *    void*; NULL = the default stream) and nothing on the forward path synchronises the host;
 *  - a linear is immutable after creation and may be shared by several threads; a scratch
 *    object belongs to one stream at a time (like the reference's one
 *    Bnb4BitLinearScratch per backend, src/models/Qwen3Bnb4Backend.hpp:54);
 *  - activations are bfloat16, row-major [seq_len][features], exactly as the reference's
 *    Tensor buffers; outputs are bfloat16 with fp32 accumulation;
 *  - there is no CPU fallback: without a usable CUDA device every compute call fails with
 *    AILA_NF4_ERR_CUDA.
 */
#ifndef AILA_NF4_H
#define AILA_NF4_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#define AILA_NF4_EXTERN extern "C"
#else
#define AILA_NF4_EXTERN extern
#endif
#define AILA_NF4_API AILA_NF4_EXTERN __attribute__((visibility("default")))

typedef struct AilaNf4Linear AilaNf4Linear;   /* opaque: one quantised weight on one GPU  */
typedef struct AilaNf4Scratch AilaNf4Scratch; /* opaque: per-stream work space            */

typedef enum AilaNf4Status {
    AILA_NF4_OK = 0,
    AILA_NF4_ERR_INVALID_ARGUMENT = 1, /* bad descriptor, shape, pointer or dtype contract    */
    AILA_NF4_ERR_UNSUPPORTED = 2,      /* valid NF4 data this build does not handle            */
    AILA_NF4_ERR_CUDA = 3,             /* a CUDA runtime/driver call failed (message has it)   */
    AILA_NF4_ERR_OUT_OF_MEMORY = 4,
    AILA_NF4_NOT_APPLICABLE = 5,       /* fused fast path does not apply: caller falls back    */
    AILA_NF4_ERR_KERNEL_TIMEOUT = 6    /* a bounded device-side wait expired (status query)    */
} AilaNf4Status;

typedef enum AilaNf4ShardMode {
    AILA_NF4_SHARD_ROWS = 0, /* split out_features (column-parallel linear): q/k/v, gate, up */
    AILA_NF4_SHARD_COLS = 1  /* split in_features (row-parallel linear): o_proj, down        */
} AilaNf4ShardMode;

/*
 * One bitsandbytes 4-bit weight in checkpoint form. Mirrors Bnb4BitWeightRef +
 * Bnb4BitQuantState (reference src/utils/SafeTensors.hpp:40-81): the same tensors, as raw
 * pointers. The library copies what it needs during creation; the caller may free
 * everything as soon as the create call returns (the reference's callers erase the
 * per-projection tensors right after fusion, src/models/Qwen3Bnb4Backend.cpp:237-243).
 */
typedef struct AilaNf4WeightDesc {
    int64_t out_features;        /* quant_state.shape[0]                                    */
    int64_t in_features;         /* quant_state.shape[1]; multiple of blocksize             */
    int32_t blocksize;           /* weights per absmax; a multiple of 64                    */
    int32_t nested;              /* 1: absmax is uint8 codes (double quant); 0: float32     */
    int32_t nested_blocksize;    /* absmax values per nested_absmax (power of two), if nested */
    float nested_offset;         /* quant_state.nested_offset                               */
    const uint8_t* packed_weight;   /* [out*in/2]; high nibble = even k                     */
    const void* absmax;             /* uint8[out*in/blocksize] if nested else float[...]    */
    const float* quant_map;         /* [16]  NF4 code book                                  */
    const float* nested_absmax;     /* [ceil(blocks/nested_blocksize)] or NULL              */
    const float* nested_quant_map;  /* [256] or NULL                                        */
    int64_t nested_absmax_count;    /* elements in nested_absmax                            */
    int32_t pointers_on_device;  /* 1: the five pointers are device memory of `device`; 0: host */
    int32_t device;              /* CUDA device ordinal that will own the linear            */
} AilaNf4WeightDesc;

/* Thread-local text of the most recent failure (never NULL). Reference analogue: the
 * std::string* error_message out-parameters of Bnb4BitLinear::init*
 * (src/ops/Bnb4BitLinear.cpp:248-252) and aila_get_last_error (include/aila_api.h). */
AILA_NF4_API const char* aila_nf4_last_error(void);

/* Library/ABI version, major*10000 + minor*100 + patch. */
AILA_NF4_API int aila_nf4_version(void);

/*
 * Create a linear from checkpoint tensors: validates the descriptor with the reference
 * loader's rules (LoadBnb4BitWeightRef, src/utils/SafeTensors.cpp:443-487), regroups
 * nibbles and absmax codes into the 16-byte-aligned unit stream and keeps the second-level
 * scales for in-kernel expansion. Replaces Bnb4BitLinear::init
 * (src/ops/Bnb4BitLinear.cpp:453-497), which expands absmax to fp32 on the host.
 * Synchronous (load time).
 */
AILA_NF4_API AilaNf4Status aila_nf4_linear_create(const AilaNf4WeightDesc* desc,
                                                  AilaNf4Linear** out);

/*
 * Create only rank `rank` of `world` of the weight described by `desc` (which describes the
 * WHOLE weight). ROWS keeps rows [rank*N/world, (rank+1)*N/world); COLS keeps input columns
 * [rank*K/world, (rank+1)*K/world) and requires K/world to be a multiple of blocksize. The
 * shard keeps the original second-level numbering, so its dequantised values are bit-equal
 * to the same slice of the whole weight. No reference counterpart (the reference is
 * single-device); net-new for the multi-GPU layer.
 */
AILA_NF4_API AilaNf4Status aila_nf4_linear_create_shard(const AilaNf4WeightDesc* desc,
                                                        AilaNf4ShardMode mode, int rank,
                                                        int world, AilaNf4Linear** out);

/*
 * Concatenate 2..4 linears along out_features into a new linear (q|k|v, gate|up). Sources
 * must share device, in_features, blocksize and quant_map (max abs difference 1e-6), the
 * checks of Bnb4BitLinear::init_fused_rows (src/ops/Bnb4BitLinear.cpp:499-629). The result
 * owns its memory; sources may be destroyed afterwards. Synchronous (load time).
 */
AILA_NF4_API AilaNf4Status aila_nf4_linear_create_fused_rows(AilaNf4Linear* const* sources,
                                                             int n_sources,
                                                             AilaNf4Linear** out);

AILA_NF4_API void aila_nf4_linear_destroy(AilaNf4Linear* linear);

/* Bnb4BitLinear::in_features() / out_features() (src/ops/Bnb4BitLinear.hpp:58-59). */
AILA_NF4_API int64_t aila_nf4_linear_in_features(const AilaNf4Linear* linear);
AILA_NF4_API int64_t aila_nf4_linear_out_features(const AilaNf4Linear* linear);
/* Bytes of device memory the linear owns (weights + scales). */
AILA_NF4_API int64_t aila_nf4_linear_device_bytes(const AilaNf4Linear* linear);
AILA_NF4_API int aila_nf4_linear_device(const AilaNf4Linear* linear);

/*
 * Work space used by forward calls: split-K partial sums and tile counters of the decode
 * kernels, and the bf16 weight buffer of the prefill route. Mirrors Bnb4BitLinearScratch
 * (src/ops/Bnb4BitLinear.hpp:12-24): grow-only, shared by all linears of one engine.
 */
AILA_NF4_API AilaNf4Status aila_nf4_scratch_create(int device, AilaNf4Scratch** out);
AILA_NF4_API void aila_nf4_scratch_destroy(AilaNf4Scratch* scratch);
/*
 * Pre-size the work space so later forward calls never allocate (call before capturing a
 * CUDA graph). Mirrors Bnb4BitLinearScratch::ensure (src/ops/Bnb4BitLinear.cpp:414-451);
 * need_weight != 0 reserves the [out,in] bf16 weight buffer the seq_len > 1 route uses; seq_len > 1
 * also reserves the fp32 accumulation tiles of the small-batch decode kernel (128 bytes per output row).
 * A decode call for more than 262,144 output rows that was not reserved for grows the work space
 * inside the call: it allocates and waits for the device, so it cannot be captured.
 */
AILA_NF4_API AilaNf4Status aila_nf4_scratch_reserve(AilaNf4Scratch* scratch, int seq_len,
                                                    int64_t in_features, int64_t out_features,
                                                    int need_weight);
/* Reads (and clears) the device-side status word: AILA_NF4_OK, or
 * AILA_NF4_ERR_KERNEL_TIMEOUT if a bounded wait inside a kernel expired since the last
 * query. Synchronises `stream`. */
AILA_NF4_API AilaNf4Status aila_nf4_scratch_check(AilaNf4Scratch* scratch, void* stream);

/*
 * y[seq_len][out] = x[seq_len][in] * W^T (+ residual), all bfloat16 device pointers.
 * Replaces Bnb4BitLinear::forward (src/ops/Bnb4BitLinear.cpp:799-949):
 *   seq_len == 1  -> streaming decode GEMV (reference packed_nf4_gemv_bf16, :271-410),
 *                    fp32 accumulation, one rounding to bf16;
 *   seq_len 2..48 -> small-batch decode launches of up to 32 rows each (one pass over the
 *                    packed weights per launch, fp32 accumulation; no reference counterpart:
 *                    the reference takes its seq_len > 1 route from two rows on);
 *   above         -> weights rounded to bf16 exactly as dequantize_weight (:723-757) does,
 *                    then a tcgen05 tensor-core GEMM with fp32 accumulation (the reference
 *                    runs an oneDNN bf16 matmul, :689-721, :944). With blocksize 128 the
 *                    reference instead takes a fused kernel (:18-136) whose result is not
 *                    x W^T; this library returns x W^T for every blocksize.
 * `residual` (or NULL) is bf16 [seq_len][out] added before the final rounding - the
 * documented meaning of add_residual (:323); the reference's SG16 branch ignores it.
 * Errors: seq_len <= 0 and NULL pointers give AILA_NF4_ERR_INVALID_ARGUMENT where the
 * reference throws std::runtime_error (:805-811).
 */
AILA_NF4_API AilaNf4Status aila_nf4_forward(const AilaNf4Linear* linear, AilaNf4Scratch* scratch,
                                            const void* x_bf16, void* y_bf16, int seq_len,
                                            const void* residual_bf16, void* stream);

/*
 * out[seq_len][ff_dim] = silu(x*Wg^T) .* (x*Wu^T) for a fused gate|up linear whose first
 * ff_dim rows are gate and last ff_dim rows are up. Replaces
 * Bnb4BitLinear::try_forward_decode_gate_up_swiglu (src/ops/Bnb4BitLinear.cpp:759-797) for
 * seq_len == 1 (gate and up stay fp32 until the product is rounded once, :241-242) and the
 * forward + ops::fused_gate_up_swiglu pair (src/ops/ElementwiseOps.cpp:247-294) for
 * seq_len > 1 (gate and up are rounded to bf16 first, as that pair does).
 * Returns AILA_NF4_NOT_APPLICABLE where the reference returns false (out_features !=
 * 2*ff_dim, :772) or when ff_dim is not a multiple of 16; the caller then uses
 * aila_nf4_forward followed by its own SwiGLU.
 */
AILA_NF4_API AilaNf4Status aila_nf4_forward_gate_up_swiglu(const AilaNf4Linear* fused_gate_up,
                                                           AilaNf4Scratch* scratch,
                                                           const void* x_bf16, void* out_bf16,
                                                           int seq_len, int64_t ff_dim,
                                                           void* stream);

/*
 * Same two operations with HOST buffers: copies x to the device, runs the operator, copies
 * the result back and waits for it. For callers that keep activations on the host, and the
 * end-to-end timing path of the benchmark. Host buffers should be pinned.
 */
AILA_NF4_API AilaNf4Status aila_nf4_forward_host(const AilaNf4Linear* linear,
                                                 AilaNf4Scratch* scratch, const void* x_host_bf16,
                                                 void* y_host_bf16, int seq_len, void* stream);
AILA_NF4_API AilaNf4Status aila_nf4_forward_gate_up_swiglu_host(
    const AilaNf4Linear* fused_gate_up, AilaNf4Scratch* scratch, const void* x_host_bf16,
    void* out_host_bf16, int seq_len, int64_t ff_dim, void* stream);

/*
 * Decode step (seq_len == 1) y = W x (+ residual) that allocates nothing, ever: no cudaMalloc,
 * no cudaFree, no scratch object. No counterpart in the reference (its Context::alloc_device,
 * src/core/Context.hpp:28-40, is always available to it); added for hosts that must keep the
 * CUDA allocator off their token loop - for instance an engine that hands all device memory to
 * its own pool at start-up, so a late cudaMalloc could fail or fragment it, or a serving loop
 * that cannot afford the device-wide synchronisation an allocation or free implies.
 * The split-K work space of the streaming kernel is a fixed array inside the library
 * (about 385 KB per GPU, held from library load to process exit). Consequences:
 *  - out_features is limited to 262,144 rows; larger or otherwise untaken shapes return
 *    AILA_NF4_ERR_UNSUPPORTED with a message, never a silent fallback;
 *  - all calls on one GPU share the array: two calls whose kernels overlap on the GPU (different
 *    streams) race on it - keep calls to this entry point on one stream per GPU;
 *  - the first call on each GPU looks up the array's device address; make that call before any
 *    stream capture begins.
 * Results are identical to aila_nf4_forward with seq_len == 1 (it always runs the streaming ring
 * kernel, whatever aila_nf4_set_gemv_kernel says). A bounded wait that runs out inside the
 * kernel leaves a code in a status word of the same array: aila_nf4_static_check(device, stream)
 * reads and clears it (synchronises the stream; allocates nothing) and returns
 * AILA_NF4_ERR_KERNEL_TIMEOUT if a wait expired since the last check.
 */
AILA_NF4_API AilaNf4Status aila_nf4_forward_decode_static(const AilaNf4Linear* linear,
                                                          const void* x_bf16, void* y_bf16,
                                                          const void* residual_bf16,
                                                          void* stream);
AILA_NF4_API AilaNf4Status aila_nf4_static_check(int device, void* stream);

/*
 * Row-parallel decode with the sum exchange folded into the GEMV. No reference counterpart
 * (the reference runs on one device). For a linear that holds a COLUMN shard of the weight
 * (aila_nf4_linear_create_shard, AILA_NF4_SHARD_COLS) every rank computes a partial y; the
 * kernel stores its fp32 row sums straight into every rank's exchange buffer over NVLink
 * (plain peer stores of 8-byte {value, tag} words; no multicast object, no load from another
 * GPU's memory) and the ranks' rows are summed in rank order - by the same launch when its grid
 * is one thread block per SM, else by a small second kernel: all ranks obtain the bit-identical
 * y = bf16(sum_r W_r x_r (+ residual)).
 *
 * Set-up, once per process group (one process per GPU, all on one node): every rank creates an
 * AilaNf4PeerBuf for `max_rows` >= the largest out_features it will be used with, exports its
 * 64-byte handle, hands it to the other ranks by any host channel, and imports theirs.
 * Rules: all ranks issue the same aila_nf4_forward_decode_allreduce calls in the same order;
 * the calls of one buffer go to one stream per GPU; the sequence may be captured in a CUDA
 * graph (all exchange state lives on the device). A rank that waits longer for another rank than
 * the scratch's wait limit (about a second unless aila_nf4_scratch_set_wait_limit changed it)
 * records AILA_NF4_ERR_KERNEL_TIMEOUT for aila_nf4_scratch_check; y is then not written, and the
 * buffers of the group must be recreated.
 */
typedef struct AilaNf4PeerBuf AilaNf4PeerBuf;
#define AILA_NF4_IPC_HANDLE_BYTES 64
AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_create(int device, int rank, int world,
                                                   int64_t max_rows, AilaNf4PeerBuf** out);
AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_export(const AilaNf4PeerBuf* buf, void* handle_out);
AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_import(AilaNf4PeerBuf* buf, int peer_rank,
                                                   const void* handle);
/* The same for a peer whose buffer was created by THIS process (one process that drives several
 * GPUs, or two ranks of a test on one GPU): no handle, the buffer itself. The peer's buffer must
 * outlive this one's use. */
AILA_NF4_API AilaNf4Status aila_nf4_peerbuf_import_local(AilaNf4PeerBuf* buf, int peer_rank,
                                                         const AilaNf4PeerBuf* peer);
AILA_NF4_API void aila_nf4_peerbuf_destroy(AilaNf4PeerBuf* buf);
/* seq_len == 1 only; x is this rank's column slice [in_features / world] (bf16, 16-byte
 * aligned), y receives all out_features rows. */
AILA_NF4_API AilaNf4Status aila_nf4_forward_decode_allreduce(const AilaNf4Linear* linear,
                                                             AilaNf4Scratch* scratch,
                                                             AilaNf4PeerBuf* buf,
                                                             const void* x_bf16, void* y_bf16,
                                                             const void* residual_bf16,
                                                             void* stream);

/*
 * Residual add + RMSNorm in front of a decode linear, folded into the linear's launch
 * (reference: ops::fused_add_rms_norm, src/ops/NormOps.cpp:141-260, launched before the qkv and
 * gate|up linears at src/models/Qwen3Bnb4Backend.cpp:403 and :422). With v = x + add (fp32, not
 * rounded): the linear's input is bf16(v * rsqrt(mean(v^2) + eps) * weight) and hidden_out, if
 * given, receives bf16(v) - the updated residual stream. seq_len == 1 only.
 * hidden_out must not alias x or add (every thread block of the launch reads them);
 * aila_add_rms_norm below is the stand-alone operator (any row count, hidden_out may alias x)
 * for the cases these entry points answer with AILA_NF4_NOT_APPLICABLE.
 */
typedef struct AilaNf4RmsNorm {
    const void* add_bf16;     /* [in_features] added to x first, or NULL                 */
    const void* weight_bf16;  /* [in_features] RMSNorm weight                            */
    float eps;
    void* hidden_out_bf16;    /* [in_features] receives bf16(x + add), or NULL           */
} AilaNf4RmsNorm;
AILA_NF4_API AilaNf4Status aila_nf4_forward_rmsnorm(const AilaNf4Linear* linear,
                                                    AilaNf4Scratch* scratch, const void* x_bf16,
                                                    const AilaNf4RmsNorm* norm, void* y_bf16,
                                                    const void* residual_bf16, void* stream);
AILA_NF4_API AilaNf4Status aila_nf4_forward_gate_up_swiglu_rmsnorm(
    const AilaNf4Linear* fused_gate_up, AilaNf4Scratch* scratch, const void* x_bf16,
    const AilaNf4RmsNorm* norm, void* out_bf16, int64_t ff_dim, void* stream);
AILA_NF4_API AilaNf4Status aila_add_rms_norm(const void* x_bf16, const void* add_bf16,
                                             const void* weight_bf16, float eps, int rows,
                                             int hidden_size, void* hidden_out_bf16,
                                             void* normed_out_bf16, int device, void* stream);

/*
 * A chain of decode (seq_len == 1) linears run by ONE kernel launch. Replaces the sequence of
 * Bnb4BitLinear::forward / try_forward_decode_gate_up_swiglu calls that the reference's decode
 * step issues back to back (src/models/Qwen3Bnb4Backend.cpp:400-418: o_proj, fused add+RMSNorm,
 * gate_up + SwiGLU, down_proj; src/models/Qwen35HybridBnb4Backend.cpp:2140-2197), where every
 * call is one queue submission. The operations run in list order; operation i may take the
 * output of operation i-1 as its input (x_bf16 == NULL, or x_bf16 equal to the previous
 * operation's y_bf16), optionally through the residual add + RMSNorm of AilaNf4RmsNorm. An
 * operation with an input of its own still starts only after the previous one has finished.
 * Rules: all linears share their code books (quant_map, nested_quant_map) and the scratch's
 * device; in_features of a linked operation equals the previous output size; at most 160
 * operations; in_features <= 40,832 (x lives in shared memory), and with double-quantized
 * absmax in_features <= 256 * blocksize (a row then changes its second-level block at most
 * once; 16,384 at blocksize 64); an operation with a fused RMSNorm takes in_features <= 11,520.
 * Buffers named in the list must
 * stay valid for the life of the chain; an operation must not read, through a pointer of its own,
 * memory that an earlier operation of the same chain writes (use the link instead).
 * The launch is cooperative (one thread block per SM, all resident) and every device-side wait is
 * bounded (aila_nf4_scratch_set_wait_limit); a wait that runs out is reported by
 * aila_nf4_scratch_check as AILA_NF4_ERR_KERNEL_TIMEOUT. One chain launch at a time per scratch.
 * Creation is synchronous (load time); aila_nf4_chain_run only enqueues and may be captured in a
 * CUDA graph.
 */
typedef struct AilaNf4Chain AilaNf4Chain;
typedef struct AilaNf4ChainOp {
    const AilaNf4Linear* linear;
    int64_t ff_dim;             /* > 0: fused gate|up linear, output silu(gate) .* up [ff_dim]   */
    const void* x_bf16;         /* [in_features] device memory; NULL: the previous output        */
    void* y_bf16;               /* [out] device memory; may be NULL when the next op consumes it */
    const void* residual_bf16;  /* [out] added before the rounding, or NULL (not with ff_dim)    */
    const AilaNf4RmsNorm* norm;        /* residual add + RMSNorm in front of the linear, or NULL */
} AilaNf4ChainOp;
AILA_NF4_API AilaNf4Status aila_nf4_chain_create(AilaNf4Scratch* scratch, const AilaNf4ChainOp* ops,
                                                 int n_ops, AilaNf4Chain** out);
AILA_NF4_API void aila_nf4_chain_destroy(AilaNf4Chain* chain);
AILA_NF4_API int aila_nf4_chain_length(const AilaNf4Chain* chain);
/* A chain whose LAST operation is row-parallel (its linear holds a column shard of the weight,
 * aila_nf4_linear_create_shard with AILA_NF4_SHARD_COLS): the launch stores that operation's fp32
 * row sums into every rank's exchange buffer and writes y_bf16 of the last operation as
 * bf16(sum over the ranks (+ residual_bf16)), bit-identical on all ranks - the exchange of
 * aila_nf4_forward_decode_allreduce inside the chained launch (for example gate|up -> down of
 * a tensor-parallel MLP in one launch per rank). The rules of both apply: every rank runs the
 * same chains in the same order on one stream per GPU; the buffer must outlive the chain. No
 * reference counterpart. */
AILA_NF4_API AilaNf4Status aila_nf4_chain_create_allreduce(AilaNf4Scratch* scratch,
                                                           const AilaNf4ChainOp* ops, int n_ops,
                                                           AilaNf4PeerBuf* peers, AilaNf4Chain** out);
AILA_NF4_API AilaNf4Status aila_nf4_chain_run(AilaNf4Chain* chain, void* stream);
/* Same with HOST buffers at both ends: copies x of the first operation (in_features bf16) to
 * the device buffer named in the list, runs the chain, copies the last operation's y back and
 * waits for it. One copy in, one launch, one copy out, one synchronisation for the whole chain. */
AILA_NF4_API AilaNf4Status aila_nf4_chain_run_host(AilaNf4Chain* chain, const void* x_host_bf16,
                                                   void* y_host_bf16, void* stream);
/* Bound, in SM clock cycles, of every device-side wait of the decode kernels launched with this
 * scratch: the chained kernel, the single-call kernel and the row-parallel exchange (default
 * 2e9, about a second). Takes effect at the next launch. No reference counterpart. */
AILA_NF4_API AilaNf4Status aila_nf4_scratch_set_wait_limit(AilaNf4Scratch* scratch,
                                                           int64_t sm_cycles);

/*
 * Dense bf16 linear y = x W^T (+ residual), W bf16 [out_features][in_features]: the unquantised
 * projection next to the NF4 linears (the lm_head). Replaces class Linear for this use
 * (reference src/ops/Ops.hpp:16-31: init(ctx, weight, in_features, out_features) and
 * forward(ctx, input, output, seq_len); src/ops/Linear.cpp:172-256; call site
 * src/models/Qwen3Bnb4Backend.cpp:432-439). seq_len == 1 runs an HBM-bound streaming GEMV,
 * seq_len > 1 the tcgen05 GEMM (needs in_features % 64 == 0). The weight is copied at creation.
 * The bias / GELU variants of the reference class (vision and audio towers) are not built.
 */
typedef struct AilaDenseLinear AilaDenseLinear;
AILA_NF4_API AilaNf4Status aila_dense_linear_create(const void* weight_bf16, int64_t out_features,
                                                    int64_t in_features, int weight_on_device,
                                                    int device, AilaDenseLinear** out);
AILA_NF4_API void aila_dense_linear_destroy(AilaDenseLinear* linear);
AILA_NF4_API int64_t aila_dense_linear_in_features(const AilaDenseLinear* linear);
AILA_NF4_API int64_t aila_dense_linear_out_features(const AilaDenseLinear* linear);
AILA_NF4_API AilaNf4Status aila_dense_linear_forward(const AilaDenseLinear* linear,
                                                     AilaNf4Scratch* scratch, const void* x_bf16,
                                                     void* y_bf16, int seq_len,
                                                     const void* residual_bf16, void* stream);
/* Greedy token choice over n bf16 logits on the device (reference ops::argmax,
 * src/ops/SamplingOps.cpp:321-365): index of the largest value, written to *d_result (device
 * memory). Equal values resolve as in the reference's 256-item reduction, which keeps the left
 * candidate at every level: the smallest bit-reversed (index % 256) wins, then the smallest index.
 * NaN and values <= -1e30 never win; if nothing wins the result is 0. */
AILA_NF4_API AilaNf4Status aila_argmax_bf16(const void* logits_bf16, int64_t n, int32_t* d_result,
                                            int device, void* stream);
/* The same over one shard of a vocabulary (no reference counterpart): logits[0] has the global
 * index index_offset, ties are resolved on global indices, *d_result is the LOCAL index. */
AILA_NF4_API AilaNf4Status aila_argmax_bf16_shard(const void* logits_bf16, int64_t n, int64_t index_offset,
                                                  int32_t* d_result, int device, void* stream);

/*
 * The operators of a decode step between the linears (the reference's callers of this path,
 * src/models/Qwen3Bnb4Backend.cpp:298-439): simple kernels with the reference's arithmetic and
 * roundings, so that a backend built on this library runs end to end.
 *   aila_embedding_lookup      ops::embedding_lookup   (src/ops/ElementwiseOps.cpp:14-27)
 *   aila_decode_prepare_qkv    ops::decode_prepare_qkv (src/ops/ElementwiseOps.cpp:105-215): per
 *       head RMSNorm of q and k (weights [head_dim]), rotation by start_pos * rope_freq[d]
 *       (rope_freq[d] = theta^(-2d/head_dim), d < head_dim/2; halves d and d + head_dim/2 pair
 *       up), in place; k and v of the new token are appended to the caches
 *       [kv_head][max_seq_len][head_dim] at start_pos.
 *   aila_attention_decode      ops::attention_decode, baseline form (src/ops/AttentionOps.cpp:
 *       73-166): one query token against cached_len cached positions, grouped-query heads,
 *       scale 1/sqrt(head_dim), fp32 softmax; at most about 51,000 cached positions.
 * position_device (may be NULL) lets the position live on the device, so that a whole decode step
 * can be one CUDA graph replayed per token: when given, aila_decode_prepare_qkv uses
 * *position_device instead of start_pos, and aila_attention_decode uses *position_device + 1
 * cached positions, of which the launch can hold `cached_len` (pass the window's size).
 */
AILA_NF4_API AilaNf4Status aila_embedding_lookup(const void* table_bf16, int64_t vocab_size,
                                                 const int32_t* token_ids_device, int seq_len,
                                                 int hidden_size, void* out_bf16, int device,
                                                 void* stream);
AILA_NF4_API AilaNf4Status aila_decode_prepare_qkv(void* q_bf16, void* k_bf16, const void* v_bf16,
                                                   const float* rope_freq, const void* q_norm_weight_bf16,
                                                   const void* k_norm_weight_bf16, void* k_cache_bf16,
                                                   void* v_cache_bf16, int max_seq_len, int start_pos,
                                                   const int32_t* position_device, int num_heads_q,
                                                   int num_kv_heads, int head_dim, float eps, int device,
                                                   void* stream);
AILA_NF4_API AilaNf4Status aila_attention_decode(const void* q_bf16, const void* k_cache_bf16,
                                                 const void* v_cache_bf16, void* out_bf16, int num_heads,
                                                 int num_kv_heads, int head_dim, int cached_len,
                                                 const int32_t* position_device, int max_seq_len, int device,
                                                 void* stream);

/*
 * Checkpoint front-end (host side, no GPU work): a memory-mapped safetensors file and the
 * assembly of one bitsandbytes 4-bit weight into an AilaNf4WeightDesc whose pointers lie
 * inside the mapping, ready for aila_nf4_linear_create (keep the file open until the create
 * call has returned). Replaces, for this path, LoadSafetensors + LoadBnb4BitWeightRef
 * (reference src/utils/SafeTensors.hpp:127-140, src/utils/SafeTensors.cpp:154-222 and
 * :370-489): same side-tensor names (<w>.absmax, <w>.quant_map, <w>.nested_absmax,
 * <w>.nested_quant_map, <w>.quant_state.bitsandbytes__nf4), same dtype rules, same size
 * invariants, same quant_state JSON keys; a violated rule returns
 * AILA_NF4_ERR_INVALID_ARGUMENT (AILA_NF4_ERR_UNSUPPORTED for a quant_type other than nf4)
 * with the reference's wording in aila_nf4_last_error().
 */
typedef struct AilaStFile AilaStFile;
typedef enum AilaStDtype {
    AILA_ST_DTYPE_UNKNOWN = 0, AILA_ST_U8, AILA_ST_I8, AILA_ST_F16, AILA_ST_BF16, AILA_ST_F32,
    AILA_ST_F64, AILA_ST_I32, AILA_ST_I64, AILA_ST_BOOL
} AilaStDtype;
#define AILA_ST_MAX_RANK 8
typedef struct AilaStTensorView {
    int32_t dtype;                 /* AilaStDtype */
    int32_t rank;
    int64_t shape[AILA_ST_MAX_RANK];
    const void* data;              /* inside the mapping; valid until aila_st_close */
    int64_t nbytes;
} AilaStTensorView;
AILA_NF4_API AilaNf4Status aila_st_open(const char* path, AilaStFile** out);
AILA_NF4_API void aila_st_close(AilaStFile* file);
AILA_NF4_API int64_t aila_st_tensor_count(const AilaStFile* file);
AILA_NF4_API const char* aila_st_tensor_name(const AilaStFile* file, int64_t index);
/* AILA_NF4_NOT_APPLICABLE when the file holds no tensor of that name. */
AILA_NF4_API AilaNf4Status aila_st_find(const AilaStFile* file, const char* name,
                                        AilaStTensorView* out);
AILA_NF4_API AilaNf4Status aila_st_load_bnb4_weight(const AilaStFile* file, const char* name,
                                                    int device, AilaNf4WeightDesc* out);
/* A model directory (reference LoadModelWeightsFromDir, src/utils/SafeTensors.cpp:491-535, and
 * parse_sharded_safetensors_index, :336-366): `model.safetensors` if it exists, otherwise the
 * shards that `model.safetensors.index.json` names in its weight_map, opened in sorted order.
 * A tensor that several shards hold is taken from the last of them (the reference's merge
 * replaces earlier entries). aila_st_dir_find / aila_st_dir_load_bnb4_weight look through all
 * shards, so the side tensors of a weight may sit in another shard than its packed bytes. The
 * reference's messages are kept ("No model.safetensors or model.safetensors.index.json found
 * in: ...", "Invalid safetensors index: missing weight_map", "Missing safetensors shard: ..."). */
typedef struct AilaStDir AilaStDir;
AILA_NF4_API AilaNf4Status aila_st_dir_open(const char* model_dir, AilaStDir** out);
AILA_NF4_API void aila_st_dir_close(AilaStDir* dir);
AILA_NF4_API int64_t aila_st_dir_shard_count(const AilaStDir* dir);
AILA_NF4_API const AilaStFile* aila_st_dir_shard(const AilaStDir* dir, int64_t index);
AILA_NF4_API AilaNf4Status aila_st_dir_find(const AilaStDir* dir, const char* name, AilaStTensorView* out);
AILA_NF4_API AilaNf4Status aila_st_dir_load_bnb4_weight(const AilaStDir* dir, const char* name, int device,
                                                        AilaNf4WeightDesc* out);

/*
 * Whole-weight dequantisation into the TRANSPOSED bf16 matrix Wt[in][out], bit-equal to
 * Bnb4BitLinear::dequantize_weight (src/ops/Bnb4BitLinear.cpp:723-757):
 * Wt[k*out + n] = bf16(quant_map[nibble(n,k)] * absmax(n, k/blocksize)).
 */
AILA_NF4_API AilaNf4Status aila_nf4_dequantize(const AilaNf4Linear* linear, void* out_bf16_kn,
                                               void* stream);
/* Same values in the natural orientation W[out][in] (what the prefill GEMM consumes). */
AILA_NF4_API AilaNf4Status aila_nf4_dequantize_rowmajor(const AilaNf4Linear* linear,
                                                        void* out_bf16_nk, void* stream);
/* fp32 absmax of every (row, block), [out][in/blocksize]: what Bnb4BitLinear::init
 * (src/ops/Bnb4BitLinear.cpp:472-488) computes on the host. */
AILA_NF4_API AilaNf4Status aila_nf4_expand_absmax(const AilaNf4Linear* linear, void* out_f32,
                                                  void* stream);

/*
 * Kernel selection for the seq_len == 1 route, for A/B measurement: 0 = automatic,
 * 1 = plain CUDA-core kernel (fp32 weights, exactly the reference's arithmetic up to
 * summation order), 2 = streaming tensor-core kernel with a shared-memory ring (what automatic
 * picks for a single call when it takes the shape), 3 = the chained kernel as a one-operation
 * launch. Process-wide; also settable with the
 * environment variable AILA_NF4_GEMV_KERNEL read at first use.
 */
AILA_NF4_API AilaNf4Status aila_nf4_set_gemv_kernel(int which);

#endif /* AILA_NF4_H */
