/*
 * nf4_oracle.c -- CPU restatement of the reference's bitsandbytes-NF4 linear path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA library; nothing the
 * library ships calls into it. It restates, in plain C, the arithmetic of the reference
 * operator src/ops/Bnb4BitLinear.cpp (Blackwood416/Aila v0.1.2). Every function cites the
 * reference lines it follows.
 *
 * PARITY PINNED AGAINST THE REFERENCE'S SOURCE: the reference holds no golden vectors,
 * known-answer tests or numeric fixtures for this path, and no SYCL compiler or oneDNN exists
 * in a CUDA-only image; instead src/ops/Bnb4BitLinear.cpp itself is compiled unmodified with
 * g++ against a serial host stand-in for the SYCL / oneDNN headers (oracle/ref_shim/,
 * oracle/ref_harness.cpp -> oracle/_ref/libaila_ref.so) and tests/test_reference_pin.py holds
 * this restatement bit-exact against it: absmax expansion, dequantisation, both GEMV branches,
 * fused rows, gate+up+SiLU, the seq_len > 1 route. Two things stay the stand-in's choice, not
 * the reference's: the order of sub-group / work-group reductions (unspecified in SYCL; a
 * balanced tree on both sides) and the bf16 matmul after dequantisation (oneDNN in the
 * reference; k-ascending fp32 accumulation on both sides). The quantiser and the code books
 * of third-party bitsandbytes are absent, so the ENCODE side stays unpinned; they are runtime
 * inputs here as in the reference. Also pinned by a second independent numpy restatement
 * (oracle/nf4_numpy.py) and hand-computed tiny cases in tests/.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: the reference source writes the double-quant expansion as a
 * multiply followed by an add; the canonical oracle keeps them as two rounded fp32 ops. A
 * fused variant is provided so the difference can be counted.
 *
 * Data layout (as stored in a bitsandbytes NF4 checkpoint and consumed by the reference):
 *   packed   u8  [N*K/2]   row-major [N][K/2]; HIGH nibble = even k, LOW nibble = odd k
 *   absmax   f32 [N*K/bs]  flat index = (n*K + k) / bs
 *   qmap     f32 [16]      NF4 codebook (runtime tensor, never hard-coded)
 *   nested: codes u8 [N*K/bs], nested_map f32 [256], nested_absmax f32 [ceil(blocks/nbs)],
 *           nested_offset f32
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

typedef uint16_t bf16_t;

/* float -> bfloat16, round-to-nearest-even, NaN kept quiet. This is the conversion
 * sycl::ext::oneapi::bfloat16(float) performs on the reference's device. */
static inline bf16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (bf16_t)(u >> 16);
}

static inline float bf16_to_f32(bf16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

int nf4o_num_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void nf4o_set_num_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Double-quant expansion. Bnb4BitLinear.cpp:472-488 (Bnb4BitLinear::init):
 *   absmax[i] = nested_quant_map[code[i]] * nested_absmax[i / nested_blocksize] + nested_offset
 * flat_base / the per-call index base lets a caller expand a slice whose first block has
 * flat index flat_base in the original tensor (used for shards); the reference always
 * passes the whole tensor (flat_base = 0). */
void nf4o_expand_absmax(const uint8_t* codes, int64_t n_blocks, const float* nested_map,
                        const float* nested_absmax, int nested_blocksize, float nested_offset,
                        int64_t flat_base, float* out) {
    for (int64_t i = 0; i < n_blocks; ++i) {
        const int64_t nb = (flat_base + i) / nested_blocksize;
        const float prod = nested_map[codes[i]] * nested_absmax[nb];
        out[i] = prod + nested_offset;
    }
}

/* Same expression contracted into one fma, the other legal reading of a -ffast-math build
 * (CMakeLists.txt:24). Only used to count how many values differ from the canonical form. */
void nf4o_expand_absmax_fused(const uint8_t* codes, int64_t n_blocks, const float* nested_map,
                              const float* nested_absmax, int nested_blocksize,
                              float nested_offset, int64_t flat_base, float* out) {
    for (int64_t i = 0; i < n_blocks; ++i) {
        const int64_t nb = (flat_base + i) / nested_blocksize;
        out[i] = fmaf(nested_map[codes[i]], nested_absmax[nb], nested_offset);
    }
}

/* Whole-weight dequantisation into the TRANSPOSED bf16 matrix Wt[K][N].
 * Bnb4BitLinear.cpp:723-757 (dequantize_weight): one item per packed byte,
 *   hi = byte >> 4 -> flat0 = 2*byte_index, lo = byte & 15 -> flat0 + 1,
 *   row = flat / K, col = flat % K, out[col*N + row] = bf16(qmap[nib] * absmax[flat / bs]). */
void nf4o_dequantize_kn(const uint8_t* packed, const float* qmap, const float* absmax,
                        int64_t N, int64_t K, int blocksize, bf16_t* out_kn) {
    const int64_t total = N * K;
    const int64_t nbytes = total / 2;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nbytes; ++b) {
        const uint8_t p = packed[b];
        const int64_t flat0 = 2 * b;
        const int64_t flat1 = flat0 + 1;
        if (flat0 < total) {
            const int64_t row = flat0 / K, col = flat0 % K;
            out_kn[col * N + row] = f32_to_bf16(qmap[(p >> 4) & 15] * absmax[flat0 / blocksize]);
        }
        if (flat1 < total) {
            const int64_t row = flat1 / K, col = flat1 % K;
            out_kn[col * N + row] = f32_to_bf16(qmap[p & 15] * absmax[flat1 / blocksize]);
        }
    }
}

/* Row-major (untransposed) dequantisation W[N][K]; same arithmetic as above, used by tests
 * that want the weight in its natural orientation. */
void nf4o_dequantize_nk(const uint8_t* packed, const float* qmap, const float* absmax,
                        int64_t N, int64_t K, int blocksize, bf16_t* out_nk) {
    const int64_t nbytes = N * K / 2;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nbytes; ++b) {
        const uint8_t p = packed[b];
        const int64_t flat0 = 2 * b;
        out_nk[flat0] = f32_to_bf16(qmap[(p >> 4) & 15] * absmax[flat0 / blocksize]);
        out_nk[flat0 + 1] = f32_to_bf16(qmap[p & 15] * absmax[(flat0 + 1) / blocksize]);
    }
}

/* pairwise tree sum of 16 lane partials: the order sycl::reduce_over_group leaves
 * unspecified; a balanced tree is the common sub-group implementation. */
static inline float tree_sum16(const float* v) {
    float t[16];
    memcpy(t, v, sizeof(t));
    for (int w = 8; w >= 1; w >>= 1)
        for (int i = 0; i < w; ++i) t[i] = t[i] + t[i + w];
    return t[0];
}

/* One output row of the decode GEMV, SG16 branch. Bnb4BitLinear.cpp:353-407:
 * lane l in [0,16) starts at byte 4*l and strides 64 bytes; per step it reads 4 packed
 * bytes (8 weights), one absmax (byte_offset / (bs/2)) and 8 bf16 inputs, and issues 8
 * sequential fma(x, qmap[nib]*am, partial); a byte-granular tail loop follows (stride 16);
 * the 16 partials are summed over the sub-group. */
static float gemv_row_sg16(const uint8_t* row_bytes, const float* row_absmax, const float* qmap,
                           const bf16_t* x, int bytes_per_row, int bytes_per_block) {
    float lane[16];
    for (int l = 0; l < 16; ++l) {
        float partial = 0.0f;
        int off = l * 4;
        for (; off + 3 < bytes_per_row; off += 64) {
            const float am = row_absmax[off / bytes_per_block];
            const int ib = off * 2;
            for (int j = 0; j < 4; ++j) {
                const uint8_t b = row_bytes[off + j];
                partial = fmaf(bf16_to_f32(x[ib + 2 * j]), qmap[b >> 4] * am, partial);
                partial = fmaf(bf16_to_f32(x[ib + 2 * j + 1]), qmap[b & 15] * am, partial);
            }
        }
        for (; off < bytes_per_row; off += 16) {
            const uint8_t b = row_bytes[off];
            const float am = row_absmax[off / bytes_per_block];
            const int ii = off * 2;
            partial = fmaf(bf16_to_f32(x[ii]), qmap[(b >> 4) & 15] * am, partial);
            partial = fmaf(bf16_to_f32(x[ii + 1]), qmap[b & 15] * am, partial);
        }
        lane[l] = partial;
    }
    return tree_sum16(lane);
}

/* One output row, small-K branch (K/2 < 256 bytes). Bnb4BitLinear.cpp:291-326: a work-group
 * of wg (=128 here, since bytes_per_row < 1024) items strides the row byte by byte with
 *   partial += x * qmap[nib] * absmax    (left-to-right: (x*q)*am, unfused add)
 * then a work-group reduce. Items beyond bytes_per_row contribute 0. */
static float gemv_row_smallk(const uint8_t* row_bytes, const float* row_absmax, const float* qmap,
                             const bf16_t* x, int bytes_per_row, int bytes_per_block) {
    enum { WG = 128 };
    float part[WG];
    for (int l = 0; l < WG; ++l) {
        float partial = 0.0f;
        for (int off = l; off < bytes_per_row; off += WG) {
            const uint8_t b = row_bytes[off];
            const float am = row_absmax[off / bytes_per_block];
            const float t0 = bf16_to_f32(x[2 * off]) * qmap[(b >> 4) & 15];
            partial = partial + t0 * am;
            const float t1 = bf16_to_f32(x[2 * off + 1]) * qmap[b & 15];
            partial = partial + t1 * am;
        }
        part[l] = partial;
    }
    for (int w = WG / 2; w >= 1; w >>= 1)
        for (int i = 0; i < w; ++i) part[i] = part[i] + part[i + w];
    return part[0];
}

/* Decode GEMV y[n] = bf16(sum_k x[k] * (qmap[nib(n,k)] * absmax[n*K/bs + k/bs])).
 * Bnb4BitLinear.cpp:271-410 (packed_nf4_gemv_bf16). Branch choice at :289
 * (use_sg16 = K/2 >= 256). `residual` follows the documented semantics y += residual[n]
 * (:323); note the reference's SG16 branch drops it (:404-407) -- pass NULL to match the
 * reference's default build, which never passes one (AILA_FUSE_RESIDUAL_ADD off). */
void nf4o_gemv(const uint8_t* packed, const float* qmap, const float* absmax, const bf16_t* x,
               int64_t N, int64_t K, int blocksize, const bf16_t* residual, bf16_t* y) {
    const int bytes_per_row = (int)(K / 2);
    const int bytes_per_block = blocksize / 2;
    const int64_t blocks_per_row = K / blocksize;
    const int use_sg16 = bytes_per_row >= 256;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* rb = packed + n * bytes_per_row;
        const float* ra = absmax + n * blocks_per_row;
        float s = use_sg16 ? gemv_row_sg16(rb, ra, qmap, x, bytes_per_row, bytes_per_block)
                           : gemv_row_smallk(rb, ra, qmap, x, bytes_per_row, bytes_per_block);
        if (residual) s = s + bf16_to_f32(residual[n]);
        y[n] = f32_to_bf16(s);
    }
}

/* fp32 (unrounded) variant of the GEMV, for error analysis in tests. */
void nf4o_gemv_f32(const uint8_t* packed, const float* qmap, const float* absmax,
                   const bf16_t* x, int64_t N, int64_t K, int blocksize, float* y) {
    const int bytes_per_row = (int)(K / 2);
    const int bytes_per_block = blocksize / 2;
    const int64_t blocks_per_row = K / blocksize;
    const int use_sg16 = bytes_per_row >= 256;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const uint8_t* rb = packed + n * bytes_per_row;
        const float* ra = absmax + n * blocks_per_row;
        y[n] = use_sg16 ? gemv_row_sg16(rb, ra, qmap, x, bytes_per_row, bytes_per_block)
                        : gemv_row_smallk(rb, ra, qmap, x, bytes_per_row, bytes_per_block);
    }
}

/* Fused gate+up+SiLU decode GEMV. Bnb4BitLinear.cpp:142-246
 * (packed_nf4_gemv_gate_up_swiglu) and :759-797 (try_forward_decode_gate_up_swiglu): the
 * fused buffer holds gate rows [0,ff) then up rows [ff,2ff); both dot products use the SG16
 * lane order; out[i] = bf16( (g / (1 + exp(-g))) * u ) with g,u kept in fp32 (:241-242).
 * native::exp is approximated by expf here; the difference is far below bf16 resolution. */
void nf4o_gemv_gate_up_swiglu(const uint8_t* packed, const float* qmap, const float* absmax,
                              const bf16_t* x, int64_t ff, int64_t K, int blocksize,
                              bf16_t* out) {
    const int bytes_per_row = (int)(K / 2);
    const int bytes_per_block = blocksize / 2;
    const int64_t blocks_per_row = K / blocksize;
    const uint8_t* up_packed = packed + ff * bytes_per_row;
    const float* up_absmax = absmax + ff * blocks_per_row;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < ff; ++i) {
        const float g = gemv_row_sg16(packed + i * bytes_per_row, absmax + i * blocks_per_row,
                                      qmap, x, bytes_per_row, bytes_per_block);
        const float u = gemv_row_sg16(up_packed + i * bytes_per_row,
                                      up_absmax + i * blocks_per_row, qmap, x, bytes_per_row,
                                      bytes_per_block);
        const float silu = g / (1.0f + expf(-g));
        out[i] = f32_to_bf16(silu * u);
    }
}

/* Prefill route at blocksize 64. Bnb4BitLinear.cpp:839-948: the weight is first rounded
 * to bf16 (dequantize_weight, :746/:754), then a bf16 x bf16 matmul with fp32 accumulation
 * produces bf16 [M][N] (oneDNN matmul, :697-709). Here w_nk is the bf16 weight in row-major
 * [N][K] (nf4o_dequantize_nk) and the accumulation runs k = 0..K-1 in order. */
void nf4o_gemm_bf16w(const bf16_t* w_nk, const bf16_t* x_mk, int64_t M, int64_t N, int64_t K,
                     bf16_t* y_mn) {
    float* wf = (float*)malloc((size_t)N * (size_t)K * sizeof(float));
    if (!wf) return;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < N * K; ++i) wf[i] = bf16_to_f32(w_nk[i]);
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        float* xf = (float*)malloc((size_t)K * sizeof(float));
        for (int64_t k = 0; k < K; ++k) xf[k] = bf16_to_f32(x_mk[m * K + k]);
        for (int64_t n = 0; n < N; ++n) {
            const float* wr = wf + n * K;
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc = fmaf(xf[k], wr[k], acc);
            y_mn[m * N + n] = f32_to_bf16(acc);
        }
        free(xf);
    }
    free(wf);
}

/* Unfused SwiGLU on a bf16 [M][2*ff] gate_up buffer. src/ops/ElementwiseOps.cpp:247-294
 * (ops::fused_gate_up_swiglu): g and u are READ AS bf16 (so they carry the bf16 rounding of
 * the preceding linear), silu(g) = g / (1 + exp(-g)) in fp32, product rounded to bf16.
 * The reference applies it row by row (gate in [0,ff), up in [ff,2ff) of each row). */
void nf4o_swiglu_rows(const bf16_t* gate_up, int64_t M, int64_t ff, bf16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        const bf16_t* row = gate_up + m * 2 * ff;
        for (int64_t i = 0; i < ff; ++i) {
            const float g = bf16_to_f32(row[i]);
            const float u = bf16_to_f32(row[ff + i]);
            const float silu = g / (1.0f + expf(-g));
            out[m * ff + i] = f32_to_bf16(silu * u);
        }
    }
}

/* Balanced tree over n = 2^k partial sums, t[i] += t[i + w] for w = n/2 .. 1: what a work-group
 * reduction does on the hardware the reference targets (SYCL leaves the order open). */
static float tree_sum_n(float* t, int n) {
    for (int w = n / 2; w >= 1; w >>= 1)
        for (int i = 0; i < w; ++i) t[i] = t[i] + t[i + w];
    return t[0];
}

/* Residual add + RMSNorm in front of a linear. NormOps.cpp:141-275 (ops::fused_add_rms_norm) and,
 * with residual == NULL, NormOps.cpp:14-75 (ops::rms_norm). v = float(in) + float(residual) in fp32,
 * hidden_out = bf16(v), inv_rms = 1/sqrt(sum(v^2) / H + eps). The reference has three routes and this
 * follows each one's order of additions and its choice of what is normalised:
 *   one row, H == 1024 (:152-187): 128 work-items of 8 consecutive elements, the eight squares added
 *     left to right; normed = bf16(v * inv_rms * w) from the UNROUNDED v;
 *   one row, other H (:189-240): 256 work-items, item l takes the 8-element chunks l, l+256, ... and
 *     then the tail elements; normed = bf16(float(bf16(v)) * inv_rms * w): the second pass re-reads
 *     the residual stream it has just stored as bf16;
 *   several rows (:243-274), and rms_norm in both of its forms: 256 work-items, item l takes elements
 *     l, l+256, ...; normed from the unrounded v.
 * The work-group sum is a balanced tree over the items' partial sums. */
void nf4o_add_rms_norm(const bf16_t* in, const bf16_t* residual, const bf16_t* weight, float eps,
                       int64_t M, int64_t H, bf16_t* hidden_out, bf16_t* normed_out) {
    const int decode_1024 = residual && M == 1 && H == 1024;
    const int decode_chunks = residual && M == 1 && H != 1024;
    for (int64_t m = 0; m < M; ++m) {
        const bf16_t* x = in + m * H;
        const bf16_t* r = residual ? residual + m * H : NULL;
        float part[256];
        int lanes = 256;
#define NF4O_V(k) (bf16_to_f32(x[k]) + (r ? bf16_to_f32(r[k]) : 0.0f))
        if (decode_1024) {
            lanes = 128;
            for (int l = 0; l < 128; ++l) {
                float acc = NF4O_V(l * 8) * NF4O_V(l * 8);
                for (int k = 1; k < 8; ++k) acc = acc + NF4O_V(l * 8 + k) * NF4O_V(l * 8 + k);
                part[l] = acc;
            }
        } else if (decode_chunks) {
            const int64_t chunks = H / 8, tail = chunks * 8;
            for (int l = 0; l < 256; ++l) {
                float acc = 0.0f;
                for (int64_t c = l; c < chunks; c += 256)
                    for (int k = 0; k < 8; ++k) acc = acc + NF4O_V(c * 8 + k) * NF4O_V(c * 8 + k);
                for (int64_t k = tail + l; k < H; k += 256) acc = acc + NF4O_V(k) * NF4O_V(k);
                part[l] = acc;
            }
        } else {
            for (int l = 0; l < 256; ++l) {
                float acc = 0.0f;
                for (int64_t k = l; k < H; k += 256) acc = acc + NF4O_V(k) * NF4O_V(k);
                part[l] = acc;
            }
        }
        const float sum = tree_sum_n(part, lanes);
        const float inv_rms = 1.0f / sqrtf(sum / (float)H + eps);
        for (int64_t k = 0; k < H; ++k) {
            const float v = NF4O_V(k);
            const bf16_t stored = f32_to_bf16(v);
            if (hidden_out) hidden_out[m * H + k] = stored;
            const float vn = decode_chunks ? bf16_to_f32(stored) : v;
            normed_out[m * H + k] = f32_to_bf16(vn * inv_rms * bf16_to_f32(weight[k]));
        }
#undef NF4O_V
    }
}

/* Row concatenation of already-expanded linears. Bnb4BitLinear.cpp:604-615
 * (init_fused_rows_impl): packed bytes and fp32 absmax of each source are appended. The
 * caller concatenates; this helper only exists so tests exercise the same byte arithmetic. */
void nf4o_concat_rows(const uint8_t* const* packed, const float* const* absmax,
                      const int64_t* rows, int n_src, int64_t K, int blocksize,
                      uint8_t* packed_out, float* absmax_out) {
    int64_t po = 0, ao = 0;
    for (int s = 0; s < n_src; ++s) {
        const int64_t pb = rows[s] * K / 2;
        const int64_t ab = rows[s] * K / blocksize;
        memcpy(packed_out + po, packed[s], (size_t)pb);
        memcpy(absmax_out + ao, absmax[s], (size_t)ab * sizeof(float));
        po += pb;
        ao += ab;
    }
}

/* bf16 helpers exported for the Python side. */
void nf4o_f32_to_bf16(const float* in, int64_t n, bf16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
void nf4o_bf16_to_f32(const bf16_t* in, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]);
}
