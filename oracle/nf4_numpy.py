"""Second, independent restatement of the NF4 path in numpy (TEST INFRASTRUCTURE ONLY).

Written without looking at nf4_oracle.c's loops: vectorised, no lane order. It pins the C
oracle's layout conventions (nibble order, absmax index, transposed output) and gives an
order-free float64 dot product to bound the C oracle's accumulation-order effects.
Reference lines: Bnb4BitLinear.cpp:472-488 (absmax), :735-756 (dequant), :374-389 (GEMV).
"""
import numpy as np


def bf16_round(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit pattern (uint16), round-to-nearest-even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def expand_absmax(codes, nested_map, nested_absmax, nested_blocksize, nested_offset):
    codes = np.asarray(codes, np.uint8).reshape(-1)
    idx = np.arange(codes.size) // nested_blocksize
    prod = (np.asarray(nested_map, np.float32)[codes] *
            np.asarray(nested_absmax, np.float32)[idx]).astype(np.float32)
    return (prod + np.float32(nested_offset)).astype(np.float32)


def codes_nk(packed, N, K):
    """4-bit codes as [N, K]: even k from the high nibble, odd k from the low nibble."""
    p = np.asarray(packed, np.uint8).reshape(N, K // 2)
    out = np.empty((N, K), np.uint8)
    out[:, 0::2] = p >> 4
    out[:, 1::2] = p & 15
    return out


def weights_f32(packed, qmap, absmax, N, K, blocksize):
    """fp32 weights q*am as the decode GEMV uses them, [N, K]."""
    c = codes_nk(packed, N, K)
    am = np.asarray(absmax, np.float32).reshape(N, K // blocksize)
    return (np.asarray(qmap, np.float32)[c] * np.repeat(am, blocksize, axis=1)).astype(np.float32)


def dequantize_kn(packed, qmap, absmax, N, K, blocksize):
    return bf16_round(weights_f32(packed, qmap, absmax, N, K, blocksize)).T.copy()


def gemv_f64(packed, qmap, absmax, x_bf16, N, K, blocksize):
    w = weights_f32(packed, qmap, absmax, N, K, blocksize).astype(np.float64)
    return w @ bf16_to_f32(x_bf16).astype(np.float64)
