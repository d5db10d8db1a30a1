"""Test helpers: host-side (numpy) packers / unpackers for the tile blob layouts of the sm_100a kernels.

The kernels keep quantised K/V in 128-byte core-matrix order (see ``csrc/common.cuh``); the reference
keeps them in mma.sync fragment order (``triattention/kernels/cuda/common_device.cuh:101-130,142-171``).
Both hold the same codes; these helpers map a blob to the logical ``[tile][key][feature]`` /
``[tile][key][channel]`` array so that codes can be compared one to one.  Inspection and test use
only: nothing on the attention path calls them.
"""
from __future__ import annotations

import numpy as np

D, BN = 128, 64
_S, _B = np.meshgrid(np.arange(4), np.arange(4), indexing="ij")
KPERM = (2 * _S + np.where(_B < 2, _B, _B + 6)).reshape(16)  # run position 4s+b -> key inside the 16-key group


def _sign4(n):
    n = np.asarray(n).astype(np.int8)
    return np.where(n > 7, n - 16, n).astype(np.int8)


def _k8_index():
    p = np.arange(8192)
    return (p // 1024) * 8 + (p // 16) % 8, ((p // 128) % 8) * 16 + p % 16          # key, feature


def _k4_index():
    p = np.arange(4096)
    key, sub, s, j = (p // 512) * 8 + (p // 64) % 8, (p // 16) % 4, (p // 4) % 4, p % 4
    return key, 32 * sub + 8 * s + j, 32 * sub + 8 * s + 4 + j                       # key, low feature, high feature


def _v8_index():
    p = np.arange(8192)
    return 16 * ((p // 128) % 4) + KPERM[p % 16], (p // 512) * 8 + (p // 16) % 8    # key, channel


def _v4_index():
    p = np.arange(4096)
    kc, ch = (p // 128) % 2, (p // 256) * 8 + (p // 16) % 8
    return 32 * kc + KPERM[p % 16], 32 * kc + 16 + KPERM[p % 16], ch                # low key, high key, channel


def _v16_index():
    p = np.arange(8192)
    return ((p // 64) % 8) * 8 + p % 8, (p // 512) * 8 + (p // 8) % 8               # key, channel


def unpack_k8(blob) -> np.ndarray:
    """uint8 [...,8192] -> int8 [...,64 keys,128 features].  Also valid for K4X blobs."""
    blob = np.asarray(blob)
    key, feat = _k8_index()
    out = np.empty(blob.shape[:-1] + (BN, D), np.int8)
    out[..., key, feat] = blob.view(np.int8)
    return out


def pack_k8(codes) -> np.ndarray:
    key, feat = _k8_index()
    return np.ascontiguousarray(np.asarray(codes, np.int8)[..., key, feat]).view(np.uint8)


def unpack_k4(blob) -> np.ndarray:
    """uint8 [...,4096] -> int8 [...,64,128] in -8..7."""
    blob = np.asarray(blob, np.uint8)
    key, flo, fhi = _k4_index()
    out = np.empty(blob.shape[:-1] + (BN, D), np.int8)
    out[..., key, flo] = _sign4(blob & 0xF)
    out[..., key, fhi] = _sign4(blob >> 4)
    return out


def unpack_v8(blob) -> np.ndarray:
    """uint8 [...,8192] -> int8 [...,64 keys,128 channels]."""
    blob = np.asarray(blob)
    key, ch = _v8_index()
    out = np.empty(blob.shape[:-1] + (BN, D), np.int8)
    out[..., key, ch] = blob.view(np.int8)
    return out


def pack_v8(codes) -> np.ndarray:
    key, ch = _v8_index()
    return np.ascontiguousarray(np.asarray(codes, np.int8)[..., key, ch]).view(np.uint8)


def unpack_v4(blob) -> np.ndarray:
    """uint8 [...,4096] -> int8 [...,64,128] in -8..7."""
    blob = np.asarray(blob, np.uint8)
    klo, khi, ch = _v4_index()
    out = np.empty(blob.shape[:-1] + (BN, D), np.int8)
    out[..., klo, ch] = _sign4(blob & 0xF)
    out[..., khi, ch] = _sign4(blob >> 4)
    return out


def unpack_v16(blob) -> np.ndarray:
    """uint8 [...,16384] -> float16 [...,64,128]."""
    half = np.ascontiguousarray(blob).view(np.float16)
    key, ch = _v16_index()
    out = np.empty(half.shape[:-1] + (BN, D), np.float16)
    out[..., key, ch] = half
    return out


def pack_v16(values) -> np.ndarray:
    key, ch = _v16_index()
    return np.ascontiguousarray(np.asarray(values, np.float16)[..., key, ch]).view(np.uint8)


def swizzle128(rows) -> np.ndarray:
    """uint8 [R,128] (R % 8 == 0) -> the 128-byte-swizzled shared-memory image a TMA tensor copy
    produces: the 16-byte chunk c of row r sits at chunk position c ^ (r % 8)."""
    r = np.asarray(rows, np.uint8).reshape(-1, 8, 16)
    out = np.empty_like(r)
    idx = np.arange(r.shape[0])
    for c in range(8):
        out[idx, c ^ (idx % 8)] = r[idx, c]
    return out.reshape(-1, 128)
