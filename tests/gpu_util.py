"""Shared helpers of the GPU parity tests (inputs, layouts, comparison)."""
import numpy as np
import torch


def perm_index(K):
    """q_perm[..., p] = q_plain[..., perm_index(K)[p]]: position 4i+j of every 16 holds k = 4j+i."""
    p = np.arange(K)
    g, r = p // 16 * 16, p % 16
    i, j = r // 4, r % 4
    return g + 4 * j + i


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    return t.cpu().numpy()


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a, np.float32), np.ascontiguousarray(b, np.float32)
    return np.array_equal(a.view(np.uint32), b.view(np.uint32))


def bf16_round(a):
    """float32 -> nearest bf16 (ties to even) -> float32, in numpy."""
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def make_w4_case(rng, N, K, gs, scale_bf16=True):
    """The W4A16 workload's distributions: codes U{0..15}, scale |N(0,0.02)|/7, zp U{0..15}."""
    G = K // gs
    q = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    codes = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    scale = (np.abs(rng.standard_normal((N, G)) * 0.02) / 7.0).astype(np.float32)
    if scale_bf16:
        scale = bf16_round(scale)
    zp = rng.integers(0, 16, size=(N, G), dtype=np.uint8)
    return q, codes, scale, zp
