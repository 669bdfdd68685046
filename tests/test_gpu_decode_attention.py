"""RoPE + KV-cache append + single-query attention in one launch, against the same arithmetic in
numpy float64 (rotate-half RoPE as in NSL's stdlib/nsl/nn/rope.nsl, causal attention of the newest
token as in stdlib/nsl/nn/gqa.nsl).  Floating point: inputs and outputs are bf16, the kernel
accumulates in fp32; bar: |err| <= 1e-2 * (|want| + rms(want)) for the output, the appended key row
within one bf16 ulp of the float64 rotation, the value row bit-equal."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


def rope64(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


@pytest.mark.parametrize("B,H,Hkv,D,max_ctx,pos", [(1, 32, 32, 100, 776, 0), (2, 32, 32, 100, 776, 517), (3, 8, 2, 128, 64, 63),
                                                   (4, 4, 4, 64, 40, 7), (64, 32, 32, 100, 776, 640),
                                                   # clusters of 8 / 4 / 2 CTAs per (b, h): empty slices, ragged last slice, slice boundaries
                                                   (1, 32, 32, 100, 776, 640), (1, 8, 8, 128, 260, 15), (1, 8, 8, 128, 260, 16), (1, 8, 8, 128, 260, 127),
                                                   (1, 8, 8, 128, 260, 128), (2, 32, 8, 64, 520, 300), (4, 32, 32, 100, 776, 333),
                                                   (8, 32, 32, 100, 776, 641)])
def test_against_float64(ops, B, H, Hkv, D, max_ctx, pos):
    rng = np.random.default_rng(B * 7 + pos)
    half = D // 2
    inv = 1.0 / (10000.0 ** (np.arange(half) / half))
    ang = np.arange(max_ctx)[:, None] * inv[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    q = bf16_round(rng.standard_normal((B, H, D)).astype(np.float32))
    kn = bf16_round(rng.standard_normal((B, Hkv, D)).astype(np.float32))
    vn = bf16_round(rng.standard_normal((B, Hkv, D)).astype(np.float32))
    kc = bf16_round(rng.standard_normal((B, Hkv, max_ctx, D)).astype(np.float32))
    vc = bf16_round(rng.standard_normal((B, Hkv, max_ctx, D)).astype(np.float32))
    t = lambda a: torch.from_numpy(a).cuda().to(torch.bfloat16).contiguous()
    kct, vct = t(kc), t(vc)
    pos_t = torch.tensor([pos], dtype=torch.int64, device="cuda")
    scale = 1.0 / np.sqrt(D)
    out = ops.decode_attention(t(q), t(kn), t(vn), kct, vct, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(),
                               pos_t, scale)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy().reshape(B, H, D)
    # float64 reference (the query and the appended key rounded to bf16, as the kernel stores them)
    c, s = cos[pos].astype(np.float64), sin[pos].astype(np.float64)
    k_rot = rope64(kn.astype(np.float64), c, s)
    q_rot = bf16_round(rope64(q.astype(np.float64), c, s).astype(np.float32)).astype(np.float64)
    K = kc.astype(np.float64).copy(); V = vc.astype(np.float64).copy()
    K[:, :, pos] = bf16_round(k_rot.astype(np.float32)); V[:, :, pos] = vn
    rep = H // Hkv
    want = np.empty((B, H, D))
    for b in range(B):
        for h in range(H):
            sc = K[b, h // rep, :pos + 1] @ q_rot[b, h] * scale
            pr = np.exp(sc - sc.max()); pr /= pr.sum()
            want[b, h] = pr @ V[b, h // rep, :pos + 1]
    rms = np.sqrt((want ** 2).mean(axis=-1, keepdims=True))
    assert np.all(np.abs(got - want) <= 1e-2 * (np.abs(want) + rms))
    # cache rows
    k_row = kct.float().cpu().numpy()[:, :, pos]
    assert np.all(np.abs(k_row - k_rot) <= 2.0 ** -7 * np.abs(k_rot) + 1e-6)
    assert np.array_equal(vct.float().cpu().numpy()[:, :, pos], vn)
    # rows other than pos untouched
    if pos > 0:
        assert np.array_equal(kct.float().cpu().numpy()[:, :, :pos], kc[:, :, :pos])


def test_column_slices_of_a_fused_projection(ops):
    """q, k, v handed over as column slices of one [B, 3*H*D] tensor give the same bytes as packed inputs."""
    B, H, D, max_ctx, pos = 3, 8, 100, 64, 20
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    qkv = torch.randn(B, 3 * H * D, device="cuda", generator=g).to(torch.bfloat16)
    kc = torch.randn(B, H, max_ctx, D, device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn(B, H, max_ctx, D, device="cuda", generator=g).to(torch.bfloat16)
    half = D // 2
    ang = torch.arange(max_ctx, device="cuda").float()[:, None] / (10000.0 ** (torch.arange(half, device="cuda").float() / half))[None, :]
    cos, sin = ang.cos(), ang.sin()
    pos_t = torch.tensor([pos], dtype=torch.int64, device="cuda")
    hd = H * D
    kc1, vc1, kc2, vc2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
    a = ops.decode_attention(qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], kc1, vc1, cos, sin, pos_t, 0.1)
    b = ops.decode_attention(qkv[:, :hd].contiguous(), qkv[:, hd:2 * hd].contiguous(), qkv[:, 2 * hd:].contiguous(), kc2, vc2,
                             cos, sin, pos_t, 0.1)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
