"""The decode-step launches that are not a quantized linear: embedding rows, final RMSNorm, greedy argmax.
Embedding and argmax are exact; the norm follows the CPU checker's nsl_tensor_rmsnorm (bit for bit when
the sum of squares does not depend on the summation order, within one ulp otherwise)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, dev, host  # noqa: E402
from nsl_b200 import NslqError, ops  # noqa: E402
from oracle import oracle as o  # noqa: E402


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_embed_gather(dt):
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    table = torch.randn(1000, 328, device="cuda", generator=g).to(dt)
    tok = torch.tensor([0, 999, 17, 17, 500], device="cuda")
    out = ops.embed_gather(table, tok)
    assert out.dtype == torch.float32 and torch.equal(out, table[tok].float())
    assert ops.device_status() == 0
    bad = torch.tensor([3, 1000, -1], device="cuda")
    out = ops.embed_gather(table, bad)
    assert torch.equal(out[0], table[3].float()) and float(out[1:].abs().sum()) == 0.0
    assert ops.device_status() == 0xA01
    assert ops.device_status() == 0


def test_rmsnorm_rows():
    rng = np.random.default_rng(4)
    M, K = 5, 3200
    w = rng.uniform(0.5, 1.5, size=K).astype(np.float32)
    x = (np.exp2(rng.integers(-8, 9, size=(M, K))) * rng.choice([-1.0, 1.0], size=(M, K))).astype(np.float32)
    want = o.rmsnorm_f32(x, w, 1e-5)
    got = host(ops.rmsnorm_rows(dev(x), dev(w), 1e-5))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    gb = host(ops.rmsnorm_rows(dev(x), dev(w), 1e-5, out_dtype=torch.bfloat16).float())
    assert np.array_equal(gb, bf16_round(want))
    x = (rng.standard_normal((M, 1001)) * 7).astype(np.float32)          # any width
    w = rng.uniform(0.5, 1.5, size=1001).astype(np.float32)
    want = o.rmsnorm_f32(x, w, 1e-5)
    got = host(ops.rmsnorm_rows(dev(x), dev(w), 1e-5))
    assert np.all(np.abs(got - want) <= 2e-7 * np.abs(want) + 1e-30)
    assert (got.view(np.uint32) == want.view(np.uint32)).mean() >= 0.999


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_argmax_rows(dt):
    rng = np.random.default_rng(9)
    M, V = 7, 32002
    x = rng.standard_normal((M, V)).astype(np.float32)
    x[1, 40] = x[1, 31999] = 9.0                       # tie: the lowest index wins
    x[2, 7] = np.nan                                   # a NaN never wins
    x[3, :] = -np.inf                                  # nothing above -inf: index 0
    x[4, :] = np.nan
    x[5, V - 1] = 50.0                                 # the last element
    xd = dev(x).to(dt)
    ref = xd.float().cpu().numpy()
    want = np.zeros(M, np.int64)
    for r in range(M):                                 # the reference's loop
        best, bi = -np.inf, 0
        for i in np.flatnonzero(ref[r] >= ref[r][~np.isnan(ref[r])].max() if (~np.isnan(ref[r])).any() else []):
            if ref[r, i] > best:
                best, bi = ref[r, i], i
        want[r] = bi
    pos = torch.full((1,), 41, device="cuda", dtype=torch.int64)
    got = ops.argmax_rows(xd, counter=pos)
    assert np.array_equal(host(got), want), (host(got), want)
    assert int(pos) == 42
    assert int(want[1]) == 40 and int(want[3]) == 0 and int(want[4]) == 0 and int(want[5]) == V - 1
    # a view with a row stride
    wide = torch.zeros(3, 600, device="cuda")
    wide[:, 512:] = 100.0                              # outside the view
    wide[0, 100] = wide[1, 511] = wide[2, 0] = 1.0
    assert host(ops.argmax_rows(wide[:, :512])).tolist() == [100, 511, 0]


@pytest.mark.parametrize("D", [100, 128, 6])
@pytest.mark.parametrize("pos0", [0, 5])
def test_rope_kv_prefill_equals_the_expression_on_fp32_tensors(D, pos0):
    """nslq_rope_kv_prefill: rotated queries, rotated keys in the cache and copied values have the bits of
    x * cos + rotate_half(x) * sin evaluated operation by operation on fp32 tensors and rounded to bf16 once;
    rows of the cache outside [pos0, pos0 + T) stay untouched; q, k, v may be column blocks of one fused tensor."""
    from nsl_b200.decoder import _rope
    B, T, H, cap = 3, 37, 4, 64
    g = torch.Generator(device="cuda")
    g.manual_seed(D + pos0)
    fused = torch.randn(B * T, 3 * H * D, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v = fused[:, :H * D], fused[:, H * D:2 * H * D], fused[:, 2 * H * D:]
    inv = 1.0 / (10000.0 ** (torch.arange(D // 2, device="cuda").float() / (D // 2)))
    ang = torch.arange(cap, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    kc = torch.full((B, H, cap, D), 7.0, device="cuda", dtype=torch.bfloat16)
    vc = torch.full((B, H, cap, D), 7.0, device="cuda", dtype=torch.bfloat16)
    want_q = _rope(q.reshape(B, T, H, D).transpose(1, 2), cos[pos0:pos0 + T], sin[pos0:pos0 + T])
    want_k = _rope(k.reshape(B, T, H, D).transpose(1, 2), cos[pos0:pos0 + T], sin[pos0:pos0 + T])
    want_v = v.reshape(B, T, H, D).transpose(1, 2).clone()
    ops.rope_kv_prefill(q, k, v, kc, vc, cos, sin, T, pos0)
    torch.cuda.synchronize()
    assert torch.equal(q.reshape(B, T, H, D).transpose(1, 2), want_q)
    assert torch.equal(kc[:, :, pos0:pos0 + T], want_k)
    assert torch.equal(vc[:, :, pos0:pos0 + T], want_v)
    assert bool((kc[:, :, :pos0] == 7).all()) and bool((kc[:, :, pos0 + T:] == 7).all())
    assert bool((vc[:, :, :pos0] == 7).all()) and bool((vc[:, :, pos0 + T:] == 7).all())
    assert ops.device_status() == 0


def test_rope_kv_prefill_with_grouped_heads_and_a_single_token():
    """Fewer key/value heads than query heads, one token per sequence appended at a later position."""
    from nsl_b200.decoder import _rope
    B, T, H, Hkv, D, cap, pos0 = 2, 1, 8, 2, 64, 16, 9
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    q = torch.randn(B * T, H * D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B * T, Hkv * D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B * T, Hkv * D, device="cuda", generator=g).to(torch.bfloat16)
    inv = 1.0 / (10000.0 ** (torch.arange(D // 2, device="cuda").float() / (D // 2)))
    ang = torch.arange(cap, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    kc = torch.zeros(B, Hkv, cap, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    want_q = _rope(q.reshape(B, T, H, D).transpose(1, 2), cos[pos0:pos0 + T], sin[pos0:pos0 + T])
    want_k = _rope(k.reshape(B, T, Hkv, D).transpose(1, 2), cos[pos0:pos0 + T], sin[pos0:pos0 + T])
    ops.rope_kv_prefill(q, k, v, kc, vc, cos, sin, T, pos0)
    torch.cuda.synchronize()
    assert torch.equal(q.reshape(B, T, H, D).transpose(1, 2), want_q)
    assert torch.equal(kc[:, :, pos0:pos0 + T], want_k)
    assert torch.equal(vc[:, :, pos0:pos0 + T], v.reshape(B, T, Hkv, D).transpose(1, 2))
    assert int((kc != 0).any(-1).sum()) <= B * Hkv * T and int((vc != 0).any(-1).sum()) <= B * Hkv * T
    with pytest.raises(NslqError):
        ops.rope_kv_prefill(q, k, v, kc, vc, cos, sin, T, cap)                      # past the end of the cache
