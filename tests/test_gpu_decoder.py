"""The decoder harness: a captured decode step replays to the same tokens as eager steps, and the
side streams of the sibling projections change nothing (every kernel on the path is deterministic)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(batch, side_streams, graph, steps=5, prompt=24):
    from nsl_b200.decoder import BitNetConfig, BitNetDecoder
    cfg = BitNetConfig(layers=2, hidden=256, heads=4, head_dim=64, ffn=512, vocab=1000)
    dec = BitNetDecoder(cfg, batch, prompt + steps + 1, seed=3, side_streams=side_streams)
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    ids = torch.randint(0, cfg.vocab, (batch, prompt), device="cuda", generator=g)
    dec.prefill(ids)
    toks = [dec.tokens.clone()]
    for _ in range(steps):
        if graph:
            dec.decode(1)
        else:
            dec._step()
        toks.append(dec.tokens.clone())
    torch.cuda.synchronize()
    assert int(dec.pos.item()) == prompt + steps
    return torch.stack(toks).cpu(), dec.k_cache.float().cpu(), dec.v_cache.float().cpu()


@pytest.mark.parametrize("batch", [1, 3, 8, 20])
def test_graph_and_side_streams_reproduce_eager(batch):
    ref_t, ref_k, ref_v = _run(batch, side_streams=False, graph=False)
    for side, graph in [(True, False), (False, True), (True, True)]:
        t, k, v = _run(batch, side_streams=side, graph=graph)
        assert torch.equal(t, ref_t), (side, graph)
        assert torch.equal(k, ref_k) and torch.equal(v, ref_v), (side, graph)


def test_decode_cannot_run_past_the_cache():
    from nsl_b200.decoder import BitNetConfig, BitNetDecoder
    cfg = BitNetConfig(layers=1, hidden=256, heads=4, head_dim=64, ffn=512, vocab=100)
    dec = BitNetDecoder(cfg, 2, 16, seed=1, side_streams=False)
    dec.prefill(torch.zeros(2, 12, dtype=torch.long, device="cuda"))
    dec.decode(4)                                            # positions 12..15: the last rows of the cache
    with pytest.raises(ValueError):
        dec.decode(1)


def test_attention_reports_a_position_outside_the_cache():
    """The kernel does nothing for such a position, but says so: status 0x901, output untouched."""
    from nsl_b200 import ops
    B, H, D, ctx = 2, 4, 64, 16
    q = torch.randn(B, H * D, device="cuda").to(torch.bfloat16)
    kc = torch.zeros(B, H, ctx, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    cos = torch.ones(ctx, D // 2, device="cuda")
    sin = torch.zeros(ctx, D // 2, device="cuda")
    out = torch.full((B, H * D), 7.0, device="cuda", dtype=torch.bfloat16)
    assert ops.device_status() == 0
    ops.decode_attention(q, q, q, kc, vc, cos, sin, torch.tensor([ctx], device="cuda"), 0.125, out=out)
    assert ops.device_status() == 0x901
    assert ops.device_status() == 0                          # reading clears it
    assert bool((out == 7.0).all()) and float(kc.abs().sum()) == 0.0


def test_one_decode_layer_against_the_cpu_checker(oracle):
    """Batch 1, layer 0 of a small decoder: RMSNorm -> q/k/v BitLinear -> RoPE + attention over the cache ->
    o BitLinear + residual -> RMSNorm -> gate/up BitLinear -> SiLU*up -> down BitLinear + residual, restated
    with the CPU checker's BitLinear and float64 glue, with the harness's roundings (bf16 projection
    outputs and attention output).  A quantised activation can land on the other side of a rounding
    boundary when its bf16 input differs in the last bit, so the comparison is to 3 % of the row rms."""
    import numpy as np
    from gpu_util import bf16_round
    from nsl_b200.decoder import BitNetConfig, BitNetDecoder
    cfg = BitNetConfig(layers=1, hidden=256, heads=4, head_dim=64, ffn=512, vocab=500)
    prompt = 20
    dec = BitNetDecoder(cfg, 1, prompt + 4, seed=5, side_streams=False)
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    dec.prefill(torch.randint(0, cfg.vocab, (1, prompt), device="cuda", generator=g))
    x = dec.embed[dec.tokens].float()
    k_before, v_before = dec.k_cache[0, 0].float().cpu().numpy().astype(np.float64), dec.v_cache[0, 0].float().cpu().numpy().astype(np.float64)
    got = dec.decode_layer(0, x.clone()).cpu().numpy()
    torch.cuda.synchronize()
    L, pos, D, H = dec.layers[0], prompt, cfg.head_dim, cfg.heads

    def lin(name, h):
        w = L[name]
        return oracle.bitlinear_forward_packed(np.ascontiguousarray(h, np.float32), w.packed.cpu().numpy(), w.N, w.weight_scale)[3]

    xn = x.cpu().numpy()
    h1 = oracle.rmsnorm_f32(xn, L["n1"].cpu().numpy(), cfg.eps)
    q, k, v = (bf16_round(lin(n, h1)).astype(np.float64).reshape(H, D) for n in ("q", "k", "v"))
    cos, sin = dec.cos[pos].cpu().numpy().astype(np.float64), dec.sin[pos].cpu().numpy().astype(np.float64)

    def rope(t):
        a, b = t[:, :D // 2], t[:, D // 2:]
        return np.concatenate([a * cos - b * sin, b * cos + a * sin], 1)

    qr, kr = bf16_round(rope(q)).astype(np.float64), bf16_round(rope(k)).astype(np.float64)
    att = np.zeros((H, D))
    for hd in range(H):
        keys = np.concatenate([k_before[hd, :pos], kr[hd:hd + 1]], 0)
        vals = np.concatenate([v_before[hd, :pos], v[hd:hd + 1]], 0)
        s = keys @ qr[hd] * dec.sm_scale
        pr = np.exp(s - s.max())
        att[hd] = (pr / pr.sum()) @ vals
    a = bf16_round(att.reshape(1, H * D))
    x1 = (lin("o", a) + xn).astype(np.float32)
    h2 = oracle.rmsnorm_f32(x1, L["n2"].cpu().numpy(), cfg.eps)
    gt, up = bf16_round(lin("gate", h2)).astype(np.float32), bf16_round(lin("up", h2)).astype(np.float32)
    hh = (gt / (1.0 + np.exp(-gt)) * up).astype(np.float32)
    want = (lin("down", hh) + x1).astype(np.float32)
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    assert np.abs(got - want).max() <= 3e-2 * rms, (np.abs(got - want).max(), rms)
