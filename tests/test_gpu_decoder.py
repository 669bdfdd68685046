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
