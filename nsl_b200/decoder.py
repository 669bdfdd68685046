"""Decoder harness for the model-shaped workloads of the benchmark (BitNet b1.58-3B shape).

At prefill, the attention over the prompt and the bf16 lm_head are plain PyTorch (library kernels), on
purpose: those pieces are outside the quantized-linear path this library replaces (NSL has them in
stdlib/nsl/nn/gqa.nsl and stdlib/nsl/inference/generate.nsl); the embedding rows, the rotary embedding with
the cache writes (nslq_rope_kv_prefill), the norms and the greedy choice are this library's launches.  Every projection of every layer (q, k, v, o, gate, up, down) runs
through nsl_b200.ops.BitLinear, i.e. the C ABI.  A decode step is library launches throughout, the
lm_head's bf16 GEMM aside: the embedding rows (nslq_embed_gather), the RMSNorms (inside the projections'
launches for one token, nslq_rmsnorm_act_quant_i8 above), the attention of the new token (RoPE, cache
append, softmax(qK)V: nslq_decode_attention), SiLU(gate)*up (inside the down projection's launch for
one token), the final norm (nslq_rmsnorm_rows) and the greedy choice (nslq_argmax_rows, which also
advances the position).  Weights are random ternary (no
checkpoint is available offline), so the numbers are throughput numbers, not quality numbers.

The residual stream is kept in fp32: the norms then need no casts, and the residual additions ride
in the BitLinear epilogue (`residual=`, added in fp32 after `weight_scale`, as NSL's finalize phase
orders it, crates/nsl-codegen/src/bitnet/phases/finalize.rs:55-80) instead of being separate kernels.

One decode step is captured in a single CUDA graph: the position and the current tokens live in
device tensors that the graph itself advances, so 256 steps are 256 replays.
"""
import math

import torch
import torch.nn.functional as F

from . import ops


class BitNetConfig:
    def __init__(self, layers=26, hidden=3200, heads=32, head_dim=100, ffn=8640, vocab=32002, rope_theta=10000.0,
                 eps=1e-5):
        self.layers, self.hidden, self.heads, self.head_dim = layers, hidden, heads, head_dim
        self.ffn, self.vocab, self.rope_theta, self.eps = ffn, vocab, rope_theta, eps

    def ternary_bytes_per_layer(self):
        return (4 * self.hidden * self.hidden + 3 * self.hidden * self.ffn) // 4


def _ternary(n, k, gen):
    c = torch.randint(0, 3, (n, k // 4, 4), device="cuda", dtype=torch.uint8, generator=gen)
    return ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).contiguous()


def _rope(x, cos, sin):
    """x [B, H, T, D]; cos/sin [T, D/2] (rotate-half convention).  The expression nslq_rope_kv_prefill is tested against."""
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class BitNetDecoder:
    """Random-init decoder of the given shape; act dtype bf16, KV cache bf16."""

    def __init__(self, cfg, batch, max_ctx, seed=0, side_streams=True):
        max_ctx = (max_ctx + 3) & ~3                                    # the attention kernel wants a multiple of 4
        self.cfg, self.B, self.max_ctx = cfg, batch, max_ctx
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed)
        h, f, hd = cfg.hidden, cfg.ffn, cfg.heads * cfg.head_dim
        dt = torch.bfloat16
        self.embed = (torch.randn(cfg.vocab, h, device="cuda", generator=gen) * 0.02).to(dt)
        self.lm_head = (torch.randn(cfg.vocab, h, device="cuda", generator=gen) * 0.02).to(dt)
        self.final_norm = torch.ones(h, device="cuda")
        self.layers = []
        for _ in range(cfg.layers):
            L = {"n1": torch.ones(h, device="cuda"), "n2": torch.ones(h, device="cuda")}
            for name, (n, k) in {"q": (hd, h), "k": (hd, h), "v": (hd, h), "o": (h, hd), "gate": (f, h), "up": (f, h),
                                 "down": (h, f)}.items():
                L[name] = ops.BitLinear(_ternary(n, k, gen), 1.0 / math.sqrt(k))
            self.layers.append(L)
        half = cfg.head_dim // 2
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(half, device="cuda").float() / half))
        ang = torch.arange(max_ctx, device="cuda").float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.k_cache = torch.zeros(cfg.layers, batch, cfg.heads, max_ctx, cfg.head_dim, device="cuda", dtype=dt)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.pos = torch.zeros(1, device="cuda", dtype=torch.long)       # next position to write
        self.tokens = torch.zeros(batch, device="cuda", dtype=torch.long)
        self.key_index = torch.arange(max_ctx, device="cuda")
        self.sm_scale = 1.0 / math.sqrt(cfg.head_dim)
        self.graph = None
        self.host_pos = 0
        # Sibling projections (q/k/v, gate/up) of a decode step run on side streams: at a few dozen rows
        # one projection occupies 25 to 68 of the 148 SMs, so three of them fit side by side.
        self.side = [torch.cuda.Stream(), torch.cuda.Stream()] if side_streams else []
        self.fork = False                                                # set while a decode step is issued

    def _siblings(self, fns):
        """Run independent launches; in a decode step the second and later ones go to side streams."""
        if not self.fork or len(fns) == 1 or not self.side:
            return [f() for f in fns]
        cur = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(cur)
        outs, joins = [None] * len(fns), []
        for i, (f, st) in enumerate(zip(fns[1:], self.side), start=1):
            st.wait_event(start)
            with torch.cuda.stream(st):
                outs[i] = f()
            done = torch.cuda.Event()
            done.record(st)
            joins.append(done)
        outs[0] = fns[0]()
        for done in joins:
            cur.wait_event(done)
        return outs

    # ------------------------------------------------------------------ linears through the C ABI
    def _lin(self, layer, x2d, residual):
        """fp32 output with the fp32 residual added in the epilogue."""
        return layer.forward(x2d, out_dtype=torch.float32, residual=residual)

    def _swiglu_down(self, layer, g, u, residual):
        """down(silu(gate) * up) + residual: one launch forms and quantises the product, one multiplies."""
        if g.shape[0] == 1:               # a decode step of one token: the product is formed inside the projection's launch
            return layer.forward_swiglu(g, u, out_dtype=torch.float32, residual=residual)
        qa = ops.swiglu_act_quant_i8(g, u, plain=False, perm=True)
        return layer.forward_quantized(qa, out_dtype=torch.float32, residual=residual)

    def _norm_lin_shared(self, layers, x2d, norm_w):
        """RMSNorm, then several projections of the normalised rows.  More than one row: one
        launch normalises and quantises (the normalised rows never reach memory) and the
        projections share the result; one row: norm and all projections are ONE launch whose CTAs each
        normalise and quantise for themselves (nslq_bitlinear_forward_multi), so neither the norm nor the
        siblings' side streams exist."""
        M = x2d.shape[0]
        if M <= 8:                        # one row: one launch in all; up to eight: the quantiser and ONE launch for all projections
            return ops.BitLinear.forward_multi(layers, x2d, norm_w, self.cfg.eps, out_dtype=torch.bfloat16)
        qa = ops.rmsnorm_act_quant_i8(x2d, norm_w, self.cfg.eps, plain=False, perm=True)
        return self._siblings([lambda l=l: l.forward_quantized(qa, out_dtype=torch.bfloat16) for l in layers])

    # ------------------------------------------------------------------ prefill
    def prefill(self, ids):
        """ids [B, T]; fills the KV cache, leaves pos = T and tokens = greedy next token."""
        cfg, B, T = self.cfg, ids.shape[0], ids.shape[1]
        x = ops.embed_gather(self.embed, ids.reshape(-1))                 # [B*T, h] residual stream, fp32
        for li, L in enumerate(self.layers):
            q, k, v = self._norm_lin_shared([L["q"], L["k"], L["v"]], x, L["n1"])
            # rotary embedding and cache writes in one launch; the attention reads keys and values from the cache
            ops.rope_kv_prefill(q, k, v, self.k_cache[li], self.v_cache[li], self.cos, self.sin, T)
            a = F.scaled_dot_product_attention(q.view(B, T, cfg.heads, cfg.head_dim).transpose(1, 2),
                                               self.k_cache[li, :, :, :T], self.v_cache[li, :, :, :T], is_causal=True)
            a = a.transpose(1, 2).reshape(B * T, cfg.heads * cfg.head_dim)
            x = self._lin(L["o"], a, x)
            g, u = self._norm_lin_shared([L["gate"], L["up"]], x, L["n2"])
            x = self._swiglu_down(L["down"], g, u, x)
        last = ops.rmsnorm_rows(x.view(B, T, cfg.hidden)[:, -1].contiguous(), self.final_norm, cfg.eps, out_dtype=torch.bfloat16)
        ops.argmax_rows(last @ self.lm_head.t(), out=self.tokens)
        self.pos.fill_(T)
        self.host_pos = T

    # ------------------------------------------------------------------ one decode step (graph-capturable)
    def _step(self):
        cfg, B = self.cfg, self.B
        self.fork = bool(self.side)
        x = ops.embed_gather(self.embed, self.tokens)                     # [B, h] residual stream, fp32
        for li in range(len(self.layers)):
            x = self.decode_layer(li, x)
        logits = ops.rmsnorm_rows(x, self.final_norm, cfg.eps, out_dtype=torch.bfloat16) @ self.lm_head.t()
        ops.argmax_rows(logits, out=self.tokens, counter=self.pos)       # next tokens, and the position moves on
        self.fork = False

    def decode_layer(self, li, x):
        """One layer of a decode step on the fp32 residual stream x [B, hidden]; appends to layer li's cache
        at the current position."""
        cfg, B, L = self.cfg, self.B, self.layers[li]
        q, k, v = self._norm_lin_shared([L["q"], L["k"], L["v"]], x, L["n1"])
        # RoPE, cache append and single-query attention: one launch of the library
        a = ops.decode_attention(q, k, v, self.k_cache[li], self.v_cache[li], self.cos, self.sin, self.pos,
                                 self.sm_scale)
        x = self._lin(L["o"], a.reshape(B, cfg.heads * cfg.head_dim), x)
        g, u = self._norm_lin_shared([L["gate"], L["up"]], x, L["n2"])
        return self._swiglu_down(L["down"], g, u, x)

    def capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        keep_pos, keep_tok = self.pos.clone(), self.tokens.clone()
        with torch.cuda.stream(s):
            self._step()                      # warm-up outside the graph (allocations, lazy init)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.pos.copy_(keep_pos)
        self.tokens.copy_(keep_tok)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step()
        self.pos.copy_(keep_pos)
        self.tokens.copy_(keep_tok)

    def decode(self, steps):
        # the position lives on the device (the graph advances it); the host keeps its own count so that a
        # loop cannot run past the end of the cache, where the attention kernel would do nothing
        if self.host_pos + steps > self.max_ctx:
            raise ValueError("decode(%d) from position %d would pass the end of the KV cache (%d rows)"
                             % (steps, self.host_pos, self.max_ctx))
        if self.graph is None:
            self.capture()
        for _ in range(steps):
            self.graph.replay()
        self.host_pos += steps

    def step_bytes(self, ctx):
        """Algorithmic HBM bytes of one decode step at context length ctx."""
        cfg = self.cfg
        w = cfg.layers * cfg.ternary_bytes_per_layer() + cfg.vocab * cfg.hidden * 2
        kv = self.B * cfg.layers * 2 * ctx * cfg.heads * cfg.head_dim * 2
        return w + kv
