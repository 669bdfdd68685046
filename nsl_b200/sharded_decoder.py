"""Column-sharded decode layers of a 7B-class ternary decoder (hidden 4096, 32 heads x 128,
FFN 11008): the multi-GPU workload of the benchmark.

Layout per layer on each of G ranks (one process per GPU):
  * every BitLinear weight is split by output rows (nsl_b200.ops.shard_rows = NSL's dim-0 shard,
    crates/nsl-runtime/src/tensor_parallel/sharding.rs:18-58); x and its quantisation are
    replicated, so shard outputs are bit-equal to the unsharded ones;
  * q, k, v outputs stay local: a rank owns 32/G heads and their KV cache (the cache of batch 256
    at context 2048 is 8.6 GB per layer in bf16 -- 275 GB for 32 layers, which is why one GPU
    cannot hold the model and why attention must be head-sharded);
  * four exchanges per layer, each an all-gather of [B, N/G] blocks into a buffer every rank
    can store into: the attention output (input of o_proj), o_proj's output, SiLU(gate)*up (the
    down projection contracts over the whole FFN width), and the down projection's output.
    The two projection outputs leave the GEMM epilogue straight into every rank's copy
    (nslq_bitlinear_forward_quantized_gathered); the two activations are pushed by
    nslq_peer_allgather_cols; nslq_peer_barrier closes each exchange.

The glue that is not a quantized linear (residual additions, SiLU*up) is PyTorch, as in
nsl_b200.decoder.  Weights are random ternary; the numbers are throughput numbers.
"""
import math

import torch
import torch.nn.functional as F

from . import ops


class Config7B:
    hidden, heads, head_dim, ffn, layers, vocab = 4096, 32, 128, 11008, 32, 32000
    eps, rope_theta = 1e-5, 10000.0


def _ternary(n, k, gen):
    c = torch.randint(0, 3, (n, k // 4, 4), device="cuda", dtype=torch.uint8, generator=gen)
    return ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).contiguous()


class ShardedDecodeLayers:
    """`n_layers` distinct layers (weights and KV caches), batch `batch`, caches pre-filled to `context`."""

    def __init__(self, comm, batch=256, context=2048, n_layers=4, cfg=Config7B, seed=0, kv_from_full=False):
        self.comm, self.cfg, self.B, self.ctx = comm, cfg, batch, context
        G, r = comm.world, comm.rank
        if cfg.heads % G or cfg.ffn % G or cfg.hidden % G:
            raise ValueError("heads, hidden and FFN width must divide by the world size")
        self.hl = cfg.heads // G                      # local heads
        h, f, d = cfg.hidden, cfg.ffn, cfg.head_dim
        self.max_ctx = (context + 4 + 3) & ~3
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed)
        self.layers = []
        for _ in range(n_layers):
            L = {"n1": torch.ones(h, device="cuda"), "n2": torch.ones(h, device="cuda")}
            for name, (n, k) in {"q": (h, h), "k": (h, h), "v": (h, h), "o": (h, h), "gate": (f, h), "up": (f, h),
                                 "down": (h, f)}.items():
                full = _ternary(n, k, gen)            # the same bytes on every rank (seeded), then this rank's rows
                r0, rows = ops.shard_rows(n, G, r)
                L[name] = ops.BitLinear(full[r0:r0 + rows].contiguous(), 1.0 / math.sqrt(k))
                del full
            if kv_from_full:      # small test shapes: draw the whole cache and keep this rank's heads, so that
                full = torch.empty(2, batch, cfg.heads, self.max_ctx, d, device="cuda", dtype=torch.bfloat16)   # every world size sees the same values
                full.normal_(0.0, 0.5, generator=gen)
                kv = full[:, :, r * self.hl:(r + 1) * self.hl].contiguous()
                del full
            else:
                kv = torch.empty(2, batch, self.hl, self.max_ctx, d, device="cuda", dtype=torch.bfloat16)
                kv.normal_(0.0, 0.5, generator=gen)
            L["k_cache"], L["v_cache"] = kv[0], kv[1]
            self.layers.append(L)
        half = d // 2
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(half, device="cuda").float() / half))
        ang = torch.arange(self.max_ctx, device="cuda").float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.pos = torch.full((1,), context, device="cuda", dtype=torch.long)
        self.sm_scale = 1.0 / math.sqrt(d)
        bf = torch.bfloat16
        # buffers every rank can store into
        self.a_full = comm.symm_empty((batch, h), bf)
        self.o_full = comm.symm_empty((batch, h), bf)
        self.h_full = comm.symm_empty((batch, f), bf)
        self.d_full = comm.symm_empty((batch, h), bf)
        self.x = torch.randn(batch, h, device="cuda", generator=gen)      # fp32 residual stream
        self.kv_bytes_per_layer = 2 * batch * self.hl * context * d * 2
        self.weight_bytes_per_layer = (4 * h * h + 3 * h * f) // 4 // G

    # ---- the pieces of one layer (each also timed on its own by the benchmark)
    def qkv(self, L, qa):
        return [L[n].forward_quantized(qa, out_dtype=torch.bfloat16) for n in ("q", "k", "v")]

    def attention(self, L, q, k, v):
        return ops.decode_attention(q, k, v, L["k_cache"], L["v_cache"], self.cos, self.sin, self.pos, self.sm_scale)

    # Each exchange ends with one barrier ("every rank's block has landed everywhere").  No barrier is needed
    # in front of the stores: a buffer is written again one layer later, after three further barriers that
    # every rank can only have passed once it finished reading that buffer (stream order on each rank).
    def gather_act(self, local, full):
        self.comm.peer_allgather_cols(local, full)
        self.comm.barrier()

    def linear_gathered(self, layer, qa, full):
        layer.forward_quantized_gathered(self.comm, qa, full)
        self.comm.barrier()

    def layer_step(self, L):
        cfg, x = self.cfg, self.x
        qa = ops.rmsnorm_act_quant_i8(x, L["n1"], cfg.eps, plain=False, perm=True)
        q, k, v = self.qkv(L, qa)
        a = self.attention(L, q, k, v)
        self.gather_act(a, self.a_full)
        qa = ops.act_quant_i8(self.a_full, plain=False, perm=True)
        self.linear_gathered(L["o"], qa, self.o_full)
        x.add_(self.o_full)
        qa = ops.rmsnorm_act_quant_i8(x, L["n2"], cfg.eps, plain=False, perm=True)
        g = L["gate"].forward_quantized(qa, out_dtype=torch.bfloat16)
        u = L["up"].forward_quantized(qa, out_dtype=torch.bfloat16)
        hl = F.silu(g) * u
        self.gather_act(hl, self.h_full)
        qa = ops.act_quant_i8(self.h_full, plain=False, perm=True)
        self.linear_gathered(L["down"], qa, self.d_full)
        x.add_(self.d_full)

    def step(self):
        for L in self.layers:
            self.layer_step(L)
