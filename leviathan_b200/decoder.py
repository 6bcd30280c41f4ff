"""A synthetic MoE decoder whose step is a list of C-ABI calls on one stream.

The host-side mirror of the reference's token loop (Gemma4Runner.forwardToken and forwardLayer,
Sources/LeviathanCore/Gemma4.swift:3611-3905) for the synthetic decode workload: embedding row ->
per layer [RMSNorm -> q, k, v -> per-head norms, rotary, cache append -> attention over the paged
cache -> output projection + residual -> RMSNorm -> routed experts -> residual] -> final RMSNorm ->
tied Q6_K head -> softcap -> greedy argmax.  Where the reference reads router scores and logits back
to the host every layer (Gemma4.swift:3796-3809, :3637-3641), every step here stays on the device:
token ids, positions and slots are device tensors, so the whole step is captured as one CUDA graph and
a replay is one decoded token per sequence with the next token id already in place.

Weights are random (seeded SplitMix64 normals, sigma 0.02, quantized with this package's encoders);
caches are filled with N(0, 1) values up to the last position.  torch holds the buffers and the
graph; every arithmetic step is a kernel of libleviathan_cuda.so.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from . import quant as Q
from .api import Context, PagedKV


@dataclass
class DecoderConfig:
    hidden: int = 2816
    layers: int = 30
    q_heads: int = 16
    kv_heads: int = 8
    head_dim: int = 256
    experts: int = 128
    top_k: int = 8
    expert_inter: int = 704
    vocab: int = 262144
    positions: int = 4096        # cached positions per sequence (the step writes the last one)
    page: int = 16               # positions per cache block (PAGE_SIZE of rust/crates/lev-forge/src/ops.rs:32)
    eps: float = 1e-6
    softcap: float = 30.0        # finalSoftcap of Gemma4.swift:3631
    rope_base: float = 10000.0
    attn_scale: float = 1.0 / 16.0   # 1 / sqrt(head_dim): cached keys are N(0, 1), not normed
    weight_type: int = Q.GGML_Q4_0
    head_type: int = Q.GGML_Q6_K
    sigma: float = 0.02
    seed: int = 0x4C455649

    def bytes_per_token(self, batch: int = 1) -> dict:
        """GGUF block bytes and cache bytes one decode step must read, per decoded token at `batch`
        sequences (weights are read once per step whatever the batch; each sequence reads its own cache)."""
        def blk(t, rows, cols):
            return rows * (cols // (32 if t == Q.GGML_Q4_0 else 256)) * {Q.GGML_Q4_0: 18, Q.GGML_Q4_K: 144, Q.GGML_Q6_K: 210}[t]

        qw, kw = self.q_heads * self.head_dim, self.kv_heads * self.head_dim
        attn = blk(self.weight_type, qw, self.hidden) + 2 * blk(self.weight_type, kw, self.hidden) + blk(self.weight_type, self.hidden, qw)
        expert = blk(self.weight_type, 2 * self.expert_inter, self.hidden) + blk(self.weight_type, self.hidden, self.expert_inter)
        router = self.experts * self.hidden * 4
        kv = 2 * self.positions * self.kv_heads * self.head_dim * 2
        head = blk(self.head_type, self.vocab, self.hidden)
        return {"attention_weights": attn, "expert": expert, "router": router, "kv_per_sequence": kv, "head": head,
                "batch_1_total": self.layers * (attn + router + self.top_k * expert + kv) + head}


@dataclass
class _Layer:
    wq: object    # narrow batches: three tensors behind one launch of the decode matvec
    wk: object
    wv: object
    wqkv: object  # wide batches: the same rows as one [q | k | v] tensor, one GEMM instead of three
    wo: object
    moe: object
    cache: PagedKV
    attn_norm: object
    ffn_norm: object
    q_norm: object
    k_norm: object


class SyntheticDecoder:
    """`batch` sequences, each with `cfg.positions - 1` cached positions; `step()` decodes one token per
    sequence.  With `advance=False` (the timing form) the position stays at the last cache row, so a
    step can repeat without running out of cache.

    Projections: up to `gemm_from - 1` sequences go through the decode matvec (f32 activations, at most eight
    columns a call); from `gemm_from` sequences on they go through the prefill dequant-GEMM on the tensor cores
    (activations rounded to bf16, one pass over the weights whatever the batch), the numerics the reference's own
    prefill path has (rust/crates/lev-forge/src/coopmat.rs:236-425).

    Several GPUs (`world` > 1, the context already joined by dist.init_from_torch): every rank decodes its own
    `batch` sequences (their caches differ by rank, the weights do not), attention and the head are local, and
    the experts are sharded -- rank r keeps experts [r * E / world, (r + 1) * E / world) -- so the MoE of a step
    is the expert-parallel layer: tokens go to the ranks that hold their experts and the expert rows come back
    to be combined in slot order on the token's rank."""

    def __init__(self, ctx: Context, cfg: DecoderConfig, batch: int = 1, device="cuda", norm_sigma: float = 0.02,
                 keep_host_copies: bool = False, gemm_from: int = 16, rank: int = 0, world: int = 1):
        import torch

        self.ctx, self.cfg, self.batch, self.dev = ctx, cfg, batch, device
        self.wide = batch >= gemm_from
        self.rank, self.world = rank, world
        if cfg.experts % world:
            raise ValueError(f"{cfg.experts} experts do not split over {world} ranks")
        H, QH, KVH, HD = cfg.hidden, cfg.q_heads, cfg.kv_heads, cfg.head_dim
        self.host = {} if keep_host_copies else None
        self._seed = cfg.seed
        blocks_per_seq = (cfg.positions + cfg.page - 1) // cfg.page
        self.layers: list[_Layer] = []
        for l in range(cfg.layers):
            wq = wk = wv = wqkv = None
            if self.wide:
                # GGUF rows are independent: the three tensors' bytes one after the other are the fused tensor's
                parts = [self._blocks(f"blk.{l}.attn_q", cfg.weight_type, QH * HD, H),
                         self._blocks(f"blk.{l}.attn_k", cfg.weight_type, KVH * HD, H),
                         self._blocks(f"blk.{l}.attn_v", cfg.weight_type, KVH * HD, H)]
                wqkv = ctx.upload(torch.cat(parts), cfg.weight_type, (QH + 2 * KVH) * HD, H)
                del parts
            else:
                wq = self._tensor(f"blk.{l}.attn_q", cfg.weight_type, QH * HD, H)
                wk = self._tensor(f"blk.{l}.attn_k", cfg.weight_type, KVH * HD, H)
                wv = self._tensor(f"blk.{l}.attn_v", cfg.weight_type, KVH * HD, H)
            wo = self._tensor(f"blk.{l}.attn_output", cfg.weight_type, H, QH * HD)
            if not self.wide:
                for w in (wq, wk, wv, wo):
                    w.release_gguf()   # only the decode kernels read these: one resident copy instead of two
            moe = self._experts(l)
            cache = PagedKV(batch * blocks_per_seq + 1, cfg.page, KVH, HD, slots=batch, max_blocks=blocks_per_seq, dtype="f16", device=device)
            for s in range(batch):
                cache.ensure(s, cfg.positions - 1)
            self._fill(cache.k, f"blk.{l}.cache_k")
            self._fill(cache.v, f"blk.{l}.cache_v")  # the two fills take their seeds in a per-rank range, see _fill
            self.layers.append(_Layer(wq, wk, wv, wqkv, wo, moe, cache,
                                      self._norm(f"blk.{l}.attn_norm", H, norm_sigma), self._norm(f"blk.{l}.ffn_norm", H, norm_sigma),
                                      self._norm(f"blk.{l}.attn_q_norm", HD, norm_sigma), self._norm(f"blk.{l}.attn_k_norm", HD, norm_sigma)))
        self.out_norm = self._norm("output_norm", H, norm_sigma)
        self.head = self._tensor("token_embd", cfg.head_type, cfg.vocab, H, slab=32768)
        self.inv_freq = (cfg.rope_base ** (-torch.arange(HD // 2, device=device, dtype=torch.float64) / (HD // 2))).float()
        B = batch
        self.tok = torch.zeros(B, dtype=torch.int32, device=device)
        self.pos = torch.full((B,), cfg.positions - 1, dtype=torch.int32, device=device)
        self.slot = torch.arange(B, dtype=torch.int32, device=device)
        self.x = torch.empty((B, H), device=device)
        self.x1 = torch.empty((B, H), device=device)
        self.h = torch.empty((B, H), device=device)
        self.mo = torch.empty((B, H), device=device)
        self.q = torch.empty((B, QH * HD), device=device)
        self.k = torch.empty((B, KVH * HD), device=device)
        self.v = torch.empty((B, KVH * HD), device=device)
        self.ao = torch.empty((B, QH, HD), device=device)
        self.logits = torch.empty((B, cfg.vocab), device=device)
        if self.wide:
            self.qkv = torch.empty((B, (QH + 2 * KVH) * HD), device=device)
            self.hb = torch.empty((B, H), dtype=torch.bfloat16, device=device)
            self.aob = torch.empty((B, QH * HD), dtype=torch.bfloat16, device=device)
        self.graph = None

    # ---- synthetic tensors ----
    def _next_seed(self) -> int:
        self._seed += 1
        return self._seed

    def _tensor(self, name, t, rows, cols, slab=None):
        return self.ctx.upload(self._blocks(name, t, rows, cols, slab), t, rows, cols)

    def _blocks(self, name, t, rows, cols, slab=None):
        import torch

        slab = rows if slab is None else min(slab, rows)
        parts = []
        for r0 in range(0, rows, slab):
            n = min(slab, rows - r0)
            parts.append(Q.quantize(t, Q.normal_torch(self._next_seed(), (n, cols), self.cfg.sigma, self.dev)))
        blocks = parts[0] if len(parts) == 1 else torch.cat(parts)
        if self.host is not None:
            self.host[name] = blocks.cpu().numpy()
        return blocks

    def _experts(self, l):
        import torch

        c = self.cfg
        E, H, I = c.experts, c.hidden, c.expert_inter
        per = E // self.world
        first = self.rank * per
        step = max(1, min(16, E // 8))   # experts per seed pair: the same walk whatever the number of ranks (up to 8)
        if per % step:
            raise ValueError(f"{per} experts per rank do not split into groups of {step}")
        gu, dn = [], []
        for e0 in range(0, E, step):
            n = min(step, E - e0)
            s_gu, s_dn = self._next_seed(), self._next_seed()   # every rank walks the same seeds
            if e0 + n <= first or e0 >= first + per:
                continue                                        # ... and builds only its own experts
            gu.append(Q.quantize(c.weight_type, Q.normal_torch(s_gu, (n * 2 * I, H), c.sigma, self.dev)))
            dn.append(Q.quantize(c.weight_type, Q.normal_torch(s_dn, (n * H, I), c.sigma, self.dev)))
        gu, dn = torch.cat(gu), torch.cat(dn)
        router = Q.normal_torch(self._next_seed(), (E, H), c.sigma, self.dev)
        if self.host is not None:
            self.host[f"blk.{l}.ffn_gate_up_exps"] = gu.cpu().numpy()
            self.host[f"blk.{l}.ffn_down_exps"] = dn.cpu().numpy()
            self.host[f"blk.{l}.ffn_gate_inp"] = router.cpu().numpy()
        moe = self.ctx.moe_upload(router, gu, dn, E, H, I, first, per)
        if self.batch * self.world * c.top_k < 512:
            moe.release_gguf()   # decode-sized calls read the repacked experts only: one resident copy
        return moe

    def _norm(self, name, n, sigma):
        w = 1.0 + Q.normal_torch(self._next_seed(), (n,), sigma, self.dev)
        if self.host is not None:
            self.host[name] = w.cpu().numpy()
        return w

    def _fill(self, pool, name):
        import torch

        flat = pool.view(-1)
        chunk = 1 << 26
        for o in range(0, flat.numel(), chunk):
            n = min(chunk, flat.numel() - o)
            # weights share their seeds over the ranks, caches do not: every rank decodes its own sequences
            seed = self._next_seed() ^ (self.rank << 40)
            flat[o:o + n] = Q.normal_torch(seed, (n,), 1.0, self.dev).to(torch.float16)

    # ---- the step ----
    def _cols(self):
        """column groups of at most eight sequences: the widest a decode matvec launch takes"""
        return [(c0, min(c0 + 8, self.batch)) for c0 in range(0, self.batch, 8)]

    def step(self, advance: bool = False):
        c, ctx = self.cfg, self.ctx
        QH, KVH, HD = c.q_heads, c.kv_heads, c.head_dim
        qw = QH * HD
        ctx.embed_rows(self.head, self.tok, math.sqrt(c.hidden), out=self.x)
        x, x1 = self.x, self.x1
        for L in self.layers:
            if self.wide:
                ctx.rmsnorm(x, L.attn_norm, c.eps, out=self.h)
                ctx.act_bf16(self.h, out=self.hb)
                ctx.gemm_prefill(L.wqkv, self.hb, out=self.qkv)
                ctx.qkv_norm_rope_append(self.qkv, QH, L.cache, self.slot, self.pos, L.q_norm, L.k_norm, c.eps, self.inv_freq)
                ctx.attn_decode_fused_rows(L.cache, self.slot, self.pos, self.qkv, QH, 0, c.attn_scale, out=self.ao)
            else:
                for a, b in self._cols():
                    ctx.matvec_multi_fused([L.wq, L.wk, L.wv], x[a:b], "rmsnorm", L.attn_norm, c.eps, outs=[self.q[a:b], self.k[a:b], self.v[a:b]])
                ctx.qkv_norm_rope_append_split(self.q, self.k, self.v, QH, L.cache, self.slot, self.pos, L.q_norm, L.k_norm, c.eps, self.inv_freq)
                ctx.attn_decode(L.cache, self.slot, self.pos, self.q.view(self.batch, QH, HD), 0, c.attn_scale, out=self.ao)
            if self.wide:
                ctx.act_bf16(self.ao.view(self.batch, qw), out=self.aob)
                ctx.gemm_prefill(L.wo, self.aob, out=self.mo)
                ctx.axpy(1.0, self.mo, x, out=x1)
            else:
                for a, b in self._cols():
                    ctx.matvec_fused(L.wo, self.ao[a:b].view(b - a, qw), None, residual=x[a:b], alpha=1.0, out=x1[a:b])
            ctx.rmsnorm(x1, L.ffn_norm, c.eps, out=self.h)
            if self.world > 1:
                ctx.moe_layer(L.moe, self.h, c.top_k, out=self.mo, expert_parallel=True)
                ctx.axpy(1.0, self.mo, x1, out=x)
            else:
                ctx.moe_layer_residual(L.moe, self.h, c.top_k, x1, 1.0, out=x)  # the residual rides in the combine launch
        self.head_step()
        if advance:
            self.pos.add_(1)
        return self.tok

    def head_step(self):
        """final norm -> tied head -> softcap -> greedy argmax into the token ids (Gemma4.swift:3622-3643)"""
        c, ctx, x = self.cfg, self.ctx, self.x
        if self.wide:
            ctx.rmsnorm(x, self.out_norm, c.eps, out=self.h)
            ctx.act_bf16(self.h, out=self.hb)
            ctx.gemm_prefill(self.head, self.hb, out=self.logits)
        else:
            for a, b in self._cols():
                ctx.matvec_fused(self.head, x[a:b], "rmsnorm", self.out_norm, c.eps, out=self.logits[a:b])
        ctx.softcap(self.logits, c.softcap)
        ctx.argmax_into(self.logits, self.tok)

    def capture(self, advance: bool = False):
        """Records `step` as one CUDA graph on the context's stream; `replay()` then decodes a token."""
        import torch

        stream = torch.cuda.current_stream()
        tok0, pos0 = self.tok.clone(), self.pos.clone()
        self.step(advance)   # the first call sizes every scratch buffer outside the capture
        stream.synchronize()
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            self.step(advance)
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        self.graph = g
        return g

    def replay(self):
        self.graph.replay()
        return self.tok

    def free(self):
        for L in self.layers:
            for w in (L.wq, L.wk, L.wv, L.wqkv, L.wo):
                if w is not None:
                    w.free()
            L.moe.free()
        self.head.free()
        self.layers = []


def _main():
    """python -m leviathan_b200.decoder [--batch B] [--layers L] [--vocab V] [--steps N] [--graph]
    builds the synthetic decoder on cuda:0, decodes N tokens per sequence and prints the rate."""
    import argparse
    import time

    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=30)
    ap.add_argument("--vocab", type=int, default=262144)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--graph", action="store_true", help="capture the step as one CUDA graph and replay it")
    a = ap.parse_args()
    ctx = Context(0)
    cfg = DecoderConfig(layers=a.layers, vocab=a.vocab)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        dec = SyntheticDecoder(ctx, cfg, batch=a.batch)
        if a.graph:
            dec.capture()
        run = dec.replay if a.graph else dec.step
        run()
        ctx.synchronize()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            run()
        ctx.synchronize()
        dt = time.perf_counter() - t0
    print(f"{a.steps} steps of {a.batch} sequences, {a.layers} layers, vocabulary {a.vocab}: {dt / a.steps * 1e3:.3f} ms per step, "
          f"{a.batch * a.steps / dt:.1f} tokens/s, last tokens {dec.tok[:4].tolist()}")
    dec.free()
    ctx.close()


if __name__ == "__main__":
    _main()
