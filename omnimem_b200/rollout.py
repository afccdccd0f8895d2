"""Causal chunk-by-chunk rollout of a Wan2.1-T2V-1.3B-shaped transformer whose self-attention is the
three-branch native sparse attention, driven through this library's block cache and kernels.

This is the CALLER of the selection path, re-typed from the shapes of the reference so that the
path can be measured where it is used: 30 blocks, width 1536, 12 heads of 128, feed-forward 8960,
patch 1x2x2 over 16 latent channels, 512 x 4096 text conditioning, random bf16 weights, synthetic
inputs.  Per chunk of three latent frames (4680 tokens) it runs four denoising forwards and one
cache-write forward at t = 0 (pipelines/pipeline_wan_causal.py:349-495); a layer does what
CausalNSSelfAttention.forward does in its rollout branch (models/transformers/
causal_wan_nsa_model.py:354-553): projections and gates, rotary embedding with the frame offset,
cache update with pooled keys / values, compressed attention over the pooled history, sliding-window
attention over the last chunks, top-k block selection and selection attention over the paged
history, gated sum, output projection.

What runs where:
  * linear layers, norms, cross-attention (SDPA), feed-forward: torch;
  * key rotary embedding + pooling + page append (one kernel), query rotary embedding, query-group
    pooling, scoring + top-k, LRU touch / evict / fetch, all THREE attention branches (the selection
    forward kernel over the selected pages; the range forward kernel over the window's pages and
    over the pooled history as a dense tensor), and the gated sum: this library.
Tokens stay in (frame, row, column) order and a block is 64 consecutive tokens (the reference pools
spatial tiles of 15 x 2 tokens; 64-token blocks cut across rows and chunk boundaries, which the block
cache is built for).  The window starts at the block that holds its first token.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .cache import BlockKVCache, RopeSpec, rope_apply
from .nsa.ops.index_topk import should_use_selection_attention


@dataclass
class WanShape:
    dim: int = 1536
    ffn_dim: int = 8960
    num_heads: int = 12
    num_layers: int = 30
    in_dim: int = 16
    out_dim: int = 16
    patch: tuple = (1, 2, 2)
    text_dim: int = 4096
    text_len: int = 512
    freq_dim: int = 256
    eps: float = 1e-6


@dataclass
class RolloutPlan:
    latent_frames: int = 21
    frames_per_chunk: int = 3
    latent_h: int = 60                      # 480 / 8
    latent_w: int = 104                     # 832 / 8
    timesteps: tuple = (1000.0, 750.0, 500.0, 250.0)
    topk: int = 16
    block: int = 64
    group: int = 64
    window_chunks: int = 3                  # sliding window of the swa branch, in chunks (the current one included)
    exclude_window_chunks: int = 3          # the selection skips what the window covers ...
    progressive_exclude: bool = True        # ... once the history is longer than the window
    cache_cap_frames: Optional[int] = None  # resident full-resolution K/V per layer, in latent frames (None: everything)
    new_prompt_every: Optional[int] = None  # a fresh conditioning tensor every this many latent frames
    seed: int = 0


class SectionTimer:
    """CUDA-event brackets per named section of a layer, summed over layers and forwards - the role
    of the reference's TripleAttnProfiler (utils/attn_profiler.py:10-133: cache, cmp, swa, slc_topk,
    slc_attn).  Off by default: the brackets cost launches of their own."""

    def __init__(self):
        self.events = {}

    class _Span:
        def __init__(self, owner, name):
            self.owner, self.name = owner, name

        def __enter__(self):
            self.a = torch.cuda.Event(enable_timing=True)
            self.b = torch.cuda.Event(enable_timing=True)
            self.a.record()

        def __exit__(self, *exc):
            self.b.record()
            self.owner.events.setdefault(self.name, []).append((self.a, self.b))

    def __call__(self, name):
        return SectionTimer._Span(self, name)

    def summary_ms(self, per: int = 1) -> dict:
        """Total milliseconds per section divided by `per` (e.g. the number of forwards)."""
        torch.cuda.synchronize()
        return {k: round(sum(a.elapsed_time(b) for a, b in v) / per, 3) for k, v in self.events.items()}


class _NoTimer:
    def __call__(self, name):
        return self

    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_TIMER = _NoTimer()


def rope_table(max_len: int, dim: int, theta: float = 10000.0) -> torch.Tensor:
    """complex128 [max_len, dim/2] (rope_params, wan_model.py:37-43)."""
    ang = torch.outer(torch.arange(max_len, dtype=torch.float64),
                      1.0 / torch.pow(theta, torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    return torch.polar(torch.ones_like(ang), ang)


def sinusoidal_embedding(dim: int, t: torch.Tensor) -> torch.Tensor:
    half = dim // 2
    pos = t.to(torch.float64)
    freq = torch.pow(10000.0, -torch.arange(half, dtype=torch.float64, device=t.device) / half)
    x = torch.outer(pos, freq)
    return torch.cat([x.cos(), x.sin()], dim=1).float()


class RMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x.float(), (x.shape[-1],), self.weight.float(), self.eps).to(x.dtype)


class NSASelfAttention(nn.Module):
    """The rollout branch of CausalNSSelfAttention over a BlockKVCache."""

    def __init__(self, shape: WanShape, plan: RolloutPlan, layer_idx: int):
        super().__init__()
        d, h = shape.dim, shape.num_heads
        self.h, self.hd, self.plan, self.layer_idx = h, d // h, plan, layer_idx
        self.q, self.k, self.v, self.o = (nn.Linear(d, d) for _ in range(4))
        self.norm_q, self.norm_k = RMSNorm(d, shape.eps), RMSNorm(d, shape.eps)
        self.g_proj = nn.Linear(d, 3 * h)
        nn.init.normal_(self.g_proj.weight, mean=0.0, std=1e-3)     # gates start at 0.5 (initialize_gate, :164-168)
        nn.init.zeros_(self.g_proj.bias)

    def forward(self, x, cache: BlockKVCache, rope: RopeSpec, start_token: int, timer=_NO_TIMER):
        p = self.plan
        _, S, _ = x.shape
        H, D = self.h, self.hd
        with timer("qkv_gate_proj"):
            q = self.norm_q(self.q(x)).view(S, H, D)
            k = self.norm_k(self.k(x)).view(S, H, D)
            v = self.v(x).view(S, H, D)
            g = self.g_proj(x).view(1, S, H, 3)
        scale = D ** -0.5
        # query rotary embedding; the keys receive theirs on the way into the pages, where they are also
        # pooled: one kernel replaces rope + four cache updates + two poolings of the reference layer
        with timer("rope_q"):
            qr = rope_apply(q, rope).unsqueeze(0)
        with timer("cache_append"):
            cache.append(k, v, pos0=start_token, rope=rope)
        nb = cache.n_blocks
        # compressed branch: attention over the pooled history, a dense [1, nb, H, D] view of the pooled
        # keys / values taken as one range of blocks
        with timer("cmp"):
            o_cmp, _ = ops.range_fwd(qr, ops.DenseKV(cache.pooled_keys(), cache.pooled_values()), 0,
                                     -(-nb // p.block), p.block, scale)
        # sliding-window branch: the pages of the last window_chunks chunks through the block table
        with timer("swa"):
            first_tok = max(0, start_token - (p.window_chunks - 1) * S)
            first_blk = first_tok // p.block
            o_swa, _ = ops.range_fwd(qr, cache.kv_source(), first_blk, nb - first_blk, p.block, scale)
        # selection branch
        q_chunk = start_token // S
        if p.progressive_exclude or should_use_selection_attention(nb * p.block, S, p.exclude_window_chunks, 0, causal=False):
            with timer("slc_topk"):
                qp = ops.pool_rows(qr, p.group)
                idx = ops.topk(qp, cache.pooled_keys(), p.topk, scale, p.block, S, S, False,
                               ex_win=p.exclude_window_chunks, prog_excl=p.progressive_exclude,
                               q_chunk_offset=q_chunk, q_group_size=p.group)
            with timer("slc_touch_fetch"):
                cache.touch(idx)
            with timer("slc_attn"):
                o_slc, _ = ops.sel_fwd(qr, cache.kv_source(), idx, p.block, 1, scale, False, p.group)
        else:
            o_slc = torch.zeros_like(qr)
        with timer("gate_sum_oproj"):
            y = ops.gate_combine(g, o_cmp, o_slc, o_swa)
            out = self.o(y.view(1, S, H * D))
        return out


class CrossAttention(nn.Module):
    def __init__(self, shape: WanShape):
        super().__init__()
        d, h = shape.dim, shape.num_heads
        self.h, self.hd = h, d // h
        self.q, self.k, self.v, self.o = (nn.Linear(d, d) for _ in range(4))
        self.norm_q, self.norm_k = RMSNorm(d, shape.eps), RMSNorm(d, shape.eps)

    def forward(self, x, context):
        B, S, _ = x.shape
        L = context.shape[1]
        q = self.norm_q(self.q(x)).view(B, S, self.h, self.hd).transpose(1, 2)
        k = self.norm_k(self.k(context)).view(B, L, self.h, self.hd).transpose(1, 2)
        v = self.v(context).view(B, L, self.h, self.hd).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v)
        return self.o(y.transpose(1, 2).reshape(B, S, self.h * self.hd))


class Block(nn.Module):
    def __init__(self, shape: WanShape, plan: RolloutPlan, layer_idx: int):
        super().__init__()
        d = shape.dim
        self.eps = shape.eps
        self.self_attn = NSASelfAttention(shape, plan, layer_idx)
        self.norm3 = nn.LayerNorm(d, eps=shape.eps)
        self.cross_attn = CrossAttention(shape)
        self.ffn = nn.Sequential(nn.Linear(d, shape.ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(shape.ffn_dim, d))
        self.modulation = nn.Parameter(torch.randn(1, 6, d) / d ** 0.5)

    def forward(self, x, e0, context, cache, rope, start_token, timer=_NO_TIMER):
        e = (self.modulation.float() + e0).unbind(1)                 # six [1, dim] rows (fp32, as the reference)
        d = x.shape[-1]
        with timer("norm_modulation"):
            h = (F.layer_norm(x.float(), (d,), eps=self.eps) * (1 + e[1]) + e[0]).to(x.dtype)
        y = self.self_attn(h, cache, rope, start_token, timer)
        with timer("norm_modulation"):
            x = x + (y.float() * e[2]).to(x.dtype)
        with timer("cross_attn"):
            x = x + self.cross_attn(self.norm3(x), context)
        with timer("ffn"):
            h = (F.layer_norm(x.float(), (d,), eps=self.eps) * (1 + e[4]) + e[3]).to(x.dtype)
            x = x + (self.ffn(h).float() * e[5]).to(x.dtype)
        return x


class CausalWanNSA(nn.Module):
    def __init__(self, shape: WanShape, plan: RolloutPlan):
        super().__init__()
        self.shape, self.plan = shape, plan
        d = shape.dim
        self.patch_embedding = nn.Conv3d(shape.in_dim, d, kernel_size=shape.patch, stride=shape.patch)
        self.text_embedding = nn.Sequential(nn.Linear(shape.text_dim, d), nn.GELU(approximate="tanh"), nn.Linear(d, d))
        self.time_embedding = nn.Sequential(nn.Linear(shape.freq_dim, d), nn.SiLU(), nn.Linear(d, d))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(d, 6 * d))
        self.blocks = nn.ModuleList([Block(shape, plan, i) for i in range(shape.num_layers)])
        self.head_norm_eps = shape.eps
        self.head = nn.Linear(d, shape.out_dim * math.prod(shape.patch))
        self.head_modulation = nn.Parameter(torch.randn(1, 2, d) / d ** 0.5)
        hd = d // shape.num_heads
        self.register_buffer("_dummy", torch.zeros(1), persistent=False)
        self.freqs = torch.cat([rope_table(1024, hd - 4 * (hd // 6)), rope_table(1024, 2 * (hd // 6)),
                                rope_table(1024, 2 * (hd // 6))], dim=1)

    def forward(self, latents, t, context_embedded, start_frame, caches: List[BlockKVCache], timer=_NO_TIMER):
        """latents [1, C, f, h, w]; t scalar timestep; returns the prediction in latent layout."""
        sh = self.shape
        x = self.patch_embedding(latents)
        _, _, f, gh, gw = x.shape
        x = x.flatten(2).transpose(1, 2).contiguous()
        S = x.shape[1]
        temb = sinusoidal_embedding(sh.freq_dim, torch.full((1,), float(t), device=x.device)).to(x.dtype)
        e = self.time_embedding(temb)
        e0 = self.time_projection(e).float().view(1, 6, sh.dim)
        rope = RopeSpec(self.freqs, (gh, gw), start_frame, (1, 1, 1))
        start_token = start_frame * gh * gw
        for blk, cache in zip(self.blocks, caches):
            x = blk(x, e0, context_embedded, cache, rope, start_token, timer)
        m = (self.head_modulation.float() + e.float().unsqueeze(1)).unbind(1)
        x = (F.layer_norm(x.float(), (sh.dim,), eps=self.head_norm_eps) * (1 + m[1]) + m[0]).to(x.dtype)
        x = self.head(x)                                                # [1, S, out * pf*ph*pw]
        pf, ph, pw = sh.patch
        x = x.view(1, f, gh, gw, pf, ph, pw, sh.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(1, sh.out_dim, f * pf, gh * ph, gw * pw)


def make_caches(shape: WanShape, plan: RolloutPlan, device) -> List[BlockKVCache]:
    """One page pool per layer.  Without a cap every block of the rollout is resident.  With one the
    pool holds cache_cap_frames frames' worth of blocks per head (at least the protected window and
    the chunk being written) PLUS room for the blocks one call can select (top-k x query groups per
    head): a call needs its window and everything it selected resident at the same time, and with
    random weights the selections of the 74 query groups hardly overlap.  The rest of the history
    lives in the pinned host tier and comes back when selected."""
    gh, gw = plan.latent_h // shape.patch[1], plan.latent_w // shape.patch[2]
    tokens = plan.latent_frames * gh * gw
    max_blocks = -(-tokens // plan.block)
    H, D = shape.num_heads, shape.dim // shape.num_heads
    chunk_blocks = -(-plan.frames_per_chunk * gh * gw // plan.block) + 1
    protect = plan.window_chunks * chunk_blocks                     # the window and the chunk being written stay resident
    if plan.cache_cap_frames is None:
        pages, host = H * max_blocks, False
    else:
        groups = -(-plan.frames_per_chunk * gh * gw // plan.group)
        pages = H * (max(-(-plan.cache_cap_frames * gh * gw // plan.block), protect + chunk_blocks) + plan.topk * groups)
        host = True
    return [BlockKVCache(H, D, pages, max_blocks, plan.block, torch.bfloat16, device, host_tier=host, protect_blocks=protect)
            for _ in range(shape.num_layers)]


@dataclass
class RolloutResult:
    seconds: float
    latent_frames: int
    forwards: int
    frames_per_second: float
    cache: dict = field(default_factory=dict)
    latents: Optional[torch.Tensor] = None


@torch.no_grad()
def rollout(model: CausalWanNSA, caches: List[BlockKVCache], plan: RolloutPlan, device, keep_latents: bool = False,
            timer=_NO_TIMER) -> RolloutResult:
    """The denoising loop of CausalWanT2VPipeline.generate (pipeline_wan_causal.py:349-495): per chunk,
    len(timesteps) denoising forwards (each rewrites the chunk's K/V in the caches), then one forward
    of the clean chunk at t = 0 that leaves the final K/V behind.  Returns the wall time of the loop
    (the reference's "Denoising Time") and latent frames per second."""
    sh = model.shape
    gen = torch.Generator(device=device).manual_seed(plan.seed)
    noise = torch.randn(1, sh.in_dim, plan.latent_frames, plan.latent_h, plan.latent_w, generator=gen, device=device,
                        dtype=torch.bfloat16)

    def new_context():
        raw = torch.randn(1, sh.text_len, sh.text_dim, generator=gen, device=device, dtype=torch.bfloat16)
        return model.text_embedding(raw)

    context = new_context()
    next_switch = plan.new_prompt_every
    latents = torch.zeros_like(noise) if keep_latents else None
    for c in caches:
        c.reset()
    forwards = 0
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    for start in range(0, plan.latent_frames, plan.frames_per_chunk):
        if next_switch is not None and start >= next_switch:
            context = new_context()
            next_switch += plan.new_prompt_every
        x_t = noise[:, :, start:start + plan.frames_per_chunk]
        x0 = x_t
        for i, t in enumerate(plan.timesteps):
            sigma = t / 1000.0
            v = model(x_t, t, context, start, caches, timer)
            forwards += 1
            x0 = (x_t.float() - sigma * v.float()).to(x_t.dtype)               # flow prediction -> clean estimate
            if i + 1 < len(plan.timesteps):
                s2 = plan.timesteps[i + 1] / 1000.0
                eps = torch.randn(x0.shape, generator=gen, device=device, dtype=x0.dtype)
                x_t = ((1.0 - s2) * x0.float() + s2 * eps.float()).to(x0.dtype)
        if latents is not None:
            latents[:, :, start:start + plan.frames_per_chunk] = x0
        model(x0, 0.0, context, start, caches, timer)                          # cache-write forward on the clean chunk
        forwards += 1
    torch.cuda.synchronize(device)
    dt = time.perf_counter() - t0
    stats = {"hits": 0, "misses": 0, "pages_evicted": 0, "pages_fetched": 0, "bytes_to_host": 0, "bytes_from_host": 0}
    for c in caches:
        c.check_status()
        s = c.stats()
        for k in stats:
            stats[k] += s[k]
    total = stats["hits"] + stats["misses"]
    stats["hit_rate"] = stats["hits"] / total if total else 0.0
    return RolloutResult(dt, plan.latent_frames, forwards, plan.latent_frames / dt, stats, latents)


def build(shape: WanShape, plan: RolloutPlan, device, seed: int = 0):
    torch.manual_seed(seed)
    model = CausalWanNSA(shape, plan).to(device=device, dtype=torch.bfloat16).eval()
    return model, make_caches(shape, plan, device)
