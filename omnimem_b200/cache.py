"""Fixed-page block KV cache with an LRU block table, resident on the device.

Re-expresses, at 64-token block granularity and without host round trips, what the
reference's ``MMCache`` does per chunk with Python lists, ``OrderedDict`` LRUs and pinned
offload buffers (models/cache.py:438-522 update_cache, :673-699 lru_touch_per_head,
:1032-1142 flush_offload) together with the selected-chunk reload of
nsa/ops/selection/padded_ptr/wrapper.py:253-362 and the block-KV kernels K1-K3
(nsa/cuda_backend/csrc/block_kv_ops.h:12-31):

* a page holds one (head, block); ``block_table[h, bid]`` maps a block to its page or -1;
* pooled keys / values of EVERY block ever appended stay on the device and remain top-k
  candidates; full-resolution K/V of evicted blocks live in fixed pinned-host slots and are
  fetched back when a selection asks for them (history is never dropped);
* the LRU clock is a per-page epoch stamp; victims are the pages with the oldest stamp
  outside the protected tail window;
* appends may start in the middle of the last page; the pooled key of a partially filled
  block is the mean of the tokens it holds and is refreshed when more arrive.

All decisions that depend on data (which selected blocks are missing, which pages to evict
for them) are taken by kernels; the host only supplies sizes it knows by construction.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib, ops
from ._lib import NSABackendError, call


class RopeSpec:
    """Rotary embedding of one chunk: `freqs` is the reference's complex128 table
    [max_len, D/2] (rope_params, wan_model.py:37-43; split D/2 - 2*(D/2//3), D/2//3, D/2//3 over
    frame / row / column), `grid_hw` the latent rows and columns of a frame, `start_frame` the
    chunk's first frame, `pool` the (f, h, w) pooling window that defines the token order."""

    def __init__(self, freqs: torch.Tensor, grid_hw, start_frame: int, pool=(1, 1, 1)):
        if freqs.dtype != torch.complex128 or freqs.dim() != 2:
            raise NSABackendError("RopeSpec: freqs must be a complex128 [max_len, D/2] table")
        self.freqs, self.grid_hw, self.start_frame, self.pool = freqs, tuple(grid_hw), int(start_frame), tuple(pool)
        self._tables = None

    def struct(self, device, D: int) -> _lib.Rope:
        c = D // 2
        if self.freqs.shape[1] != c:
            raise NSABackendError(f"RopeSpec: freqs has {self.freqs.shape[1]} columns, head dim {D} needs {c}")
        if self._tables is None or self._tables[0].device != device:
            parts = self.freqs.split([c - 2 * (c // 3), c // 3, c // 3], dim=1)
            self._tables = [torch.view_as_real(p.contiguous()).to(device).contiguous() for p in parts]
        s = _lib.Rope()
        s.freqs_f, s.freqs_h, s.freqs_w = (t.data_ptr() for t in self._tables)
        s.c_f, s.c_h, s.c_w = c - 2 * (c // 3), c // 3, c // 3
        s.grid_h, s.grid_w = self.grid_hw
        s.pool_f, s.pool_h, s.pool_w = self.pool
        s.start_frame = self.start_frame
        return s


def rope_apply(x: torch.Tensor, rope: RopeSpec) -> torch.Tensor:
    """Rotary embedding of a chunk of queries x [S,H,D] (bf16 / fp16) -> a new contiguous tensor;
    the query-side use of causal_reorder_rope_apply (causal_wan_nsa_model.py:72-105, 463-466)."""
    if not x.is_cuda or x.dim() != 3:
        raise NSABackendError("rope_apply: x must be a CUDA tensor [S,H,D]")
    x = ops._rows16(x)
    S, H, D = x.shape
    out = torch.empty(S, H, D, dtype=x.dtype, device=x.device)
    spec = rope.struct(x.device, D)
    with torch.cuda.device(x.device):
        call("nsa_rope_apply", x.data_ptr(), (C.c_int64 * 3)(x.stride(0), x.stride(1), 0), S, H, D, out.data_ptr(),
             ops._dtype(x), C.byref(spec), torch.cuda.current_stream(x.device).cuda_stream)
    return out


class BlockKVCache:
    _drain_streams = {}                       # device index -> the stream the write-behind copies run on

    def __init__(self, num_heads: int, head_dim: int, num_pages: int, max_blocks: int,
                 page_tokens: int = 64, dtype: torch.dtype = torch.bfloat16, device="cuda",
                 host_tier: bool = True, protect_blocks: int = 0, write_behind: bool = True):
        """`write_behind`: the pages an append evicts go to a staging buffer on the device (so they are
        free at once) and from there to the host tier on a stream of their own, beside the work that
        follows; which pages are evicted, and when, does not change."""
        dev = torch.device(device)
        if dev.type != "cuda":
            raise NSABackendError("BlockKVCache lives on a CUDA device")
        self.H, self.D, self.page_tokens = num_heads, head_dim, page_tokens
        self.num_pages, self.max_blocks = num_pages, max_blocks
        self.dtype, self.device = dtype, dev
        self.protect_blocks = protect_blocks
        # Zero-filled, not empty: the rows of a partly filled page behind the block's last token are
        # read by the attention kernels (their keys get probability 0, but 0 x NaN would still be NaN
        # in the P V and dS K products), so the pool must never hold non-finite bit patterns.
        self.k_pool = torch.zeros(num_pages, page_tokens, head_dim, dtype=dtype, device=dev)
        self.v_pool = torch.zeros_like(self.k_pool)
        self.block_table = torch.full((num_heads, max_blocks), -1, dtype=torch.int32, device=dev)
        self.page_owner = torch.full((num_pages,), -1, dtype=torch.int32, device=dev)
        self.page_stamp = torch.zeros(num_pages, dtype=torch.int64, device=dev)
        self.k_pooled = torch.zeros(num_heads, max_blocks, head_dim, dtype=dtype, device=dev)
        self.v_pooled = torch.zeros_like(self.k_pooled)
        self._stamp32 = torch.zeros(num_heads * max_blocks, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.host_k = self.host_v = None
        if host_tier:
            # one fixed slot per (head, block); pinned memory is addressable from the device
            self.host_k = torch.zeros(num_heads * max_blocks, page_tokens, head_dim, dtype=dtype, pin_memory=True)
            self.host_v = torch.zeros(num_heads * max_blocks, page_tokens, head_dim, dtype=dtype, pin_memory=True)
        # LRU statistics kept on the device (MMCache's hit / miss counters, models/cache.py:156-163,
        # 713-716): [0] selected blocks found resident, [1] selected blocks that had no page,
        # [2] pages evicted, [3] pages fetched back from the host tier
        self.counters = torch.zeros(4, dtype=torch.int64, device=dev)
        self.n_tokens = 0
        self.epoch = 0
        self._evicted_any = False
        self.page_bytes = page_tokens * head_dim * self.k_pool.element_size()
        self._dtype_code = ops._dtype(self.k_pool)
        self.write_behind = bool(write_behind) and host_tier
        self._stage_k = self._stage_v = self._stage_keys = None
        self._drain_event = None                 # recorded behind the last copy from the staging buffer to the host

    # ------------------------------------------------------------------------------ helpers
    @property
    def n_blocks(self) -> int:
        return -(-self.n_tokens // self.page_tokens)

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def pooled_keys(self) -> torch.Tensor:
        """[1, n_blocks, H, D] view of the pooled keys (the top-k's `k` argument)."""
        return self.k_pooled[:, : self.n_blocks].permute(1, 0, 2).unsqueeze(0)

    def pooled_values(self) -> torch.Tensor:
        return self.v_pooled[:, : self.n_blocks].permute(1, 0, 2).unsqueeze(0)

    def kv_source(self) -> ops.PagedKV:
        return ops.PagedKV(self.k_pool, self.v_pool, self.block_table, self.n_tokens, self.page_tokens)

    def check_status(self) -> None:
        """Synchronising read of the device status word; raises if a kernel reported a problem."""
        st = int(self.status.item())
        if st != 0:
            self.status.zero_()
            raise NSABackendError(f"block cache: device status {st} (page pool exhausted)")

    def stats(self) -> dict:
        """Synchronising read of the LRU counters (the role of MMCache.lru_hit_rate_overall,
        models/cache.py:713-716): hits and misses count unique selected (head, block) pairs per
        `touch`; bytes moved are whole pages, K and V."""
        hits, misses, evicted, fetched = (int(x) for x in self.counters.tolist())
        total = hits + misses
        return {"hits": hits, "misses": misses, "hit_rate": hits / total if total else 0.0,
                "pages_evicted": evicted, "pages_fetched": fetched,
                "bytes_to_host": evicted * 2 * self.page_bytes if self.host_k is not None else 0,
                "bytes_from_host": fetched * 2 * self.page_bytes}

    def _select_victims(self, n: int, n_dev: Optional[torch.Tensor], cap: int, protect_from: Optional[int] = None
                        ) -> torch.Tensor:
        victims = torch.full((max(cap, 1),), -1, dtype=torch.int32, device=self.device)
        if protect_from is None:
            protect_from = max(self.n_blocks - self.protect_blocks, 0)
        call("nsa_cache_select_victims", self.page_owner.data_ptr(), self.page_stamp.data_ptr(), self.num_pages,
             self.max_blocks, protect_from, self.epoch, n, None if n_dev is None else n_dev.data_ptr(), cap,
             victims.data_ptr(), self.status.data_ptr(), self._stream())
        return victims

    def _move(self, direction: int, pages, keys, n: int, n_dev, cap: int) -> None:
        call("nsa_cache_move_pages", direction, pages.data_ptr(), None if keys is None else keys.data_ptr(), n,
             None if n_dev is None else n_dev.data_ptr(), cap, self.k_pool.data_ptr(), self.v_pool.data_ptr(),
             self.page_bytes, None if self.host_k is None else self.host_k.data_ptr(),
             None if self.host_v is None else self.host_v.data_ptr(), self.block_table.data_ptr(),
             self.page_owner.data_ptr(), self.page_stamp.data_ptr(), self.epoch, self.counters.data_ptr(),
             self._stream())

    def _wait_drain(self) -> None:
        """Order the current stream behind the last write-behind copy (before the staging buffer is
        reused and before anything reads the host tier)."""
        if self._drain_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self._drain_event)
            self._drain_event = None

    def _evict_write_behind(self, pages: torch.Tensor, n: int) -> None:
        """Evict `n` listed pages (free ones pass through): to the staging buffer now, to the host
        tier on the drain stream."""
        self._wait_drain()
        if self._stage_keys is None or self._stage_keys.numel() < n:
            self._stage_k = torch.empty(n, self.page_tokens, self.D, dtype=self.dtype, device=self.device)
            self._stage_v = torch.empty_like(self._stage_k)
            self._stage_keys = torch.empty(n, dtype=torch.int32, device=self.device)
        cur = torch.cuda.current_stream(self.device)
        call("nsa_cache_move_pages", 2, pages.data_ptr(), self._stage_keys.data_ptr(), n, None, n,
             self.k_pool.data_ptr(), self.v_pool.data_ptr(), self.page_bytes, self._stage_k.data_ptr(),
             self._stage_v.data_ptr(), self.block_table.data_ptr(), self.page_owner.data_ptr(),
             self.page_stamp.data_ptr(), self.epoch, self.counters.data_ptr(), cur.cuda_stream)
        side = BlockKVCache._drain_streams.get(self.device.index)
        if side is None:
            side = BlockKVCache._drain_streams[self.device.index] = torch.cuda.Stream(self.device)
        staged = torch.cuda.Event()
        staged.record(cur)
        side.wait_event(staged)
        call("nsa_cache_move_pages", 3, None, self._stage_keys.data_ptr(), n, None, n,
             self._stage_k.data_ptr(), self._stage_v.data_ptr(), self.page_bytes, self.host_k.data_ptr(),
             self.host_v.data_ptr(), None, None, None, 0, None, side.cuda_stream)
        self._drain_event = torch.cuda.Event()
        self._drain_event.record(side)

    def _make_resident(self, ids: torch.Tensor, T: int, count: bool, protect_from: Optional[int] = None):
        """Stamp the pages of the listed blocks with the current epoch and bring the ones that have
        no page back from the host tier, evicting (free pages first, then least recently used)
        to make room - all on the device.  ids: flat int32 in [.., H, T] order."""
        cap = min(ids.numel(), self.H * self.max_blocks)
        uniq = torch.empty(1 + cap, dtype=torch.int32, device=self.device)
        miss = torch.empty(1 + cap, dtype=torch.int32, device=self.device)
        wsb = _lib.load().nsa_cache_dedup_workspace_bytes(self.H * self.max_blocks)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=self.device)
        call("nsa_cache_dedup_touch", ids.data_ptr(), ids.numel(), self.H, T, self.max_blocks, self.max_blocks,
             self._stamp32.data_ptr(), self.epoch, self.block_table.data_ptr(), self.page_stamp.data_ptr(),
             self.epoch, uniq.data_ptr(), miss.data_ptr(), cap, self.counters.data_ptr() if count else None,
             ws.data_ptr(), wsb, self._stream())
        if self._evicted_any and self.host_k is not None:
            self._wait_drain()                   # a missing block may still be on its way to the host tier
            n_dev = miss[:1]
            victims = self._select_victims(0, n_dev, cap, protect_from)
            self._move(0, victims, None, 0, n_dev, cap)
            self._move(1, victims, miss, 0, n_dev, cap)
        return uniq, miss

    # ------------------------------------------------------------------------------- append
    def append(self, k_new: torch.Tensor, v_new: torch.Tensor, pos0: Optional[int] = None,
               rope: Optional["RopeSpec"] = None) -> None:
        """Write k_new / v_new [S,H,D] at token position pos0 (default: the end).  Re-writing
        existing positions is allowed (each denoising step of a chunk overwrites the chunk).
        With `rope` the keys are given WITHOUT their rotary embedding and receive it on the way
        into the pages (causal_reorder_rope_apply, causal_wan_nsa_model.py:72-105).

        Blocks the call touches are never chosen as victims for the pages it needs, and a touched
        block that was evicted earlier comes back from the host tier before it is rewritten, so a
        rewrite that covers part of a block keeps the rest of it."""
        S = k_new.shape[0]
        if S == 0:
            return
        pos0 = self.n_tokens if pos0 is None else int(pos0)
        if pos0 > self.n_tokens:
            raise NSABackendError(f"append at {pos0} would leave a gap after {self.n_tokens} tokens")
        k_new, v_new = ops._rows16(k_new), ops._rows16(v_new)
        if v_new.stride() != k_new.stride():
            v_new = v_new.contiguous()
            k_new = k_new.contiguous()
        first, last = pos0 // self.page_tokens, (pos0 + S - 1) // self.page_tokens
        if last >= self.max_blocks:
            raise NSABackendError(f"token {pos0 + S - 1} is past the block table ({self.max_blocks} blocks)")
        n_touched = last - first + 1
        n_new = max(0, last + 1 - self.n_blocks)            # blocks that have never had a page
        n_exist = n_touched - n_new                         # touched blocks that were appended before
        self.epoch += 1
        # pages for this call may only come from blocks in front of the ones it touches
        protect_from = max(min(first, self.n_blocks - self.protect_blocks), 0)
        with torch.cuda.device(self.device):
            if n_exist and self._evicted_any:
                if self.host_k is None:
                    raise NSABackendError("rewriting blocks after evictions needs the host tier (a dropped block "
                                          "cannot be completed again)")
                ids = torch.arange(first, first + n_exist, dtype=torch.int32, device=self.device).repeat_interleave(self.H)
                self._make_resident(ids, 1, count=False, protect_from=protect_from)
            new_pages = torch.full((self.H, n_touched), -1, dtype=torch.int32, device=self.device)
            need = n_new * self.H
            if need:
                pages = self._select_victims(need, None, need, protect_from)
                if self.write_behind:
                    self._evict_write_behind(pages, need)             # free pages pass through untouched
                else:
                    self._move(0, pages, None, need, None, need)
                new_pages[:, n_exist:] = pages.view(self.H, n_new)
                if self.n_blocks * self.H + need > self.num_pages:
                    self._evicted_any = True
            args = (k_new.data_ptr(), v_new.data_ptr(),
                    (C.c_int64 * 3)(k_new.stride(0), k_new.stride(1), 0), S, pos0, self.n_tokens, self.H, self.D,
                    self.k_pool.data_ptr(), self.v_pool.data_ptr(), self.page_tokens, self.block_table.data_ptr(),
                    self.max_blocks, new_pages.data_ptr(), n_touched, self.page_owner.data_ptr(),
                    self.page_stamp.data_ptr(), self.epoch, self.k_pooled.data_ptr(), self.v_pooled.data_ptr(),
                    self.status.data_ptr(), self._dtype_code)
            if rope is None:
                call("nsa_cache_append", *args, self._stream())
            else:
                spec = rope.struct(self.device, self.D)
                call("nsa_cache_append_rope", *args, C.byref(spec), self._stream())
        self.n_tokens = max(self.n_tokens, pos0 + S)

    # ------------------------------------------------------------------- selection residency
    def touch(self, block_indices: torch.Tensor, return_lists: bool = False):
        """LRU-touch the selected blocks and make the missing ones resident (evicting the least
        recently used pages to make room) - all on the device.  block_indices int32 [1,MG,H,T]."""
        ids = block_indices.contiguous().view(-1)
        T = block_indices.shape[-1]
        self.epoch += 1
        with torch.cuda.device(self.device):
            uniq, miss = self._make_resident(ids, T, count=True)
        return (uniq, miss) if return_lists else None

    def evict_all(self) -> None:
        """Move every resident page to the host tier and free it (the block cache's form of
        MMCache.flush_offload with nothing protected, models/cache.py:1032-1142)."""
        if self.host_k is None:
            raise NSABackendError("evict_all needs the host tier")
        with torch.cuda.device(self.device):
            self._wait_drain()
            pages = torch.arange(self.num_pages, dtype=torch.int32, device=self.device)
            self._move(0, pages, None, self.num_pages, None, self.num_pages)
        self._evicted_any = True

    def selection_attention(self, q: torch.Tensor, block_indices: torch.Tensor, scale: Optional[float] = None,
                            group_size: int = 64, return_lse: bool = False):
        """Selection attention of q [1,M,H,D] over the selected blocks of this cache (the role of
        selection_attention_block_store, padded_ptr/block_wrapper.py:15-89)."""
        if q.shape[0] != 1:
            raise NSABackendError("the block cache serves batch size 1")
        self.touch(block_indices)
        sc = q.shape[-1] ** -0.5 if scale is None else scale
        out, lse = ops.sel_fwd(q, self.kv_source(), block_indices, self.page_tokens, 1, sc, False, group_size)
        return (out, lse) if return_lse else out

    def reset(self) -> None:
        self._wait_drain()
        self.block_table.fill_(-1)
        self.page_owner.fill_(-1)
        self.page_stamp.zero_()
        self._stamp32.zero_()
        self.status.zero_()
        self.counters.zero_()
        self.n_tokens = 0
        self.epoch = 0
        self._evicted_any = False


class BlockKVStore:
    """One BlockKVCache per transformer layer: the block-level store that the reference's
    selection_attention_block_store expects behind ``kv_cache.block_store``
    (padded_ptr/block_wrapper.py:51-85) and that its repository does not ship."""

    def __init__(self, num_layers: int, num_heads: int, head_dim: int, num_pages: int, max_blocks: int,
                 page_tokens: int = 64, dtype: torch.dtype = torch.bfloat16, device="cuda", host_tier: bool = True,
                 protect_blocks: int = 0):
        self.layers = [BlockKVCache(num_heads, head_dim, num_pages, max_blocks, page_tokens, dtype, device, host_tier,
                                    protect_blocks) for _ in range(num_layers)]
        self.block_tokens, self.head_dim, self.num_heads = page_tokens, head_dim, num_heads

    @property
    def block_store(self):
        return self

    def layer(self, layer_idx: int) -> BlockKVCache:
        return self.layers[layer_idx]

    def reset(self) -> None:
        for c in self.layers:
            c.reset()

    def stats(self) -> dict:
        total = {}
        for c in self.layers:
            for k, v in c.stats().items():
                if k != "hit_rate":
                    total[k] = total.get(k, 0) + v
        n = total.get("hits", 0) + total.get("misses", 0)
        total["hit_rate"] = total.get("hits", 0) / n if n else 0.0
        return total
