// Fixed-page block KV cache kernels: append (+ pooled key/value refresh), selected-block
// dedup + LRU touch, LRU victim selection, evict / fetch page moves with publish-after-copy,
// and the reference's three block-KV entry points.  All byte / integer work, 16-byte
// vectorised, no host synchronisation: data-dependent counts stay on the device.
#include "common.cuh"

namespace nsa {
namespace {

__device__ __forceinline__ void copy16(char* dst, const char* src, int64_t bytes) {
  for (int64_t i = static_cast<int64_t>(threadIdx.x) * 16; i < bytes; i += static_cast<int64_t>(blockDim.x) * 16)
    *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
}

// ------------------------------------------------------------------------------------ append
struct AppendParams {
  const char* k_new; const char* v_new;
  int64_t s_stride, h_stride;      // elements
  int64_t S, pos0;
  int64_t n_tokens_before;         // tokens the cache held before this call (a rewrite may end before them)
  int H, D, page_tokens, max_blocks, n_touched;
  int hc;                          // heads per thread block of the append kernel
  char* k_pool; char* v_pool;
  int32_t* block_table; const int32_t* new_pages;
  int32_t* page_owner; int64_t* page_stamp; int64_t epoch;
  char* k_pooled; char* v_pooled;
  int32_t* status;
  // optional rotary embedding of the new keys (causal_reorder_rope_apply,
  // models/transformers/causal_wan_nsa_model.py:72-105): token t of the chunk, in the reordered
  // order (f h w fs hs ws), sits at frame / row / column (fr, hr, wr) of the chunk's latent grid;
  // complex pair j of a head takes its factor from the frame table (j < c_f, row start_frame + fr),
  // the row table (next c_h pairs) or the column table (last c_w pairs); products in float64.
  const double2* rope_f; const double2* rope_h; const double2* rope_w;
  int c_f, c_h, c_w;
  int grid_h, grid_w, pool_f, pool_h, pool_w, start_frame;
};

// frame / row / column of token t of a chunk stored in (f h w fs hs ws) order
template <typename I>
__device__ __forceinline__ void rope_position_t(const AppendParams& p, I t, int& fr, int& hr, int& wr) {
  const I pw = static_cast<I>(p.pool_w), ph = static_cast<I>(p.pool_h), pf = static_cast<I>(p.pool_f);
  const int ws = static_cast<int>(t % pw); t /= pw;
  const int hs = static_cast<int>(t % ph); t /= ph;
  const int fs = static_cast<int>(t % pf); t /= pf;
  const I wq = static_cast<I>(p.grid_w / p.pool_w), hq = static_cast<I>(p.grid_h / p.pool_h);
  const int wo = static_cast<int>(t % wq); t /= wq;
  const int ho = static_cast<int>(t % hq); t /= hq;
  fr = static_cast<int>(t) * p.pool_f + fs;
  hr = ho * p.pool_h + hs;
  wr = wo * p.pool_w + ws;
}
// (five divisions per call: in 32 bits whenever the token index allows, a 64-bit division costs
// several times as many instructions and this runs once per row and thread)
__device__ __forceinline__ void rope_position(const AppendParams& p, int64_t t, int& fr, int& hr, int& wr) {
  if (static_cast<uint64_t>(t) <= 0xffffffffull) rope_position_t<uint32_t>(p, static_cast<uint32_t>(t), fr, hr, wr);
  else rope_position_t<int64_t>(p, t, fr, hr, wr);
}

// One thread block per (touched block, group of `hc` neighbouring heads).  A thread owns one 16-byte
// column piece of one head and one eighth of the block's rows, so that the block reads CONTIGUOUS
// pieces of the [S, H, D] source rows (hc x D elements each) and writes whole page rows; reading one
// head's 256 bytes out of every source row left the DRAM pages half used.  The pooled key / value of
// a block written as a whole come from the rows on their way through the registers; a block the call
// covers only in part is read back from its page.  Sums are fp32: the rows of a part in ascending
// order, then the eight parts in order.
constexpr int kAppendSlices = 8;
constexpr int kRopeRows = 128;              // page sizes up to this keep their rows' positions in shared memory

template <typename T, bool ROPE>
__global__ void __launch_bounds__(768) cache_append_kernel(const AppendParams p) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int UNROLL = ROPE ? 2 : 4;
  extern __shared__ float s_part[];          // [slices][hc][2][D] partial sums of K and V
  __shared__ int s_page[64];
  __shared__ int s_pos[ROPE ? 3 * kRopeRows : 1];   // ROPE: frame / row / column of each row of the block
  chain_release();
  chain_wait();
  const int cpr = p.D / VEC;
  const int j = blockIdx.x;
  const int h0 = blockIdx.y * p.hc;
  const int nh = p.H - h0 < p.hc ? p.H - h0 : p.hc;
  const int per_slice = p.hc * cpr;
  const int slice = threadIdx.x / per_slice, rem = threadIdx.x % per_slice;
  const int hl = rem / cpr, col = rem % cpr;
  const bool live = hl < nh;
  const int h = h0 + hl;
  const int64_t first_block = p.pos0 / p.page_tokens;
  const int64_t bid = first_block + j;
  const int64_t key = static_cast<int64_t>(h) * p.max_blocks + bid;
  if (live && slice == 0 && col == 0) {
    int page = p.block_table[key];
    if (page < 0) {
      page = p.new_pages ? p.new_pages[static_cast<int64_t>(h) * p.n_touched + j] : -1;
      if (page >= 0) {
        p.block_table[key] = page;
        p.page_owner[page] = static_cast<int32_t>(key);
      } else {
        atomicExch(p.status, NSA_ERR_EXHAUSTED);
      }
    }
    if (page >= 0) p.page_stamp[page] = p.epoch;
    s_page[hl] = page;
  }
  // ROPE: what a pair of a thread's piece is multiplied with depends on the row's position and on the
  // pair's index alone, so the table, its row length and the coordinate that indexes it are chosen once
  // per thread (a warp's threads sit in different tables: choosing inside the row loop diverged), and
  // the positions of the block's rows are worked out once per thread block
  const double2* tb[VEC / 2];
  int tb_len[VEC / 2], tb_sel[VEC / 2];
  if (ROPE) {
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      const int jj = col * (VEC / 2) + i;                  // complex pair of the head
      if (jj < p.c_f) { tb[i] = p.rope_f + static_cast<int64_t>(p.start_frame) * p.c_f + jj; tb_len[i] = p.c_f; tb_sel[i] = 0; }
      else if (jj < p.c_f + p.c_h) { tb[i] = p.rope_h + (jj - p.c_f); tb_len[i] = p.c_h; tb_sel[i] = 1; }
      else { tb[i] = p.rope_w + (jj - p.c_f - p.c_h); tb_len[i] = p.c_w; tb_sel[i] = 2; }
    }
    if (p.page_tokens <= kRopeRows) {
      const int64_t t0 = bid * p.page_tokens - p.pos0;     // chunk-local index of the block's first row (may be < 0)
      for (int r = threadIdx.x; r < p.page_tokens; r += blockDim.x) {
        int fr = 0, hr = 0, wr = 0;
        if (t0 + r >= 0 && t0 + r < p.S) rope_position(p, t0 + r, fr, hr, wr);
        s_pos[r] = fr; s_pos[kRopeRows + r] = hr; s_pos[2 * kRopeRows + r] = wr;
      }
    }
  }
  __syncthreads();
  const int page = live ? s_page[hl] : -1;
  const int64_t blk0 = bid * p.page_tokens;
  const int64_t lo = max(p.pos0, blk0), hi = min(p.pos0 + p.S, blk0 + p.page_tokens);
  const int64_t held = min(p.n_tokens_before, blk0 + p.page_tokens);
  const int n_present = static_cast<int>(max(hi, held) - blk0);   // rows the block holds after this call
  const int row_lo = static_cast<int>(lo - blk0), row_hi = static_cast<int>(hi - blk0);
  const bool whole = row_lo == 0 && row_hi == n_present;
  const int rows_per_slice = (p.page_tokens + kAppendSlices - 1) / kAppendSlices;
  const int s_begin = slice * rows_per_slice, s_end = min(s_begin + rows_per_slice, p.page_tokens);
  const int64_t row_bytes = static_cast<int64_t>(p.D) * sizeof(T);
  float ak[VEC], av[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) ak[i] = av[i] = 0.f;
  if (page >= 0) {
    char* kp = p.k_pool + static_cast<int64_t>(page) * p.page_tokens * row_bytes + col * 16;
    char* vp = p.v_pool + static_cast<int64_t>(page) * p.page_tokens * row_bytes + col * 16;
    // ---- copy the rows of this thread's part that the call writes
    const int c_begin = max(s_begin, row_lo), c_end = min(s_end, row_hi);
    const int64_t src_row = p.s_stride * sizeof(T);
    const char* ksrc = p.k_new + ((blk0 - p.pos0) * p.s_stride + h * p.h_stride) * sizeof(T) + col * 16;
    const char* vsrc = p.v_new + ((blk0 - p.pos0) * p.s_stride + h * p.h_stride) * sizeof(T) + col * 16;
    for (int rb = c_begin; rb < c_end; rb += UNROLL) {
      uint4 kq[UNROLL], vq[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {                 // all loads of the batch first
        if (rb + u < c_end) {
          kq[u] = *reinterpret_cast<const uint4*>(ksrc + (rb + u) * src_row);
          vq[u] = *reinterpret_cast<const uint4*>(vsrc + (rb + u) * src_row);
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int r = rb + u;
        if (r >= c_end) continue;
        if (ROPE) {
          int pos[3];
          if (p.page_tokens <= kRopeRows) { pos[0] = s_pos[r]; pos[1] = s_pos[kRopeRows + r]; pos[2] = s_pos[2 * kRopeRows + r]; }
          else rope_position(p, blk0 - p.pos0 + r, pos[0], pos[1], pos[2]);
          T* e = reinterpret_cast<T*>(&kq[u]);
#pragma unroll
          for (int i = 0; i < VEC / 2; ++i) {
            const int at = tb_sel[i] == 0 ? pos[0] : tb_sel[i] == 1 ? pos[1] : pos[2];
            const double2 w = tb[i][static_cast<int64_t>(at) * tb_len[i]];
            const double xr = static_cast<double>(to_f32<T>(e[2 * i])), xi = static_cast<double>(to_f32<T>(e[2 * i + 1]));
            // float64 product, then float64 -> float32 -> T, as view_as_real(...).type_as(x) does
            e[2 * i] = from_f32<T>(static_cast<float>(xr * w.x - xi * w.y));
            e[2 * i + 1] = from_f32<T>(static_cast<float>(xr * w.y + xi * w.x));
          }
        }
        *reinterpret_cast<uint4*>(kp + r * row_bytes) = kq[u];
        *reinterpret_cast<uint4*>(vp + r * row_bytes) = vq[u];
        if (whole) {
          const T* ea = reinterpret_cast<const T*>(&kq[u]);
          const T* eb = reinterpret_cast<const T*>(&vq[u]);
#pragma unroll
          for (int i = 0; i < VEC; ++i) { ak[i] += to_f32<T>(ea[i]); av[i] += to_f32<T>(eb[i]); }
        }
      }
    }
  }
  if (!whole) {
    // pooled key / value over the rows the block now holds, [0, n_present): a rewrite that covers
    // part of the block leaves the other rows in place, so read the page back (the rows this thread
    // block just wrote are visible to it after the barrier)
    __syncthreads();
    if (page >= 0) {
      const char* kp = p.k_pool + static_cast<int64_t>(page) * p.page_tokens * row_bytes + col * 16;
      const char* vp = p.v_pool + static_cast<int64_t>(page) * p.page_tokens * row_bytes + col * 16;
      for (int r = s_begin; r < min(s_end, n_present); ++r) {
        const uint4 a = *reinterpret_cast<const uint4*>(kp + r * row_bytes);
        const uint4 b = *reinterpret_cast<const uint4*>(vp + r * row_bytes);
        const T* ea = reinterpret_cast<const T*>(&a);
        const T* eb = reinterpret_cast<const T*>(&b);
#pragma unroll
        for (int i = 0; i < VEC; ++i) { ak[i] += to_f32<T>(ea[i]); av[i] += to_f32<T>(eb[i]); }
      }
    }
  }
  if (slice < kAppendSlices) {
    float* mine = s_part + (static_cast<int64_t>(slice) * p.hc + hl) * 2 * p.D + col * VEC;
#pragma unroll
    for (int i = 0; i < VEC; ++i) { mine[i] = ak[i]; mine[p.D + i] = av[i]; }
  }
  __syncthreads();
  if (slice == 0 && page >= 0) {
    const float inv = 1.f / static_cast<float>(n_present);
    uint4 ok, ov;
    T* ek = reinterpret_cast<T*>(&ok);
    T* ev = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float sk = 0.f, sv = 0.f;
      for (int sl = 0; sl < kAppendSlices; ++sl) {
        const float* part = s_part + (static_cast<int64_t>(sl) * p.hc + hl) * 2 * p.D + col * VEC;
        sk += part[i];
        sv += part[p.D + i];
      }
      ek[i] = from_f32<T>(sk * inv);
      ev[i] = from_f32<T>(sv * inv);
    }
    *reinterpret_cast<uint4*>(p.k_pooled + key * row_bytes + col * 16) = ok;
    if (p.v_pooled) *reinterpret_cast<uint4*>(p.v_pooled + key * row_bytes + col * 16) = ov;
  }
}

// Rotary embedding of a chunk of QUERIES (same rule and rounding as the keys above): one thread per
// 16-byte piece of a row, x [S,H,D] by stride -> out [S,H,D] contiguous.
template <typename T>
__global__ void __launch_bounds__(256) rope_apply_kernel(const AppendParams p, char* __restrict__ out) {
  constexpr int VEC = 16 / sizeof(T);
  const int cpr = p.D / VEC;
  const int64_t total = p.S * p.H * cpr;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int cc, h;
    int64_t t;
    if (total <= 0xffffffffll) {
      const uint32_t i32 = static_cast<uint32_t>(i), sh = i32 / static_cast<uint32_t>(cpr);
      cc = static_cast<int>(i32 - sh * static_cast<uint32_t>(cpr));
      const uint32_t t32 = sh / static_cast<uint32_t>(p.H);
      h = static_cast<int>(sh - t32 * static_cast<uint32_t>(p.H));
      t = t32;
    } else {
      cc = static_cast<int>(i % cpr);
      const int64_t sh = i / cpr;
      h = static_cast<int>(sh % p.H);
      t = sh / p.H;
    }
    uint4 q = *reinterpret_cast<const uint4*>(p.k_new + (t * p.s_stride + h * p.h_stride) * sizeof(T) + cc * 16);
    int fr, hr, wr;
    rope_position(p, t, fr, hr, wr);
    T* e = reinterpret_cast<T*>(&q);
#pragma unroll
    for (int k = 0; k < VEC / 2; ++k) {
      const int j = cc * (VEC / 2) + k;
      // one load through a selected table instead of three branches: a warp's threads sit in different tables
      const bool in_f = j < p.c_f, in_h = j < p.c_f + p.c_h;
      const double2* tbp = in_f ? p.rope_f + j : in_h ? p.rope_h + (j - p.c_f) : p.rope_w + (j - p.c_f - p.c_h);
      const int len = in_f ? p.c_f : in_h ? p.c_h : p.c_w;
      const int at = in_f ? p.start_frame + fr : in_h ? hr : wr;
      const double2 w = tbp[static_cast<int64_t>(at) * len];
      const double xr = static_cast<double>(to_f32<T>(e[2 * k])), xi = static_cast<double>(to_f32<T>(e[2 * k + 1]));
      e[2 * k] = from_f32<T>(static_cast<float>(xr * w.x - xi * w.y));
      e[2 * k + 1] = from_f32<T>(static_cast<float>(xr * w.y + xi * w.x));
    }
    *reinterpret_cast<uint4*>(out + ((t * p.H + h) * static_cast<int64_t>(p.D)) * sizeof(T) + cc * 16) = q;
  }
}

// ------------------------------------------------------------------------ dedup + LRU touch
constexpr int kTileKeys = 1024;

// key of (head h, block bid) = (cid*H + h)*bpc + loc with cid = bid / bpc, loc = bid % bpc; with
// bpc == max_blocks this is h*max_blocks + bid, the index into the [H][max_blocks] block table.
__global__ void dedup_mark_kernel(const int32_t* __restrict__ ids, int64_t n_entries, int H, int T,
                                  int max_blocks, int bpc, int32_t* __restrict__ stamp, int32_t epoch) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_entries) return;
  const int32_t bid = ids[i];
  if (bid < 0 || bid >= max_blocks) return;
  const int h = static_cast<int>((i / T) % H);
  const int cid = bid / bpc, loc = bid - cid * bpc;
  stamp[(static_cast<int64_t>(cid) * H + h) * bpc + loc] = epoch;   // idempotent store
}

// counts[2*tile] = keys marked this epoch, counts[2*tile+1] = marked keys with no page
__global__ void __launch_bounds__(kTileKeys) dedup_count_kernel(const int32_t* __restrict__ stamp, int32_t epoch,
                                                                const int32_t* __restrict__ table, int64_t n_keys,
                                                                int32_t* __restrict__ counts) {
  const int64_t key = static_cast<int64_t>(blockIdx.x) * kTileKeys + threadIdx.x;
  const bool hit = key < n_keys && stamp[key] == epoch;
  const bool miss = hit && table && table[key] < 0;
  const int a = __syncthreads_count(hit);
  const int b = __syncthreads_count(miss);
  if (threadIdx.x == 0) { counts[2 * blockIdx.x] = a; counts[2 * blockIdx.x + 1] = b; }
}

// single block: exclusive scan of the tile counts; writes totals to out_unique[0] / out_missing[0]
// counters (may be null): [0] += unique blocks found resident (hits), [1] += unique blocks without
// a page (misses) - the device form of the hit / miss counts of MMCache.lru_touch_per_head
// (models/cache.py:156-163, 673-699)
__global__ void dedup_scan_kernel(int32_t* __restrict__ counts, int n_tiles, int32_t* out_unique,
                                  int32_t* out_missing, int64_t* counters) {
  if (threadIdx.x != 0) return;
  int a = 0, b = 0;
  for (int t = 0; t < n_tiles; ++t) {
    const int ca = counts[2 * t], cb = counts[2 * t + 1];
    counts[2 * t] = a; counts[2 * t + 1] = b;
    a += ca; b += cb;
  }
  out_unique[0] = a;
  if (out_missing) out_missing[0] = b;
  if (counters) { counters[0] += a - b; counters[1] += b; }
}

__global__ void __launch_bounds__(kTileKeys) dedup_compact_kernel(
    const int32_t* __restrict__ stamp, int32_t epoch, const int32_t* __restrict__ table, int64_t n_keys,
    const int32_t* __restrict__ offsets, int64_t* __restrict__ page_stamp, int64_t epoch64,
    int32_t* __restrict__ out_unique, int32_t* __restrict__ out_missing, int cap) {
  __shared__ int s_warp[2][32];
  const int64_t key = static_cast<int64_t>(blockIdx.x) * kTileKeys + threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool hit = key < n_keys && stamp[key] == epoch;
  const int page = (hit && table) ? table[key] : 0;
  const bool miss = hit && page < 0;
  if (hit && table && page >= 0 && page_stamp) page_stamp[page] = epoch64;       // LRU touch
  const unsigned mh = __ballot_sync(0xffffffffu, hit), mm = __ballot_sync(0xffffffffu, miss);
  if (lane == 0) { s_warp[0][warp] = __popc(mh); s_warp[1][warp] = __popc(mm); }
  __syncthreads();
  int ph = offsets[2 * blockIdx.x], pm = offsets[2 * blockIdx.x + 1];
  for (int w = 0; w < warp; ++w) { ph += s_warp[0][w]; pm += s_warp[1][w]; }
  ph += __popc(mh & ((1u << lane) - 1));
  pm += __popc(mm & ((1u << lane) - 1));
  if (hit && ph < cap) out_unique[1 + ph] = static_cast<int32_t>(key);
  if (miss && out_missing && pm < cap) out_missing[1 + pm] = static_cast<int32_t>(key);
}

// ------------------------------------------------------------------------- victim selection
// Single block.  Picks n pages to (re)use: free pages first (owner < 0, ascending page id), then
// the least recently used owned pages: owner's block id below protect_from_bid, stamp < epoch (not
// touched by the current call), order (stamp, page) ascending.
__global__ void __launch_bounds__(1024) select_victims_kernel(
    const int32_t* __restrict__ page_owner, const int64_t* __restrict__ page_stamp, int num_pages,
    int max_blocks, int protect_from_bid, int64_t epoch, int n_host, const int32_t* __restrict__ n_dev,
    int cap, int32_t* __restrict__ victims, int32_t* status) {
  __shared__ unsigned long long s_red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int n = n_dev ? *n_dev : n_host;
  if (n > cap) n = cap;
  auto key_at = [&](int pg) -> unsigned long long {
    const int owner = page_owner[pg];
    if (owner < 0) return static_cast<unsigned long long>(pg);        // free: before every owned page
    if (owner % max_blocks >= protect_from_bid) return ~0ull;
    const int64_t st = page_stamp[pg];
    if (st >= epoch) return ~0ull;
    return (static_cast<unsigned long long>(st + 1) << 24) | static_cast<unsigned>(pg);
  };
  auto scan_above = [&](unsigned long long bound, bool any) {
    unsigned long long best = ~0ull;
    for (int pg = threadIdx.x; pg < num_pages; pg += blockDim.x) {
      const unsigned long long k = key_at(pg);
      if ((any || k > bound) && k < best) best = k;
    }
    return best;
  };
  unsigned long long local = scan_above(0ull, true);
  for (int r = 0; r < n; ++r) {
    unsigned long long best = local;
#pragma unroll
    for (int d = 16; d; d >>= 1) {
      const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, d);
      best = o < best ? o : best;
    }
    if (lane == 0) s_red[warp] = best;
    __syncthreads();
    best = s_red[0];
    for (int w = 1; w < nw; ++w) best = s_red[w] < best ? s_red[w] : best;
    __syncthreads();
    if (best == ~0ull) {          // fewer evictable pages than requested
      if (threadIdx.x == 0) atomicExch(status, NSA_ERR_EXHAUSTED);
      for (int i = r + threadIdx.x; i < n; i += blockDim.x) victims[i] = -1;
      return;
    }
    if (threadIdx.x == 0) victims[r] = static_cast<int32_t>(best & 0xffffffu);
    if (local == best) local = scan_above(best, false);
  }
}

// The same selection without a rescan per victim.  The scan kernel above costs milliseconds when
// a new chunk needs a page for every (head, block) it brings (888 pages out of 14040 at a 48-frame
// cap); this one finds the n-th smallest key by radix selection (eight passes over the pool, one
// byte of the 64-bit key each, histogram in shared memory), gathers the n keys that do not exceed
// it into shared memory, sorts them there (bitonic) and writes them out in ascending order: tens
// of microseconds whatever n is.  n is limited by the shared-memory list to kSelectMax victims.
constexpr int kSelectMax = 16384;
constexpr int kBatch = 8;               // pages a thread examines per batch of loads

__device__ __forceinline__ unsigned long long victim_key_of(int owner, int64_t st, int pg, int max_blocks,
                                                            int protect_from_bid, int64_t epoch) {
  if (owner < 0) return static_cast<unsigned long long>(pg);           // free: before every owned page
  if (owner % max_blocks >= protect_from_bid) return ~0ull;
  if (st >= epoch) return ~0ull;
  return (static_cast<unsigned long long>(st + 1) << 24) | static_cast<unsigned>(pg);
}

// Keys of the kBatch pages pg0, pg0 + stride, ...: both arrays are read for every page, without a
// branch in between, so that the 2 x kBatch loads are in flight together.
__device__ __forceinline__ void victim_keys(const int32_t* __restrict__ page_owner, const int64_t* __restrict__ page_stamp,
                                            int pg0, int stride, int num_pages, int max_blocks, int protect_from_bid,
                                            int64_t epoch, unsigned long long* ks);

__device__ __forceinline__ void victim_keys(const int32_t* __restrict__ page_owner, const int64_t* __restrict__ page_stamp,
                                            int pg0, int stride, int num_pages, int max_blocks, int protect_from_bid,
                                            int64_t epoch, unsigned long long* ks) {
  int owner[kBatch];
  int64_t st[kBatch];
#pragma unroll
  for (int u = 0; u < kBatch; ++u) {
    const int pg = pg0 + u * stride;
    const int pc = pg < num_pages ? pg : 0;
    owner[u] = page_owner[pc];
    st[u] = page_stamp[pc];
  }
#pragma unroll
  for (int u = 0; u < kBatch; ++u) {
    const int pg = pg0 + u * stride;
    ks[u] = pg < num_pages ? victim_key_of(owner[u], st[u], pg, max_blocks, protect_from_bid, epoch) : ~0ull;
  }
}

// PPT > 0: a thread keeps the keys of its PPT pages (page = i * 1024 + thread) in registers, computed
// once; PPT == 0: any pool size, keys recomputed from the two arrays in every pass.  With one thread
// block the kernel is bound by the instructions one SM can issue, and the key (two loads, a modulo)
// costs five times what a pass does with it.
template <int PPT>
__global__ void __launch_bounds__(1024) select_victims_radix_kernel(
    const int32_t* __restrict__ page_owner, const int64_t* __restrict__ page_stamp, int num_pages,
    int max_blocks, int protect_from_bid, int64_t epoch, int n_host, const int32_t* __restrict__ n_dev,
    int cap, int32_t* __restrict__ victims, int32_t* status) {
  extern __shared__ unsigned long long s_list[];            // the selected keys, padded to a power of two
  __shared__ unsigned int s_hist[256];
  __shared__ unsigned long long s_prefix, s_or, s_and;
  __shared__ int s_remaining, s_count, s_total;
  constexpr int kKeep = PPT > 0 ? PPT : 1;
  int n = n_dev ? *n_dev : n_host;
  if (n > cap) n = cap;
  if (n > kSelectMax) n = kSelectMax;                       // the host sends larger requests to the scan kernel
  if (n <= 0) return;
  if (threadIdx.x == 0) { s_prefix = 0ull; s_remaining = n; s_count = 0; s_total = 0; s_or = 0ull; s_and = ~0ull; }
  __syncthreads();
  unsigned long long keep[kKeep];
  if (PPT > 0) {
#pragma unroll
    for (int b0 = 0; b0 < PPT; b0 += kBatch)
      victim_keys(page_owner, page_stamp, b0 * 1024 + threadIdx.x, 1024, num_pages, max_blocks, protect_from_bid, epoch,
                  keep + b0);
  }
  const int n_batches = PPT > 0 ? PPT / kBatch : (num_pages + kBatch * 1024 - 1) / (kBatch * 1024);
  // batch bt of this thread's keys (pages (bt * kBatch + u) * 1024 + thread)
  auto batch = [&](int bt, unsigned long long* ks) {
    if (PPT > 0) {
#pragma unroll
      for (int b0 = 0; b0 < PPT; b0 += kBatch)
        if (b0 == bt * kBatch) {
#pragma unroll
          for (int u = 0; u < kBatch; ++u) ks[u] = keep[b0 + u];
        }
    } else {
      victim_keys(page_owner, page_stamp, bt * kBatch * 1024 + threadIdx.x, 1024, num_pages, max_blocks, protect_from_bid,
                  epoch, ks);
    }
  };
  // ---- bytes on which every candidate key agrees need no pass (the free flag and the high bytes of
  // stamp and page id are alike for all of them: five or six of the eight): OR and AND of the keys
  {
    unsigned long long o = 0ull, a = ~0ull;
    int cnt = 0;
    for (int bt = 0; bt < n_batches; ++bt) {
      unsigned long long ks[kBatch];
      batch(bt, ks);
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (ks[u] != ~0ull) { o |= ks[u]; a &= ks[u]; ++cnt; }
    }
    const unsigned lo_o = __reduce_or_sync(0xffffffffu, static_cast<unsigned>(o)), hi_o = __reduce_or_sync(0xffffffffu, static_cast<unsigned>(o >> 32));
    const unsigned lo_a = __reduce_and_sync(0xffffffffu, static_cast<unsigned>(a)), hi_a = __reduce_and_sync(0xffffffffu, static_cast<unsigned>(a >> 32));
    cnt = __reduce_add_sync(0xffffffffu, cnt);
    if ((threadIdx.x & 31) == 0) {
      atomicOr(&s_or, (static_cast<unsigned long long>(hi_o) << 32) | lo_o);
      atomicAnd(&s_and, (static_cast<unsigned long long>(hi_a) << 32) | lo_a);
      atomicAdd(&s_total, cnt);
    }
    __syncthreads();
  }
  const unsigned long long all_or = s_or, differs = s_or ^ s_and;
  const bool enough = s_total >= n;                         // else every candidate is taken and no digit matters
  // ---- the n-th smallest key, one byte at a time from the top
  for (int byte = 7; byte >= 0 && enough; --byte) {
    if (((differs >> (8 * byte)) & 255ull) == 0ull) {       // block-uniform
      if (threadIdx.x == 0) s_prefix = (s_prefix << 8) | ((all_or >> (8 * byte)) & 255ull);
      __syncthreads();
      continue;
    }
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_hist[i] = 0u;
    __syncthreads();
    const unsigned long long prefix = s_prefix;
    for (int bt = 0; bt < n_batches; ++bt) {                // block-uniform trip count
      unsigned long long ks[kBatch];
      batch(bt, ks);
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        // one shared-memory atomic per distinct digit of the warp, not per page: the high bytes of the
        // keys are all alike, and a warp's 32 increments of one counter would run one after the other
        const unsigned long long k = ks[u];
        const bool in = k != ~0ull && (byte == 7 || (k >> (8 * (byte + 1))) == prefix);
        const unsigned digit = in ? static_cast<unsigned>((k >> (8 * byte)) & 255u) : 256u;
        const unsigned peers = __match_any_sync(0xffffffffu, digit);
        if (in && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&s_hist[digit], static_cast<unsigned>(__popc(peers)));
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // the first digit at which the running count reaches what is still wanted: lane l owns bins
      // 8l .. 8l+7, a warp scan gives the counts in front of each lane
      const int lane = threadIdx.x;
      unsigned int bins[8], mine = 0u;
#pragma unroll
      for (int i = 0; i < 8; ++i) { bins[i] = s_hist[8 * lane + i]; mine += bins[i]; }
      unsigned int incl = mine;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      const unsigned int total_all = __shfl_sync(0xffffffffu, incl, 31);
      const unsigned int remaining = static_cast<unsigned int>(s_remaining);
      const unsigned int before = incl - mine;
      const bool here = before < remaining && incl >= remaining;        // at most one lane
      const unsigned int who = __ballot_sync(0xffffffffu, here);
      if (who == 0u) {
        // fewer candidates than asked for: every candidate is taken (digit 255)
        if (lane == 0) { s_remaining = static_cast<int>(remaining - total_all); s_prefix = (prefix << 8) | 255ull; }
      } else if (here) {
        unsigned int seen = before;
        int digit = 8 * lane + 7;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (seen + bins[i] >= remaining) { digit = 8 * lane + i; break; }
          seen += bins[i];
        }
        s_remaining = static_cast<int>(remaining - seen);
        s_prefix = (prefix << 8) | static_cast<unsigned long long>(digit);
      }
    }
    __syncthreads();
  }
  const int total = s_total;
  const int take = total < n ? total : n;                   // keys that exist
  const unsigned long long threshold = total < n ? ~0ull - 1ull : s_prefix;
  // ---- gather the keys up to the threshold (exactly `take` of them: keys are unique), sort, write
  int n_pow2 = 2;
  while (n_pow2 < take) n_pow2 <<= 1;
  for (int i = threadIdx.x; i < n_pow2; i += blockDim.x) s_list[i] = ~0ull;
  __syncthreads();
  for (int bt = 0; bt < n_batches; ++bt) {
    unsigned long long ks[kBatch];
    batch(bt, ks);
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const bool take_it = ks[u] != ~0ull && ks[u] <= threshold;
      const unsigned takers = __ballot_sync(0xffffffffu, take_it);       // one counter update per warp
      if (takers != 0u) {
        const int lane = threadIdx.x & 31;
        int first = 0;
        if (lane == __ffs(takers) - 1) first = atomicAdd(&s_count, __popc(takers));
        first = __shfl_sync(0xffffffffu, first, __ffs(takers) - 1);
        const int pos = first + __popc(takers & ((1u << lane) - 1u));
        if (take_it && pos < n_pow2) s_list[pos] = ks[u];
      }
    }
  }
  __syncthreads();
  for (int k = 2; k <= n_pow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n_pow2; i += blockDim.x) {
        const int l = i ^ j;
        if (l > i) {
          const unsigned long long a = s_list[i], b = s_list[l];
          const bool ascending = (i & k) == 0;
          if ((a > b) == ascending) { s_list[i] = b; s_list[l] = a; }
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    victims[i] = i < take ? static_cast<int32_t>(s_list[i] & 0xffffffu) : -1;
  if (threadIdx.x == 0 && take < n) atomicExch(status, NSA_ERR_EXHAUSTED);
}

// ----------------------------------------------------------------------------- page movement
struct MoveParams {
  const int32_t* pages;        // [n] page per move (evict: the victim; fetch: the destination)
  const int32_t* keys;         // fetch: [1 + n] list written by the dedup (count first); evict: null
  int n_host; const int32_t* n_dev;
  char* k_pool; char* v_pool; int64_t page_bytes;
  char* host_k; char* host_v;  // slot of key = base + key * page_bytes (device-mapped pinned memory)
  int32_t* block_table; int32_t* page_owner; int64_t* page_stamp; int64_t epoch;
  unsigned long long* counters;  // may be null: [2] += pages evicted, [3] += pages fetched
};

template <bool FETCH>
__global__ void __launch_bounds__(256) move_pages_kernel(const MoveParams p) {
  const int i = blockIdx.x;
  const int n = p.n_dev ? *p.n_dev : p.n_host;
  if (i >= n) return;
  const int page = p.pages[i];
  if (page < 0) return;
  char* kp = p.k_pool + static_cast<int64_t>(page) * p.page_bytes;
  char* vp = p.v_pool + static_cast<int64_t>(page) * p.page_bytes;
  if (FETCH) {
    const int key = p.keys[1 + i];
    copy16(kp, p.host_k + static_cast<int64_t>(key) * p.page_bytes, p.page_bytes);
    copy16(vp, p.host_v + static_cast<int64_t>(key) * p.page_bytes, p.page_bytes);
    __threadfence();
    __syncthreads();             // publish only after the whole page has landed
    if (threadIdx.x == 0) {
      p.page_owner[page] = key;
      p.page_stamp[page] = p.epoch;
      p.block_table[key] = page;
      if (p.counters) atomicAdd(p.counters + 3, 1ull);
    }
  } else {
    const int key = p.page_owner[page];
    if (key < 0) return;
    if (p.host_k) {
      copy16(p.host_k + static_cast<int64_t>(key) * p.page_bytes, kp, p.page_bytes);
      copy16(p.host_v + static_cast<int64_t>(key) * p.page_bytes, vp, p.page_bytes);
      __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      p.block_table[key] = -1;
      p.page_owner[page] = -1;
      if (p.counters) atomicAdd(p.counters + 2, 1ull);
    }
  }
}

// Write-behind eviction, first half: like an evict, but the page goes to slot i of a staging
// buffer in device memory (host_k / host_v hold the staging bases here) and its key to stage_keys[i]
// (-1: nothing staged); tables are updated at once, so the page is free for the caller.
__global__ void __launch_bounds__(256) stage_pages_kernel(const MoveParams p, int32_t* __restrict__ stage_keys) {
  const int i = blockIdx.x;
  const int n = p.n_dev ? *p.n_dev : p.n_host;
  int key = -1;
  const int page = i < n ? p.pages[i] : -1;
  if (page >= 0) key = p.page_owner[page];
  if (key >= 0) {
    copy16(p.host_k + static_cast<int64_t>(i) * p.page_bytes, p.k_pool + static_cast<int64_t>(page) * p.page_bytes, p.page_bytes);
    copy16(p.host_v + static_cast<int64_t>(i) * p.page_bytes, p.v_pool + static_cast<int64_t>(page) * p.page_bytes, p.page_bytes);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    stage_keys[i] = key;
    if (key >= 0) {
      p.block_table[key] = -1;
      p.page_owner[page] = -1;
      if (p.counters) atomicAdd(p.counters + 2, 1ull);
    }
  }
}

// Second half, on a stream of its own: staging slot i -> the host slot of stage_keys[i].
// (k_pool / v_pool hold the staging bases here.)
__global__ void __launch_bounds__(256) drain_pages_kernel(const MoveParams p) {
  const int i = blockIdx.x;
  const int key = p.keys[i];
  if (key < 0) return;
  copy16(p.host_k + static_cast<int64_t>(key) * p.page_bytes, p.k_pool + static_cast<int64_t>(i) * p.page_bytes, p.page_bytes);
  copy16(p.host_v + static_cast<int64_t>(key) * p.page_bytes, p.v_pool + static_cast<int64_t>(i) * p.page_bytes, p.page_bytes);
  __threadfence_system();
}

// --------------------------------------------- the reference's K1 / K2 contracts, re-expressed
__global__ void gather_publish_clear_kernel(const int64_t* __restrict__ desc, int64_t n_fetch,
                                            int64_t n_clear, int64_t block_bytes, int wide) {
  const int64_t i = blockIdx.x;
  if (i < n_fetch) {
    const char* src_k = reinterpret_cast<const char*>(desc[i]);
    const char* src_v = reinterpret_cast<const char*>(desc[n_fetch + i]);
    char* dst_k = reinterpret_cast<char*>(desc[2 * n_fetch + i]);
    char* dst_v = reinterpret_cast<char*>(desc[3 * n_fetch + i]);
    int64_t* pub_k = reinterpret_cast<int64_t*>(desc[4 * n_fetch + i]);
    int64_t* pub_v = reinterpret_cast<int64_t*>(desc[5 * n_fetch + i]);
    const bool v16 = wide && block_bytes % 16 == 0 &&
                     ((desc[i] | desc[n_fetch + i] | desc[2 * n_fetch + i] | desc[3 * n_fetch + i]) & 15) == 0;
    if (v16) {
      copy16(dst_k, src_k, block_bytes);
      copy16(dst_v, src_v, block_bytes);
    } else if (wide) {
      for (int64_t o = static_cast<int64_t>(threadIdx.x) * 8; o < block_bytes; o += static_cast<int64_t>(blockDim.x) * 8) {
        *reinterpret_cast<uint64_t*>(dst_k + o) = *reinterpret_cast<const uint64_t*>(src_k + o);
        *reinterpret_cast<uint64_t*>(dst_v + o) = *reinterpret_cast<const uint64_t*>(src_v + o);
      }
    } else {
      for (int64_t o = static_cast<int64_t>(threadIdx.x) * 2; o < block_bytes; o += static_cast<int64_t>(blockDim.x) * 2) {
        *reinterpret_cast<uint16_t*>(dst_k + o) = *reinterpret_cast<const uint16_t*>(src_k + o);
        *reinterpret_cast<uint16_t*>(dst_v + o) = *reinterpret_cast<const uint16_t*>(src_v + o);
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      *pub_k = reinterpret_cast<int64_t>(dst_k);
      *pub_v = reinterpret_cast<int64_t>(dst_v);
    }
  } else {
    const int64_t base = (i - n_fetch) * 256;
    for (int64_t e = threadIdx.x; e < 256; e += blockDim.x)
      if (base + e < n_clear) *reinterpret_cast<int64_t*>(desc[6 * n_fetch + base + e]) = 0;
  }
}

__global__ void block_range_kernel(int64_t* __restrict__ table, int32_t* __restrict__ n_valid, int H,
                                   int64_t MB, int64_t first_bid, int64_t n_blocks, int64_t k_base,
                                   int64_t v_base, int64_t head_stride, int64_t block_bytes,
                                   int64_t n_valid_value, int write_k, int write_v, int clear) {
  const int h = blockIdx.x;
  const int64_t j = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
  if (j < n_blocks) {
    const int64_t off = h * head_stride + j * block_bytes;
    if (write_k) table[(0 * H + h) * MB + first_bid + j] = clear ? 0 : k_base + off;
    if (write_v) table[(1 * H + h) * MB + first_bid + j] = clear ? 0 : v_base + off;
  }
  if (blockIdx.y == 0 && threadIdx.x == 0 && n_valid_value >= 0) n_valid[h] = static_cast<int32_t>(n_valid_value);
}

}  // namespace
}  // namespace nsa

using namespace nsa;

static int set_rope(const nsa_rope* rope, int64_t S, int32_t D, AppendParams* p) {
  NSA_REQUIRE(rope->freqs_f && rope->freqs_h && rope->freqs_w, NSA_ERR_INVALID, "rope: null frequency table");
  NSA_REQUIRE(rope->c_f >= 0 && rope->c_h >= 0 && rope->c_w >= 0 && 2 * (rope->c_f + rope->c_h + rope->c_w) == D,
              NSA_ERR_INVALID, "rope: c_f + c_h + c_w must be D / 2");
  NSA_REQUIRE(rope->pool_f > 0 && rope->pool_h > 0 && rope->pool_w > 0 && rope->grid_h > 0 && rope->grid_w > 0 &&
                  rope->grid_h % rope->pool_h == 0 && rope->grid_w % rope->pool_w == 0 && rope->start_frame >= 0,
              NSA_ERR_INVALID, "rope: bad grid / pooling window");
  NSA_REQUIRE(S % (static_cast<int64_t>(rope->grid_h) * rope->grid_w * rope->pool_f) == 0, NSA_ERR_INVALID,
              "rope: S must be whole groups of pool_f frames of grid_h x grid_w tokens");
  p->rope_f = static_cast<const double2*>(rope->freqs_f); p->rope_h = static_cast<const double2*>(rope->freqs_h);
  p->rope_w = static_cast<const double2*>(rope->freqs_w);
  p->c_f = rope->c_f; p->c_h = rope->c_h; p->c_w = rope->c_w;
  p->grid_h = rope->grid_h; p->grid_w = rope->grid_w; p->pool_f = rope->pool_f; p->pool_h = rope->pool_h;
  p->pool_w = rope->pool_w; p->start_frame = rope->start_frame;
  return NSA_OK;
}

static int cache_append_impl(const void* k_new, const void* v_new, const int64_t kv_stride[2],
                             int64_t S, int64_t pos0, int64_t n_tokens, int32_t H, int32_t D, void* k_pool,
                             void* v_pool, int32_t page_tokens, int32_t* block_table,
                             int32_t max_blocks, const int32_t* new_pages, int32_t n_touched_blocks,
                             int32_t* page_owner, int64_t* page_stamp, int64_t epoch,
                             void* k_pooled, void* v_pooled, int32_t* status, int32_t dtype,
                             const nsa_rope* rope, void* stream) {
  NSA_REQUIRE(S >= 0 && pos0 >= 0 && H > 0 && D > 0 && page_tokens > 0 && max_blocks > 0, NSA_ERR_INVALID,
              "cache_append: bad size");
  NSA_REQUIRE(n_tokens >= 0 && pos0 <= n_tokens, NSA_ERR_INVALID,
              "cache_append: pos0 = %lld would leave a gap behind the %lld tokens the cache holds",
              static_cast<long long>(pos0), static_cast<long long>(n_tokens));
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_F16, NSA_ERR_UNSUPPORTED, "cache_append: bf16 / fp16 only");
  if (S == 0) return NSA_OK;
  const int esz = 2;
  NSA_REQUIRE((D * esz) % 16 == 0 && D * esz / 16 <= 128, NSA_ERR_UNSUPPORTED, "cache_append: head dim %d", D);
  const int64_t first = pos0 / page_tokens, last = (pos0 + S - 1) / page_tokens;
  NSA_REQUIRE(last < max_blocks, NSA_ERR_INVALID, "cache_append: token %lld is past the block table (%d blocks)",
              static_cast<long long>(pos0 + S - 1), max_blocks);
  NSA_REQUIRE(n_touched_blocks == last - first + 1, NSA_ERR_INVALID,
              "cache_append: n_touched_blocks must be %lld", static_cast<long long>(last - first + 1));
  NSA_REQUIRE(k_new && v_new && k_pool && v_pool && block_table && page_owner && page_stamp && k_pooled && status,
              NSA_ERR_INVALID, "cache_append: null pointer");
  NSA_REQUIRE(aligned16(k_new) && aligned16(v_new) && (kv_stride[0] * esz) % 16 == 0 && (kv_stride[1] * esz) % 16 == 0,
              NSA_ERR_LAYOUT, "cache_append: new K/V rows must be 16-byte aligned");
  NSA_REQUIRE(static_cast<int64_t>(n_touched_blocks) * H <= 0x7fffffff, NSA_ERR_INVALID, "cache_append: too many blocks");
  AppendParams p{static_cast<const char*>(k_new), static_cast<const char*>(v_new), kv_stride[0], kv_stride[1],
                 S, pos0, n_tokens, H, D, page_tokens, max_blocks, n_touched_blocks, H, static_cast<char*>(k_pool),
                 static_cast<char*>(v_pool), block_table, new_pages, page_owner, page_stamp, epoch,
                 static_cast<char*>(k_pooled), static_cast<char*>(v_pooled), status};
  if (rope != nullptr) {
    const int rc = set_rope(rope, S, D, &p);
    if (rc) return rc;
  }
  // heads per thread block: whole source rows when the touched blocks alone fill the GPU, else the
  // heads are split (down to 512-byte pieces); 8 row parts x hc heads x (D / 8) pieces <= 768 threads
  const int cpr = D * esz / 16;
  int hc = H;
  const int min_hc = (512 + D * esz - 1) / (D * esz);
  while (hc > min_hc && static_cast<int64_t>(n_touched_blocks) * cdiv(H, hc) < 148) hc = cdiv(hc, 2);
  while (hc > 1 && kAppendSlices * hc * cpr > 768) hc = cdiv(hc, 2);
  NSA_REQUIRE(kAppendSlices * hc * cpr <= 768 && hc <= 64, NSA_ERR_UNSUPPORTED, "cache_append: head dim %d too wide", D);
  p.hc = hc;
  const int threads = kAppendSlices * hc * cpr;
  const size_t smem = static_cast<size_t>(kAppendSlices) * hc * 2 * D * sizeof(float);
  const dim3 grid(static_cast<unsigned>(n_touched_blocks), cdiv(H, hc));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (smem + 4096 > 48 * 1024) {                  // (static shared memory counts against the 48 KiB default)
    if (rope != nullptr) {
      if (dtype == NSA_BF16) NSA_CUDA_OK(cudaFuncSetAttribute(cache_append_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      else NSA_CUDA_OK(cudaFuncSetAttribute(cache_append_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    } else {
      if (dtype == NSA_BF16) NSA_CUDA_OK(cudaFuncSetAttribute(cache_append_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      else NSA_CUDA_OK(cudaFuncSetAttribute(cache_append_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
  }
  // (a programmatic dependent launch: back-to-back appends overlap one launch's ramp with the tail of the one before)
  if (rope != nullptr) {
    if (dtype == NSA_BF16) NSA_CUDA_OK(launch_chained(kChainSmall, cache_append_kernel<__nv_bfloat16, true>, grid, dim3(threads), smem, s, p));
    else NSA_CUDA_OK(launch_chained(kChainSmall, cache_append_kernel<__half, true>, grid, dim3(threads), smem, s, p));
  } else {
    if (dtype == NSA_BF16) NSA_CUDA_OK(launch_chained(kChainSmall, cache_append_kernel<__nv_bfloat16, false>, grid, dim3(threads), smem, s, p));
    else NSA_CUDA_OK(launch_chained(kChainSmall, cache_append_kernel<__half, false>, grid, dim3(threads), smem, s, p));
  }
  NSA_LAUNCH_OK("cache_append_kernel");
  return NSA_OK;
}

extern "C" int nsa_cache_append(const void* k_new, const void* v_new, const int64_t kv_stride[2],
                                int64_t S, int64_t pos0, int64_t n_tokens, int32_t H, int32_t D, void* k_pool,
                                void* v_pool, int32_t page_tokens, int32_t* block_table,
                                int32_t max_blocks, const int32_t* new_pages, int32_t n_touched_blocks,
                                int32_t* page_owner, int64_t* page_stamp, int64_t epoch,
                                void* k_pooled, void* v_pooled, int32_t* status, int32_t dtype,
                                void* stream) {
  return cache_append_impl(k_new, v_new, kv_stride, S, pos0, n_tokens, H, D, k_pool, v_pool, page_tokens, block_table,
                           max_blocks, new_pages, n_touched_blocks, page_owner, page_stamp, epoch, k_pooled,
                           v_pooled, status, dtype, nullptr, stream);
}

extern "C" int nsa_cache_append_rope(const void* k_new, const void* v_new, const int64_t kv_stride[2],
                                     int64_t S, int64_t pos0, int64_t n_tokens, int32_t H, int32_t D, void* k_pool,
                                     void* v_pool, int32_t page_tokens, int32_t* block_table,
                                     int32_t max_blocks, const int32_t* new_pages, int32_t n_touched_blocks,
                                     int32_t* page_owner, int64_t* page_stamp, int64_t epoch,
                                     void* k_pooled, void* v_pooled, int32_t* status, int32_t dtype,
                                     const nsa_rope* rope, void* stream) {
  NSA_REQUIRE(rope != nullptr, NSA_ERR_INVALID, "cache_append_rope: rope is null");
  return cache_append_impl(k_new, v_new, kv_stride, S, pos0, n_tokens, H, D, k_pool, v_pool, page_tokens, block_table,
                           max_blocks, new_pages, n_touched_blocks, page_owner, page_stamp, epoch, k_pooled,
                           v_pooled, status, dtype, rope, stream);
}

extern "C" int nsa_rope_apply(const void* x, const int64_t x_stride[2], int64_t S, int32_t H, int32_t D, void* out,
                              int32_t dtype, const nsa_rope* rope, void* stream) {
  NSA_REQUIRE(S >= 0 && H > 0 && D > 0, NSA_ERR_INVALID, "rope_apply: bad size");
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_F16, NSA_ERR_UNSUPPORTED, "rope_apply: bf16 / fp16 only");
  NSA_REQUIRE((D * 2) % 16 == 0, NSA_ERR_UNSUPPORTED, "rope_apply: head dim %d", D);
  NSA_REQUIRE(rope != nullptr, NSA_ERR_INVALID, "rope_apply: rope is null");
  if (S == 0) return NSA_OK;
  NSA_REQUIRE(x && out && aligned16(x) && aligned16(out) && (x_stride[0] * 2) % 16 == 0 && (x_stride[1] * 2) % 16 == 0,
              NSA_ERR_LAYOUT, "rope_apply: rows must be 16-byte aligned");
  AppendParams p{};
  p.k_new = static_cast<const char*>(x); p.s_stride = x_stride[0]; p.h_stride = x_stride[1];
  p.S = S; p.H = H; p.D = D;
  int rc;
  if ((rc = set_rope(rope, S, D, &p))) return rc;
  const int64_t total = S * H * (D * 2 / 16);
  const int blocks = static_cast<int>(cdiv64(total, 256) < 148 * 16 ? cdiv64(total, 256) : 148 * 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == NSA_BF16) rope_apply_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p, static_cast<char*>(out));
  else rope_apply_kernel<__half><<<blocks, 256, 0, s>>>(p, static_cast<char*>(out));
  NSA_LAUNCH_OK("rope_apply_kernel");
  return NSA_OK;
}

extern "C" size_t nsa_cache_dedup_workspace_bytes(int64_t n_keys) {
  return align_up(static_cast<size_t>(cdiv64(n_keys, kTileKeys)) * 2 * sizeof(int32_t), 256);
}

extern "C" int nsa_cache_dedup_touch(const int32_t* block_indices, int64_t n_entries, int32_t H,
                                     int32_t T, int32_t max_blocks, int32_t bpc, int32_t* stamp, int32_t epoch32,
                                     const int32_t* block_table, int64_t* page_stamp, int64_t epoch,
                                     int32_t* out_unique, int32_t* out_missing, int32_t cap,
                                     int64_t* counters, void* workspace, size_t workspace_bytes, void* stream) {
  NSA_REQUIRE(n_entries >= 0 && H > 0 && T > 0 && max_blocks > 0 && cap >= 0, NSA_ERR_INVALID, "cache_dedup: bad size");
  NSA_REQUIRE(stamp && out_unique, NSA_ERR_INVALID, "cache_dedup: null pointer");
  NSA_REQUIRE(bpc > 0 && max_blocks % bpc == 0, NSA_ERR_INVALID, "cache_dedup: bpc must divide max_blocks");
  NSA_REQUIRE(epoch32 >= 1, NSA_ERR_INVALID, "cache_dedup: epoch must be >= 1");
  NSA_REQUIRE(block_table == nullptr || bpc == max_blocks, NSA_ERR_INVALID,
              "cache_dedup: a block table needs bpc == max_blocks (keys index the table)");
  const int64_t n_keys = static_cast<int64_t>(H) * max_blocks;
  NSA_REQUIRE(n_keys <= 0x7fffffff, NSA_ERR_INVALID, "cache_dedup: too many keys");
  NSA_REQUIRE(workspace && workspace_bytes >= nsa_cache_dedup_workspace_bytes(n_keys), NSA_ERR_WORKSPACE,
              "cache_dedup: workspace too small");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* counts = static_cast<int32_t*>(workspace);
  const int n_tiles = static_cast<int>(cdiv64(n_keys, kTileKeys));
  if (n_entries > 0) {
    NSA_REQUIRE(block_indices != nullptr, NSA_ERR_INVALID, "cache_dedup: block_indices is null");
    dedup_mark_kernel<<<static_cast<unsigned>(cdiv64(n_entries, 256)), 256, 0, s>>>(block_indices, n_entries, H, T,
                                                                                    max_blocks, bpc, stamp, epoch32);
    NSA_LAUNCH_OK("dedup_mark_kernel");
  }
  dedup_count_kernel<<<n_tiles, kTileKeys, 0, s>>>(stamp, epoch32, block_table, n_keys, counts);
  NSA_LAUNCH_OK("dedup_count_kernel");
  dedup_scan_kernel<<<1, 32, 0, s>>>(counts, n_tiles, out_unique, out_missing, block_table ? counters : nullptr);
  NSA_LAUNCH_OK("dedup_scan_kernel");
  dedup_compact_kernel<<<n_tiles, kTileKeys, 0, s>>>(stamp, epoch32, block_table, n_keys, counts, page_stamp,
                                                     epoch, out_unique, out_missing, cap);
  NSA_LAUNCH_OK("dedup_compact_kernel");
  return NSA_OK;
}

extern "C" int nsa_cache_select_victims(const int32_t* page_owner, const int64_t* page_stamp,
                                        int32_t num_pages, int32_t max_blocks, int32_t protect_from_bid,
                                        int64_t epoch, int32_t n, const int32_t* n_dev, int32_t cap,
                                        int32_t* victims, int32_t* status, void* stream) {
  NSA_REQUIRE(num_pages > 0 && num_pages < (1 << 24) && max_blocks > 0 && cap >= 0 && n >= 0, NSA_ERR_INVALID,
              "cache_select_victims: bad size");
  NSA_REQUIRE(page_owner && page_stamp && victims && status, NSA_ERR_INVALID, "cache_select_victims: null pointer");
  NSA_REQUIRE(n_dev != nullptr || n <= cap, NSA_ERR_INVALID, "cache_select_victims: n > cap");
  if (cap == 0 || (!n_dev && n == 0)) return NSA_OK;
  // test hook: OMNIMEM_B200_VICTIMS_KERNEL=scan keeps the rescanning kernel for every pool size
  const char* env = getenv("OMNIMEM_B200_VICTIMS_KERNEL");
  const bool scan_only = env != nullptr && env[0] == 's';
  const int n_max = n_dev ? cap : n;                        // the most victims this call can ask for
  if (n_max <= kSelectMax && !scan_only) {
    int n_pow2 = 2;
    while (n_pow2 < n_max) n_pow2 <<= 1;
    const size_t smem = static_cast<size_t>(n_pow2) * sizeof(unsigned long long);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (num_pages <= 16 * 1024) {
      NSA_CUDA_OK(cudaFuncSetAttribute(select_victims_radix_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelectMax * 8));
      select_victims_radix_kernel<16><<<1, 1024, smem, st>>>(page_owner, page_stamp, num_pages, max_blocks, protect_from_bid,
                                                             epoch, n, n_dev, cap, victims, status);
    } else if (num_pages <= 32 * 1024) {
      NSA_CUDA_OK(cudaFuncSetAttribute(select_victims_radix_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelectMax * 8));
      select_victims_radix_kernel<32><<<1, 1024, smem, st>>>(page_owner, page_stamp, num_pages, max_blocks, protect_from_bid,
                                                             epoch, n, n_dev, cap, victims, status);
    } else {
      NSA_CUDA_OK(cudaFuncSetAttribute(select_victims_radix_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelectMax * 8));
      select_victims_radix_kernel<0><<<1, 1024, smem, st>>>(page_owner, page_stamp, num_pages, max_blocks, protect_from_bid,
                                                            epoch, n, n_dev, cap, victims, status);
    }
    NSA_LAUNCH_OK("select_victims_radix_kernel");
    return NSA_OK;
  }
  select_victims_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      page_owner, page_stamp, num_pages, max_blocks, protect_from_bid, epoch, n, n_dev, cap, victims, status);
  NSA_LAUNCH_OK("select_victims_kernel");
  return NSA_OK;
}

extern "C" int nsa_cache_move_pages(int32_t direction, const int32_t* pages, const int32_t* keys,
                                    int32_t n, const int32_t* n_dev, int32_t cap, void* k_pool,
                                    void* v_pool, int64_t page_bytes, void* host_k, void* host_v,
                                    int32_t* block_table, int32_t* page_owner, int64_t* page_stamp,
                                    int64_t epoch, int64_t* counters, void* stream) {
  NSA_REQUIRE(direction >= 0 && direction <= 3, NSA_ERR_INVALID, "cache_move_pages: direction must be 0 .. 3");
  NSA_REQUIRE(n >= 0 && cap >= 0 && page_bytes > 0 && page_bytes % 16 == 0, NSA_ERR_INVALID, "cache_move_pages: bad size");
  NSA_REQUIRE(k_pool && v_pool, NSA_ERR_INVALID, "cache_move_pages: null pointer");
  NSA_REQUIRE(direction == 3 || (pages && block_table && page_owner && page_stamp), NSA_ERR_INVALID,
              "cache_move_pages: null pointer");
  NSA_REQUIRE(direction == 0 || (keys && host_k && host_v), NSA_ERR_INVALID,
              "cache_move_pages: fetch, stage and drain need keys and the second set of slots");
  const int grid = n_dev ? cap : n;
  if (grid == 0) return NSA_OK;
  if (direction >= 2) {
    MoveParams sp{pages, keys, n, n_dev, static_cast<char*>(k_pool), static_cast<char*>(v_pool), page_bytes,
                  static_cast<char*>(host_k), static_cast<char*>(host_v), block_table, page_owner, page_stamp, epoch,
                  reinterpret_cast<unsigned long long*>(counters)};
    if (direction == 2) stage_pages_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(sp, const_cast<int32_t*>(keys));
    else drain_pages_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(sp);
    NSA_LAUNCH_OK("stage / drain pages kernel");
    return NSA_OK;
  }
  MoveParams p{pages, keys, n, n_dev, static_cast<char*>(k_pool), static_cast<char*>(v_pool), page_bytes,
               static_cast<char*>(host_k), static_cast<char*>(host_v), block_table, page_owner, page_stamp, epoch,
               reinterpret_cast<unsigned long long*>(counters)};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (direction == 1) move_pages_kernel<true><<<grid, 256, 0, s>>>(p);
  else move_pages_kernel<false><<<grid, 256, 0, s>>>(p);
  NSA_LAUNCH_OK("move_pages_kernel");
  return NSA_OK;
}

extern "C" int nsa_gather_publish_clear(const int64_t* desc, int64_t n_fetch, int64_t n_clear,
                                        int64_t block_bytes, int32_t wide, int32_t num_warps,
                                        int64_t* ctas_launched, void* stream) {
  if (ctas_launched) *ctas_launched = 0;
  if (n_fetch == 0 && n_clear == 0) return NSA_OK;
  NSA_REQUIRE(n_fetch >= 0 && n_clear >= 0, NSA_ERR_INVALID, "gather_publish_clear: n_fetch / n_clear must be >= 0");
  NSA_REQUIRE(block_bytes > 0 && block_bytes % 2 == 0, NSA_ERR_INVALID,
              "gather_publish_clear: block_bytes=%lld must be a positive multiple of 2", static_cast<long long>(block_bytes));
  NSA_REQUIRE(!wide || block_bytes % 8 == 0, NSA_ERR_INVALID, "gather_publish_clear: wide copies need block_bytes % 8 == 0");
  NSA_REQUIRE(num_warps >= 1 && num_warps <= 32, NSA_ERR_INVALID, "gather_publish_clear: num_warps=%d outside [1, 32]", num_warps);
  const int64_t ctas = n_fetch + cdiv64(n_clear, 256);
  if (ctas_launched) *ctas_launched = ctas;
  NSA_REQUIRE(desc != nullptr, NSA_ERR_INVALID, "gather_publish_clear: desc is null");
  NSA_REQUIRE(ctas <= 0x7fffffff, NSA_ERR_INVALID, "gather_publish_clear: too many blocks");
  gather_publish_clear_kernel<<<static_cast<unsigned>(ctas), 32 * num_warps, 0, static_cast<cudaStream_t>(stream)>>>(
      desc, n_fetch, n_clear, block_bytes, wide);
  NSA_LAUNCH_OK("gather_publish_clear_kernel");
  return NSA_OK;
}

extern "C" int nsa_block_range(int64_t* table, int32_t* n_valid, int32_t H, int64_t MB, int64_t first_bid,
                               int64_t n_blocks, int64_t k_base, int64_t v_base, int64_t head_stride_bytes,
                               int64_t block_bytes, int64_t n_valid_value, int32_t write_k, int32_t write_v,
                               int32_t clear, void* stream) {
  NSA_REQUIRE(H > 0 && H <= 65535 && MB > 0, NSA_ERR_INVALID, "block_range: bad table shape");
  NSA_REQUIRE(n_blocks > 0 && first_bid >= 0 && first_bid + n_blocks <= MB, NSA_ERR_INVALID,
              "block_range: range [%lld, %lld) is outside the table (%lld blocks)", static_cast<long long>(first_bid),
              static_cast<long long>(first_bid + n_blocks), static_cast<long long>(MB));
  NSA_REQUIRE(table && n_valid, NSA_ERR_INVALID, "block_range: null pointer");
  const dim3 grid(H, static_cast<unsigned>(cdiv64(n_blocks, 128)));
  block_range_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(table, n_valid, H, MB, first_bid, n_blocks,
                                                                          k_base, v_base, head_stride_bytes, block_bytes,
                                                                          n_valid_value, write_k, write_v, clear);
  NSA_LAUNCH_OK("block_range_kernel");
  return NSA_OK;
}
