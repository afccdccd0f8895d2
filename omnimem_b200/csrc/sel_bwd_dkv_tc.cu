// Selection attention backward, dK/dV half, on tcgen05 / TMEM / TMA for the page geometry
// (bf16, D = 128, 64-token blocks, query groups of up to 64 rows, dense or paged K/V).
//
// Ownership as in the general kernel: one work item = one (batch, head, KV block); the item's
// dK / dV tile is produced by exactly one thread block, from the block's bucket of query groups
// in ascending group order - no atomics, bit-reproducible.  Persistent thread blocks (one per
// SM) walk the items round-robin; inside a block the roles are pipelined across steps AND
// across items:
//   warp 8   TMA producer: K, V tile of the item; per step the Q and dO rows of TWO groups of
//            the bucket, stacked into 128-row tiles (two-stage ring)
//   warp 9   MMA issuer 1, per step:  S  = [Qa;Qb] K^T, dP = [dOa;dOb] V^T   (M=128, N=64, K=128)
//   warp 10  MMA issuer 2, per step:  dV^T += [dOa;dOb]^T P,  dK^T += [Qa;Qb]^T dS
//                                   (M=128 = head dim, N=64 keys, K=128 query rows)
//            (two issuing threads: each spends a good part of a step in its barrier waits)
//   warps 0-3  one query row per thread: P = exp2(S c - LSE), dS = P (dP - delta) scale, written
//            as bf16 rows into shared memory in the 128-byte-swizzled layout the MMA reads
//   warps 4-7  epilogue: one head-dim lane per thread, read dV^T / dK^T from TMEM and store the
//            transposed tile; items with an empty bucket are zero-filled here
// Both operands of every MMA are full (two real groups fill the 128 rows), so no tensor work
// is wasted; S/dP and the dV^T/dK^T accumulators are double buffered in TMEM (512 columns).
#include "sel_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <string>

namespace nsa {

int device_status_address(int32_t** out);
int make_qkv_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                  CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV);

#ifdef NSA_TC_TRACE
// Debug build only: clock64 stamps of thread block 0; [0] MMA issuer, [1] math thread 0, [2] producer, [3] epilogue.
__device__ long long g_trace_dkv[4][1024];
#define TRACE(role, slot) do { if (blockIdx.x == 0 && (slot) < 1024) g_trace_dkv[role][slot] = clock64(); } while (0)
#else
#define TRACE(role, slot) do { } while (0)
#endif

namespace {

using namespace tc;

constexpr int kThreads = 352;
constexpr uint32_t kKVBytes = 32768;     // K tile 16 KiB + V tile 16 KiB
constexpr uint32_t kQdOBytes = 65536;    // Q2 32 KiB + dO2 32 KiB per stage
constexpr uint32_t kPdSBytes = 32768;    // P 16 KiB + dS 16 KiB
constexpr uint32_t kSmemTiles = kKVBytes + 2 * kQdOBytes + kPdSBytes;

// TMEM columns: S / dP double buffered (64 columns each), accumulators double buffered
__device__ __forceinline__ uint32_t col_s(int buf) { return buf * 128; }
__device__ __forceinline__ uint32_t col_dp(int buf) { return buf * 128 + 64; }
__device__ __forceinline__ uint32_t col_dv(int acc) { return 256 + acc * 128; }
__device__ __forceinline__ uint32_t col_dk(int acc) { return 256 + acc * 128 + 64; }

struct TcDkvParams {
  const int32_t* groups;     // [B,H,MG*T] buckets, ascending inside a bucket
  const int32_t* offsets;    // [B,H,NS+1]
  const float* lse;          // [B,H,M]
  const float* delta;        // [B,H,M]
  char* dk; char* dv;        // contiguous [B,N,H,D]
  const int32_t* block_table;
  int max_blocks, paged;
  int64_t n_tokens, M, NS;
  int B, H, T, G, MG, chunk_size, causal;
  float scale, scale_log2;
  int32_t* status;
  int32_t* counter;          // zeroed before the launch: next work item to hand out
};

struct Item { int b, h, blk, beg, n_ent, row; bool active; };

// Decodes work item i (block fastest, then head, then batch) and its bucket.
__device__ __forceinline__ Item get_item(const TcDkvParams& p, int64_t i) {
  Item it;
  const uint32_t iu = static_cast<uint32_t>(i), ns = static_cast<uint32_t>(p.NS);   // the host keeps B*H*NS below 2^31
  const uint32_t r = iu / ns;
  it.blk = static_cast<int>(iu - r * ns);
  it.b = static_cast<int>(r / static_cast<uint32_t>(p.H));
  it.h = static_cast<int>(r - static_cast<uint32_t>(it.b) * static_cast<uint32_t>(p.H));
  const int32_t* offs = p.offsets + (static_cast<int64_t>(it.b) * p.H + it.h) * (p.NS + 1);
  it.beg = offs[it.blk];
  it.n_ent = offs[it.blk + 1] - it.beg;
  it.row = it.blk * 64;
  if (p.paged) {
    const int page = it.blk < p.max_blocks ? p.block_table[static_cast<int64_t>(it.h) * p.max_blocks + it.blk] : -1;
    it.row = page * 64;
    if (page < 0) it.n_ent = 0;
  }
  it.active = it.n_ent > 0;
  return it;
}
// Work items are handed out through a global counter (buckets differ a lot in length, a static
// split leaves thread blocks idle).  The producer thread takes the ticket, decodes the item and
// publishes it in a 4-deep shared-memory ring that the other roles follow; n_ent = -1 ends it.
__device__ __forceinline__ Item fetch_item(const TcDkvParams& p, int64_t n_items) {
  const int64_t t = atomicAdd(p.counter, 1);
  if (t < n_items) return get_item(p, t);
  Item it{0, 0, 0, 0, -1, 0, false};
  return it;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1)
sel_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapDO,
                      const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                      const TcDkvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sKV = tiles;                               // K [2][64][128 B], V [2][64][128 B]
  uint8_t* sQdO = tiles + kKVBytes;                   // [stage]{ Q2 [2][128][128 B], dO2 [2][128][128 B] }
  uint8_t* sP = tiles + kKVBytes + 2 * kQdOBytes;     // [128 q][128 B] swizzled
  uint8_t* sdS = sP + 16384;

  __shared__ uint64_t kv_full, kv_empty, qdo_full[2], qdo_empty[2], sdp_full[2], sdp_free[2], pds_full, pds_free,
      acc_full[2], acc_free[2];
  __shared__ uint64_t sched_full[4], sched_empty[4];
  __shared__ Item s_items[4];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < 4; ++i) { mbar_init(&sched_full[i], 1); mbar_init(&sched_empty[i], 258); }
    mbar_init(&kv_full, 1); mbar_init(&kv_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1);
      mbar_init(&sdp_full[i], 1); mbar_init(&sdp_free[i], 128);
      mbar_init(&acc_full[i], 1); mbar_init(&acc_free[i], 128);
    }
    mbar_init(&pds_full, 128); mbar_init(&pds_free, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapDO); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_base_s;
  volatile int* abort = &s_abort;
  const int64_t n_items = static_cast<int64_t>(p.B) * p.H * p.NS;
  const int64_t bucket_row = static_cast<int64_t>(p.MG) * p.T;

  if (warp == 8) {
    // ======================= TMA producer =======================
    if (lane == 0) {
      uint32_t ic = 0, sc = 0;
      bool ok = true;
      Item nxt = fetch_item(p, n_items);
      for (uint32_t n = 0; ok; ++n) {
        const Item it = nxt;
        if (!mbar_wait(&sched_empty[n & 3], ((n >> 2) & 1) ^ 1, abort)) break;
        s_items[n & 3] = it;
        mbar_arrive(&sched_full[n & 3]);
        if (it.n_ent < 0) break;
        nxt = fetch_item(p, n_items);          // decoded while this item's copies are issued
        if (!it.active) continue;
        TRACE(2, 16 + sc * 4 + 0);
        if (!mbar_wait(&kv_empty, (ic & 1) ^ 1, abort)) break;
        TRACE(2, 16 + sc * 4 + 1);
        mbar_expect_tx(&kv_full, kKVBytes);
        for (int dh = 0; dh < 2; ++dh) {
          if (p.paged) {
            tma_load_2d(sKV + dh * 8192, &mapK, dh * 64, it.row, &kv_full);
            tma_load_2d(sKV + 16384 + dh * 8192, &mapV, dh * 64, it.row, &kv_full);
          } else {
            tma_load_4d(sKV + dh * 8192, &mapK, dh * 64, it.h, it.row, it.b, &kv_full);
            tma_load_4d(sKV + 16384 + dh * 8192, &mapV, dh * 64, it.h, it.row, it.b, &kv_full);
          }
        }
        const int32_t* bucket = p.groups + (static_cast<int64_t>(it.b) * p.H + it.h) * bucket_row + it.beg;
        const int nsteps = (it.n_ent + 1) >> 1;
        for (int t = 0; t < nsteps; ++t, ++sc) {
          const int st = sc & 1, ph = (sc >> 1) & 1;
          if (!mbar_wait(&qdo_empty[st], ph ^ 1, abort)) { ok = false; break; }
          TRACE(2, 16 + sc * 4 + 2);
          const int ga = bucket[2 * t], gb = (2 * t + 1 < it.n_ent) ? bucket[2 * t + 1] : ga;
          uint8_t* dq = sQdO + st * kQdOBytes;
          mbar_expect_tx(&qdo_full[st], kQdOBytes);
          for (int dh = 0; dh < 2; ++dh) {
            tma_load_4d(dq + dh * 16384, &mapQ, dh * 64, it.h, ga * p.G, it.b, &qdo_full[st]);
            tma_load_4d(dq + dh * 16384 + 8192, &mapQ, dh * 64, it.h, gb * p.G, it.b, &qdo_full[st]);
            tma_load_4d(dq + 32768 + dh * 16384, &mapDO, dh * 64, it.h, ga * p.G, it.b, &qdo_full[st]);
            tma_load_4d(dq + 32768 + dh * 16384 + 8192, &mapDO, dh * 64, it.h, gb * p.G, it.b, &qdo_full[st]);
          }
        }
        ++ic;
      }
      if (*abort) {
        // consumers have stopped: wait (bounded) for the copies still in flight
        if (ic > 0) mbar_wait(&kv_full, (ic - 1) & 1, abort);
        for (uint32_t u = (sc > 1 ? sc - 2 : 0); u < sc; ++u) mbar_wait(&qdo_full[u & 1], (u >> 1) & 1, abort);
      }
    }
  } else if (warp == 9) {
    // ======================= MMA issuer 1: S and dP of every step =======================
    if (lane == 0) {
      constexpr uint32_t idesc_first = instr_desc_bf16(128, 64, 0, 0);    // both operands K-major
      const uint64_t dK = smem_desc(smem_u32(sKV), 16, 1024), dV = smem_desc(smem_u32(sKV + 16384), 16, 1024);
      uint32_t ic = 0, sc = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        if (!mbar_wait(&sched_full[n & 3], (n >> 2) & 1, abort)) break;
        const int n_ent = s_items[n & 3].n_ent;
        mbar_arrive(&sched_empty[n & 3]);
        if (n_ent < 0) break;
        if (n_ent == 0) continue;
        TRACE(0, 16 + sc * 8 + 0);
        if (!mbar_wait(&kv_full, ic & 1, abort)) break;
        TRACE(0, 16 + sc * 8 + 1);
        const int nsteps = (n_ent + 1) >> 1;
        for (int t = 0; t < nsteps; ++t, ++sc) {
          const int st = sc & 1, ph = (sc >> 1) & 1;
          if (!mbar_wait(&qdo_full[st], ph, abort)) { ok = false; break; }
          TRACE(0, 16 + sc * 8 + 2);
          if (!mbar_wait(&sdp_free[st], ph ^ 1, abort)) { ok = false; break; }
          tc_fence_after();
          const uint32_t aQ = smem_u32(sQdO + st * kQdOBytes);
          const uint64_t dQ = smem_desc(aQ, 16, 1024), dDO = smem_desc(aQ + 32768, 16, 1024);
          const uint32_t ts = tm + col_s(st), tdp = tm + col_dp(st);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(ts, desc_advance(dQ, (kk >> 2) * 16384 + (kk & 3) * 32),
                    desc_advance(dK, (kk >> 2) * 8192 + (kk & 3) * 32), idesc_first, kk > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tdp, desc_advance(dDO, (kk >> 2) * 16384 + (kk & 3) * 32),
                    desc_advance(dV, (kk >> 2) * 8192 + (kk & 3) * 32), idesc_first, kk > 0 ? 1u : 0u);
          umma_commit(&sdp_full[st]);
          if (t == nsteps - 1) umma_commit(&kv_empty);
          TRACE(0, 16 + sc * 8 + 3);
        }
        ++ic;
      }
    }
  } else if (warp == 10) {
    // ======================= MMA issuer 2: dV^T and dK^T of every step =======================
    // A thread of its own, so that these products start the moment P / dS are in shared memory
    // while issuer 1 already waits for the tiles of the next step.
    if (lane == 0) {
      constexpr uint32_t idesc_second = instr_desc_bf16(128, 64, 1, 1);   // both operands MN-major
      const uint64_t dP = smem_desc(smem_u32(sP), 16, 1024), dDS = smem_desc(smem_u32(sdS), 16, 1024);
      uint32_t ic = 0, sc = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        if (!mbar_wait(&sched_full[n & 3], (n >> 2) & 1, abort)) break;
        const int n_ent = s_items[n & 3].n_ent;
        mbar_arrive(&sched_empty[n & 3]);
        if (n_ent < 0) break;
        if (n_ent == 0) continue;
        const int acc = ic & 1;
        const int nsteps = (n_ent + 1) >> 1;
        for (int t = 0; t < nsteps; ++t, ++sc) {
          const int st = sc & 1;
          if (!mbar_wait(&pds_full, sc & 1, abort)) { ok = false; break; }
          TRACE(0, 16 + sc * 8 + 4);
          if (t == 0 && !mbar_wait(&acc_free[acc], ((ic >> 1) & 1) ^ 1, abort)) { ok = false; break; }
          TRACE(0, 16 + sc * 8 + 5);
          tc_fence_after();
          const uint32_t aQ = smem_u32(sQdO + st * kQdOBytes);
          const uint64_t dQmn = smem_desc(aQ, 16384, 1024), dDOmn = smem_desc(aQ + 32768, 16384, 1024);
          const uint32_t acc0 = t == 0 ? 0u : 1u;
          const uint32_t tdv = tm + col_dv(acc), tdk = tm + col_dk(acc);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tdv, desc_advance(dDOmn, kk * 2048), desc_advance(dP, kk * 2048), idesc_second, kk > 0 ? 1u : acc0);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tdk, desc_advance(dQmn, kk * 2048), desc_advance(dDS, kk * 2048), idesc_second, kk > 0 ? 1u : acc0);
          umma_commit(&qdo_empty[st]);
          umma_commit(&pds_free);
          if (t == nsteps - 1) umma_commit(&acc_full[acc]);
          TRACE(0, 16 + sc * 8 + 6);
        }
        ++ic;
      }
    }
  } else if (warp < 4) {
    // ======================= per-row math: P and dS of one query row per thread =======================
    const int half = warp >> 1, r = threadIdx.x & 63;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int row = threadIdx.x;                       // row of the stacked 128-row tiles
    uint8_t* prow = sP + row * 128;
    uint8_t* dsrow = sdS + row * 128;
    uint32_t sc = 0;
    bool ok = true;
    for (uint32_t n = 0; ok; ++n) {
      ok = __all_sync(0xffffffffu, mbar_wait(&sched_full[n & 3], (n >> 2) & 1, abort));
      if (!ok) break;
      const Item it = s_items[n & 3];
      mbar_arrive(&sched_empty[n & 3]);
      if (it.n_ent < 0) break;
      if (!it.active) continue;
      const int32_t* bucket = p.groups + (static_cast<int64_t>(it.b) * p.H + it.h) * bucket_row + it.beg;
      const int64_t t0 = static_cast<int64_t>(it.blk) * 64;
      const int n_blk = static_cast<int>(p.n_tokens - t0 < 64 ? p.n_tokens - t0 : 64);
      const int64_t bh = (static_cast<int64_t>(it.b) * p.H + it.h) * p.M;
      const int nsteps = (it.n_ent + 1) >> 1;
      for (int t = 0; t < nsteps; ++t, ++sc) {
        const int st = sc & 1, ph = (sc >> 1) & 1;
        const int ent = 2 * t + half;
        const bool valid = ent < it.n_ent;
        const int g = valid ? bucket[ent] : 0;
        const int64_t m0 = static_cast<int64_t>(g) * p.G;
        const int nq = valid ? static_cast<int>(p.M - m0 < p.G ? p.M - m0 : p.G) : 0;
        const bool rowok = r < nq;
        const float lse2 = rowok ? p.lse[bh + m0 + r] * kLog2e : INFINITY;
        const float dl = rowok ? p.delta[bh + m0 + r] : 0.f;
        int nkv = n_blk;
        if (p.causal) {
          const int64_t lim = (m0 / p.chunk_size + 1) * p.chunk_size - t0;
          if (lim < nkv) nkv = static_cast<int>(lim < 0 ? 0 : lim);
        }
        if (!rowok) nkv = 0;
        if (threadIdx.x == 0) TRACE(1, 16 + sc * 8 + 0);
        ok = __all_sync(0xffffffffu, mbar_wait(&sdp_full[st], ph, abort));
        if (!ok) break;
        if (threadIdx.x == 0) TRACE(1, 16 + sc * 8 + 1);
        tc_fence_after();
        uint32_t pp[32], dd[32];                       // packed bf16 pairs of the 64 keys
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          uint32_t x[32], y[32];
          tmem_ld32_nowait(tm + lane_base + col_s(st) + hc * 32, x);
          tmem_ld32_nowait(tm + lane_base + col_dp(st) + hc * 32, y);
          tmem_ld_wait();
          if (hc == 1) { tc_fence_before(); mbar_arrive(&sdp_free[st]); }
          const float sl = p.scale_log2, nl = -lse2, sc_ = p.scale, nds = -dl * p.scale;
          if (nkv == 64) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(x[2 * j]), sl, nl));
              const float p1 = fast_exp2(fmaf(__uint_as_float(x[2 * j + 1]), sl, nl));
              pp[hc * 16 + j] = pack2<__nv_bfloat16>(p0, p1);
              dd[hc * 16 + j] = pack2<__nv_bfloat16>(p0 * fmaf(__uint_as_float(y[2 * j]), sc_, nds),
                                                     p1 * fmaf(__uint_as_float(y[2 * j + 1]), sc_, nds));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int c0 = hc * 32 + 2 * j;
              const float p0 = (c0 < nkv) ? fast_exp2(fmaf(__uint_as_float(x[2 * j]), sl, nl)) : 0.f;
              const float p1 = (c0 + 1 < nkv) ? fast_exp2(fmaf(__uint_as_float(x[2 * j + 1]), sl, nl)) : 0.f;
              pp[hc * 16 + j] = pack2<__nv_bfloat16>(p0, p1);
              dd[hc * 16 + j] = pack2<__nv_bfloat16>(p0 * fmaf(__uint_as_float(y[2 * j]), sc_, nds),
                                                     p1 * fmaf(__uint_as_float(y[2 * j + 1]), sc_, nds));
            }
          }
        }
        if (threadIdx.x == 0) TRACE(1, 16 + sc * 8 + 2);
        // P / dS of the previous step must have been consumed before the rows are overwritten
        ok = __all_sync(0xffffffffu, mbar_wait(&pds_free, (sc & 1) ^ 1, abort));
        if (!ok) break;
        if (threadIdx.x == 0) TRACE(1, 16 + sc * 8 + 3);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int off = ((c ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(prow + off) = make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
          *reinterpret_cast<uint4*>(dsrow + off) = make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);
        }
        fence_async_smem();                           // make the rows visible to the tensor core's reads
        mbar_arrive(&pds_full);
        if (threadIdx.x == 0) TRACE(1, 16 + sc * 8 + 4);
      }
    }
  } else if (warp < 8) {
    // ======================= epilogue (warps 4-7): one head-dim lane per thread =======================
    const int d = (warp - 4) * 32 + lane;
    const int te = threadIdx.x - 128;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t ic = 0;
    bool ok = true;
    for (uint32_t n = 0; ok; ++n) {
      ok = __all_sync(0xffffffffu, mbar_wait(&sched_full[n & 3], (n >> 2) & 1, abort));
      if (!ok) break;
      const Item it = s_items[n & 3];
      mbar_arrive(&sched_empty[n & 3]);
      if (it.n_ent < 0) break;
      const int64_t t0 = static_cast<int64_t>(it.blk) * 64;
      const int n_blk = static_cast<int>(p.n_tokens - t0 < 64 ? p.n_tokens - t0 : 64);
      const int64_t row_bytes = static_cast<int64_t>(p.H) * 256;
      const int64_t base = ((static_cast<int64_t>(it.b) * p.n_tokens + t0) * p.H + it.h) * 256;
      if (!it.active) {
        for (int c = te; c < n_blk * 16; c += 128) {
          const int64_t off = base + (c >> 4) * row_bytes + (c & 15) * 16;
          *reinterpret_cast<uint4*>(p.dk + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(p.dv + off) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int acc = ic & 1, ph = (ic >> 1) & 1;
      if (te == 0) TRACE(3, 16 + ic * 4 + 0);
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], ph, abort));
      if (!ok) break;
      if (te == 0) TRACE(3, 16 + ic * 4 + 1);
      tc_fence_after();
#pragma unroll
      for (int mat = 0; mat < 2; ++mat) {
        char* outp = (mat == 0 ? p.dv : p.dk) + base;
        const uint32_t col = mat == 0 ? col_dv(acc) : col_dk(acc);
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          uint32_t x[32];
          tmem_ld32_nowait(tm + lane_base + col + hc * 32, x);
          tmem_ld_wait();
          // lanes d (even) and d+1 trade values so that each writes one packed pair of head dims
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float a = __uint_as_float(x[2 * j]), c = __uint_as_float(x[2 * j + 1]);
            const float got = __shfl_xor_sync(0xffffffffu, (lane & 1) ? a : c, 1);
            const int key = hc * 32 + 2 * j + (lane & 1);
            const uint32_t w = (lane & 1) ? pack2<__nv_bfloat16>(got, c) : pack2<__nv_bfloat16>(a, got);
            if (key < n_blk) *reinterpret_cast<uint32_t*>(outp + key * row_bytes + (d & ~1) * 2) = w;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_free[acc]);
      if (te == 0) TRACE(3, 16 + ic * 4 + 2);
      ++ic;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (threadIdx.x == 0 && s_abort) atomicExch(p.status, NSA_ERR_CUDA);
}

}  // namespace

// Launches the tensor-core dK/dV kernel when it covers the call (*launched = true).  `groups`
// must be sorted ascending inside each bucket (nsa_inverted_index does that).
int try_launch_sel_bwd_dkv_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* groups,
                              const int32_t* offsets, const float* lse, const float* delta, const void* d_out,
                              const int64_t* do_stride, void* dk, void* dv, int B, int64_t M, int H, int D, int T,
                              int block_size, int chunk_size, int causal, int G, float scale, int dtype,
                              int32_t* counter, cudaStream_t stream, bool* launched) {
  *launched = false;
  if (counter == nullptr) return NSA_OK;
  const char* env = getenv("OMNIMEM_B200_BWD_KERNEL");
  if (env != nullptr && std::string(env) == "general") return NSA_OK;
  if (dtype != NSA_BF16 || D != 128 || block_size != 64 || G > 64 || G < 16 || H == 1) return NSA_OK;
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  CUtensorMap mapQ, mapDO, mapK, mapV;
  int rc;
  if ((rc = make_qkv_maps(q, q_stride, kv, B, M, H, &mapQ, &mapK, &mapV))) return rc;
  if ((rc = make_qkv_maps(d_out, do_stride, nullptr, B, M, H, &mapDO, nullptr, nullptr))) return rc;
  TcDkvParams p;
  p.groups = groups; p.offsets = offsets; p.lse = lse; p.delta = delta;
  p.dk = static_cast<char*>(dk); p.dv = static_cast<char*>(dv);
  p.block_table = kv->block_table; p.max_blocks = kv->max_blocks; p.paged = kv->mode == NSA_KV_PAGED;
  p.n_tokens = kv->n_tokens; p.M = M; p.NS = cdiv64(kv->n_tokens, 64);
  p.B = B; p.H = H; p.T = T; p.G = G; p.MG = static_cast<int>(cdiv64(M, G)); p.chunk_size = chunk_size; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  if ((rc = device_status_address(&p.status))) return rc;
  p.counter = counter;
  NSA_CUDA_OK(cudaMemsetAsync(counter, 0, sizeof(int32_t), stream));
  int dev = 0, sms = 0;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int64_t n_items = static_cast<int64_t>(B) * H * p.NS;
  if (n_items > 0x7fffffff) return NSA_OK;
  const int grid = static_cast<int>(n_items < sms ? n_items : sms);
  const size_t smem = kSmemTiles + 1024;
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  sel_bwd_dkv_tc_kernel<<<grid, kThreads, smem, stream>>>(mapQ, mapDO, mapK, mapV, p);
  NSA_LAUNCH_OK("sel_bwd_dkv_tc_kernel");
  *launched = true;
  return NSA_OK;
}

}  // namespace nsa

#ifdef NSA_TC_TRACE
extern "C" int nsa_debug_trace_dkv(long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace_dkv, sizeof(long long) * 4 * 1024));
  return NSA_OK;
}
#endif
