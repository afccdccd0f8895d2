// Selection attention backward, dK/dV half, on tcgen05 / TMEM / TMA for the page geometry
// (bf16, D = 128, 64-token blocks, query groups of up to 64 rows, dense or paged K/V).
//
// Ownership as in the general kernel: one work item = one (batch, head, KV block); the item's
// dK / dV tile is produced by exactly one thread block, from the block's bucket of query groups
// in ascending group order - no atomics, bit-reproducible.  Persistent thread blocks (one per
// SM) take items from a global counter.  A step is ONE bucket entry (one query group against
// the item's block); most buckets hold one to three entries, so small steps in a deep pipeline
// beat wide ones.  Roles, pipelined across steps and across items:
//   warp 11  scheduler: item tickets from the global counter, decoded a few items ahead and
//            published, with the bucket's first entries, in a small ring the other roles follow
//   warp 8   producer (one lane): nothing but copies - the K, V tile of the item and, per step,
//            the Q and dO rows of the group into a four-stage ring, one TMA copy per tile
//   warp 9   MMA issuer 1, per step:  S = Q K^T, dP = dO V^T          (M=64, N=64, K=128)
//   warp 10  MMA issuer 2, per step:  dV^T += dO^T P,  dK^T += Q^T dS  (M=128 = head dim, N=64 keys, K=64 rows)
//   warps 0-3 and 12-15  row arithmetic on the accumulator fragments (16 rows x 64 keys per warp;
//            the first group takes the even steps, the second the odd ones):
//            P = exp2(S c - LSE), dS = P (dP - delta) scale, stored as bf16 with stmatrix into
//            the 128-byte-swizzled shared-memory tiles the second products read; each thread
//            loads its rows' LSE and delta itself while S and dP are being computed
//   warps 4-7  epilogue: read dV^T / dK^T from TMEM, transpose into the ring stage of the item's
//            last step and store the two tiles with TMA; items with an empty bucket are zero-filled here
// S/dP, the P/dS tiles and the dV^T/dK^T accumulators are double buffered.
#include "sel_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <string>

namespace nsa {

int device_status_address(int32_t** out);
int make_tile_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                   CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV);

#ifdef NSA_TC_TRACE
// Debug build only: clock64 stamps of thread block 0; [0] MMA issuers, [1] row thread 0, [2] producer, [3] epilogue.
__device__ long long g_trace_dkv[4][1024];
#define TRACE(role, slot) do { if (blockIdx.x == 0 && (slot) < 1024) g_trace_dkv[role][slot] = clock64(); } while (0)
__device__ unsigned long long g_trace_dkv_span[256][2];   // per thread block: globaltimer at start and end
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#else
#define TRACE(role, slot) do { } while (0)
#endif

namespace {

using namespace tc;

constexpr int kThreads = 512;
constexpr int kStages = 4;               // Q / dO ring
constexpr uint32_t kKVBytes = 32768;     // K tile 16 KiB + V tile 16 KiB
constexpr uint32_t kQdOBytes = 32768;    // Q 16 KiB + dO 16 KiB per stage
constexpr uint32_t kPdSBytes = 16384;    // P 8 KiB + dS 8 KiB per buffer
// The epilogue stages the item's dV and dK tiles (16 KiB each) in the ring stage of the item's
// LAST step: that stage is dead once the last products have run, and handing it back to the
// producer a little later costs less than a staging buffer that would take a ring stage away.
constexpr uint32_t kSmemTiles = 2 * kKVBytes + kStages * kQdOBytes + 2 * kPdSBytes;

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

constexpr uint32_t kSched = 4;           // items the scheduler may run ahead of the slowest role
constexpr int kItemGroups = 16;          // bucket entries the scheduler copies into the item
struct Item {
  int b, h, blk, beg, n_ent, row;
  bool active;
  int g[kItemGroups];                    // the bucket's first entries (query groups); later ones are read from global memory
};

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
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Zeroes the scheduling counter as a kernel, so that the launch chain dQ kernel -> this -> dK/dV
// kernel stays a chain of kernels (a memset between two kernels would end the early start).
__global__ void zero_counter_kernel(int32_t* counter) {
  chain_release();
  chain_wait();                                // completes only after the kernel before it: the next kernel's wait relies on that
  *counter = 0;
}

__global__ void __launch_bounds__(kThreads, 1)
sel_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapDO,
                      const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                      const __grid_constant__ CUtensorMap mapDK, const __grid_constant__ CUtensorMap mapDV,
                      const TcDkvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sKV = tiles;                               // [buffer]{ K [2][64][128 B], V [2][64][128 B] }, item i in buffer i & 1
  uint8_t* sQdO = tiles + 2 * kKVBytes;               // [stage]{ Q [2][64][128 B], dO [2][64][128 B] }
  uint8_t* sPdS = sQdO + kStages * kQdOBytes;         // [buffer]{ P [64 q][128 B], dS [64 q][128 B] } swizzled

  __shared__ uint64_t kv_full[2], kv_empty[2], qdo_full[kStages], qdo_empty[kStages], sdp_full[2], sdp_free[2], pds_full[2],
      pds_free[2], acc_full[2], acc_free[2];
  __shared__ uint64_t sched_full[kSched], sched_empty[kSched];
  __shared__ Item s_items[kSched];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

#ifdef NSA_TC_TRACE
  if (threadIdx.x == 0 && blockIdx.x < 256) g_trace_dkv_span[blockIdx.x][0] = global_ns();
#endif
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    // The host sizes the dynamic segment as the tiles plus the padding up to the next 1 KiB
    // boundary after the static variables; refuse to run if that did not work out.
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (tiles + kSmemTiles > smem_raw + dyn_bytes) {
      if (threadIdx.x == 0) atomicExch(p.status, NSA_ERR_CUDA);
      return;
    }
  }
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kSched; ++i) { mbar_init(&sched_full[i], 1); mbar_init(&sched_empty[i], 387); }
    for (int i = 0; i < kStages; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1);
      mbar_init(&sdp_full[i], 1); mbar_init(&sdp_free[i], 256);
      mbar_init(&pds_full[i], 256); mbar_init(&pds_free[i], 1);
      mbar_init(&acc_full[i], 1); mbar_init(&acc_free[i], 128);
    }
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapDO); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  chain_wait();                                // everything above needs no result of the kernels before this one
  const uint32_t tm = tmem_base_s;
  volatile int* abort = &s_abort;
  const int64_t n_items = static_cast<int64_t>(p.B) * p.H * p.NS;
  const int64_t bucket_row = static_cast<int64_t>(p.MG) * p.T;

  if (warp == 8) {
    // ======================= producer (one lane) =======================
    // Issues copies and nothing else: the item and its bucket entries come from the scheduler's
    // ring, so no global load sits between two copies.
    if (lane == 0) {
      uint32_t ic = 0, sc = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        ok = mbar_wait(&sched_full[n % kSched], (n / kSched) & 1, abort);
        if (!ok) break;
        const Item* it = &s_items[n % kSched];
        const int n_ent = it->n_ent;
        if (n_ent <= 0) {
          mbar_arrive(&sched_empty[n % kSched]);
          if (n_ent < 0) break;
          continue;
        }
        const int ib = it->b, ih = it->h, irow = it->row;
        TRACE(2, 16 + sc * 4 + 0);
        const int kb = ic & 1;
        ok = mbar_wait(&kv_empty[kb], ((ic >> 1) & 1) ^ 1, abort);
        if (!ok) break;
        TRACE(2, 16 + sc * 4 + 1);
        {
          uint8_t* kvb = sKV + kb * kKVBytes;
          mbar_expect_tx(&kv_full[kb], kKVBytes);
          if (p.paged) {
            tma_load_3d(kvb, &mapK, 0, irow, 0, &kv_full[kb]);
            tma_load_3d(kvb + 16384, &mapV, 0, irow, 0, &kv_full[kb]);
          } else {
            tma_load_5d(kvb, &mapK, 0, ih, irow, 0, ib, &kv_full[kb]);
            tma_load_5d(kvb + 16384, &mapV, 0, ih, irow, 0, ib, &kv_full[kb]);
          }
        }
        const int32_t* bucket = p.groups + (static_cast<int64_t>(ib) * p.H + ih) * bucket_row + it->beg;
        for (int t = 0; t < n_ent; ++t, ++sc) {
          const int st = sc % kStages, ph = (sc / kStages) & 1;
          const int g = t < kItemGroups ? it->g[t] : bucket[t];
          const int m0 = g * p.G;
          TRACE(2, 16 + sc * 4 + 3);
          ok = mbar_wait(&qdo_empty[st], ph ^ 1, abort);
          if (!ok) break;
          TRACE(2, 16 + sc * 4 + 2);
          uint8_t* dq = sQdO + st * kQdOBytes;
          mbar_expect_tx(&qdo_full[st], kQdOBytes);
          tma_load_5d(dq, &mapQ, 0, ih, m0, 0, ib, &qdo_full[st]);
          tma_load_5d(dq + 16384, &mapDO, 0, ih, m0, 0, ib, &qdo_full[st]);
        }
        mbar_arrive(&sched_empty[n % kSched]);              // the item's bucket entries are no longer needed
        ++ic;
      }
      if (*abort) {
        // consumers have stopped: wait (bounded) for the copies still in flight
        for (uint32_t u = (ic > 2 ? ic - 2 : 0); u < ic; ++u) mbar_wait(&kv_full[u & 1], (u >> 1) & 1, abort);
        for (uint32_t u = (sc > kStages ? sc - kStages : 0); u < sc; ++u) mbar_wait(&qdo_full[u % kStages], (u / kStages) & 1, abort);
      }
    }
  } else if (warp == 9) {
    // ======================= MMA issuer 1: S and dP of every step =======================
    // The whole warp runs the loop (warp-uniform control flow keeps the descriptor arithmetic in
    // uniform registers); one elected lane issues.
    {
      constexpr uint32_t idesc_first = instr_desc_bf16(64, 64, 0, 0);     // both operands K-major
      const uint32_t el = elect_one();
      uint32_t ic = 0, sc = 0;
      bool ok = true;
      // A wait on a barrier whose phase is long complete still costs a round trip of a few hundred
      // cycles, and this warp has up to four of them per step.  So the barriers of the NEXT step
      // (and, on an item's last step, of the next item) are tested before this step's products
      // are issued and the answers read afterwards: a phase seen complete stays complete until
      // this warp itself has used it.
      bool have_sched = false, have_kv = false, have_step = false;
      for (uint32_t n = 0; ok; ++n) {
        if (!have_sched && !__all_sync(0xffffffffu, mbar_wait(&sched_full[n % kSched], (n / kSched) & 1, abort))) break;
        have_sched = false;
        const int n_ent = s_items[n % kSched].n_ent;
        __syncwarp();
        if (el) mbar_arrive(&sched_empty[n % kSched]);
        if (n_ent < 0) break;
        if (n_ent == 0) continue;
        if (!have_kv && !__all_sync(0xffffffffu, mbar_wait(&kv_full[ic & 1], (ic >> 1) & 1, abort))) break;
        have_kv = false;
        const uint32_t aKV = smem_u32(sKV + (ic & 1) * kKVBytes);
        const uint64_t dK = smem_desc(aKV, 16, 1024), dV = smem_desc(aKV + 16384, 16, 1024);
        for (int t = 0; t < n_ent; ++t, ++sc) {
          const int st = sc % kStages, sb = sc & 1;
          if (!have_step) {
            ok = __all_sync(0xffffffffu, mbar_wait(&qdo_full[st], (sc / kStages) & 1, abort) &&
                                         mbar_wait(&sdp_free[sb], ((sc >> 1) & 1) ^ 1, abort));
            if (!ok) break;
          }
          TRACE(0, 16 + sc * 8 + 2);
          tc_fence_after();
          const uint32_t sn = sc + 1, icn = ic + 1, nn = n + 1;
          const bool last = t == n_ent - 1;
          const bool nxt_q = mbar_test(&qdo_full[sn % kStages], (sn / kStages) & 1);
          const bool nxt_s = mbar_test(&sdp_free[sn & 1], ((sn >> 1) & 1) ^ 1);
          const bool nxt_kv = last && mbar_test(&kv_full[icn & 1], (icn >> 1) & 1);
          const bool nxt_it = last && mbar_test(&sched_full[nn % kSched], (nn / kSched) & 1);
          const uint32_t aQ = smem_u32(sQdO + st * kQdOBytes);
          const uint64_t dQ = smem_desc(aQ, 16, 1024), dDO = smem_desc(aQ + 16384, 16, 1024);
          const uint32_t ts = tm + col_s(sb), tdp = tm + col_dp(sb);
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ss(ts, desc_advance(dQ, (kk >> 2) * 8192 + (kk & 3) * 32),
                      desc_advance(dK, (kk >> 2) * 8192 + (kk & 3) * 32), idesc_first, kk > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ss(tdp, desc_advance(dDO, (kk >> 2) * 8192 + (kk & 3) * 32),
                      desc_advance(dV, (kk >> 2) * 8192 + (kk & 3) * 32), idesc_first, kk > 0 ? 1u : 0u);
            umma_commit(&sdp_full[sb]);
            if (last) umma_commit(&kv_empty[ic & 1]);
          }
          __syncwarp();
          have_step = __all_sync(0xffffffffu, nxt_q && nxt_s);
          if (last) {
            have_kv = __all_sync(0xffffffffu, nxt_kv);
            have_sched = __all_sync(0xffffffffu, nxt_it);
          }
          TRACE(0, 16 + sc * 8 + 3);
        }
        ++ic;
      }
    }
  } else if (warp == 10) {
    // ======================= MMA issuer 2: dV^T and dK^T of every step =======================
    // A warp of its own, so that these products start the moment P / dS are in shared memory
    // while issuer 1 already waits for the tiles of a later step.
    {
      constexpr uint32_t idesc_second = instr_desc_bf16(128, 64, 1, 1);   // both operands MN-major
      const uint32_t el = elect_one();
      uint32_t ic = 0, sc = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        if (!__all_sync(0xffffffffu, mbar_wait(&sched_full[n % kSched], (n / kSched) & 1, abort))) break;
        const int n_ent = s_items[n % kSched].n_ent;
        __syncwarp();
        if (el) mbar_arrive(&sched_empty[n % kSched]);
        if (n_ent < 0) break;
        if (n_ent == 0) continue;
        const int acc = ic & 1;
        for (int t = 0; t < n_ent; ++t, ++sc) {
          const int st = sc % kStages, pb = sc & 1;
          // the accumulator of two items ago is normally long drained: ask first, so that the round
          // trip of that wait passes while P / dS are still being written
          ok = __all_sync(0xffffffffu, (t > 0 || mbar_wait(&acc_free[acc], ((ic >> 1) & 1) ^ 1, abort)) &&
                                       mbar_wait(&pds_full[pb], (sc >> 1) & 1, abort));
          if (!ok) break;
          TRACE(0, 16 + sc * 8 + 5);
          tc_fence_after();
          const uint32_t aQ = smem_u32(sQdO + st * kQdOBytes), aP = smem_u32(sPdS + pb * kPdSBytes);
          // A: Q^T / dO^T, head dim contiguous, two 64-column boxes 8 KiB apart; B: P / dS, keys contiguous
          const uint64_t dQmn = smem_desc(aQ, 8192, 1024), dDOmn = smem_desc(aQ + 16384, 8192, 1024);
          const uint64_t dP = smem_desc(aP, 16, 1024), dDS = smem_desc(aP + 8192, 16, 1024);
          const uint32_t acc0 = t == 0 ? 0u : 1u;
          const uint32_t tdv = tm + col_dv(acc), tdk = tm + col_dk(acc);
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ss(tdv, desc_advance(dDOmn, kk * 2048), desc_advance(dP, kk * 2048), idesc_second, kk > 0 ? 1u : acc0);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ss(tdk, desc_advance(dQmn, kk * 2048), desc_advance(dDS, kk * 2048), idesc_second, kk > 0 ? 1u : acc0);
            // the stage of the item's last step goes to the epilogue, which hands it back
            if (t != n_ent - 1) umma_commit(&qdo_empty[st]);
            umma_commit(&pds_free[pb]);
            if (t == n_ent - 1) umma_commit(&acc_full[acc]);
          }
          __syncwarp();
          TRACE(0, 16 + sc * 8 + 6);
        }
        ++ic;
      }
    }
  } else if (warp == 11) {
    // ======================= scheduler (whole warp) =======================
    // Takes tickets from the global counter (buckets differ a lot in length, a static split
    // leaves thread blocks idle), decodes each item (bucket bounds, page) and copies the bucket's
    // first entries, one per lane; publishes it in the ring the other roles follow, so the
    // dependent global loads behind one item are paid here, several items ahead of the copies.
    // The ticket of the next item is taken while the current one is decoded; n_ent = -1 ends it.
    int tk = lane == 0 ? atomicAdd(p.counter, 1) : 0;
    for (uint32_t n = 0;; ++n) {
      tk = __shfl_sync(0xffffffffu, tk, 0);
      const bool live = tk < n_items;
      int tk_next = 0;
      if (lane == 0 && live) tk_next = atomicAdd(p.counter, 1);
      Item it{0, 0, 0, 0, -1, 0, false, {}};
      int gl = 0;
      if (live) {
        it = get_item(p, tk);
        if (lane < it.n_ent && lane < kItemGroups)
          gl = p.groups[(static_cast<int64_t>(it.b) * p.H + it.h) * bucket_row + it.beg + lane];
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&sched_empty[n % kSched], ((n / kSched) & 1) ^ 1, abort))) break;
      Item* slot = &s_items[n % kSched];
      if (lane == 0) {
        slot->b = it.b; slot->h = it.h; slot->blk = it.blk; slot->beg = it.beg;
        slot->n_ent = it.n_ent; slot->row = it.row; slot->active = it.active;
      }
      if (lane < kItemGroups) slot->g[lane] = gl;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sched_full[n % kSched]);
      if (it.n_ent < 0) break;
      tk = tk_next;
    }
  } else if (warp < 4 || warp >= 12) {
    // ======================= row arithmetic: P and dS on accumulator fragments =======================
    // Two groups of four warps share every step: warps 0-3 take keys 0-31, warps 12-15 keys 32-63,
    // which halves the time from S / dP to P / dS, a link of the chain that bounds a ring stage's life.
    // Warp w (of its group) owns rows 16w .. 16w+15 of the step's query group (TMEM lanes 32w ..
    // 32w+15 of an M=64 accumulator); thread t holds rows 16w + t/4 and + 8, keys 32 grp + 8i + 2(t%4), +1.
    const int grp = warp >= 12 ? 1 : 0, w4 = warp & 3;
    const bool tracer = threadIdx.x == 0;
    const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;
    const int r0 = w4 * 16 + (lane >> 2), r1 = r0 + 8;
    const int cq = (lane & 3) * 2;
    // stmatrix: this thread supplies the address of row (lane%8) of matrix (lane/8); the four
    // matrices of one instruction are (rows +0, keys 8i), (rows +8, keys 8i), (rows +0, keys 8i+8), (rows +8, keys 8i+8)
    const int st_row = w4 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int st_chunk = lane >> 4;                    // + 2 * instruction index
    uint32_t sc = 0;
    bool ok = true;
    for (uint32_t n = 0; ok; ++n) {
      ok = __all_sync(0xffffffffu, mbar_wait(&sched_full[n % kSched], (n / kSched) & 1, abort));
      if (!ok) break;
      const Item* it = &s_items[n % kSched];
      const int n_ent = it->n_ent;
      if (n_ent <= 0) {
        mbar_arrive(&sched_empty[n % kSched]);
        if (n_ent < 0) break;
        continue;
      }
      const int64_t bh = (static_cast<int64_t>(it->b) * p.H + it->h) * p.M;
      const int32_t* bucket = p.groups + (static_cast<int64_t>(it->b) * p.H + it->h) * bucket_row + it->beg;
      const int64_t t0 = static_cast<int64_t>(it->blk) * 64;
      const int n_blk = static_cast<int>(p.n_tokens - t0 < 64 ? p.n_tokens - t0 : 64);
      for (int t = 0; t < n_ent; ++t, ++sc) {
        const int sb = sc & 1, ph = (sc >> 1) & 1;
        if (tracer) TRACE(1, 16 + sc * 8 + 0);
        // This thread's two rows of the step's query group: LSE * log2(e) (+inf = no such row) and
        // delta, and the step's visible key count; the loads fly while S and dP are computed.
        const int g = t < kItemGroups ? it->g[t] : bucket[t];
        const int64_t m_first = static_cast<int64_t>(g) * p.G;
        const int nq = static_cast<int>(p.M - m_first < p.G ? p.M - m_first : p.G);
        float2 m0, m1;
        m0.x = r0 < nq ? p.lse[bh + m_first + r0] * kLog2e : INFINITY;
        m0.y = r0 < nq ? p.delta[bh + m_first + r0] : 0.f;
        m1.x = r1 < nq ? p.lse[bh + m_first + r1] * kLog2e : INFINITY;
        m1.y = r1 < nq ? p.delta[bh + m_first + r1] : 0.f;
        int nkv = n_blk;
        if (p.causal) {
          const int64_t lim = (static_cast<int64_t>(static_cast<uint32_t>(m_first) / static_cast<uint32_t>(p.chunk_size)) + 1) * p.chunk_size - t0;
          if (lim < nkv) nkv = static_cast<int>(lim < 0 ? 0 : lim);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&sdp_full[sb], ph, abort));
        if (!ok) break;
        if (tracer) TRACE(1, 16 + sc * 8 + 1);
        tc_fence_after();
        uint32_t x[16], y[16];
        tmem_ld_16x256b_x4_nowait(tm + lane_base + col_s(sb) + 32 * grp, x);
        tmem_ld_16x256b_x4_nowait(tm + lane_base + col_dp(sb) + 32 * grp, y);
        // the buffer's previous P / dS (two steps ago) must have been consumed: normally long true,
        // so poll once here, where the round trip hides behind the TMEM load
        const bool pds_ok = mbar_try(&pds_free[sb], ph ^ 1);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&sdp_free[sb]);
        const float sl = p.scale_log2, sc_ = p.scale;
        const float nl0 = -m0.x, nl1 = -m1.x, nd0 = -m0.y * sc_, nd1 = -m1.y * sc_;
        // x[4i], x[4i+1]: row r0, keys 32 grp + 8i + cq, +1;  x[4i+2], x[4i+3]: row r1, same keys.
        // Afterwards x[2i], x[2i+1] hold the packed P of (r0, r1) for key block i, y[2i], y[2i+1] the packed dS.
        if (nkv == 64) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float p00 = fast_exp2(fmaf(__uint_as_float(x[4 * i]), sl, nl0));
            const float p01 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 1]), sl, nl0));
            const float p10 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 2]), sl, nl1));
            const float p11 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 3]), sl, nl1));
            const uint32_t d0 = pack2<__nv_bfloat16>(p00 * fmaf(__uint_as_float(y[4 * i]), sc_, nd0),
                                                     p01 * fmaf(__uint_as_float(y[4 * i + 1]), sc_, nd0));
            const uint32_t d1 = pack2<__nv_bfloat16>(p10 * fmaf(__uint_as_float(y[4 * i + 2]), sc_, nd1),
                                                     p11 * fmaf(__uint_as_float(y[4 * i + 3]), sc_, nd1));
            x[2 * i] = pack2<__nv_bfloat16>(p00, p01);
            x[2 * i + 1] = pack2<__nv_bfloat16>(p10, p11);
            y[2 * i] = d0;
            y[2 * i + 1] = d1;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int c = 32 * grp + 8 * i + cq;
            const float p00 = (c < nkv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i]), sl, nl0)) : 0.f;
            const float p01 = (c + 1 < nkv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 1]), sl, nl0)) : 0.f;
            const float p10 = (c < nkv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 2]), sl, nl1)) : 0.f;
            const float p11 = (c + 1 < nkv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 3]), sl, nl1)) : 0.f;
            const uint32_t d0 = pack2<__nv_bfloat16>(p00 * fmaf(__uint_as_float(y[4 * i]), sc_, nd0),
                                                     p01 * fmaf(__uint_as_float(y[4 * i + 1]), sc_, nd0));
            const uint32_t d1 = pack2<__nv_bfloat16>(p10 * fmaf(__uint_as_float(y[4 * i + 2]), sc_, nd1),
                                                     p11 * fmaf(__uint_as_float(y[4 * i + 3]), sc_, nd1));
            x[2 * i] = pack2<__nv_bfloat16>(p00, p01);
            x[2 * i + 1] = pack2<__nv_bfloat16>(p10, p11);
            y[2 * i] = d0;
            y[2 * i + 1] = d1;
          }
        }
        if (tracer) TRACE(1, 16 + sc * 8 + 2);
        if (!__all_sync(0xffffffffu, pds_ok)) {
          ok = __all_sync(0xffffffffu, mbar_wait(&pds_free[sb], ph ^ 1, abort));
          if (!ok) break;
        }
        if (tracer) TRACE(1, 16 + sc * 8 + 3);
        const uint32_t aP = smem_u32(sPdS + sb * kPdSBytes) + st_row * 128;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint32_t off = static_cast<uint32_t>(((4 * grp + 2 * q + st_chunk) ^ (st_row & 7)) << 4);
          stmatrix_x4(aP + off, x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
          stmatrix_x4(aP + 8192 + off, y[4 * q], y[4 * q + 1], y[4 * q + 2], y[4 * q + 3]);
        }
        fence_async_smem();                           // make the rows visible to the tensor core's reads
        mbar_arrive(&pds_full[sb]);
        if (tracer) TRACE(1, 16 + sc * 8 + 4);
      }
      if (ok) mbar_arrive(&sched_empty[n % kSched]);        // the item's bucket entries are no longer needed
    }
  } else if (warp < 8) {
    // ======================= epilogue (warps 4-7): one head-dim lane per thread =======================
    const int te = threadIdx.x - 128;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t ic = 0, sc = 0;
    bool ok = true;
    for (uint32_t n = 0; ok; ++n) {
      ok = __all_sync(0xffffffffu, mbar_wait(&sched_full[n % kSched], (n / kSched) & 1, abort));
      if (!ok) break;
      const Item it = s_items[n % kSched];
      mbar_arrive(&sched_empty[n % kSched]);
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
      // acc_full also says that every product reading the last step's Q / dO stage has run:
      // the stage now holds { dV, dK }[2][64 keys][128 B] swizzled, for the tile stores
      sc += static_cast<uint32_t>(it.n_ent);
      const int st_last = static_cast<int>((sc - 1) % kStages);
      uint8_t* sOut = sQdO + st_last * kQdOBytes;
      // Accumulator fragments (16 head-dim lanes x 64 keys per load) are packed to bf16 pairs of
      // adjacent keys and stored TRANSPOSED, 8 x 8 at a time, into the [key][head dim] tiles.
#pragma unroll
      for (int mat = 0; mat < 2; ++mat) {
        const uint32_t col = mat == 0 ? col_dv(acc) : col_dk(acc);
#pragma unroll
        for (int lh = 0; lh < 2; ++lh) {                 // lanes 0-15 and 16-31 of this warp's quadrant
          uint32_t x[32];
          tmem_ld_16x256b_x8_nowait(tm + lane_base + (static_cast<uint32_t>(lh * 16) << 16) + col, x);
          tmem_ld_wait();
          if (mat == 1 && lh == 1) { tc_fence_before(); mbar_arrive(&acc_free[acc]); }
          // x[4i], x[4i+1]: head dim D0 + lane/4, keys 8i + 2(lane%4), +1;  x[4i+2], x[4i+3]: head dim + 8
          const int D0 = (warp - 4) * 32 + lh * 16;
          const int dsel = D0 + ((lane >> 3) & 1) * 8;   // head dims of the matrix this lane addresses
          const uint32_t boxa = smem_u32(sOut + mat * 16384 + (dsel >> 6) * 8192);
          const uint32_t dchunk = static_cast<uint32_t>((dsel & 63) >> 3);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int i0 = 2 * q, i1 = 2 * q + 1;
            const uint32_t a0 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i0]), __uint_as_float(x[4 * i0 + 1]));
            const uint32_t b0 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i0 + 2]), __uint_as_float(x[4 * i0 + 3]));
            const uint32_t a1 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i1]), __uint_as_float(x[4 * i1 + 1]));
            const uint32_t b1 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i1 + 2]), __uint_as_float(x[4 * i1 + 3]));
            // matrices: (keys 8 i0.., dims D0..), (keys 8 i0.., dims D0+8..), (keys 8 i1.., D0..), (keys 8 i1.., D0+8..)
            const int key = 8 * (2 * q + (lane >> 4)) + (lane & 7);
            stmatrix_x4_trans(boxa + key * 128 + ((dchunk ^ static_cast<uint32_t>(key & 7)) << 4), a0, b0, a1, b1);
          }
        }
      }
      fence_async_smem();
      named_barrier(3, 128);
      if (te == 0) {
        const int tok = static_cast<int>(t0);
        tma_store_5d(&mapDV, sOut, 0, it.h, tok, 0, it.b);
        tma_store_5d(&mapDK, sOut + 16384, 0, it.h, tok, 0, it.b);
        bulk_commit_group();
        bulk_wait_read_all();                          // the stores have read the stage: back to the producer
        mbar_arrive(&qdo_empty[st_last]);
        TRACE(3, 16 + ic * 4 + 2);
      }
      ++ic;
    }
    if (te == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
#ifdef NSA_TC_TRACE
  if (threadIdx.x == 0 && blockIdx.x < 256) g_trace_dkv_span[blockIdx.x][1] = global_ns();
#endif
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
  if (!(scale > 0.f)) return NSA_OK;   // the kernel folds log2(scale) into the exponent
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  CUtensorMap mapQ, mapDO, mapK, mapV, mapDK, mapDV;
  int rc;
  if ((rc = make_tile_maps(q, q_stride, kv, B, M, H, &mapQ, &mapK, &mapV))) return rc;
  if ((rc = make_tile_maps(d_out, do_stride, nullptr, B, M, H, &mapDO, nullptr, nullptr))) return rc;
  {
    // dK / dV are contiguous [B, N, H, 128]: the same tile boxes as the loads, used for tile stores
    const int64_t N = kv->n_tokens;
    const int64_t st[4] = {N * H * 128, static_cast<int64_t>(H) * 128, 128, 1};
    if ((rc = make_tile_maps(dk, st, nullptr, B, N, H, &mapDK, nullptr, nullptr))) return rc;
    if ((rc = make_tile_maps(dv, st, nullptr, B, N, H, &mapDV, nullptr, nullptr))) return rc;
  }
  TcDkvParams p;
  p.groups = groups; p.offsets = offsets; p.lse = lse; p.delta = delta;
  p.dk = static_cast<char*>(dk); p.dv = static_cast<char*>(dv);
  p.block_table = kv->block_table; p.max_blocks = kv->max_blocks; p.paged = kv->mode == NSA_KV_PAGED;
  p.n_tokens = kv->n_tokens; p.M = M; p.NS = cdiv64(kv->n_tokens, 64);
  p.B = B; p.H = H; p.T = T; p.G = G; p.MG = static_cast<int>(cdiv64(M, G)); p.chunk_size = chunk_size; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  if ((rc = device_status_address(&p.status))) return rc;
  p.counter = counter;
  int dev = 0, sms = 0;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int64_t n_items = static_cast<int64_t>(B) * H * p.NS;
  if (n_items > 0x7fffffff) return NSA_OK;
  const int grid = static_cast<int>(n_items < sms ? n_items : sms);
  // the tiles start at the first 1 KiB boundary after the kernel's static shared variables
  cudaFuncAttributes fa;
  NSA_CUDA_OK(cudaFuncGetAttributes(&fa, sel_bwd_dkv_tc_kernel));
  const size_t smem = kSmemTiles + (1024 - fa.sharedSizeBytes % 1024) % 1024;
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  NSA_CUDA_OK(launch_chained(kChainDkv, zero_counter_kernel, dim3(1), dim3(1), 0, stream, counter));
  NSA_CUDA_OK(launch_chained(kChainDkv, sel_bwd_dkv_tc_kernel, dim3(grid), dim3(kThreads), smem, stream, mapQ, mapDO, mapK, mapV, mapDK, mapDV, p));
  NSA_LAUNCH_OK("sel_bwd_dkv_tc_kernel");
  *launched = true;
  return NSA_OK;
}

}  // namespace nsa

#ifdef NSA_TC_TRACE
extern "C" int nsa_debug_trace_dkv_span(unsigned long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace_dkv_span, sizeof(unsigned long long) * 512));
  return NSA_OK;
}
extern "C" int nsa_debug_trace_dkv(long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace_dkv, sizeof(long long) * 4 * 1024));
  return NSA_OK;
}
#endif
