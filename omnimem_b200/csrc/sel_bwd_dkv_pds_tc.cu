// Selection attention backward, dK/dV half, from STORED probabilities: the variant of the
// tcgen05 dK/dV kernel that runs after a dQ kernel which wrote P and dS of every (query group, head,
// selected block) pair to a scratch buffer (bf16, one 8 KiB tile each, in the 128-byte-swizzled
// [row][64 keys] image an MMA operand has in shared memory).  S, dP and the exponentials are then
// not computed a second time: this kernel only streams operands and issues the two products
//     dV^T += dO^T P      dK^T += Q^T dS        (M=128 = head dim, N=64 keys, K=64 rows)
// and needs neither the K / V tiles nor LSE / delta.
//
// Ownership as in the recomputing kernel: one work item = one (batch, head, KV block), its dK / dV
// tile produced by exactly one thread block from the block's bucket of query groups in ascending
// (group, slot) order - no atomics, bit-reproducible.  Persistent thread blocks (one per SM) take
// items from a global counter.  A step is one bucket entry.  Roles:
//   warp 6   scheduler: item tickets, decoded a few items ahead and published with the bucket's
//            first entries (group and slot) in a small ring the other roles follow
//   warps 4, 7  producers (one lane each): per step one stage of the ring = the group's Q and dO rows
//            (warp 4: two TMA tile copies) and the pair's P / dS tiles (warp 7: one 16 KiB bulk copy);
//            an issue costs a thread a few hundred cycles, so the two halves have a thread each
//   warp 5   MMA issuer: the two products of every step; accumulators double buffered across items
//   warps 0-3  epilogue: read dV^T / dK^T from TMEM, transpose into two staging tiles and store them
//            with TMA; items with an empty bucket are zero-filled here
#include "sel_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <string>

namespace nsa {

int device_status_address(int32_t** out);
int make_tile_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                   CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV);

#ifdef NSA_TC_TRACE
// Debug build only: clock64 stamps of thread block 0; [0] MMA issuer, [1] producer, [2] epilogue.
__device__ long long g_trace_pds[3][1024];
#define TRACE(role, slot) do { if (blockIdx.x == 0 && (slot) < 1024) g_trace_pds[role][slot] = clock64(); } while (0)
#else
#define TRACE(role, slot) do { } while (0)
#endif

namespace {

using namespace tc;

constexpr int kThreads = 256;
constexpr int kStages = 4;
constexpr uint32_t kQdOBytes = 32768;    // Q 16 KiB + dO 16 KiB
constexpr uint32_t kPdSBytes = 16384;    // P 8 KiB + dS 8 KiB
constexpr uint32_t kStageBytes = kQdOBytes + kPdSBytes;
constexpr uint32_t kOutBytes = 32768;     // the epilogue's staging tiles: dV 16 KiB + dK 16 KiB
constexpr uint32_t kSmemTiles = kStages * kStageBytes + kOutBytes;
constexpr uint32_t kTmemCols = 256;      // two accumulator pairs of 2 x 64 columns

__device__ __forceinline__ uint32_t col_dv(int acc) { return acc * 128; }
__device__ __forceinline__ uint32_t col_dk(int acc) { return acc * 128 + 64; }

struct PdsDkvParams {
  const int32_t* groups;     // [B,H,MG*T] buckets, ascending inside a bucket
  const int32_t* slots;      // same layout: the entry's position in its group's id list
  const int32_t* offsets;    // [B,H,NS+1]
  const char* pds;           // [B,MG,H,T] x { P 8 KiB, dS 8 KiB }
  char* dk; char* dv;        // contiguous [B,N,H,D]
  const int32_t* block_table;
  int max_blocks, paged;
  int64_t n_tokens, M, NS;
  int B, H, T, G, MG;
  int32_t* status;
  int32_t* counter;          // zeroed before the launch: next work item to hand out
};

constexpr uint32_t kSched = 4;           // items the scheduler may run ahead of the slowest role
constexpr int kItemGroups = 16;          // bucket entries the scheduler copies into the item
struct Item {
  int b, h, blk, beg, n_ent;
  bool active;
  int g[kItemGroups], slot[kItemGroups];
};

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void zero_counter_pds_kernel(int32_t* counter) {
  chain_release();
  chain_wait();                                // completes only after the kernel before it: the next kernel's wait relies on that
  *counter = 0;
}

__global__ void __launch_bounds__(kThreads, 1)
sel_bwd_dkv_pds_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapDO,
                          const __grid_constant__ CUtensorMap mapDK, const __grid_constant__ CUtensorMap mapDV,
                          const PdsDkvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // stage: { Q [2][64][128 B], dO [2][64][128 B], P [64 q][128 B], dS [64 q][128 B] }

  __shared__ uint64_t st_full[kStages], st_empty[kStages], acc_full[2], acc_free[2];
  __shared__ uint64_t sched_full[kSched], sched_empty[kSched];
  __shared__ Item s_items[kSched];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (tiles + kSmemTiles > smem_raw + dyn_bytes) {
      if (threadIdx.x == 0) atomicExch(p.status, NSA_ERR_CUDA);
      return;
    }
  }
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kSched; ++i) { mbar_init(&sched_full[i], 1); mbar_init(&sched_empty[i], 131); }
    for (int i = 0; i < kStages; ++i) { mbar_init(&st_full[i], 2); mbar_init(&st_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_free[i], 128); }
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, kTmemCols);
  if (warp == 4 && lane == 0) { tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapDO); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  chain_wait();                                // everything above needs no result of the kernels before this one
  const uint32_t tm = tmem_base_s;
  volatile int* abort = &s_abort;
  const int64_t n_items = static_cast<int64_t>(p.B) * p.H * p.NS;
  const int64_t bucket_row = static_cast<int64_t>(p.MG) * p.T;

  if (warp == 4 || warp == 7) {
    // ======================= producers (one lane each) =======================
    // warp 4: the step's Q and dO rows; warp 7: its P / dS tiles.  Both follow the item ring and the
    // stage ring on their own; a stage is full when both halves have landed.
    const bool rows = warp == 4;
    if (lane == 0) {
      uint32_t sc = 0;
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
        const int ib = it->b, ih = it->h;
        const int64_t brow = (static_cast<int64_t>(ib) * p.H + ih) * bucket_row + it->beg;
        for (int t = 0; t < n_ent; ++t, ++sc) {
          const int st = sc % kStages, ph = (sc / kStages) & 1;
          const int g = t < kItemGroups ? it->g[t] : p.groups[brow + t];
          if (rows) TRACE(1, 8 + sc * 2);
          ok = mbar_wait(&st_empty[st], ph ^ 1, abort);
          if (!ok) break;
          if (rows) TRACE(1, 8 + sc * 2 + 1);
          uint8_t* sg = tiles + st * kStageBytes;
          if (rows) {
            const int m0 = g * p.G;
            mbar_expect_tx(&st_full[st], kQdOBytes);
            tma_load_5d(sg, &mapQ, 0, ih, m0, 0, ib, &st_full[st]);
            tma_load_5d(sg + 16384, &mapDO, 0, ih, m0, 0, ib, &st_full[st]);
          } else {
            const int slot = t < kItemGroups ? it->slot[t] : p.slots[brow + t];
            const char* src = p.pds + (((((static_cast<int64_t>(ib) * p.MG + g) * p.H + ih) * p.T) + slot) << 14);
            mbar_expect_tx(&st_full[st], kPdSBytes);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(sg + kQdOBytes)), "l"(src), "r"(kPdSBytes), "r"(smem_u32(&st_full[st])) : "memory");
          }
        }
        mbar_arrive(&sched_empty[n % kSched]);              // the item's bucket entries are no longer needed
      }
      if (*abort) {
        // consumers have stopped: wait (bounded) for the copies still in flight
        for (uint32_t u = (sc > kStages ? sc - kStages : 0); u < sc; ++u) mbar_wait(&st_full[u % kStages], (u / kStages) & 1, abort);
      }
    }
  } else if (warp == 5) {
    // ======================= MMA issuer: dV^T and dK^T of every step =======================
    // The whole warp runs the loop (warp-uniform control flow); one elected lane issues.
    constexpr uint32_t idesc = instr_desc_bf16(128, 64, 1, 1);          // both operands MN-major
    const uint32_t el = elect_one();
    uint32_t ic = 0, sc = 0;
    bool ok = true;
    // A wait on a barrier whose phase is long complete still costs a round trip of a few hundred
    // cycles.  So the barriers of the NEXT step (and, on an item's last step, of the next item) are
    // tested before this step's products are issued and the answers read afterwards: a phase seen
    // complete stays complete until this warp itself has used it.
    bool have_sched = false, have_acc = false, have_step = false;
    for (uint32_t n = 0; ok; ++n) {
      if (!have_sched && !__all_sync(0xffffffffu, mbar_wait(&sched_full[n % kSched], (n / kSched) & 1, abort))) break;
      have_sched = false;
      const int n_ent = s_items[n % kSched].n_ent;
      __syncwarp();
      if (el) mbar_arrive(&sched_empty[n % kSched]);
      if (n_ent < 0) break;
      if (n_ent == 0) continue;
      const int acc = ic & 1;
      for (int t = 0; t < n_ent; ++t, ++sc) {
        const int st = sc % kStages;
        TRACE(0, 8 + sc * 2);
        if (t == 0 && !have_acc) {
          ok = __all_sync(0xffffffffu, mbar_wait(&acc_free[acc], ((ic >> 1) & 1) ^ 1, abort));
          if (!ok) break;
        }
        if (!have_step) {
          ok = __all_sync(0xffffffffu, mbar_wait(&st_full[st], (sc / kStages) & 1, abort));
          if (!ok) break;
        }
        TRACE(0, 8 + sc * 2 + 1);
        tc_fence_after();
        const uint32_t sn = sc + 1, icn = ic + 1, nn = n + 1;
        const bool last = t == n_ent - 1;
        const bool nxt_step = mbar_test(&st_full[sn % kStages], (sn / kStages) & 1);
        const bool nxt_acc = last && mbar_test(&acc_free[icn & 1], ((icn >> 1) & 1) ^ 1);
        const bool nxt_it = last && mbar_test(&sched_full[nn % kSched], (nn / kSched) & 1);
        const uint32_t aQ = smem_u32(tiles + st * kStageBytes), aP = aQ + kQdOBytes;
        // A: Q^T / dO^T, head dim contiguous, two 64-column boxes 8 KiB apart; B: P / dS, keys contiguous
        const uint64_t dQmn = smem_desc(aQ, 8192, 1024), dDOmn = smem_desc(aQ + 16384, 8192, 1024);
        const uint64_t dP = smem_desc(aP, 16, 1024), dDS = smem_desc(aP + 8192, 16, 1024);
        const uint32_t acc0 = t == 0 ? 0u : 1u;
        const uint32_t tdv = tm + col_dv(acc), tdk = tm + col_dk(acc);
        if (el) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tdv, desc_advance(dDOmn, kk * 2048), desc_advance(dP, kk * 2048), idesc, kk > 0 ? 1u : acc0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tdk, desc_advance(dQmn, kk * 2048), desc_advance(dDS, kk * 2048), idesc, kk > 0 ? 1u : acc0);
          umma_commit(&st_empty[st]);
          if (t == n_ent - 1) umma_commit(&acc_full[acc]);
        }
        __syncwarp();
        have_step = __all_sync(0xffffffffu, nxt_step);
        if (last) {
          have_acc = __all_sync(0xffffffffu, nxt_acc);
          have_sched = __all_sync(0xffffffffu, nxt_it);
        }
      }
      ++ic;
    }
  } else if (warp == 6) {
    // ======================= scheduler (whole warp) =======================
    int tk = lane == 0 ? atomicAdd(p.counter, 1) : 0;
    for (uint32_t n = 0;; ++n) {
      tk = __shfl_sync(0xffffffffu, tk, 0);
      const bool live = tk < n_items;
      int tk_next = 0;
      if (lane == 0 && live) tk_next = atomicAdd(p.counter, 1);
      int ib = 0, ih = 0, blk = 0, beg = 0, n_ent = -1, gl = 0, sl = 0;
      if (live) {
        const uint32_t iu = static_cast<uint32_t>(tk), ns = static_cast<uint32_t>(p.NS);   // the host keeps B*H*NS below 2^31
        const uint32_t r = iu / ns;
        blk = static_cast<int>(iu - r * ns);
        ib = static_cast<int>(r / static_cast<uint32_t>(p.H));
        // heads in ascending order: the dQ kernel takes the heads from the last to the first, so the tiles
        // of the first heads were written last and are the ones still in L2
        ih = static_cast<int>(r - static_cast<uint32_t>(ib) * static_cast<uint32_t>(p.H));
        const int32_t* offs = p.offsets + (static_cast<int64_t>(ib) * p.H + ih) * (p.NS + 1);
        beg = offs[blk];
        n_ent = offs[blk + 1] - beg;
        if (p.paged) {
          const int page = blk < p.max_blocks ? p.block_table[static_cast<int64_t>(ih) * p.max_blocks + blk] : -1;
          if (page < 0) n_ent = 0;
        }
        if (lane < n_ent && lane < kItemGroups) {
          const int64_t at = (static_cast<int64_t>(ib) * p.H + ih) * bucket_row + beg + lane;
          gl = p.groups[at];
          sl = p.slots[at];
          // the entry's P / dS tiles on their way into L2, several steps before the producer asks for them
          const char* src = p.pds + (((((static_cast<int64_t>(ib) * p.MG + gl) * p.H + ih) * p.T) + sl) << 14);
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(kPdSBytes) : "memory");
        }
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&sched_empty[n % kSched], ((n / kSched) & 1) ^ 1, abort))) break;
      Item* slot = &s_items[n % kSched];
      if (lane == 0) {
        slot->b = ib; slot->h = ih; slot->blk = blk; slot->beg = beg; slot->n_ent = n_ent; slot->active = n_ent > 0;
      }
      if (lane < kItemGroups) { slot->g[lane] = gl; slot->slot[lane] = sl; }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sched_full[n % kSched]);
      if (n_ent < 0) break;
      tk = tk_next;
    }
  } else if (warp < 4) {
    // ======================= epilogue (warps 0-3): one head-dim lane per thread =======================
    const int te = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    uint32_t ic = 0;
    bool ok = true;
    for (uint32_t n = 0; ok; ++n) {
      ok = __all_sync(0xffffffffu, mbar_wait(&sched_full[n % kSched], (n / kSched) & 1, abort));
      if (!ok) break;
      const int ib = s_items[n % kSched].b, ih = s_items[n % kSched].h, blk = s_items[n % kSched].blk;
      const int n_ent = s_items[n % kSched].n_ent;
      mbar_arrive(&sched_empty[n % kSched]);
      if (n_ent < 0) break;
      const int64_t t0 = static_cast<int64_t>(blk) * 64;
      const int n_blk = static_cast<int>(p.n_tokens - t0 < 64 ? p.n_tokens - t0 : 64);
      const int64_t row_bytes = static_cast<int64_t>(p.H) * 256;
      const int64_t base = ((static_cast<int64_t>(ib) * p.n_tokens + t0) * p.H + ih) * 256;
      if (n_ent == 0) {
        for (int c = te; c < n_blk * 16; c += 128) {
          const int64_t off = base + (c >> 4) * row_bytes + (c & 15) * 16;
          *reinterpret_cast<uint4*>(p.dk + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(p.dv + off) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int acc = ic & 1, ph = (ic >> 1) & 1;
      if (te == 0) TRACE(2, 8 + ic * 4);
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], ph, abort));
      if (!ok) break;
      if (te == 0) TRACE(2, 8 + ic * 4 + 1);
      tc_fence_after();
      // the staging tiles { dV, dK }[2][64 keys][128 B] swizzled: free once the previous item's stores have read them
      uint8_t* sOut = tiles + kStages * kStageBytes;
      if (te == 0) bulk_wait_read_all();
      named_barrier(3, 128);
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
          const int D0 = warp * 32 + lh * 16;
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
            const int key = 8 * (2 * q + (lane >> 4)) + (lane & 7);
            stmatrix_x4_trans(boxa + key * 128 + ((dchunk ^ static_cast<uint32_t>(key & 7)) << 4), a0, b0, a1, b1);
          }
        }
      }
      fence_async_smem();
      named_barrier(3, 128);
      if (te == 0) {
        const int tok = static_cast<int>(t0);
        tma_store_5d(&mapDV, sOut, 0, ih, tok, 0, ib);
        tma_store_5d(&mapDK, sOut + 16384, 0, ih, tok, 0, ib);
        bulk_commit_group();
        TRACE(2, 8 + ic * 4 + 2);
      }
      ++ic;
    }
    if (te == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, kTmemCols);
  if (threadIdx.x == 0 && s_abort) atomicExch(p.status, NSA_ERR_CUDA);
}

}  // namespace

// Launches the stored-probabilities dK/dV kernel when it covers the call (*launched = true).
// `pds` must have been written by the tcgen05 dQ kernel for the same call; `groups` / `slots` are
// nsa_inverted_index_slots' outputs.
int try_launch_sel_bwd_dkv_pds_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* groups,
                                  const int32_t* slots, const int32_t* offsets, const void* pds, const void* d_out,
                                  const int64_t* do_stride, void* dk, void* dv, int B, int64_t M, int H, int D, int T,
                                  int block_size, int G, int dtype, int32_t* counter, cudaStream_t stream,
                                  bool* launched) {
  *launched = false;
  if (counter == nullptr || pds == nullptr || slots == nullptr) return NSA_OK;
  if (dtype != NSA_BF16 || D != 128 || block_size != 64 || G > 64 || G < 16 || H == 1) return NSA_OK;
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  CUtensorMap mapQ, mapDO, mapDK, mapDV;
  int rc;
  if ((rc = make_tile_maps(q, q_stride, nullptr, B, M, H, &mapQ, nullptr, nullptr))) return rc;
  if ((rc = make_tile_maps(d_out, do_stride, nullptr, B, M, H, &mapDO, nullptr, nullptr))) return rc;
  {
    const int64_t N = kv->n_tokens;
    const int64_t st[4] = {N * H * 128, static_cast<int64_t>(H) * 128, 128, 1};
    if ((rc = make_tile_maps(dk, st, nullptr, B, N, H, &mapDK, nullptr, nullptr))) return rc;
    if ((rc = make_tile_maps(dv, st, nullptr, B, N, H, &mapDV, nullptr, nullptr))) return rc;
  }
  PdsDkvParams p;
  p.groups = groups; p.slots = slots; p.offsets = offsets; p.pds = static_cast<const char*>(pds);
  p.dk = static_cast<char*>(dk); p.dv = static_cast<char*>(dv);
  p.block_table = kv->block_table; p.max_blocks = kv->max_blocks; p.paged = kv->mode == NSA_KV_PAGED;
  p.n_tokens = kv->n_tokens; p.M = M; p.NS = cdiv64(kv->n_tokens, 64);
  p.B = B; p.H = H; p.T = T; p.G = G; p.MG = static_cast<int>(cdiv64(M, G));
  if ((rc = device_status_address(&p.status))) return rc;
  p.counter = counter;
  int dev = 0, sms = 0;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int64_t n_items = static_cast<int64_t>(B) * H * p.NS;
  if (n_items > 0x7fffffff) return NSA_OK;
  const int grid = static_cast<int>(n_items < sms ? n_items : sms);
  cudaFuncAttributes fa;
  NSA_CUDA_OK(cudaFuncGetAttributes(&fa, sel_bwd_dkv_pds_tc_kernel));
  const size_t smem = kSmemTiles + (1024 - fa.sharedSizeBytes % 1024) % 1024;
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_bwd_dkv_pds_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  NSA_CUDA_OK(launch_chained(kChainDkv, zero_counter_pds_kernel, dim3(1), dim3(1), 0, stream, counter));
  NSA_CUDA_OK(launch_chained(kChainDkv, sel_bwd_dkv_pds_tc_kernel, dim3(grid), dim3(kThreads), smem, stream, mapQ, mapDO, mapDK, mapDV, p));
  NSA_LAUNCH_OK("sel_bwd_dkv_pds_tc_kernel");
  *launched = true;
  return NSA_OK;
}

}  // namespace nsa

#ifdef NSA_TC_TRACE
extern "C" int nsa_debug_trace_pds(long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace_pds, sizeof(long long) * 3 * 1024));
  return NSA_OK;
}
#endif
