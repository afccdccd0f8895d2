// Selection attention backward, dQ half, on tcgen05 / TMEM / TMA for the page geometry
// (bf16, D = 128, 64-token blocks, query groups of up to 64 rows, dense or paged K/V).
//
// One thread block per (batch, query group, head), TWO thread blocks resident per SM (104 KiB of
// tiles and 256 TMEM columns each): the block-list / delta prologue and the store epilogue of one
// block run beside the main loop of the other, and the tensor pipe always has a second queue to
// draw from.  A step is ONE selected block (64 keys):
//     S    = Q  K^T         (M=64, N=64, K=128)    Q is the A operand read from TMEM  warp 9 issues
//     dP   = dO V^T         (M=64, N=64, K=128)                                       warp 9 issues
//     dS   = exp2(S c - LSE + log2 scale) (dP - delta)   on accumulator fragments, stored as bf16
//            with stmatrix into a swizzled shared tile                                warps 0-7 (two groups, half the keys each)
//     dQ^T += K^T dS^T      (M=128 head dims, N=64 rows, K=64 keys; the K tile is read MN-major
//            in place as A, dS K-major as B)                                          warp 10 issues
// Accumulating dQ transposed takes 64 TMEM columns instead of 128; the 64 columns saved hold Q,
// which the row warps move from its landing tile into TMEM in the prologue (tcgen05.st.16x128b),
// so S reads only K from shared memory and the landing tile becomes a third K stage - a K tile
// is held from S(t) to dQ(t), two stages left the copy of K(t+2) on the path every other step.
// Warp 8 builds the list of visible selected blocks and issues every TMA copy (Q and dO once,
// K through a three-stage, V through a two-stage ring).  delta = sum_d(O dO) is reduced in the
// prologue and stored for the dK/dV kernel.  The epilogue packs the dQ^T fragments to bf16 and
// stores them transposed (stmatrix.trans) into the first K stage, dead by then, from where TMA
// tile stores write them.
//
// With a P / dS buffer (STORE = true) the row warps also produce P = exp2(S c - LSE log2e) itself, as a
// second swizzled 8 KiB tile, and the warp that issues dQ^T hands both tiles of the step to a bulk
// store into the (group, head, slot) pair's place in the buffer: the dK/dV kernel then needs no S, dP
// or exponential of its own.  The P tile makes it 112 KiB of tiles: two thread blocks still share an
// SM because the static variables shrink to half a KiB (lists of at most 64 slots).
#include "sel_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <string>

namespace nsa {

int device_status_address(int32_t** out);

#ifdef NSA_TC_TRACE
// Debug build only: clock64 stamps of thread block (0,0,0); [0][..] MMA issuers, [1][..] row thread 0.
__device__ long long g_trace_dq[2][512];
#define TRACE(role, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (slot) < 512) g_trace_dq[role][slot] = clock64(); } while (0)
#else
#define TRACE(role, slot) do { } while (0)
#endif

namespace {

using namespace tc;

constexpr int kThreads = 352;
constexpr int kProducerWarp = 8, kScoreWarp = 9, kGradWarp = 10;   // warps 0-7 do the row arithmetic
constexpr int kMaxSlots = 256;
constexpr uint32_t kTile = 16384;                 // 64 rows x 256 bytes, as two 64-column halves of 8 KiB
constexpr uint32_t kSmemTiles = kTile + 3 * kTile + 2 * kTile + 8192;   // dO, K x3, V x2, dS
constexpr uint32_t kSmemTilesStore = kSmemTiles + 8192;                 // + P
constexpr int kMaxSlotsStore = 64;

constexpr uint32_t kColS = 0;      // 64: S (M=64 rows x 64 keys, fp32)
constexpr uint32_t kColDP = 64;    // 64: dP
constexpr uint32_t kColDQ = 128;   // 64: dQ^T (M=128 head dims x 64 rows, fp32)
constexpr uint32_t kColQ = 192;    // 64: Q as the A operand of S (64 rows x 128 bf16, two per column)
constexpr uint32_t kTmemCols = 256;

struct TcDqParams {
  const int32_t* ids;
  int64_t i_sb, i_sg, i_sh, i_st;
  const char* o; int64_t o_sb, o_sm, o_sh;      // forward output (for delta)
  const char* dO; int64_t do_sb, do_sm, do_sh;
  char* dq; int64_t dq_sb, dq_sm, dq_sh;         // only for zero-filling rows of groups without visible blocks
  const float* lse;
  float* delta;
  const int32_t* block_table;
  int max_blocks, paged;
  int64_t n_tokens, M;
  int H, T, G, chunk_size, causal;
  float scale, scale_log2;
  int32_t* status;
  char* pds;            // optional: P and dS of every (group, head, slot) as 2 x 8 KiB swizzled tiles, for the dK/dV kernel
  int MG;
};

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <bool STORE>
__global__ void __launch_bounds__(kThreads, 2)
sel_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapDO,
                     const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                     const __grid_constant__ CUtensorMap mapDQ, const TcDqParams p) {
  constexpr int kKStages = 3;
  constexpr int kSlots = STORE ? kMaxSlotsStore : kMaxSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sDO = tiles;                                 // [2][64][128 B]
  uint8_t* sK = tiles + kTile;                          // kKStages stages; the last one first receives Q (moved to TMEM
                                                        // in the prologue), the first one is the epilogue's dQ staging tile
  uint8_t* sV = tiles + (1 + kKStages) * kTile;         // 2 stages
  // dS [64 q][128 B] swizzled; with STORE the P tile (same image) comes first, so that { P, dS } is one 16 KiB piece
  uint8_t* sP = tiles + (3 + kKStages) * kTile;
  uint8_t* sDS = STORE ? sP + 8192 : sP;
  uint8_t* sQ = sK + (kKStages - 1) * kTile;            // landing tile of Q
  uint8_t* sOut = sK;                                   // dQ staging tile

  __shared__ uint64_t qdo_full, q_moved, k_full[3], k_empty[3], v_full[2], v_empty[2], sdp_full, sdp_free, ds_full,
      ds_free, dq_final, tile_stored;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort, s_nb;
  __shared__ int s_row[kSlots];
  __shared__ uint8_t s_nvis[kSlots];             // visible tokens of a listed block (1..64)
  __shared__ uint8_t s_slot[kSlots];             // position of a visible block in the group's id list
  // the partial sums of delta: in a tile nothing has touched yet when they are needed
  float* s_part = reinterpret_cast<float*>(sDS);

  if (STORE) {
    // the host sizes the dynamic segment as the tiles plus the padding up to the next 1 KiB boundary
    // after the static variables; refuse to run if that did not work out
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (tiles + kSmemTilesStore > smem_raw + dyn_bytes) {
      if (threadIdx.x == 0) atomicExch(p.status, NSA_ERR_CUDA);
      return;
    }
  }
  // heads in descending order: the forward, which ran just before in a training step, read the K / V of
  // the last heads last, so they are the ones still in L2
  const int g = blockIdx.x, h = p.H - 1 - static_cast<int>(blockIdx.y), b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t m0 = static_cast<int64_t>(g) * p.G;
  const int n_q = static_cast<int>(p.M - m0 < p.G ? p.M - m0 : p.G);
  const int q_chunk = static_cast<int>(m0 / p.chunk_size);
  const int64_t bhm = (static_cast<int64_t>(b) * p.H + h) * p.M + m0;

  chain_release();
  if (threadIdx.x == 0) TRACE(1, 0);
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(&qdo_full, 1);
    mbar_init(&q_moved, 256);
    for (int i = 0; i < kKStages; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(&sdp_full, 1); mbar_init(&sdp_free, 256);
    mbar_init(&ds_full, 256); mbar_init(&ds_free, 1);
    mbar_init(&dq_final, 1);
    mbar_init(&tile_stored, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, kTmemCols);
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapDO); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  chain_wait();                                // everything above needs no result of the kernel before this one
  // ---- row warps start the loads for delta = sum_d O dO right away: thread j takes query row j / 4,
  // head dims [32 (j & 3), +32)
  const int drow_q = threadIdx.x >> 2, dquarter = threadIdx.x & 3;
  uint4 ro_[4], rd_[4];
  if (warp < 8 && drow_q < n_q) {
    const uint4* orow = reinterpret_cast<const uint4*>(p.o + (b * p.o_sb + (m0 + drow_q) * p.o_sm + h * p.o_sh) * 2) + dquarter * 4;
    const uint4* drow = reinterpret_cast<const uint4*>(p.dO + (b * p.do_sb + (m0 + drow_q) * p.do_sm + h * p.do_sh) * 2) + dquarter * 4;
#pragma unroll
    for (int c = 0; c < 4; ++c) { ro_[c] = orow[c]; rd_[c] = drow[c]; }
  }
  // ---- list of the visible selected blocks (TMA row coordinate, visible tokens), compacted by the producer warp
  if (warp == kProducerWarp) {
    int base = 0;
    for (int t0 = 0; t0 < p.T; t0 += 32) {
      const int t = t0 + lane;
      int row = -1, nv = 0;
      if (t < p.T) {
        const int bid = p.ids[b * p.i_sb + g * p.i_sg + h * p.i_sh + t * p.i_st];
        if (bid >= 0) {
          const int64_t tok0 = static_cast<int64_t>(bid) * 64;
          if (tok0 < p.n_tokens) {
            int64_t n = p.n_tokens - tok0 < 64 ? p.n_tokens - tok0 : 64;
            bool ok = true;
            if (p.causal) {
              if (tok0 / p.chunk_size > q_chunk) ok = false;
              const int64_t lim = static_cast<int64_t>(q_chunk + 1) * p.chunk_size - tok0;
              if (lim < n) n = lim;
              if (n <= 0) ok = false;
            }
            if (ok) {
              if (p.paged) {
                const int page = bid < p.max_blocks ? p.block_table[static_cast<int64_t>(h) * p.max_blocks + bid] : -1;
                if (page >= 0) { row = page * 64; nv = static_cast<int>(n); }
              } else {
                row = static_cast<int>(tok0);
                nv = static_cast<int>(n);
              }
            }
          }
        }
      }
      const unsigned live = __ballot_sync(0xffffffffu, nv > 0);
      if (nv > 0) {
        const int pos = base + __popc(live & ((1u << lane) - 1u));
        s_row[pos] = row;
        s_nvis[pos] = static_cast<uint8_t>(nv);
        s_slot[pos] = static_cast<uint8_t>(t);
      }
      base += __popc(live);
    }
    if (lane == 0) s_nb = base;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_base_s;
  volatile int* abort = &s_abort;
  const int nb = s_nb;
  if (threadIdx.x == 0) TRACE(1, 1);

  if (warp == kProducerWarp) {
    // ======================= TMA producer =======================
    if (lane == 0 && nb > 0) {
      mbar_expect_tx(&qdo_full, 2 * kTile);
      tma_load_5d(sQ, &mapQ, 0, h, static_cast<int>(m0), 0, b, &qdo_full);
      tma_load_5d(sDO, &mapDO, 0, h, static_cast<int>(m0), 0, b, &qdo_full);
      int t = 0;
      for (; t < nb; ++t) {
        const int st = t & 1, ph = (t >> 1) & 1;
        const int ks = t % kKStages, kph = (t / kKStages) & 1;
        const int row = s_row[t];
        // the last K stage held Q until the row warps moved it to TMEM
        if (t == kKStages - 1 && !mbar_wait(&q_moved, 0, abort)) break;
        if (!mbar_wait(&k_empty[ks], kph ^ 1, abort)) break;
        mbar_expect_tx(&k_full[ks], kTile);
        if (p.paged) tma_load_3d(sK + ks * kTile, &mapK, 0, row, 0, &k_full[ks]);
        else tma_load_5d(sK + ks * kTile, &mapK, 0, h, row, 0, b, &k_full[ks]);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort)) { ++t; break; }
        mbar_expect_tx(&v_full[st], kTile);
        if (p.paged) tma_load_3d(sV + st * kTile, &mapV, 0, row, 0, &v_full[st]);
        else tma_load_5d(sV + st * kTile, &mapV, 0, h, row, 0, b, &v_full[st]);
      }
      if (*abort) {
        // the other roles have stopped consuming: wait (bounded) for the copies still in flight
        for (int u = (t > kKStages ? t - kKStages : 0); u < t; ++u) mbar_wait(&k_full[u % kKStages], (u / kKStages) & 1, abort);
        for (int u = (t > 2 ? t - 2 : 0); u < t; ++u) mbar_wait(&v_full[u & 1], (u >> 1) & 1, abort);
        mbar_wait(&qdo_full, 0, abort);
      }
    }
  } else if (warp == kScoreWarp) {
    // ======================= MMA issuer 1: S and dP (whole warp runs the loop, one elected lane issues) =======================
    if (nb > 0) {
      constexpr uint32_t idesc = instr_desc_bf16(64, 64, 0, 0);        // both operands K-major
      const uint32_t el = elect_one();
      const uint64_t dDO = smem_desc(smem_u32(sDO), 16, 1024);
      // dO has landed (qdo_full) and Q sits in TMEM (q_moved)
      bool ok = __all_sync(0xffffffffu, mbar_wait(&qdo_full, 0, abort) && mbar_wait(&q_moved, 0, abort));
      for (int t = 0; ok && t < nb; ++t) {
        const int st = t & 1, ph = (t >> 1) & 1;
        const int ks = t % kKStages;
        ok = __all_sync(0xffffffffu, mbar_wait(&k_full[ks], (t / kKStages) & 1, abort) && mbar_wait(&v_full[st], ph, abort) &&
                                     (t == 0 || mbar_wait(&sdp_free, (t - 1) & 1, abort)));    // S / dP of step t-1 were read
        if (!ok) break;
        tc_fence_after();
        TRACE(0, 8 + t * 8 + 0);
        const uint64_t dK = smem_desc(smem_u32(sK + ks * kTile), 16, 1024), dV = smem_desc(smem_u32(sV + st * kTile), 16, 1024);
        if (el) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (kk >> 2) * 8192 + (kk & 3) * 32;
            umma_ts(tm + kColS, tm + kColQ + kk * 8, desc_advance(dK, off), idesc, kk > 0 ? 1u : 0u);   // A = Q from TMEM
          }
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (kk >> 2) * 8192 + (kk & 3) * 32;
            umma_ss(tm + kColDP, desc_advance(dDO, off), desc_advance(dV, off), idesc, kk > 0 ? 1u : 0u);
          }
          umma_commit(&sdp_full);
          umma_commit(&v_empty[st]);
        }
        __syncwarp();
        TRACE(0, 8 + t * 8 + 1);
      }
    }
  } else if (warp == kGradWarp) {
    // ======================= MMA issuer 2: dQ += dS K =======================
    if (nb > 0) {
      // dQ^T += K^T dS^T: the accumulator is (128 head dims) x (64 rows) and takes 64 TMEM columns instead of 128
      constexpr uint32_t idesc = instr_desc_bf16(128, 64, 1, 0);       // A (K tile, head dim as M) MN-major, B (dS) K-major
      const uint32_t el = elect_one();
      const uint64_t dDS = smem_desc(smem_u32(sDS), 16, 1024);
      for (int t = 0; t < nb; ++t) {
        const int ks = t % kKStages;
        if (!__all_sync(0xffffffffu, mbar_wait(&ds_full, t & 1, abort))) break;
        tc_fence_after();
        TRACE(0, 8 + t * 8 + 2);
        // K tile [64 keys][128 dims] as two 64-column boxes 8 KiB apart, read with the head dim as M
        const uint64_t dKmn = smem_desc(smem_u32(sK + ks * kTile), 8192, 1024);
        if (el) {
          if (STORE) {
            // the step's { P, dS } tiles go to the pair's place in the buffer, one 16 KiB bulk store issued
            // before the products so that it reads shared memory while they are being issued; the row
            // warps overwrite the tiles only after the product (ds_free) AND the store (tile_stored) have read them
            char* dst = p.pds + (((((static_cast<int64_t>(b) * p.MG + g) * p.H + h) * p.T) + s_slot[t]) << 14);
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 16384;" ::"l"(dst), "r"(smem_u32(sP)) : "memory");
            bulk_commit_group();
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tm + kColDQ, desc_advance(dKmn, kk * 2048), desc_advance(dDS, kk * 32), idesc, (t > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&k_empty[ks]);
          umma_commit(&ds_free);
          if (t == nb - 1) umma_commit(&dq_final);
          if (STORE) {
            bulk_wait_read_all();
            mbar_arrive(&tile_stored);
          }
        }
        __syncwarp();
        TRACE(0, 8 + t * 8 + 3);
      }
      if (STORE && el) bulk_wait_all();
    }
  } else if (warp < 8) {
    // ======================= row arithmetic on accumulator fragments (warps 0-7) =======================
    // Two groups of four warps share every step: warps 0-3 take keys 0-31 of the block, warps 4-7 keys
    // 32-63, which halves the time from S / dP to dS, the link of the chain that bounds a step.  Warps w and
    // w + 4 own query rows 16(w%4) .. +15 (TMEM lanes 32(w%4) .. +15 of the M=64 accumulators); thread t holds
    // rows r0 = 16(w%4) + t/4 and r1 = r0 + 8, keys 32 grp + 8i + 2(t%4), +1 of every 8-key block i of its half.
    const int grp = warp >> 2, wq = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const int r0 = wq * 16 + (lane >> 2), r1 = r0 + 8;
    const int cq = 32 * grp + (lane & 3) * 2;
    // stmatrix: this thread supplies the address of row (lane%8) of matrix (lane/8); the four matrices of
    // one instruction are (rows +0, block 2q), (rows +8, block 2q), (rows +0, block 2q+1), (rows +8, block 2q+1)
    const int st_row = wq * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int st_chunk = 4 * grp + (lane >> 4);
    // delta = sum_d O dO: thread j reduced a quarter of a row from the loads issued at the top of the kernel
    {
      float part = 0.f;
      if (drow_q < n_q) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t aw[4] = {ro_[c].x, ro_[c].y, ro_[c].z, ro_[c].w}, dw[4] = {rd_[c].x, rd_[c].y, rd_[c].z, rd_[c].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = unpack2<__nv_bfloat16>(aw[e]), y = unpack2<__nv_bfloat16>(dw[e]);
            part += x.x * y.x + x.y * y.y;
          }
        }
      }
      s_part[threadIdx.x] = part;
    }
    named_barrier(2, 256);
    const float delta0 = (s_part[4 * r0] + s_part[4 * r0 + 1]) + (s_part[4 * r0 + 2] + s_part[4 * r0 + 3]);
    const float delta1 = (s_part[4 * r1] + s_part[4 * r1 + 1]) + (s_part[4 * r1 + 2] + s_part[4 * r1 + 3]);
    if (grp == 0 && (lane & 3) == 0) {
      if (r0 < n_q) p.delta[bhm + r0] = delta0;
      if (r1 < n_q) p.delta[bhm + r1] = delta1;
    }
    named_barrier(2, 256);                             // the partial sums are read: their tile may be written
    if (nb == 0) {
      if (drow_q < n_q) {
        char* drow = p.dq + (b * p.dq_sb + (m0 + drow_q) * p.dq_sm + h * p.dq_sh) * 2 + dquarter * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(drow + c * 16) = make_uint4(0, 0, 0, 0);
      }
    } else {
      // exponent offsets: LSE log2e - log2 scale (the scale of dS is folded into the exponent); +inf = no such row
      const float lg = log2f(p.scale);
      const float nl0 = r0 < n_q ? -(p.lse[bhm + r0] * kLog2e - lg) : -INFINITY;
      const float nl1 = r1 < n_q ? -(p.lse[bhm + r1] * kLog2e - lg) : -INFINITY;
      const float sl = p.scale_log2;
      // exponent offsets of P itself (no scale folded in)
      const float np0 = r0 < n_q ? -(p.lse[bhm + r0] * kLog2e) : -INFINITY;
      const float np1 = r1 < n_q ? -(p.lse[bhm + r1] * kLog2e) : -INFINITY;
      // ---- Q from its landing tile into TMEM, in the layout of an M=64 A operand: row r in the lane of
      // accumulator row r, head dims 2c, 2c+1 in column c.  With tcgen05.st.16x128b a thread supplies, per
      // four-column block j, the word (row r0, column 4j + t%4) and the same column of row r1.  Group g
      // moves head dims [64 g, +64).
      bool ok = __all_sync(0xffffffffu, mbar_wait(&qdo_full, 0, abort));
      if (ok) {
        const uint8_t* box = sQ + grp * 8192;
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          w[2 * j] = *reinterpret_cast<const uint32_t*>(box + r0 * 128 + ((j ^ (r0 & 7)) << 4) + 4 * (lane & 3));
          w[2 * j + 1] = *reinterpret_cast<const uint32_t*>(box + r1 * 128 + ((j ^ (r1 & 7)) << 4) + 4 * (lane & 3));
        }
        tmem_st_16x128b_x8_nowait(tm + lane_base + kColQ + grp * 32, w);
        tmem_st_wait();
        tc_fence_before();
      }
      mbar_arrive(&q_moved);
      if (threadIdx.x == 0) TRACE(1, 2);
      for (int t = 0; t < nb; ++t) {
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 0);
        ok = __all_sync(0xffffffffu, mbar_wait(&sdp_full, t & 1, abort));
        if (!ok) break;
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 1);
        tc_fence_after();
        uint32_t x[16], y[16];
        tmem_ld_16x256b_x4_nowait(tm + lane_base + kColS + 32 * grp, x);
        tmem_ld_16x256b_x4_nowait(tm + lane_base + kColDP + 32 * grp, y);
        const int nv = s_nvis[t];
        // the dS tile of the previous step must have been consumed: normally long true, so poll once
        // here, where the round trip hides behind the TMEM load
        const bool ds_ok = t == 0 || mbar_try(&ds_free, (t - 1) & 1);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&sdp_free);
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 2);
        // x[4i], x[4i+1]: row r0, keys 8i+cq, +1;  x[4i+2], x[4i+3]: row r1.  Afterwards x[2i], x[2i+1]
        // hold the packed dS of (r0, r1) for key block i of this group's half.
        uint32_t pp[8];                               // STORE: the packed P of (r0, r1) per key block
        if (STORE) {
          // P = exp2(S c - LSE log2e) (masked keys: 0) and dS = P (dP - delta) scale from the same exponential
          const float sc_ = p.scale;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int c = 8 * i + cq;
            const float p00 = (c < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i]), sl, np0)) : 0.f;
            const float p01 = (c + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 1]), sl, np0)) : 0.f;
            const float p10 = (c < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 2]), sl, np1)) : 0.f;
            const float p11 = (c + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 3]), sl, np1)) : 0.f;
            pp[2 * i] = pack2<__nv_bfloat16>(p00, p01);
            pp[2 * i + 1] = pack2<__nv_bfloat16>(p10, p11);
            const float d00 = p00 * ((__uint_as_float(y[4 * i]) - delta0) * sc_);
            const float d01 = p01 * ((__uint_as_float(y[4 * i + 1]) - delta0) * sc_);
            const float d10 = p10 * ((__uint_as_float(y[4 * i + 2]) - delta1) * sc_);
            const float d11 = p11 * ((__uint_as_float(y[4 * i + 3]) - delta1) * sc_);
            x[2 * i] = pack2<__nv_bfloat16>(d00, d01);
            x[2 * i + 1] = pack2<__nv_bfloat16>(d10, d11);
          }
        } else if (nv == 64) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float d00 = fast_exp2(fmaf(__uint_as_float(x[4 * i]), sl, nl0)) * (__uint_as_float(y[4 * i]) - delta0);
            const float d01 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 1]), sl, nl0)) * (__uint_as_float(y[4 * i + 1]) - delta0);
            const float d10 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 2]), sl, nl1)) * (__uint_as_float(y[4 * i + 2]) - delta1);
            const float d11 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 3]), sl, nl1)) * (__uint_as_float(y[4 * i + 3]) - delta1);
            x[2 * i] = pack2<__nv_bfloat16>(d00, d01);
            x[2 * i + 1] = pack2<__nv_bfloat16>(d10, d11);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int c = 8 * i + cq;
            const float d00 = (c < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i]), sl, nl0)) * (__uint_as_float(y[4 * i]) - delta0) : 0.f;
            const float d01 = (c + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 1]), sl, nl0)) * (__uint_as_float(y[4 * i + 1]) - delta0) : 0.f;
            const float d10 = (c < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 2]), sl, nl1)) * (__uint_as_float(y[4 * i + 2]) - delta1) : 0.f;
            const float d11 = (c + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 3]), sl, nl1)) * (__uint_as_float(y[4 * i + 3]) - delta1) : 0.f;
            x[2 * i] = pack2<__nv_bfloat16>(d00, d01);
            x[2 * i + 1] = pack2<__nv_bfloat16>(d10, d11);
          }
        }
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 3);
        if (!__all_sync(0xffffffffu, ds_ok)) {
          ok = __all_sync(0xffffffffu, mbar_wait(&ds_free, (t - 1) & 1, abort));
          if (!ok) break;
        }
        if (STORE && t > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(&tile_stored, (t - 1) & 1, abort));
          if (!ok) break;
        }
        const uint32_t aDS = smem_u32(sDS) + st_row * 128;
#pragma unroll
        for (int q = 0; q < 2; ++q)
          stmatrix_x4(aDS + static_cast<uint32_t>(((2 * q + st_chunk) ^ (st_row & 7)) << 4), x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
        if (STORE) {
          const uint32_t aP = smem_u32(sP) + st_row * 128;
#pragma unroll
          for (int q = 0; q < 2; ++q)
            stmatrix_x4(aP + static_cast<uint32_t>(((2 * q + st_chunk) ^ (st_row & 7)) << 4), pp[4 * q], pp[4 * q + 1], pp[4 * q + 2], pp[4 * q + 3]);
        }
        fence_async_smem();                           // make the rows visible to the tensor core's reads
        mbar_arrive(&ds_full);
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 4);
      }
      if (threadIdx.x == 0) TRACE(1, 3);
      // ---- epilogue: dQ^T fragments (16 head-dim lanes x 64 rows per load) -> bf16 pairs of adjacent rows,
      // stored TRANSPOSED 8 x 8 at a time into the swizzled [row][head dim] staging tile (the first K stage,
      // dead once every product has run) -> TMA tile stores.  Group g takes lanes 16 g .. +15 of its quadrant.
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&dq_final, 0, abort));
      if (ok) {
        tc_fence_after();
        const int lh = grp;
        uint32_t x[32];
        tmem_ld_16x256b_x8_nowait(tm + lane_base + (static_cast<uint32_t>(lh * 16) << 16) + kColDQ, x);
        tmem_ld_wait();
        // x[4i], x[4i+1]: head dim D0 + lane/4, rows 8i + 2(lane%4), +1;  x[4i+2], x[4i+3]: head dim + 8
        const int D0 = wq * 32 + lh * 16;
        const int dsel = D0 + ((lane >> 3) & 1) * 8;     // head dims of the matrix this lane addresses
        const uint32_t boxa = smem_u32(sOut + (dsel >> 6) * 8192);
        const uint32_t dchunk = static_cast<uint32_t>((dsel & 63) >> 3);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i0 = 2 * q, i1 = 2 * q + 1;
          const uint32_t a0 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i0]), __uint_as_float(x[4 * i0 + 1]));
          const uint32_t b0 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i0 + 2]), __uint_as_float(x[4 * i0 + 3]));
          const uint32_t a1 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i1]), __uint_as_float(x[4 * i1 + 1]));
          const uint32_t b1 = pack2<__nv_bfloat16>(__uint_as_float(x[4 * i1 + 2]), __uint_as_float(x[4 * i1 + 3]));
          // matrices: (rows 8 i0.., dims D0..), (rows 8 i0.., dims D0+8..), (rows 8 i1.., D0..), (rows 8 i1.., D0+8..)
          const int qrow = 8 * (2 * q + (lane >> 4)) + (lane & 7);
          stmatrix_x4_trans(boxa + qrow * 128 + ((dchunk ^ static_cast<uint32_t>(qrow & 7)) << 4), a0, b0, a1, b1);
        }
        fence_async_smem();
      }
      named_barrier(1, 256);
      if (ok && threadIdx.x == 0) {
        for (int dh = 0; dh < 2; ++dh) tma_store_4d(&mapDQ, sOut + dh * 8192, dh * 64, h, static_cast<int>(m0), b);
        bulk_commit_group();
        bulk_wait_all();
      }
    }
  }

  if (threadIdx.x == 0) TRACE(1, 4);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, kTmemCols);
  if (threadIdx.x == 0) TRACE(1, 5);
  if (threadIdx.x == 0 && s_abort) atomicExch(p.status, NSA_ERR_CUDA);
}

}  // namespace

int make_tile_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                   CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV);
int make_rows_map(const void* q, const int64_t* q_stride, int B, int64_t M, int H, int box_rows, CUtensorMap* map);

// Launches the tensor-core dQ kernel when it covers the call (*launched = true).
int try_launch_sel_bwd_dq_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* ids,
                             const int64_t* idx_stride, const void* out, const int64_t* out_stride, const float* lse,
                             const void* d_out, const int64_t* do_stride, void* dq, const int64_t* dq_stride,
                             float* delta, int B, int64_t M, int H, int D, int T, int block_size, int chunk_size,
                             int causal, int G, float scale, int dtype, cudaStream_t stream, bool* launched,
                             void* pds) {
  *launched = false;
  const char* env = getenv("OMNIMEM_B200_BWD_KERNEL");
  if (env != nullptr && std::string(env) == "general") return NSA_OK;
  if (dtype != NSA_BF16 || D != 128 || block_size != 64 || G > 64 || G < 16 || T > kMaxSlots || H == 1) return NSA_OK;
  if (pds != nullptr && T > kMaxSlotsStore) pds = nullptr;   // (the caller is told: max_store_slots)
  if (!(scale > 0.f)) return NSA_OK;   // the kernel folds log2(scale) into the exponent
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  // dQ leaves through TMA tile stores: 16-byte aligned rows
  if ((reinterpret_cast<uintptr_t>(dq) & 15) != 0 || (dq_stride[0] * 2) % 16 != 0 || (dq_stride[1] * 2) % 16 != 0 ||
      (dq_stride[2] * 2) % 16 != 0)
    return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  CUtensorMap mapQ, mapDO, mapK, mapV, mapDQ;
  int rc;
  if ((rc = make_tile_maps(q, q_stride, kv, B, M, H, &mapQ, &mapK, &mapV))) return rc;
  if ((rc = make_tile_maps(d_out, do_stride, nullptr, B, M, H, &mapDO, nullptr, nullptr))) return rc;
  // the store box holds G rows: a group shorter than 64 rows must not write into the next group
  if ((rc = make_rows_map(dq, dq_stride, B, M, H, G, &mapDQ))) return rc;
  TcDqParams p;
  p.ids = ids; p.i_sb = idx_stride[0]; p.i_sg = idx_stride[1]; p.i_sh = idx_stride[2]; p.i_st = idx_stride[3];
  p.o = static_cast<const char*>(out); p.o_sb = out_stride[0]; p.o_sm = out_stride[1]; p.o_sh = out_stride[2];
  p.dO = static_cast<const char*>(d_out); p.do_sb = do_stride[0]; p.do_sm = do_stride[1]; p.do_sh = do_stride[2];
  p.dq = static_cast<char*>(dq); p.dq_sb = dq_stride[0]; p.dq_sm = dq_stride[1]; p.dq_sh = dq_stride[2];
  p.lse = lse; p.delta = delta;
  p.block_table = kv->block_table; p.max_blocks = kv->max_blocks; p.paged = kv->mode == NSA_KV_PAGED;
  p.n_tokens = kv->n_tokens; p.M = M; p.H = H; p.T = T; p.G = G; p.chunk_size = chunk_size; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.pds = static_cast<char*>(pds); p.MG = static_cast<int>(cdiv64(M, G));
  if ((rc = device_status_address(&p.status))) return rc;
  size_t smem = kSmemTiles + 1024;
  auto kernel = pds != nullptr ? sel_bwd_dq_tc_kernel<true> : sel_bwd_dq_tc_kernel<false>;
  if (pds != nullptr) {
    // 112 KiB of tiles start at the first 1 KiB boundary after the static variables: exactly half an SM
    cudaFuncAttributes fa;
    NSA_CUDA_OK(cudaFuncGetAttributes(&fa, kernel));
    smem = kSmemTilesStore + (1024 - fa.sharedSizeBytes % 1024) % 1024;
  }
  NSA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  NSA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   static_cast<int>(cudaSharedmemCarveoutMaxShared)));
  NSA_CUDA_OK(launch_chained(kChainDq, kernel, dim3(static_cast<unsigned>(cdiv64(M, G)), H, B), dim3(kThreads), smem, stream,
                             mapQ, mapDO, mapK, mapV, mapDQ, p));
  NSA_LAUNCH_OK("sel_bwd_dq_tc_kernel");
  *launched = true;
  return NSA_OK;
}

}  // namespace nsa

#ifdef NSA_TC_TRACE
extern "C" int nsa_debug_trace_dq(long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace_dq, sizeof(long long) * 2 * 512));
  return NSA_OK;
}
#endif
