// Selection attention backward, dQ half, on tcgen05 / TMEM / TMA for the page geometry
// (bf16, D = 128, 64-token blocks, query groups of up to 64 rows, dense or paged K/V).
//
// Same skeleton as the tensor-core forward: one thread block per (batch, query group, head);
// warp 4 feeds the K ring, warp 6 the V ring (plus the Q and dO tiles once), warp 5 issues
// the MMAs, warps 0-3 own one TMEM lane (matrix row) per thread.  Q and dO are loaded twice
// (rows 0-63 and 64-127 of their A tiles); per step two selected blocks (128 keys) are
// processed: rows 0-63 work on the even block (columns 0-63 of S and dP), rows 64-127 on the
// odd block (columns 64-127); the other half of each dS row is zero.  Per step:
//     S  = [Q;Q]   K^T          (M=128, N=128, K=128)   recomputed scores
//     dP = [dO;dO] V^T          (M=128, N=128, K=128)
//     dS = exp2(S c - LSE) (dP - delta) scale           (threads, written to TMEM as bf16)
//     dQ += dS K                (M=128, N=128, K=128, A from TMEM, K tile read MN-major)
// The two halves of dQ are summed in the epilogue.  delta = sum_d(O dO) is computed in the
// prologue and stored for the dK/dV kernel.
#include "sel_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <string>

namespace nsa {

int device_status_address(int32_t** out);

#ifdef NSA_TC_TRACE
// Debug build only: clock64 stamps of thread block (0,0,0); [0][..] MMA issuer, [1][..] row thread 0.
__device__ long long g_trace_dq[4][512];
#define TRACE(role, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (slot) < 512) g_trace_dq[role][slot] = clock64(); } while (0)
#else
#define TRACE(role, slot) do { } while (0)
#endif

namespace {

using namespace tc;

constexpr int kThreads = 288;
constexpr int kMaxSlots = 128;
constexpr int kStagesK = 3;
constexpr uint32_t kTileBytes = 32768;
constexpr uint32_t kSmemTiles = 7 * kTileBytes;   // Q, dO, K x3, V x2

constexpr uint32_t kColS = 0;      // 2 x 128: scores of even / odd steps; dS (64 columns of bf16 pairs) is written over them
constexpr uint32_t kColDP = 256;   // 128
constexpr uint32_t kColDQ = 384;   // 128

struct TcDqParams {
  const int32_t* ids;
  int64_t i_sb, i_sg, i_sh, i_st;
  const char* o; int64_t o_sb, o_sm, o_sh;      // forward output (for delta)
  const char* dO; int64_t do_sb, do_sm, do_sh;
  char* dq; int64_t dq_sb, dq_sm, dq_sh;
  const float* lse;
  float* delta;
  const int32_t* block_table;
  int max_blocks, paged;
  int64_t n_tokens, M;
  int H, T, G, chunk_size, causal;
  float scale, scale_log2;
  int32_t* status;
};

__global__ void __launch_bounds__(kThreads, 1)
sel_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapDO,
                     const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                     const TcDqParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = tiles;
  uint8_t* sDO = tiles + kTileBytes;
  uint8_t* sK = tiles + 2 * kTileBytes;
  uint8_t* sV = tiles + 5 * kTileBytes;
  float* stage = reinterpret_cast<float*>(tiles + 2 * kTileBytes);   // epilogue: 128 x 129 floats over the rings

  __shared__ uint64_t qdo_full, k_full[kStagesK], k_empty[kStagesK], v_full[2], v_empty[2], s_full[2], s_free[2], ds_full[2], dp_full, dp_free, dq_final;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort, s_nb;
  __shared__ int s_row[kMaxSlots], s_nvis[kMaxSlots];
  __shared__ float s_delta[128];

  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t m0 = static_cast<int64_t>(g) * p.G;
  const int n_q = static_cast<int>(p.M - m0 < p.G ? p.M - m0 : p.G);
  const int q_chunk = static_cast<int>(m0 / p.chunk_size);

  if (threadIdx.x == 0) TRACE(1, 0);
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(&qdo_full, 1);
    for (int i = 0; i < kStagesK; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 1); mbar_init(&ds_full[i], 128);
    }
    mbar_init(&dp_full, 1);
    mbar_init(&dp_free, 128);
    mbar_init(&dq_final, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapDO); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  // ---- row threads start the loads for delta = sum_d O dO right away: the two threads that own
  // a query row (rows r and 64 + r of the duplicated tiles) each take one 64-column half
  const int half = (warp >> 1) & 1;
  const int qrow = threadIdx.x & 63;
  uint4 ro_[8], rd_[8];
  if (warp < 4 && qrow < n_q) {
    const uint4* orow = reinterpret_cast<const uint4*>(p.o + (b * p.o_sb + (m0 + qrow) * p.o_sm + h * p.o_sh) * 2) + half * 8;
    const uint4* drow = reinterpret_cast<const uint4*>(p.dO + (b * p.do_sb + (m0 + qrow) * p.do_sm + h * p.do_sh) * 2) + half * 8;
#pragma unroll
    for (int c = 0; c < 8; ++c) { ro_[c] = orow[c]; rd_[c] = drow[c]; }
  }
  // ---- list of the visible selected blocks (TMA row coordinate, visible tokens), compacted by warp 4
  if (warp == 4) {
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
        s_nvis[pos] = nv;
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
  const int NT = (nb + 1) >> 1;
  if (threadIdx.x == 0) TRACE(1, 1);
  char* dq_row0 = p.dq + (b * p.dq_sb + m0 * p.dq_sm + h * p.dq_sh) * 2;
  const int64_t bhm = (static_cast<int64_t>(b) * p.H + h) * p.M + m0;

  auto load_tile = [&](uint8_t* dst, const CUtensorMap* map, int re, int ro, uint64_t* bar) {
    mbar_expect_tx(bar, kTileBytes);
    if (p.paged) {
      tma_load_2d(dst, map, 0, re, bar);
      tma_load_2d(dst + 8192, map, 0, ro, bar);
      tma_load_2d(dst + 16384, map, 64, re, bar);
      tma_load_2d(dst + 24576, map, 64, ro, bar);
    } else {
      tma_load_4d(dst, map, 0, h, re, b, bar);
      tma_load_4d(dst + 8192, map, 0, h, ro, b, bar);
      tma_load_4d(dst + 16384, map, 64, h, re, b, bar);
      tma_load_4d(dst + 24576, map, 64, h, ro, b, bar);
    }
  };

  if (warp == 4 || warp == 6) {
    // ======================= TMA producers =======================
    if (lane == 0) {
      const bool isK = warp == 4;
      uint64_t* full = isK ? k_full : v_full;
      uint64_t* empty = isK ? k_empty : v_empty;
      uint8_t* ring = isK ? sK : sV;
      const CUtensorMap* map = isK ? &mapK : &mapV;
      const int ns = isK ? kStagesK : 2;
      if (isK) {
        mbar_expect_tx(&qdo_full, 2 * kTileBytes);
        for (int dh = 0; dh < 2; ++dh)
          for (int dup = 0; dup < 2; ++dup) {
            tma_load_4d(sQ + dh * 16384 + dup * 8192, &mapQ, dh * 64, h, static_cast<int>(m0), b, &qdo_full);
            tma_load_4d(sDO + dh * 16384 + dup * 8192, &mapDO, dh * 64, h, static_cast<int>(m0), b, &qdo_full);
          }
      }
      int t = 0;
      for (; t < NT; ++t) {
        const int s = t % ns, ph = (t / ns) & 1;
        const int re = s_row[2 * t], ro = (2 * t + 1 < nb) ? s_row[2 * t + 1] : re;
        if (!mbar_wait(&empty[s], ph ^ 1, abort)) break;
        TRACE(isK ? 2 : 3, t);
        load_tile(ring + s * kTileBytes, map, re, ro, &full[s]);
      }
      if (*abort || nb == 0) {
        // the other roles have stopped (or never started) consuming: wait (bounded) for the copies in flight
        for (int u = (t > ns ? t - ns : 0); u < t && u < NT; ++u) mbar_wait(&full[u % ns], (u / ns) & 1, abort);
        if (isK) mbar_wait(&qdo_full, 0, abort);
      }
    }
  } else if (warp == 5 || warp == 7 || warp == 8) {
    // ======================= MMA issuers =======================
    // Three issuing threads, one per product, so that the tensor pipe is fed while each of them
    // sits in its own barrier waits: warp 5 issues S(t) (double-buffered, reused once dQ(t-2) has
    // read the dS written over it), warp 7 issues dP(t) as soon as the row threads have read
    // dP(t-1), warp 8 issues dQ(t) when dS(t) is in TMEM.  A K tile is held from S(t) to dQ(t),
    // hence the three-stage K ring.
    // Whole warps run these loops (warp-uniform control flow keeps descriptor arithmetic in uniform
    // registers); one elected lane issues.
    if (nb > 0) {
      constexpr uint32_t idesc_kk = instr_desc_bf16(128, 128, 0, 0);   // both operands K-major
      constexpr uint32_t idesc_mn = instr_desc_bf16(128, 128, 0, 1);   // B read MN-major
      const uint32_t el = elect_one();
      if (warp == 5) {
        const uint64_t dQ = smem_desc(smem_u32(sQ), 16, 1024);
        bool ok = __all_sync(0xffffffffu, mbar_wait(&qdo_full, 0, abort));
        TRACE(0, 0);
        for (int t = 0; ok && t < NT; ++t) {
          const int s = t & 1, ks = t % kStagesK;
          ok = __all_sync(0xffffffffu, mbar_wait(&k_full[ks], (t / kStagesK) & 1, abort) &&
                                       (t < 2 || mbar_wait(&s_free[s], ((t - 2) >> 1) & 1, abort)));   // dQ(t-2) done
          if (!ok) break;
          tc_fence_after();
          TRACE(0, 8 + t * 8 + 0);
          const uint64_t dK = smem_desc(smem_u32(sK + ks * kTileBytes), 16, 1024);
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
              umma_ss(tm + kColS + s * 128, desc_advance(dQ, off), desc_advance(dK, off), idesc_kk, kk > 0 ? 1u : 0u);
            }
            umma_commit(&s_full[s]);
          }
          __syncwarp();
          TRACE(0, 8 + t * 8 + 1);
        }
      } else if (warp == 7) {
        const uint64_t dDO = smem_desc(smem_u32(sDO), 16, 1024);
        bool ok = __all_sync(0xffffffffu, mbar_wait(&qdo_full, 0, abort));
        for (int t = 0; ok && t < NT; ++t) {
          const int s = t & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(&v_full[s], (t >> 1) & 1, abort) &&
                                       (t < 1 || mbar_wait(&dp_free, (t - 1) & 1, abort)));             // dP(t-1) has been read
          if (!ok) break;
          tc_fence_after();
          TRACE(0, 8 + t * 8 + 2);
          const uint64_t dV = smem_desc(smem_u32(sV + s * kTileBytes), 16, 1024);
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
              umma_ss(tm + kColDP, desc_advance(dDO, off), desc_advance(dV, off), idesc_kk, kk > 0 ? 1u : 0u);
            }
            umma_commit(&dp_full);
            umma_commit(&v_empty[s]);
          }
          __syncwarp();
          TRACE(0, 8 + t * 8 + 3);
        }
      } else {
        for (int t = 0; t < NT; ++t) {
          const int s = t & 1, ks = t % kStagesK;
          if (!__all_sync(0xffffffffu, mbar_wait(&ds_full[s], (t >> 1) & 1, abort))) break;
          tc_fence_after();
          TRACE(0, 8 + t * 8 + 4);
          const uint64_t dKmn = smem_desc(smem_u32(sK + ks * kTileBytes), 16384, 1024);
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ts(tm + kColDQ, tm + kColS + s * 128 + kk * 8, desc_advance(dKmn, kk * 2048), idesc_mn,
                      (t > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&k_empty[ks]);
            umma_commit(&s_free[s]);
            if (t == NT - 1) umma_commit(&dq_final);
          }
          __syncwarp();
          TRACE(0, 8 + t * 8 + 5);
        }
      }
    }
  } else if (warp < 4) {
    // ======================= per-row math (warps 0-3) =======================
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    // delta = sum_d O dO of this thread's query row: each of the row's two threads reduces the half
    // it loaded at the top of the kernel, the halves meet in shared memory
    float delta = 0.f, lse2 = INFINITY, lse2s = INFINITY;
    if (qrow < n_q) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t aw[4] = {ro_[c].x, ro_[c].y, ro_[c].z, ro_[c].w}, dw[4] = {rd_[c].x, rd_[c].y, rd_[c].z, rd_[c].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = unpack2<__nv_bfloat16>(aw[e]), y = unpack2<__nv_bfloat16>(dw[e]);
          delta += x.x * y.x + x.y * y.y;
        }
      }
      lse2 = p.lse[bhm + qrow] * kLog2e;
      lse2s = lse2 - log2f(p.scale);
    }
    s_delta[threadIdx.x] = delta;
    named_barrier(2, 128);
    delta = s_delta[qrow] + s_delta[64 + qrow];
    if (qrow < n_q && half == 0) p.delta[bhm + qrow] = delta;
    if (nb == 0) {
      if (qrow < n_q) {
        char* drow = dq_row0 + qrow * p.dq_sm * 2 + half * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(drow + c * 16) = make_uint4(0, 0, 0, 0);
      }
    } else {
      bool ok = true;
      if (threadIdx.x == 0) TRACE(1, 2);
      for (int t = 0; t < NT; ++t) {
        const int s = t & 1;
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 0);
        ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (t >> 1) & 1, abort) && mbar_wait(&dp_full, t & 1, abort));
        if (!ok) break;
        tc_fence_after();
        uint32_t x0[32], x1[32], y0[32], y1[32];
        tmem_ld32_nowait(tm + lane_base + kColS + s * 128 + half * 64, x0);
        tmem_ld32_nowait(tm + lane_base + kColS + s * 128 + half * 64 + 32, x1);
        tmem_ld32_nowait(tm + lane_base + kColDP + half * 64, y0);
        tmem_ld32_nowait(tm + lane_base + kColDP + half * 64 + 32, y1);
        tmem_ld_wait();
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 1);
        tc_fence_before();
        mbar_arrive(&dp_free);
        const int blk = 2 * t + half;
        const int nv = blk < nb ? s_nvis[blk] : 0;
        // dS = P (dP - delta) scale with the scale folded into the exponent (lse2s = LSE log2e - log2 scale)
        uint32_t pk[32];
        {
          const float sl = p.scale_log2, nl = -lse2s;
          if (nv == 64) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float d0 = fast_exp2(fmaf(__uint_as_float(x0[2 * j]), sl, nl)) * (__uint_as_float(y0[2 * j]) - delta);
              const float d1 = fast_exp2(fmaf(__uint_as_float(x0[2 * j + 1]), sl, nl)) * (__uint_as_float(y0[2 * j + 1]) - delta);
              const float d2 = fast_exp2(fmaf(__uint_as_float(x1[2 * j]), sl, nl)) * (__uint_as_float(y1[2 * j]) - delta);
              const float d3 = fast_exp2(fmaf(__uint_as_float(x1[2 * j + 1]), sl, nl)) * (__uint_as_float(y1[2 * j + 1]) - delta);
              pk[j] = pack2<__nv_bfloat16>(d0, d1);
              pk[16 + j] = pack2<__nv_bfloat16>(d2, d3);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float d0 = (2 * j < nv) ? fast_exp2(fmaf(__uint_as_float(x0[2 * j]), sl, nl)) * (__uint_as_float(y0[2 * j]) - delta) : 0.f;
              const float d1 = (2 * j + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(x0[2 * j + 1]), sl, nl)) * (__uint_as_float(y0[2 * j + 1]) - delta) : 0.f;
              const float d2 = (2 * j + 32 < nv) ? fast_exp2(fmaf(__uint_as_float(x1[2 * j]), sl, nl)) * (__uint_as_float(y1[2 * j]) - delta) : 0.f;
              const float d3 = (2 * j + 33 < nv) ? fast_exp2(fmaf(__uint_as_float(x1[2 * j + 1]), sl, nl)) * (__uint_as_float(y1[2 * j + 1]) - delta) : 0.f;
              pk[j] = pack2<__nv_bfloat16>(d0, d1);
              pk[16 + j] = pack2<__nv_bfloat16>(d2, d3);
            }
          }
        }
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 2);
        // dS over the score columns of this step: this row's 64 values in its own half, zeros in the other
        tmem_st32_nowait(tm + lane_base + kColS + s * 128 + half * 32, pk);
#pragma unroll
        for (int j = 0; j < 32; ++j) pk[j] = 0u;
        tmem_st32_nowait(tm + lane_base + kColS + s * 128 + (1 - half) * 32, pk);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&ds_full[s]);
        if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 3);
      }
      if (threadIdx.x == 0) TRACE(1, 3);
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&dq_final, 0, abort));
      if (threadIdx.x == 0) TRACE(1, 4);
      if (ok) {
        tc_fence_after();
        const int tid = threadIdx.x;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32_nowait(tm + lane_base + kColDQ + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) stage[tid * 129 + c * 32 + j] = __uint_as_float(o[j]);
        }
      }
      named_barrier(1, 128);
      if (ok && qrow < n_q) {
        const float* ra = stage + qrow * 129 + half * 64;
        const float* rb = stage + (64 + qrow) * 129 + half * 64;
        char* drow = dq_row0 + qrow * p.dq_sm * 2 + half * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w[e] = pack2<__nv_bfloat16>(ra[c * 8 + 2 * e] + rb[c * 8 + 2 * e], ra[c * 8 + 2 * e + 1] + rb[c * 8 + 2 * e + 1]);
          *reinterpret_cast<uint4*>(drow + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }

  if (threadIdx.x == 0) TRACE(1, 5);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
  if (threadIdx.x == 0) TRACE(1, 6);
  if (threadIdx.x == 0 && s_abort) atomicExch(p.status, NSA_ERR_CUDA);
}

}  // namespace

int make_qkv_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                  CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV);

// Launches the tensor-core dQ kernel when it covers the call (*launched = true).
int try_launch_sel_bwd_dq_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* ids,
                             const int64_t* idx_stride, const void* out, const int64_t* out_stride, const float* lse,
                             const void* d_out, const int64_t* do_stride, void* dq, const int64_t* dq_stride,
                             float* delta, int B, int64_t M, int H, int D, int T, int block_size, int chunk_size,
                             int causal, int G, float scale, int dtype, cudaStream_t stream, bool* launched) {
  *launched = false;
  const char* env = getenv("OMNIMEM_B200_BWD_KERNEL");
  if (env != nullptr && std::string(env) == "general") return NSA_OK;
  if (dtype != NSA_BF16 || D != 128 || block_size != 64 || G > 64 || G < 16 || T > kMaxSlots || H == 1) return NSA_OK;
  if (!(scale > 0.f)) return NSA_OK;   // the kernel folds log2(scale) into the exponent
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  CUtensorMap mapQ, mapDO, mapK, mapV;
  int rc;
  if ((rc = make_qkv_maps(q, q_stride, kv, B, M, H, &mapQ, &mapK, &mapV))) return rc;
  if ((rc = make_qkv_maps(d_out, do_stride, nullptr, B, M, H, &mapDO, nullptr, nullptr))) return rc;
  TcDqParams p;
  p.ids = ids; p.i_sb = idx_stride[0]; p.i_sg = idx_stride[1]; p.i_sh = idx_stride[2]; p.i_st = idx_stride[3];
  p.o = static_cast<const char*>(out); p.o_sb = out_stride[0]; p.o_sm = out_stride[1]; p.o_sh = out_stride[2];
  p.dO = static_cast<const char*>(d_out); p.do_sb = do_stride[0]; p.do_sm = do_stride[1]; p.do_sh = do_stride[2];
  p.dq = static_cast<char*>(dq); p.dq_sb = dq_stride[0]; p.dq_sm = dq_stride[1]; p.dq_sh = dq_stride[2];
  p.lse = lse; p.delta = delta;
  p.block_table = kv->block_table; p.max_blocks = kv->max_blocks; p.paged = kv->mode == NSA_KV_PAGED;
  p.n_tokens = kv->n_tokens; p.M = M; p.H = H; p.T = T; p.G = G; p.chunk_size = chunk_size; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  if ((rc = device_status_address(&p.status))) return rc;
  const size_t smem = kSmemTiles + 1024;
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  sel_bwd_dq_tc_kernel<<<dim3(static_cast<unsigned>(cdiv64(M, G)), H, B), kThreads, smem, stream>>>(mapQ, mapDO, mapK, mapV, p);
  NSA_LAUNCH_OK("sel_bwd_dq_tc_kernel");
  *launched = true;
  return NSA_OK;
}

}  // namespace nsa

#ifdef NSA_TC_TRACE
extern "C" int nsa_debug_trace_dq(long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace_dq, sizeof(long long) * 4 * 512));
  return NSA_OK;
}
#endif
