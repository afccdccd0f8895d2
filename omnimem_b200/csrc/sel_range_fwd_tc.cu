// Attention of every query over ONE contiguous range of KV blocks, on tcgen05 / TMEM / TMA
// (bf16, D = 128, 64-token blocks; K/V dense or in the fixed-page pool).  This is what the layer's
// compressed branch (all pooled rows) and sliding-window branch (the last chunks' pages) compute:
// the same softmax attention as the selection forward with every query group listing the same
// blocks.  Because the list is shared, a thread block takes 128 query rows instead of one group of
// 64: the products run on full-height tiles and every K / V tile serves twice the rows.
//
// One thread block per (batch, 128 query rows, head), two resident per SM (96 KiB of tiles, 256
// TMEM columns each).  A step is one block of the range (64 keys):
//   warp 4  producer: the list of the range's resident blocks, Q once (128 rows), K and V tiles
//           through two-stage rings (TMA), K one step ahead of V;
//   warp 5  issues S = Q K^T (M=128, N=64, K=128) into a double-buffered TMEM tile;
//   warps 0-3  online softmax, ONE ROW PER THREAD (TMEM lane = query row): running maximum, the
//           exponentials, the row sum; P goes back into TMEM as packed bf16 pairs over the first 32
//           of S(t)'s 64 columns, the A operand of the second product;
//   warp 6  issues O += P V (M=128, N=128, K=64), V read MN-major in place.
// O stays in TMEM and is rescaled only when a row's maximum grows by more than 2^8.  The epilogue
// normalises O, stages it as bf16 in the dead Q tile and writes it with one TMA tile store.
//
// A long range over few query tiles does not fill the machine evenly (444 tiles on 296 slots run as
// one full wave and one half-empty one), so the launch may cut the range into `splits` spans of
// steps: the thread block of (tile, span) writes a partial output and its log-sum-exp into a
// workspace and nsa_merge_partials joins the spans exactly.
#include "sel_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <string>

namespace nsa {

int device_status_address(int32_t** out);
int make_tile_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                   CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV);

namespace {

using namespace tc;

constexpr int kThreads = 224;
constexpr int kMaxRange = 1024;                // blocks of a range one launch serves
constexpr uint32_t kTile = 16384;              // 64 rows x 256 bytes, as two 64-column halves of 8 KiB
constexpr uint32_t kQTile = 32768;             // 128 rows x 256 bytes, as two 64-column halves of 16 KiB
constexpr uint32_t kSmemTiles = kQTile + 2 * kTile + 2 * kTile;   // Q, K x2, V x2
constexpr float kRescaleGap = 8.f;             // log2 units
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0;      // 2 x 64 fp32 score columns (double buffered); P(t) is packed over the first 32 of S(t)'s
constexpr uint32_t kColO = 128;    // 128

struct RangeFwdParams {
  float* lse;
  const int32_t* block_table;
  int max_blocks, paged;
  int64_t n_tokens, M;
  int H, B, first_block, n_blocks, splits;
  float scale_log2;
  char* out; int64_t o_sb, o_sm, o_sh;     // only for zero-filling when nothing is visible
  int32_t* status;
};

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 2)
sel_range_fwd_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                        const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO,
                        const RangeFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = tiles;                   // [2][128][128 B]; reused as the output staging tile by the epilogue
  uint8_t* sK = tiles + kQTile;          // 2 stages
  uint8_t* sV = sK + 2 * kTile;          // 2 stages

  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], p_free[2], pv_done, o_final;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort, s_nb;
  __shared__ int s_row[kMaxRange];
  __shared__ int s_last_nv;

  const int h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = static_cast<int>(blockIdx.x) % p.splits;
  const int bo = split * p.B + b;               // batch coordinate of the output (partials: [splits][B])
  const int64_t m0 = static_cast<int64_t>(blockIdx.x / p.splits) * 128;
  const int n_q = static_cast<int>(p.M - m0 < 128 ? p.M - m0 : 128);

  chain_release();
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128); mbar_init(&p_free[i], 1);
    }
    mbar_init(&pv_done, 1);
    mbar_init(&o_final, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, kTmemCols);
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  chain_wait();                                // everything above needs no result of the kernel before this one
  // ---- the range's resident blocks (TMA row coordinate), compacted by warp 4; only the last block of
  // the KV can be partly filled
  if (warp == 4) {
    int base = 0, last_nv = 64;
    for (int t0 = 0; t0 < p.n_blocks; t0 += 32) {
      const int t = t0 + lane;
      int row = -1, nv = 0;
      if (t < p.n_blocks) {
        const int bid = p.first_block + t;
        const int64_t tok0 = static_cast<int64_t>(bid) * 64;
        if (bid >= 0 && tok0 < p.n_tokens) {
          nv = static_cast<int>(p.n_tokens - tok0 < 64 ? p.n_tokens - tok0 : 64);
          if (p.paged) {
            const int page = bid < p.max_blocks ? p.block_table[static_cast<int64_t>(h) * p.max_blocks + bid] : -1;
            if (page >= 0) row = page * 64; else nv = 0;
          } else {
            row = static_cast<int>(tok0);
          }
        }
      }
      const unsigned live = __ballot_sync(0xffffffffu, nv > 0);
      if (nv > 0) s_row[base + __popc(live & ((1u << lane) - 1u))] = row;
      // (blocks are in ascending order: a partly filled one can only be the last listed)
      const unsigned part = __ballot_sync(0xffffffffu, nv > 0 && nv < 64);
      if (part) last_nv = __shfl_sync(0xffffffffu, nv, 31 - __clz(part));
      base += __popc(live);
    }
    if (lane == 0) { s_nb = base; s_last_nv = last_nv; }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_base_s;
  volatile int* abort = &s_abort;
  // this thread block's span of the list
  const int nb_all = s_nb;
  const int lo = static_cast<int>(static_cast<int64_t>(nb_all) * split / p.splits);
  const int nb = static_cast<int>(static_cast<int64_t>(nb_all) * (split + 1) / p.splits) - lo;
  const int* rows = s_row + lo;
  const int t_part = nb_all - 1 - lo;           // the step of the partly filled block, if it falls in this span
  float* lse_row0 = p.lse + (static_cast<int64_t>(bo) * p.H + h) * p.M + m0;

  if (nb == 0) {
    // nothing to attend: O = 0, LSE = -inf
    char* out_row0 = p.out + (bo * p.o_sb + m0 * p.o_sm + h * p.o_sh) * 2;
    for (int i = threadIdx.x; i < n_q * 16; i += blockDim.x)
      *reinterpret_cast<uint4*>(out_row0 + (i >> 4) * p.o_sm * 2 + (i & 15) * 16) = make_uint4(0, 0, 0, 0);
    for (int r = threadIdx.x; r < n_q; r += blockDim.x) lse_row0[r] = -INFINITY;
  } else if (warp == 4) {
    // ======================= TMA producer =======================
    if (lane == 0) {
      mbar_expect_tx(&q_full, kQTile);
      tma_load_5d(sQ, &mapQ, 0, h, static_cast<int>(m0), 0, b, &q_full);
      int kt = 0, vt = 0;                             // copies issued so far
      auto load_k = [&](int t) {
        const int ks = t & 1;
        if (!mbar_wait(&k_empty[ks], ((t >> 1) & 1) ^ 1, abort)) return false;
        mbar_expect_tx(&k_full[ks], kTile);
        if (p.paged) tma_load_3d(sK + ks * kTile, &mapK, 0, rows[t], 0, &k_full[ks]);
        else tma_load_5d(sK + ks * kTile, &mapK, 0, h, rows[t], 0, b, &k_full[ks]);
        ++kt;
        return true;
      };
      bool okp = load_k(0);
      for (int t = 0; okp && t < nb; ++t) {
        if (t + 1 < nb && !(okp = load_k(t + 1))) break;
        const int st = t & 1, ph = (t >> 1) & 1;
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort)) break;
        mbar_expect_tx(&v_full[st], kTile);
        if (p.paged) tma_load_3d(sV + st * kTile, &mapV, 0, rows[t], 0, &v_full[st]);
        else tma_load_5d(sV + st * kTile, &mapV, 0, h, rows[t], 0, b, &v_full[st]);
        ++vt;
      }
      if (*abort) {
        // the other roles have stopped consuming: wait (bounded) for the copies still in flight
        for (int u = (kt > 2 ? kt - 2 : 0); u < kt; ++u) mbar_wait(&k_full[u & 1], (u >> 1) & 1, abort);
        for (int u = (vt > 2 ? vt - 2 : 0); u < vt; ++u) mbar_wait(&v_full[u & 1], (u >> 1) & 1, abort);
        mbar_wait(&q_full, 0, abort);
      }
    }
  } else if (warp == 5) {
    // ======================= MMA issuer 1: S = Q K^T (whole warp runs the loop, one elected lane issues) =======================
    constexpr uint32_t idesc = instr_desc_bf16(128, 64, 0, 0);         // both operands K-major
    const uint32_t el = elect_one();
    const uint64_t dQ = smem_desc(smem_u32(sQ), 16, 1024);
    bool ok = __all_sync(0xffffffffu, mbar_wait(&q_full, 0, abort));
    for (int t = 0; ok && t < nb; ++t) {
      const int st = t & 1;
      // P(t-2) lives in the columns of S(t-2): they are free once P V of step t-2 has run
      ok = __all_sync(0xffffffffu, mbar_wait(&k_full[st], (t >> 1) & 1, abort) &&
                                   (t < 2 || mbar_wait(&p_free[st], ((t - 2) >> 1) & 1, abort)));
      if (!ok) break;
      tc_fence_after();
      const uint64_t dK = smem_desc(smem_u32(sK + st * kTile), 16, 1024);
      if (el) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tm + kColS + st * 64, desc_advance(dQ, (kk >> 2) * 16384 + (kk & 3) * 32),
                  desc_advance(dK, (kk >> 2) * 8192 + (kk & 3) * 32), idesc, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
      }
      __syncwarp();
    }
  } else if (warp == 6) {
    // ======================= MMA issuer 2: O += P V =======================
    constexpr uint32_t idesc = instr_desc_bf16(128, 128, 0, 1);        // A (P) K-major from TMEM, B (V tile) MN-major
    const uint32_t el = elect_one();
    for (int t = 0; t < nb; ++t) {
      const int st = t & 1, ph = (t >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&v_full[st], ph, abort) && mbar_wait(&p_full[st], ph, abort))) break;
      tc_fence_after();
      // V tile [64 keys][128 dims] as two 64-column boxes 8 KiB apart, read with the head dim as N
      const uint64_t dVmn = smem_desc(smem_u32(sV + st * kTile), 8192, 1024);
      if (el) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts(tm + kColO, tm + kColS + st * 64 + kk * 8, desc_advance(dVmn, kk * 2048), idesc, (t > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&v_empty[st]);
        umma_commit(&p_free[st]);
        umma_commit(&pv_done);
        if (t == nb - 1) umma_commit(&o_final);
      }
      __syncwarp();
    }
  } else if (warp < 4) {
    // ======================= softmax, one query row per thread (warps 0-3) =======================
    // Thread (warp w, lane l) owns row 32w + l = TMEM lane 32w + l of the M=128 accumulators.
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int row = warp * 32 + lane;
    const float sl = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int t = 0; t < nb; ++t) {
      const int sb = t & 1, ph = (t >> 1) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], ph, abort));
      if (!ok) break;
      tc_fence_after();
      uint32_t x[32], y[32];                              // keys 0-31 and 32-63 of the block
      tmem_ld32_nowait(tm + lane_base + kColS + sb * 64, x);
      tmem_ld32_nowait(tm + lane_base + kColS + sb * 64 + 32, y);
      const int nv = t == t_part ? s_last_nv : 64;
      tmem_ld_wait();
      // running maximum on the unscaled scores (the scale is positive)
      float tmax = -INFINITY;
      if (nv == 64) {
        float u0 = -INFINITY, u1 = -INFINITY, u2 = -INFINITY, u3 = -INFINITY;     // four chains, not one of 32
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          u0 = fmaxf(u0, fmaxf(__uint_as_float(x[4 * i]), __uint_as_float(y[4 * i])));
          u1 = fmaxf(u1, fmaxf(__uint_as_float(x[4 * i + 1]), __uint_as_float(y[4 * i + 1])));
          u2 = fmaxf(u2, fmaxf(__uint_as_float(x[4 * i + 2]), __uint_as_float(y[4 * i + 2])));
          u3 = fmaxf(u3, fmaxf(__uint_as_float(x[4 * i + 3]), __uint_as_float(y[4 * i + 3])));
        }
        tmax = fmaxf(fmaxf(u0, u1), fmaxf(u2, u3));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i < nv) tmax = fmaxf(tmax, __uint_as_float(x[i]));
          if (32 + i < nv) tmax = fmaxf(tmax, __uint_as_float(y[i]));
        }
      }
      tmax *= sl;
      const bool need = tmax > m_run + kRescaleGap;          // true at the first step (m = -inf)
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = need ? tmax : m_run;
        if (t > 0) {
          // O holds sums relative to the old maximum: rescale it once P V of step t-1 has completed
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done, (t - 1) & 1, abort));
          if (!ok) break;
          tc_fence_after();
          const float c = need ? fast_exp2(m_run - m_new) : 1.f;
          l_run *= c;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t o[32];
            tmem_ld32_nowait(tm + lane_base + kColO + c4 * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * c);
            tmem_st32_nowait(tm + lane_base + kColO + c4 * 32, o);
          }
          tmem_st_wait();
          tc_fence_before();
        }
        m_run = m_new;
      }
      // probabilities, packed in place: x[i] = keys (2i, 2i+1) for i < 16, then keys (32 + 2(i-16), +1)
      // from y once the upper half of x is dead
      {
        const float g = -m_run;
        float a0 = 0.f, a1 = 0.f;
        if (nv == 64) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(x[2 * i]), sl, g));
            const float p1 = fast_exp2(fmaf(__uint_as_float(x[2 * i + 1]), sl, g));
            a0 += p0; a1 += p1;
            x[i] = pack2<__nv_bfloat16>(p0, p1);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p2 = fast_exp2(fmaf(__uint_as_float(y[2 * i]), sl, g));
            const float p3 = fast_exp2(fmaf(__uint_as_float(y[2 * i + 1]), sl, g));
            a0 += p2; a1 += p3;
            x[16 + i] = pack2<__nv_bfloat16>(p2, p3);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = 2 * i < nv ? fast_exp2(fmaf(__uint_as_float(x[2 * i]), sl, g)) : 0.f;
            const float p1 = 2 * i + 1 < nv ? fast_exp2(fmaf(__uint_as_float(x[2 * i + 1]), sl, g)) : 0.f;
            a0 += p0; a1 += p1;
            x[i] = pack2<__nv_bfloat16>(p0, p1);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p2 = 32 + 2 * i < nv ? fast_exp2(fmaf(__uint_as_float(y[2 * i]), sl, g)) : 0.f;
            const float p3 = 33 + 2 * i < nv ? fast_exp2(fmaf(__uint_as_float(y[2 * i + 1]), sl, g)) : 0.f;
            a0 += p2; a1 += p3;
            x[16 + i] = pack2<__nv_bfloat16>(p2, p3);
          }
        }
        l_run += a0 + a1;
        // P stays in TMEM, packed over the first 32 of S(t)'s 64 columns, as the A operand of P V
        tmem_st32_nowait(tm + lane_base + kColS + sb * 64, x);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[sb]);
    }
    // ---- epilogue: normalise the row of O, stage it as bf16 in the dead Q tile ([half][128 rows][128 B],
    // 16-byte pieces swizzled by the row), one TMA tile store
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&o_final, 0, abort));
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      if (row < n_q) lse_row0[row] = l_run > 0.f ? (m_run + log2f(l_run)) * kLn2 : -INFINITY;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t o[32];
        tmem_ld32_nowait(tm + lane_base + kColO + c4 * 32, o);
        tmem_ld_wait();
        uint8_t* dst = sQ + (c4 >> 1) * 16384 + row * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack2<__nv_bfloat16>(__uint_as_float(o[8 * j]) * inv, __uint_as_float(o[8 * j + 1]) * inv);
          v.y = pack2<__nv_bfloat16>(__uint_as_float(o[8 * j + 2]) * inv, __uint_as_float(o[8 * j + 3]) * inv);
          v.z = pack2<__nv_bfloat16>(__uint_as_float(o[8 * j + 4]) * inv, __uint_as_float(o[8 * j + 5]) * inv);
          v.w = pack2<__nv_bfloat16>(__uint_as_float(o[8 * j + 6]) * inv, __uint_as_float(o[8 * j + 7]) * inv);
          const int chunk = (c4 & 1) * 4 + j;
          *reinterpret_cast<uint4*>(dst + ((chunk ^ (row & 7)) << 4)) = v;
        }
      }
      fence_async_smem();
    }
    named_barrier(1, 128);
    if (ok && threadIdx.x == 0) {
      tma_store_5d(&mapO, sQ, 0, h, static_cast<int>(m0), 0, bo);
      bulk_commit_group();
      bulk_wait_all();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, kTmemCols);
  if (threadIdx.x == 0 && s_abort) atomicExch(p.status, NSA_ERR_CUDA);
}

// 5-D map of a dense [B,M,H,128] bf16 tensor whose box is 128 rows of one head, landing as two
// 64-column halves of 16 KiB each ([half][128 rows][128 B], 128-byte swizzled).
int make_rows128_map(const void* base, const int64_t* stride, int B, int64_t rows, int H, CUtensorMap* map) {
  const uint32_t box5[5] = {64, 1, 128, 2, 1};
  const uint64_t dims[5] = {64, static_cast<uint64_t>(H), static_cast<uint64_t>(rows), 2, static_cast<uint64_t>(B)};
  const uint64_t st[4] = {static_cast<uint64_t>(stride[2]) * 2, static_cast<uint64_t>(stride[1]) * 2, 128,
                          B > 1 ? static_cast<uint64_t>(stride[0]) * 2 : static_cast<uint64_t>(stride[1]) * 2 * rows};
  return tc::make_bf16_map(map, base, 5, dims, st, box5);
}

}  // namespace

// Spans to cut a range of n_blocks steps into, for `items` (batch, tile, head) thread blocks on
// 2 x SM-count resident slots.  Cost of a count = waves x (steps per span + a fixed cost per thread
// block); a last wave that fills at most half the slots runs one thread block per SM, which measured
// 1.7x faster than two sharing one (so it counts 0.65 of a wave).  1 on ties.
int range_fwd_splits(int B, int64_t M, int H, int n_blocks) {
  static int slots = 0;
  if (slots == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    slots = 2 * sms;
  }
  const char* env = getenv("OMNIMEM_B200_RANGE_SPLITS");      // test hook: a fixed count
  if (env != nullptr && atoi(env) >= 1) return atoi(env) > 8 ? 8 : atoi(env);
  const int64_t items = cdiv64(M, 128) * H * B;
  int best = 1;
  int64_t best_cost = 0;
  for (int s = 1; s <= 8; ++s) {
    const int64_t n = items * s, rem = n % slots;
    const int64_t waves100 = (n / slots) * 100 + (rem == 0 ? 0 : rem * 2 <= slots ? 65 : 100);
    int64_t cost = waves100 * (cdiv64(n_blocks, s) + 10);
    if (s > 1) cost += cost / 50 + 200;            // the merge pass
    if (s == 1 || cost < best_cost) { best = s; best_cost = cost; }
  }
  return best;
}

// Launches the range forward when it covers the call (*launched = true); NSA_OK with *launched = false
// leaves the call to the selection forward.  With splits > 1, `out` / `lse` are the partial buffers
// [splits][B,M,H,128] / [splits][B,H,M] (contiguous) that nsa_merge_partials joins.
int try_launch_sel_range_fwd_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int first_block,
                                int n_blocks, void* out, const int64_t* out_stride, float* lse, int B, int64_t M,
                                int H, int D, int block_size, float scale, int dtype, int splits,
                                cudaStream_t stream, bool* launched) {
  *launched = false;
  if (splits < 1 || cdiv64(M, 128) * splits > 0x7fffffff) return NSA_OK;
  if (dtype != NSA_BF16 || D != 128 || block_size != 64 || H == 1 || n_blocks > kMaxRange || n_blocks < 0 || first_block < 0)
    return NSA_OK;
  if (!(scale > 0.f)) return NSA_OK;   // the running maximum is taken on the unscaled scores
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0 || (out_stride[0] * 2) % 16 != 0 || (out_stride[1] * 2) % 16 != 0 ||
      (out_stride[2] * 2) % 16 != 0)
    return NSA_OK;
  CUtensorMap mapQ, mapK, mapV, mapO, unused;
  int rc;
  if ((rc = make_tile_maps(q, q_stride, kv, B, M, H, &unused, &mapK, &mapV))) return rc;
  if ((rc = make_rows128_map(q, q_stride, B, M, H, &mapQ))) return rc;
  if ((rc = make_rows128_map(out, out_stride, B * splits, M, H, &mapO))) return rc;
  RangeFwdParams p;
  p.lse = lse;
  p.block_table = kv->block_table; p.max_blocks = kv->max_blocks; p.paged = kv->mode == NSA_KV_PAGED;
  p.n_tokens = kv->n_tokens; p.M = M; p.H = H; p.B = B; p.first_block = first_block; p.n_blocks = n_blocks;
  p.splits = splits;
  p.scale_log2 = scale * kLog2e;
  p.out = static_cast<char*>(out); p.o_sb = out_stride[0]; p.o_sm = out_stride[1]; p.o_sh = out_stride[2];
  if ((rc = device_status_address(&p.status))) return rc;
  const size_t smem = kSmemTiles + 1024;
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_range_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_range_fwd_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   static_cast<int>(cudaSharedmemCarveoutMaxShared)));
  NSA_CUDA_OK(launch_chained(kChainFwd, sel_range_fwd_tc_kernel, dim3(static_cast<unsigned>(cdiv64(M, 128) * splits), H, B), dim3(kThreads),
                             smem, stream, mapQ, mapK, mapV, mapO, p));
  NSA_LAUNCH_OK("sel_range_fwd_tc_kernel");
  *launched = true;
  return NSA_OK;
}

}  // namespace nsa
