// Selection attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA) for
// the page geometry: bf16, D = 128, 64-token blocks, query groups of up to 64 rows, K/V read
// from a dense [B,N,H,D] tensor or straight from the fixed-page pool through the block table.
//
// One thread block per (batch, query group, head), TWO thread blocks resident per SM (96 KiB
// of tiles and 256 TMEM columns each), so that the list-building prologue and the store epilogue
// of one block run beside the main loop of the other.  A step is ONE selected block (64 keys):
//   warp 4  producer: block list (ballot compaction), Q once, K tiles through a three-stage and V tiles
//           through a two-stage ring (TMA), K one step ahead of V;
//   warp 5  issues S = Q K^T (M=64, N=64, K=128) into a double-buffered TMEM tile, so the scores of
//           step t+1 are computed while the softmax of step t runs;
//   warps 0-3  online softmax on the accumulator fragments (16 rows x 64 keys per warp, the four
//           threads of a quad share a row); P never leaves TMEM: the packed bf16 pairs of the
//           fragment are stored (tcgen05.st.16x128b) over the first 32 of S(t)'s 64 columns;
//   warp 6  issues O += P V (M=64, N=128, K=64) with P as the A operand read from TMEM and the V
//           tile read MN-major in place; S(t+2) is issued once P V of step t has run.
// O stays in TMEM across steps; it is rescaled only when a row's running maximum grows by more than
// 2^8 (the reference maximum is otherwise kept, which is exact because P and the row sum use the
// same reference).  The epilogue normalises the O fragments, stages them with stmatrix in the dead
// Q tile and writes them with TMA tile stores whose box holds one group's rows.
#include "sel_common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <mutex>
#include <string>

namespace nsa {
namespace tc {

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_bf16_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                  const uint32_t* box) {
  EncodeTiledFn enc = encode_tiled_fn();
  NSA_REQUIRE(enc != nullptr, NSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t d[5], s[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), d, s, bx, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NSA_REQUIRE(r == CUDA_SUCCESS, NSA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return NSA_OK;
}

}  // namespace tc

// Sticky device-side status of the tensor-core kernels: set to a negative nsa_status when a
// bounded wait gave up; read (and cleared) by nsa_device_status().
__device__ int g_device_status = 0;

#ifdef NSA_TC_TRACE
// Debug build only: clock64 stamps of thread block (0,0,0); [0][..] MMA issuer, [1][..] softmax thread 0,
// [2][..] producer.
__device__ long long g_trace[3][512];
#define TRACE(role, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (slot) < 512) g_trace[role][slot] = clock64(); } while (0)
#else
#define TRACE(role, slot) do { } while (0)
#endif

namespace {

using namespace tc;

constexpr int kTcThreads = 224;
constexpr int kMaxSlots = 256;
constexpr uint32_t kTile = 16384;              // 64 rows x 256 bytes, as two 64-column halves of 8 KiB
constexpr int kKStages = 3;
constexpr uint32_t kSmemTiles = kTile + kKStages * kTile + 2 * kTile;   // Q, K x3, V x2
constexpr float kRescaleGap = 8.f;             // log2 units
constexpr uint32_t kTmemCols = 256;            // per thread block; two blocks share an SM's 512

// TMEM columns
constexpr uint32_t kColS = 0;      // 2 x 64 fp32 score columns (double buffered); P(t) is packed over the first 32 of S(t)'s
constexpr uint32_t kColO = 128;    // 128

struct TcFwdParams {
  const int32_t* ids;
  int64_t i_sb, i_sg, i_sh, i_st;
  char* out;
  int64_t o_sb, o_sm, o_sh;
  float* lse;
  const int32_t* block_table;
  int max_blocks;
  int paged;
  int64_t n_tokens, M;
  int H, T, G, chunk_size, causal;
  float scale_log2;
  int32_t* status;
};

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

__global__ void __launch_bounds__(kTcThreads, 2)
sel_fwd_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO,
                  const TcFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = tiles;                   // [2][64][128 B]; reused as the output staging tile by the epilogue
  uint8_t* sK = tiles + kTile;                     // kKStages stages
  uint8_t* sV = tiles + (1 + kKStages) * kTile;    // 2 stages

  __shared__ uint64_t q_full, k_full[kKStages], k_empty[kKStages], v_full[2], v_empty[2], s_full[2], p_full[2], p_free[2],
      pv_done, o_final;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort, s_nb;
  __shared__ int s_row[kMaxSlots], s_nvis[kMaxSlots];

  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t m0 = static_cast<int64_t>(g) * p.G;
  const int n_q = static_cast<int>(p.M - m0 < p.G ? p.M - m0 : p.G);
  const int q_chunk = static_cast<int>(m0 / p.chunk_size);

  chain_release();
  if (threadIdx.x == 0) TRACE(1, 0);
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128); mbar_init(&p_free[i], 1);
    }
    for (int i = 0; i < kKStages; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    mbar_init(&pv_done, 1);
    mbar_init(&o_final, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, kTmemCols);
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  chain_wait();                                // everything above needs no result of the kernel before this one
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
  char* out_row0 = p.out + (b * p.o_sb + m0 * p.o_sm + h * p.o_sh) * 2;
  float* lse_row0 = p.lse + (static_cast<int64_t>(b) * p.H + h) * p.M + m0;
  if (threadIdx.x == 0) TRACE(1, 1);

  if (nb == 0) {
    // nothing visible: O = 0, LSE = -inf
    for (int i = threadIdx.x; i < n_q * 16; i += blockDim.x)
      *reinterpret_cast<uint4*>(out_row0 + (i >> 4) * p.o_sm * 2 + (i & 15) * 16) = make_uint4(0, 0, 0, 0);
    for (int r = threadIdx.x; r < n_q; r += blockDim.x) lse_row0[r] = -INFINITY;
  } else if (warp == 4) {
    // ======================= TMA producer =======================
    if (lane == 0) {
      mbar_expect_tx(&q_full, kTile);
      tma_load_5d(sQ, &mapQ, 0, h, static_cast<int>(m0), 0, b, &q_full);
      // K runs one step ahead of V: K(t+1) is asked for before V(t), so that a K tile is in flight
      // while the step before it still holds both V stages
      int kt = 0, vt = 0;                             // copies issued so far
      auto load_k = [&](int t) {
        const int ks = t % kKStages;
        if (!mbar_wait(&k_empty[ks], ((t / kKStages) & 1) ^ 1, abort)) return false;
        mbar_expect_tx(&k_full[ks], kTile);
        if (p.paged) tma_load_3d(sK + ks * kTile, &mapK, 0, s_row[t], 0, &k_full[ks]);
        else tma_load_5d(sK + ks * kTile, &mapK, 0, h, s_row[t], 0, b, &k_full[ks]);
        ++kt;
        return true;
      };
      bool okp = load_k(0);
      for (int t = 0; okp && t < nb; ++t) {
        if (t + 1 < nb && !(okp = load_k(t + 1))) break;
        const int st = t & 1, ph = (t >> 1) & 1;
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort)) break;
        mbar_expect_tx(&v_full[st], kTile);
        if (p.paged) tma_load_3d(sV + st * kTile, &mapV, 0, s_row[t], 0, &v_full[st]);
        else tma_load_5d(sV + st * kTile, &mapV, 0, h, s_row[t], 0, b, &v_full[st]);
        ++vt;
      }
      if (*abort) {
        // the other roles have stopped consuming: wait (bounded) for the copies still in flight
        for (int u = (kt > kKStages ? kt - kKStages : 0); u < kt; ++u) mbar_wait(&k_full[u % kKStages], (u / kKStages) & 1, abort);
        for (int u = (vt > 2 ? vt - 2 : 0); u < vt; ++u) mbar_wait(&v_full[u & 1], (u >> 1) & 1, abort);
        mbar_wait(&q_full, 0, abort);
      }
    }
  } else if (warp == 5) {
    // ======================= MMA issuer 1: S = Q K^T (whole warp runs the loop, one elected lane issues) =======================
    constexpr uint32_t idesc = instr_desc_bf16(64, 64, 0, 0);          // both operands K-major
    const uint32_t el = elect_one();
    const uint64_t dQ = smem_desc(smem_u32(sQ), 16, 1024);
    bool ok = __all_sync(0xffffffffu, mbar_wait(&q_full, 0, abort));
    TRACE(0, 0);
    for (int t = 0; ok && t < nb; ++t) {
      const int st = t & 1, ph = (t >> 1) & 1;
      // P(t-2) lives in the columns of S(t-2): they are free once P V of step t-2 has run
      const int ks = t % kKStages;
      ok = __all_sync(0xffffffffu, mbar_wait(&k_full[ks], (t / kKStages) & 1, abort) &&
                                   (t < 2 || mbar_wait(&p_free[st], ((t - 2) >> 1) & 1, abort)));
      if (!ok) break;
      tc_fence_after();
      TRACE(0, 8 + t * 8 + 0);
      const uint64_t dK = smem_desc(smem_u32(sK + ks * kTile), 16, 1024);
      if (el) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tm + kColS + st * 64, desc_advance(dQ, off), desc_advance(dK, off), idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[ks]);
      }
      __syncwarp();
      TRACE(0, 8 + t * 8 + 1);
    }
  } else if (warp == 6) {
    // ======================= MMA issuer 2: O += P V =======================
    constexpr uint32_t idesc = instr_desc_bf16(64, 128, 0, 1);         // A (P) K-major, B (V tile) MN-major
    const uint32_t el = elect_one();
    for (int t = 0; t < nb; ++t) {
      const int st = t & 1, ph = (t >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&v_full[st], ph, abort) && mbar_wait(&p_full[st], ph, abort))) break;
      tc_fence_after();
      TRACE(0, 8 + t * 8 + 2);
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
      TRACE(0, 8 + t * 8 + 3);
    }
  } else if (warp < 4) {
    // ======================= softmax on accumulator fragments (warps 0-3) =======================
    // Warp w owns query rows 16w .. 16w+15 (TMEM lanes 32w .. 32w+15 of the M=64 accumulators); thread t
    // holds rows r0 = 16w + t/4 and r1 = r0 + 8, columns 8i + 2(t%4), +1 of every 8-column block i; the
    // four threads of a quad share a row and keep its running maximum identical (quad shuffles).
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int cq = (lane & 3) * 2;
    const int st_row = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);   // stmatrix: row this lane addresses
    const int st_chunk = lane >> 4;
    const float sl = p.scale_log2;
    float m_0 = -INFINITY, m_1 = -INFINITY, l_0 = 0.f, l_1 = 0.f;        // l: this thread's share of the row sums
    bool ok = true;
    for (int t = 0; t < nb; ++t) {
      const int sb = t & 1, ph = (t >> 1) & 1;
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 0);
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], ph, abort));
      if (!ok) break;
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 1);
      tc_fence_after();
      uint32_t x[32];
      tmem_ld_16x256b_x8_nowait(tm + lane_base + kColS + sb * 64, x);
      const int nv = s_nvis[t];
      tmem_ld_wait();
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 2);
      // running maxima on the unscaled scores (the scale is positive)
      float t0 = -INFINITY, t1 = -INFINITY;
      if (nv == 64) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          t0 = fmaxf(t0, fmaxf(__uint_as_float(x[4 * i]), __uint_as_float(x[4 * i + 1])));
          t1 = fmaxf(t1, fmaxf(__uint_as_float(x[4 * i + 2]), __uint_as_float(x[4 * i + 3])));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = 8 * i + cq;
          if (c < nv) { t0 = fmaxf(t0, __uint_as_float(x[4 * i])); t1 = fmaxf(t1, __uint_as_float(x[4 * i + 2])); }
          if (c + 1 < nv) { t0 = fmaxf(t0, __uint_as_float(x[4 * i + 1])); t1 = fmaxf(t1, __uint_as_float(x[4 * i + 3])); }
        }
      }
      t0 = quad_max(t0) * sl;
      t1 = quad_max(t1) * sl;
      const bool need0 = t0 > m_0 + kRescaleGap, need1 = t1 > m_1 + kRescaleGap;   // true at the first step (m = -inf)
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 3);
      if (__any_sync(0xffffffffu, need0 || need1)) {
        const float n0 = need0 ? t0 : m_0, n1 = need1 ? t1 : m_1;
        if (t > 0) {
          // O holds sums relative to the old maxima: rescale it once P V of step t-1 has completed
          // (P V of step t-2 is known complete from p_free, so this wait cannot alias a phase)
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done, (t - 1) & 1, abort));
          if (!ok) break;
          tc_fence_after();
          const float c0 = need0 ? fast_exp2(m_0 - n0) : 1.f, c1 = need1 ? fast_exp2(m_1 - n1) : 1.f;
          l_0 *= c0;
          l_1 *= c1;
#pragma unroll
          for (int dh = 0; dh < 2; ++dh) {
            uint32_t o[32];
            tmem_ld_16x256b_x8_nowait(tm + lane_base + kColO + dh * 64, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              o[4 * i] = __float_as_uint(__uint_as_float(o[4 * i]) * c0);
              o[4 * i + 1] = __float_as_uint(__uint_as_float(o[4 * i + 1]) * c0);
              o[4 * i + 2] = __float_as_uint(__uint_as_float(o[4 * i + 2]) * c1);
              o[4 * i + 3] = __float_as_uint(__uint_as_float(o[4 * i + 3]) * c1);
            }
            tmem_st_16x256b_x8_nowait(tm + lane_base + kColO + dh * 64, o);
          }
          tmem_st_wait();
          tc_fence_before();
        }
        m_0 = n0;
        m_1 = n1;
      }
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 4);
      // probabilities, packed in place: x[2i] = row r0 / x[2i+1] = row r1 of key block i
      {
        const float g0 = -m_0, g1 = -m_1;
        float a0 = 0.f, a1 = 0.f;
        if (nv == 64) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float p00 = fast_exp2(fmaf(__uint_as_float(x[4 * i]), sl, g0));
            const float p01 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 1]), sl, g0));
            const float p10 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 2]), sl, g1));
            const float p11 = fast_exp2(fmaf(__uint_as_float(x[4 * i + 3]), sl, g1));
            a0 += p00 + p01;
            a1 += p10 + p11;
            x[2 * i] = pack2<__nv_bfloat16>(p00, p01);
            x[2 * i + 1] = pack2<__nv_bfloat16>(p10, p11);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = 8 * i + cq;
            const float p00 = (c < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i]), sl, g0)) : 0.f;
            const float p01 = (c + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 1]), sl, g0)) : 0.f;
            const float p10 = (c < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 2]), sl, g1)) : 0.f;
            const float p11 = (c + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(x[4 * i + 3]), sl, g1)) : 0.f;
            a0 += p00 + p01;
            a1 += p10 + p11;
            x[2 * i] = pack2<__nv_bfloat16>(p00, p01);
            x[2 * i + 1] = pack2<__nv_bfloat16>(p10, p11);
          }
        }
        l_0 += a0;
        l_1 += a1;
      }
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 5);
      // P stays in TMEM, packed over the first 32 of S(t)'s 64 columns, as the A operand of P V
      tmem_st_16x128b_x8_nowait(tm + lane_base + kColS + sb * 64, x);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[sb]);
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 6);
    }
    if (threadIdx.x == 0) TRACE(1, 2);
    // ---- epilogue: normalise the O fragments, stage them as bf16 in the dead Q tile, TMA tile stores
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&o_final, 0, abort));
    if (threadIdx.x == 0) TRACE(1, 3);
    if (ok) {
      tc_fence_after();
      const float L0 = quad_sum(l_0), L1 = quad_sum(l_1);
      const float i0 = L0 > 0.f ? 1.f / L0 : 0.f, i1 = L1 > 0.f ? 1.f / L1 : 0.f;
      if ((lane & 3) == 0) {
        if (r0 < n_q) lse_row0[r0] = L0 > 0.f ? (m_0 + log2f(L0)) * kLn2 : -INFINITY;
        if (r1 < n_q) lse_row0[r1] = L1 > 0.f ? (m_1 + log2f(L1)) * kLn2 : -INFINITY;
      }
#pragma unroll
      for (int dh = 0; dh < 2; ++dh) {
        uint32_t o[32];
        tmem_ld_16x256b_x8_nowait(tm + lane_base + kColO + dh * 64, o);
        tmem_ld_wait();
        const uint32_t aO = smem_u32(sQ) + dh * 8192 + st_row * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j0 = 2 * q, j1 = 2 * q + 1;
          const uint32_t a0 = pack2<__nv_bfloat16>(__uint_as_float(o[4 * j0]) * i0, __uint_as_float(o[4 * j0 + 1]) * i0);
          const uint32_t b0 = pack2<__nv_bfloat16>(__uint_as_float(o[4 * j0 + 2]) * i1, __uint_as_float(o[4 * j0 + 3]) * i1);
          const uint32_t a1 = pack2<__nv_bfloat16>(__uint_as_float(o[4 * j1]) * i0, __uint_as_float(o[4 * j1 + 1]) * i0);
          const uint32_t b1 = pack2<__nv_bfloat16>(__uint_as_float(o[4 * j1 + 2]) * i1, __uint_as_float(o[4 * j1 + 3]) * i1);
          stmatrix_x4(aO + static_cast<uint32_t>(((2 * q + st_chunk) ^ (st_row & 7)) << 4), a0, b0, a1, b1);
        }
      }
      fence_async_smem();
    }
    named_barrier(1, 128);
    if (ok && threadIdx.x == 0) {
      for (int dh = 0; dh < 2; ++dh) tma_store_4d(&mapO, sQ + dh * 8192, dh * 64, h, static_cast<int>(m0), b);
      bulk_commit_group();
      bulk_wait_all();
    }
  }

  if (threadIdx.x == 0) TRACE(1, 4);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, kTmemCols);
  if (threadIdx.x == 0) TRACE(1, 5);
  if (threadIdx.x == 0 && s_abort) atomicExch(p.status ? p.status : &g_device_status, NSA_ERR_CUDA);
}

}  // namespace

// Device address of the sticky status word, for kernels in other translation units (looked up
// once per device with that device current).
int device_status_address(int32_t** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int32_t* cached[kMaxDevices] = {};
  int dev = -1;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_REQUIRE(dev >= 0 && dev < kMaxDevices, NSA_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    NSA_CUDA_OK(cudaGetSymbolAddress(&p, g_device_status));
    cached[dev] = static_cast<int32_t*>(p);
  }
  *out = cached[dev];
  return NSA_OK;
}

// Maps whose box is a whole 64-row x 128-column tile of one head, landing in shared memory as
// the two 64-column halves one after the other ([half][row][64], each half 128-byte swizzled):
// the head dimension is split into (64, 2) and the half index is placed ABOVE the row dimension.
// Dense tensors [B,M,H,128]: coordinates (0, head, row, 0, batch); paged K/V [rows,128]:
// coordinates (0, row, 0).  One copy instruction per tile instead of two.
int make_tile_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                   CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV) {
  int rc;
  const uint32_t box5[5] = {64, 1, 64, 2, 1};
  auto dense = [&](CUtensorMap* map, const void* base, const int64_t* stride, int64_t rows) {
    const uint64_t dims[5] = {64, static_cast<uint64_t>(H), static_cast<uint64_t>(rows), 2, static_cast<uint64_t>(B)};
    const uint64_t st[4] = {static_cast<uint64_t>(stride[2]) * 2, static_cast<uint64_t>(stride[1]) * 2, 128,
                            B > 1 ? static_cast<uint64_t>(stride[0]) * 2 : static_cast<uint64_t>(stride[1]) * 2 * rows};
    return tc::make_bf16_map(map, base, 5, dims, st, box5);
  };
  if (q != nullptr && (rc = dense(mapQ, q, q_stride, M))) return rc;
  if (kv == nullptr) return NSA_OK;
  if (kv->mode == NSA_KV_DENSE) {
    if ((rc = dense(mapK, kv->k, kv->k_stride, kv->n_tokens))) return rc;
    if ((rc = dense(mapV, kv->v, kv->v_stride, kv->n_tokens))) return rc;
  } else {
    const uint64_t rows = kv->num_pages > 0 ? static_cast<uint64_t>(kv->num_pages) * 64 : (1ull << 31);
    const uint64_t dims[3] = {64, rows, 2};
    const uint64_t st[2] = {256, 128};
    const uint32_t box[3] = {64, 64, 2};
    if ((rc = tc::make_bf16_map(mapK, kv->k, 3, dims, st, box))) return rc;
    if ((rc = tc::make_bf16_map(mapV, kv->v, 3, dims, st, box))) return rc;
  }
  return NSA_OK;
}

// 4-D map of a [B,M,H,128] bf16 tensor whose box holds `box_rows` rows of one head (64 columns):
// for tile stores of a query group shorter than 64 rows, which must not touch the next group.
int make_rows_map(const void* q, const int64_t* q_stride, int B, int64_t M, int H, int box_rows, CUtensorMap* map) {
  const uint32_t box4[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  const uint64_t dims[4] = {128, static_cast<uint64_t>(H), static_cast<uint64_t>(M), static_cast<uint64_t>(B)};
  const uint64_t st[3] = {static_cast<uint64_t>(q_stride[2]) * 2, static_cast<uint64_t>(q_stride[1]) * 2,
                          B > 1 ? static_cast<uint64_t>(q_stride[0]) * 2 : static_cast<uint64_t>(q_stride[1]) * 2 * M};
  return tc::make_bf16_map(map, q, 4, dims, st, box4);
}

// Returns NSA_OK after launching, or NSA_ERR_UNSUPPORTED (without setting an error) when the
// tensor-core kernel does not cover the call and the caller should use the general kernel.
int try_launch_sel_fwd_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* ids,
                          const int64_t* idx_stride, void* out, const int64_t* out_stride, float* lse, int B,
                          int64_t M, int H, int D, int T, int block_size, int chunk_size, int causal, int G,
                          float scale, int dtype, int32_t* status, cudaStream_t stream, bool* launched) {
  *launched = false;
  // test hook: OMNIMEM_B200_FWD_KERNEL=general sends every shape to the general kernel
  const char* env = getenv("OMNIMEM_B200_FWD_KERNEL");
  if (env != nullptr && std::string(env) == "general") return NSA_OK;
  if (dtype != NSA_BF16 || D != 128 || block_size != 64 || G > 64 || G < 16 || T > kMaxSlots) return NSA_OK;
  if (!(scale > 0.f)) return NSA_OK;   // the running maximum is taken on the unscaled scores
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  const int64_t MG = cdiv64(M, G);

  if (H == 1) return NSA_OK;   // a size-1 head dimension may carry an arbitrary stride: leave it to the general kernel
  // the output leaves through TMA tile stores: 16-byte aligned rows
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0 || (out_stride[0] * 2) % 16 != 0 || (out_stride[1] * 2) % 16 != 0 ||
      (out_stride[2] * 2) % 16 != 0)
    return NSA_OK;
  CUtensorMap mapQ, mapK, mapV, mapO;
  int rc;
  if ((rc = make_tile_maps(q, q_stride, kv, B, M, H, &mapQ, &mapK, &mapV))) return rc;
  // the store box holds G rows: a group shorter than 64 rows must not write into the next group
  if ((rc = make_rows_map(out, out_stride, B, M, H, G, &mapO))) return rc;

  TcFwdParams p;
  p.ids = ids;
  p.i_sb = idx_stride[0]; p.i_sg = idx_stride[1]; p.i_sh = idx_stride[2]; p.i_st = idx_stride[3];
  p.out = static_cast<char*>(out);
  p.o_sb = out_stride[0]; p.o_sm = out_stride[1]; p.o_sh = out_stride[2];
  p.lse = lse;
  p.block_table = kv->block_table; p.max_blocks = kv->max_blocks; p.paged = kv->mode == NSA_KV_PAGED;
  p.n_tokens = kv->n_tokens; p.M = M;
  p.H = H; p.T = T; p.G = G; p.chunk_size = chunk_size; p.causal = causal;
  p.scale_log2 = scale * kLog2e;
  p.status = status;
  const size_t smem = kSmemTiles + 1024;
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_fwd_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                   static_cast<int>(cudaSharedmemCarveoutMaxShared)));
  NSA_CUDA_OK(launch_chained(kChainFwd, sel_fwd_tc_kernel, dim3(static_cast<unsigned>(MG), H, B), dim3(kTcThreads), smem, stream, mapQ, mapK, mapV,
                             mapO, p));
  NSA_LAUNCH_OK("sel_fwd_tc_kernel");
  *launched = true;
  return NSA_OK;
}

}  // namespace nsa

extern "C" int nsa_device_status(int32_t* value) {
  NSA_REQUIRE(value != nullptr, NSA_ERR_INVALID, "device_status: null pointer");
  int v = 0;
  NSA_CUDA_OK(cudaMemcpyFromSymbol(&v, nsa::g_device_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NSA_CUDA_OK(cudaMemcpyToSymbol(nsa::g_device_status, &zero, sizeof(int)));
  }
  *value = v;
  return NSA_OK;
}

#ifdef NSA_TC_TRACE
extern "C" int nsa_debug_trace(long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace, sizeof(long long) * 3 * 512));
  return NSA_OK;
}
#endif
