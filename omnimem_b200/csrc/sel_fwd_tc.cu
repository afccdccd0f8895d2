// Selection attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA) for
// the page geometry: bf16, D = 128, 64-token blocks, query groups of up to 64 rows, K/V read
// from a dense [B,N,H,D] tensor or straight from the fixed-page pool through the block table.
//
// One thread block per (batch, query group, head), TWO thread blocks resident per SM (96 KiB of
// tiles and 256 TMEM columns each), so that the load / list-building prologue and the
// merge-and-store epilogue of one block run beside the main loop of the other.  Roles:
//   warp 4  TMA producer: Q once, then per step the K tile of TWO selected blocks (128 keys),
//           coordinates taken from the compacted block list;   warp 6: the same for V;
//   warp 5  MMA issuer: S = [Q;Q] K^T (M=128, N=128, K=128) into TMEM;
//   warp 7  MMA issuer: once the softmax warps have written P over the score columns,
//           O += P V with P read from TMEM;
//   warps 0-3  softmax: one TMEM lane (matrix row) per thread.
// The 64 query rows are loaded twice, into rows 0-63 and 64-127 of the A tile: rows 0-63 do
// the online softmax over the EVEN block of each step (S columns 0-63), rows 64-127 over the
// ODD block (columns 64-127); the other half of each P row is zero, so the two halves
// accumulate attention over disjoint key sets in their own O rows and are merged exactly
// (log-sum-exp weights) in the epilogue.  Every softmax thread therefore has 64 useful
// columns per step and no cross-thread reduction is needed.
// O stays in TMEM across steps; it is rescaled only when a row's running maximum grows by
// more than 2^8 (the reference maximum is otherwise kept, which is exact because P and the
// row sum use the same reference).
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

constexpr int kTcThreads = 256;
constexpr int kMaxSlots = 256;
constexpr uint32_t kTileBytes = 32768;        // 128 rows x 256 bytes, as two 64-column halves of 16 KiB
constexpr uint32_t kSmemTiles = 3 * kTileBytes;   // Q, K, V
constexpr float kRescaleGap = 8.f;            // log2 units
constexpr uint32_t kTmemCols = 256;           // per thread block; two blocks share an SM's 512

// TMEM columns
constexpr uint32_t kColS = 0;      // 128 fp32 score columns; P (64 columns of bf16 pairs) is written over them
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

__global__ void __launch_bounds__(kTcThreads, 2)
sel_fwd_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const TcFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = tiles;
  uint8_t* sK = tiles + kTileBytes;
  uint8_t* sV = tiles + 2 * kTileBytes;
  float* stage = reinterpret_cast<float*>(tiles);   // epilogue: 128 x 129 floats over the dead Q/K/V tiles

  __shared__ uint64_t q_full, k_full, k_empty, v_full, v_empty, s_full, p_full, pv_done, o_final;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort, s_nb;
  __shared__ int s_row[kMaxSlots], s_nvis[kMaxSlots];
  __shared__ float s_m[128], s_l[128];

  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t m0 = static_cast<int64_t>(g) * p.G;
  const int n_q = static_cast<int>(p.M - m0 < p.G ? p.M - m0 : p.G);
  const int q_chunk = static_cast<int>(m0 / p.chunk_size);

  if (threadIdx.x == 0) TRACE(1, 0);
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(&q_full, 1);
    mbar_init(&k_full, 1); mbar_init(&k_empty, 1);
    mbar_init(&v_full, 1); mbar_init(&v_empty, 1);
    mbar_init(&s_full, 1); mbar_init(&p_full, 128);
    mbar_init(&pv_done, 1);
    mbar_init(&o_final, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, kTmemCols);
  if (warp == 4 && lane == 0) {
    // Q does not depend on the block list: start its copy at once (its barrier is initialised by
    // this same thread only when threadIdx.x == 0 is, so the copy is issued after the sync below)
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  // ---- list of the visible selected blocks (TMA row coordinate, visible tokens), compacted by one warp
  if (warp == 1) {
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
  const int NT = (nb + 1) >> 1;
  if (threadIdx.x == 0) TRACE(1, 1);

  // K / V tile of one step: the even block in rows 0-63, the odd block in rows 64-127 of each
  // 64-column half (the even block again when the step has no odd block).
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

  if (nb == 0) {
    // nothing visible: O = 0, LSE = -inf
    for (int i = threadIdx.x; i < n_q * 16; i += blockDim.x)
      *reinterpret_cast<uint4*>(out_row0 + (i >> 4) * p.o_sm * 2 + (i & 15) * 16) = make_uint4(0, 0, 0, 0);
    for (int r = threadIdx.x; r < n_q; r += blockDim.x) lse_row0[r] = -INFINITY;
  } else if (warp == 4 || warp == 6) {
    // ======================= TMA producers: warp 4 loads Q and the K tiles, warp 6 the V tiles =======================
    if (lane == 0) {
      const bool isK = warp == 4;
      uint64_t* full = isK ? &k_full : &v_full;
      uint64_t* empty = isK ? &k_empty : &v_empty;
      uint8_t* dst = isK ? sK : sV;
      const CUtensorMap* map = isK ? &mapK : &mapV;
      if (isK) {
        mbar_expect_tx(&q_full, kTileBytes);
        for (int dh = 0; dh < 2; ++dh)
          for (int dup = 0; dup < 2; ++dup)
            tma_load_4d(sQ + dh * 16384 + dup * 8192, &mapQ, dh * 64, h, static_cast<int>(m0), b, &q_full);
      }
      int t = 0;
      for (; t < NT; ++t) {
        const int re = s_row[2 * t], ro = (2 * t + 1 < nb) ? s_row[2 * t + 1] : re;
        if (!mbar_wait(empty, (t & 1) ^ 1, abort)) break;
        load_tile(dst, map, re, ro, full);
      }
      if (*abort) {
        // the other roles have stopped consuming: wait (bounded) for the copy still in flight
        if (t > 0) mbar_wait(full, (t - 1) & 1, abort);
        if (isK) mbar_wait(&q_full, 0, abort);
      }
    }
  } else if (warp == 5 || warp == 7) {
    // ======================= MMA issuers =======================
    // Per step: S = [Q;Q] K^T (warp 5), softmax writes P over S, O += P V (warp 7).  The next S
    // overwrites P, so it is issued only after the P V product that reads it has completed.
    // Two issuing threads, because each passed barrier wait costs the thread a few hundred cycles.
    // Whole warps run these loops (warp-uniform control flow keeps descriptor arithmetic in uniform
    // registers); one elected lane issues.
    {
      const uint32_t el = elect_one();
      if (warp == 5) {
        constexpr uint32_t idesc_s = instr_desc_bf16(128, 128, 0, 0);
        const uint64_t dQ = smem_desc(smem_u32(sQ), 16, 1024);
        const uint64_t dK = smem_desc(smem_u32(sK), 16, 1024);
        bool ok = __all_sync(0xffffffffu, mbar_wait(&q_full, 0, abort));
        TRACE(0, 0);
        for (int t = 0; ok && t < NT; ++t) {
          const uint32_t ph = t & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(&k_full, ph, abort) && (t == 0 || mbar_wait(&pv_done, ph ^ 1, abort)));
          if (!ok) break;
          TRACE(0, 8 + t * 8 + 0);
          tc_fence_after();
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ss(tm + kColS, desc_advance(dQ, (kk >> 2) * 16384 + (kk & 3) * 32),
                      desc_advance(dK, (kk >> 2) * 16384 + (kk & 3) * 32), idesc_s, kk > 0 ? 1u : 0u);
            umma_commit(&s_full);
            umma_commit(&k_empty);
          }
          __syncwarp();
          TRACE(0, 8 + t * 8 + 1);
        }
      } else {
        constexpr uint32_t idesc_pv = instr_desc_bf16(128, 128, 0, 1);
        const uint64_t dV = smem_desc(smem_u32(sV), 16384, 1024);
        for (int t = 0; t < NT; ++t) {
          const uint32_t ph = t & 1;
          if (!__all_sync(0xffffffffu, mbar_wait(&v_full, ph, abort) && mbar_wait(&p_full, ph, abort))) break;
          TRACE(0, 8 + t * 8 + 2);
          tc_fence_after();
          if (el) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ts(tm + kColO, tm + kColS + kk * 8, desc_advance(dV, kk * 2048), idesc_pv, (t > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&v_empty);
            umma_commit(&pv_done);
            if (t == NT - 1) umma_commit(&o_final);
          }
          __syncwarp();
          TRACE(0, 8 + t * 8 + 3);
        }
      }
    }
  } else if (warp < 4) {
    // ======================= softmax (warps 0-3), one matrix row per thread =======================
    const int half = warp >> 1;                       // 0: even block of each step, 1: odd block
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int t = 0; t < NT; ++t) {
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 0);
      // s_full is committed after the previous step's P V was issued, so its completion also
      // means that O is quiescent and may be rescaled below
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full, t & 1, abort));
      if (!ok) break;
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 1);
      tc_fence_after();
      uint32_t x0[32], x1[32];
      tmem_ld32_nowait(tm + lane_base + kColS + half * 64, x0);
      tmem_ld32_nowait(tm + lane_base + kColS + half * 64 + 32, x1);
      tmem_ld_wait();
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 2);
      const int blk = 2 * t + half;
      const int nv = blk < nb ? s_nvis[blk] : 0;
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float a = __uint_as_float(x0[j]) * p.scale_log2, c = __uint_as_float(x1[j]) * p.scale_log2;
        x0[j] = __float_as_uint(a);
        x1[j] = __float_as_uint(c);
        if (j < nv) tmax = fmaxf(tmax, a);
        if (j + 32 < nv) tmax = fmaxf(tmax, c);
      }
      const bool need = tmax > m_ref + kRescaleGap;      // also true for the first visible key (m_ref = -inf)
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 3);
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = need ? tmax : m_ref;
        if (t > 0) {
          const float sc = need ? fast_exp2(m_ref - m_new) : 1.f;
          l_sum *= sc;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32_nowait(tm + lane_base + kColO + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * sc);
            tmem_st32_nowait(tm + lane_base + kColO + c * 32, o);
          }
        }
        m_ref = m_new;
      }
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 4);
      uint32_t pk[32];
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float a0 = (2 * j < nv) ? fast_exp2(__uint_as_float(x0[2 * j]) - m_ref) : 0.f;
        const float a1 = (2 * j + 1 < nv) ? fast_exp2(__uint_as_float(x0[2 * j + 1]) - m_ref) : 0.f;
        const float c0 = (2 * j + 32 < nv) ? fast_exp2(__uint_as_float(x1[2 * j]) - m_ref) : 0.f;
        const float c1 = (2 * j + 33 < nv) ? fast_exp2(__uint_as_float(x1[2 * j + 1]) - m_ref) : 0.f;
        rs += (a0 + a1) + (c0 + c1);
        pk[j] = pack2<__nv_bfloat16>(a0, a1);
        pk[16 + j] = pack2<__nv_bfloat16>(c0, c1);
      }
      l_sum += rs;
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 5);
      // P over the score columns: this row's 64 probabilities in its own half, zeros in the other
      tmem_st32_nowait(tm + lane_base + kColS + half * 32, pk);
#pragma unroll
      for (int j = 0; j < 32; ++j) pk[j] = 0u;
      tmem_st32_nowait(tm + lane_base + kColS + (1 - half) * 32, pk);
      tmem_st_wait();
      if (threadIdx.x == 0) TRACE(1, 8 + t * 8 + 6);
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    if (threadIdx.x == 0) TRACE(1, 2);
    // ---- epilogue: wait for the last P V, merge the two halves, normalise, store
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&o_final, 0, abort));
    if (threadIdx.x == 0) TRACE(1, 3);
    if (ok) {
      tc_fence_after();
      const int tid = threadIdx.x;                    // 0..127 = TMEM lane = A-tile row
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32_nowait(tm + lane_base + kColO + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[tid * 129 + c * 32 + j] = __uint_as_float(o[j]);
      }
      s_m[tid] = m_ref;
      s_l[tid] = l_sum;
    }
    named_barrier(1, 128);
    if (ok) {
      const int qrow = threadIdx.x & 63;
      if (qrow < n_q) {
        const float ma = s_m[qrow], mb = s_m[64 + qrow];
        const float m = fmaxf(ma, mb);
        const float wa = (ma == -INFINITY) ? 0.f : fast_exp2(ma - m);
        const float wb = (mb == -INFINITY) ? 0.f : fast_exp2(mb - m);
        const float L = s_l[qrow] * wa + s_l[64 + qrow] * wb;
        const float inv = L > 0.f ? 1.f / L : 0.f;
        const float* ra = stage + qrow * 129 + half * 64;
        const float* rb = stage + (64 + qrow) * 129 + half * 64;
        char* orow = out_row0 + qrow * p.o_sm * 2 + half * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w[e] = pack2<__nv_bfloat16>((ra[c * 8 + 2 * e] * wa + rb[c * 8 + 2 * e] * wb) * inv,
                                        (ra[c * 8 + 2 * e + 1] * wa + rb[c * 8 + 2 * e + 1] * wb) * inv);
          *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (half == 0) lse_row0[qrow] = L > 0.f ? (m + log2f(L)) * kLn2 : -INFINITY;
      }
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

// Tensor maps of the tensor-core kernels: a [B,M,H,128] bf16 query-like tensor as a 4-D map
// (box = 64 columns x 64 rows of one head) and, when `kv` is given, K and V either as 4-D maps of
// the dense tensors or as 2-D maps over the page pool [num_pages*64, 128].
int make_qkv_maps(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int B, int64_t M, int H,
                  CUtensorMap* mapQ, CUtensorMap* mapK, CUtensorMap* mapV) {
  int rc;
  const uint32_t box4[4] = {64, 1, 64, 1};
  {
    const uint64_t dims[4] = {128, static_cast<uint64_t>(H), static_cast<uint64_t>(M), static_cast<uint64_t>(B)};
    const uint64_t st[3] = {static_cast<uint64_t>(q_stride[2]) * 2, static_cast<uint64_t>(q_stride[1]) * 2,
                            B > 1 ? static_cast<uint64_t>(q_stride[0]) * 2 : static_cast<uint64_t>(q_stride[1]) * 2 * M};
    if ((rc = tc::make_bf16_map(mapQ, q, 4, dims, st, box4))) return rc;
  }
  if (kv == nullptr) return NSA_OK;
  if (kv->mode == NSA_KV_DENSE) {
    const uint64_t N = static_cast<uint64_t>(kv->n_tokens);
    const uint64_t dims[4] = {128, static_cast<uint64_t>(H), N, static_cast<uint64_t>(B)};
    const uint64_t sk[3] = {static_cast<uint64_t>(kv->k_stride[2]) * 2, static_cast<uint64_t>(kv->k_stride[1]) * 2,
                            B > 1 ? static_cast<uint64_t>(kv->k_stride[0]) * 2 : static_cast<uint64_t>(kv->k_stride[1]) * 2 * N};
    const uint64_t sv[3] = {static_cast<uint64_t>(kv->v_stride[2]) * 2, static_cast<uint64_t>(kv->v_stride[1]) * 2,
                            B > 1 ? static_cast<uint64_t>(kv->v_stride[0]) * 2 : static_cast<uint64_t>(kv->v_stride[1]) * 2 * N};
    if ((rc = tc::make_bf16_map(mapK, kv->k, 4, dims, sk, box4))) return rc;
    if ((rc = tc::make_bf16_map(mapV, kv->v, 4, dims, sv, box4))) return rc;
  } else {
    const uint64_t rows = kv->num_pages > 0 ? static_cast<uint64_t>(kv->num_pages) * 64 : (1ull << 31);
    const uint64_t dims[2] = {128, rows};
    const uint64_t st[1] = {256};
    const uint32_t box[2] = {64, 64};
    if ((rc = tc::make_bf16_map(mapK, kv->k, 2, dims, st, box))) return rc;
    if ((rc = tc::make_bf16_map(mapV, kv->v, 2, dims, st, box))) return rc;
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
  if (kv->mode != NSA_KV_DENSE && kv->mode != NSA_KV_PAGED) return NSA_OK;
  if (kv->n_tokens <= 0 || M <= 0 || M > 0x7fffffff || kv->n_tokens > 0x7fffffff) return NSA_OK;
  if (encode_tiled_fn() == nullptr) return NSA_OK;
  const int64_t MG = cdiv64(M, G);

  if (H == 1) return NSA_OK;   // a size-1 head dimension may carry an arbitrary stride: leave it to the general kernel
  CUtensorMap mapQ, mapK, mapV;
  int rc;
  if ((rc = make_qkv_maps(q, q_stride, kv, B, M, H, &mapQ, &mapK, &mapV))) return rc;

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
  sel_fwd_tc_kernel<<<dim3(static_cast<unsigned>(MG), H, B), kTcThreads, smem, stream>>>(mapQ, mapK, mapV, p);
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
