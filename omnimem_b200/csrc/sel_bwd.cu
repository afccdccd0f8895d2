// Selection attention backward, general geometry (bf16 / fp16, D in {64,128}):
//   * inverted (block -> query groups) CSR index: histogram, per-(b,h) scan, scatter;
//   * dQ kernel: one thread block per (b, group, h), same packed K/V tiles as the forward;
//     computes delta = sum(O*dO) in its prologue and stores it for the dK/dV kernel;
//   * dK/dV kernel: one thread block OWNS a 64-token tile of one (b, h, block) and walks the
//     block's bucket of query groups in ascending group order - no atomics, results are
//     bit-reproducible from run to run.
#include "sel_common.cuh"

namespace nsa {
namespace {

__host__ __device__ __forceinline__ int64_t min64(int64_t a, int64_t b) { return a < b ? a : b; }
constexpr int kIdxThreads = 256;
constexpr int kSortCap = 1024;   // bucket entries sorted in shared memory

struct IdxParams {
  const int32_t* ids;
  int64_t i_sb, i_sg, i_sh, i_st;
  int B, MG, H, T;
  int64_t NS;
  int block_size, chunk_size, causal, G;
  int32_t* slots;          // optional second output (same layout as groups): the entry's position in its group's id list
};

// With a slot output the entries travel as (group << 8 | slot) through scatter and sort (T <= 256,
// MG < 2^23), so that equal groups stay ordered by slot, and are taken apart at the end.
constexpr int kSlotBits = 8;
__device__ __forceinline__ int32_t inv_entry(const IdxParams& p, int g, int t) {
  return p.slots != nullptr ? ((g << kSlotBits) | t) : g;
}

__device__ __forceinline__ bool pair_bucket(const IdxParams& p, int b, int g, int h, int t,
                                            int& bucket) {
  const int32_t bid = p.ids[b * p.i_sb + g * p.i_sg + h * p.i_sh + t * p.i_st];
  if (bid < 0 || bid >= p.NS) return false;
  if (p.causal) {
    const int64_t kc = (static_cast<int64_t>(bid) * p.block_size) / p.chunk_size;
    const int64_t qc = (static_cast<int64_t>(g) * p.G) / p.chunk_size;
    if (kc > qc) return false;
  }
  bucket = bid;
  return true;
}

template <bool SCATTER>
__global__ void inv_pass_kernel(const IdxParams p, int32_t* __restrict__ counts,
                                int32_t* __restrict__ groups) {
  const int64_t pair = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (pair >= static_cast<int64_t>(p.MG) * p.T) return;
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = static_cast<int>(pair / p.T), t = static_cast<int>(pair % p.T);
  int bucket;
  if (!pair_bucket(p, b, g, h, t, bucket)) return;
  const int64_t row = static_cast<int64_t>(b) * p.H + h;
  const int pos = atomicAdd(&counts[row * p.NS + bucket], 1);
  if (SCATTER) groups[row * p.MG * p.T + pos] = inv_entry(p, g, t);
}

// One thread block per (b, h) row: exclusive scan of the NS counts -> offsets[NS+1]; the
// counts are replaced by the offsets so the scatter pass can use them as cursors.
__global__ void inv_scan_kernel(int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                int64_t NS) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int64_t row = blockIdx.x;
  int32_t* c = counts + row * NS;
  int32_t* o = offsets + row * (NS + 1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < NS; base += blockDim.x) {
    const int64_t i = base + threadIdx.x;
    const int v = i < NS ? c[i] : 0;
    int x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = lane < nw ? warp_sums[lane] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      warp_sums[lane] = w;   // inclusive sums of the warps
    }
    __syncthreads();
    const int carry = carry_s;
    const int excl = carry + (warp ? warp_sums[warp - 1] : 0) + x - v;
    if (i < NS) { o[i] = excl; c[i] = excl; }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry_s = carry + warp_sums[nw - 1];
    __syncthreads();
  }
  if (threadIdx.x == 0) o[NS] = carry_s;
}

// One thread per bucket: insertion sort of its group ids (buckets are short; the scatter pass
// fills them in arrival order), so every consumer sees ascending groups and sums in a fixed order.
__global__ void inv_sort_kernel(const int32_t* __restrict__ offsets, int32_t* __restrict__ groups, int64_t NS,
                                int64_t groups_row, int64_t n_buckets, int32_t* __restrict__ slots) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_buckets) return;
  const int64_t row = i / NS, s = i % NS;
  const int32_t* o = offsets + row * (NS + 1);
  int32_t* gp = groups + row * groups_row + o[s];
  const int n = o[s + 1] - o[s];
  for (int a = 1; a < n; ++a) {
    const int32_t v = gp[a];
    int c = a - 1;
    while (c >= 0 && gp[c] > v) { gp[c + 1] = gp[c]; --c; }
    gp[c + 1] = v;
  }
  if (slots != nullptr) {
    int32_t* sp = slots + row * groups_row + o[s];
    for (int a = 0; a < n; ++a) {
      const int32_t v = gp[a];
      gp[a] = v >> kSlotBits;
      sp[a] = v & ((1 << kSlotBits) - 1);
    }
  }
}

// The whole index of one (b, h) row in a single thread block when its NS counters fit in shared
// memory: histogram and cursors in shared memory, scatter, then one thread per bucket sorts it.
// STAGED: the row's pairs also fit, so scatter and sort run in shared memory and the bucket
// array is written out once, coalesced.
template <bool STAGED>
__global__ void __launch_bounds__(1024) inv_fused_kernel(const IdxParams p, int32_t* __restrict__ groups,
                                                         int32_t* __restrict__ offsets) {
  extern __shared__ int s_cnt[];                   // [NS] (+ [pairs] when STAGED)
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int h = blockIdx.x % p.H, b = blockIdx.x / p.H;
  const int64_t row = blockIdx.x;
  const int NS = static_cast<int>(p.NS);
  const int pairs = p.MG * p.T;
  int32_t* o = offsets + row * (p.NS + 1);
  int32_t* gr_out = groups + row * static_cast<int64_t>(pairs);
  int32_t* gr = STAGED ? s_cnt + NS : gr_out;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < NS; i += blockDim.x) s_cnt[i] = 0;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int pr = threadIdx.x; pr < pairs; pr += blockDim.x) {
    int bucket;
    if (pair_bucket(p, b, pr / p.T, h, pr % p.T, bucket)) atomicAdd(&s_cnt[bucket], 1);
  }
  __syncthreads();
  for (int base = 0; base < NS; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int v = i < NS ? s_cnt[i] : 0;
    int x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = lane < nw ? warp_sums[lane] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    const int excl = carry + (warp ? warp_sums[warp - 1] : 0) + x - v;
    if (i < NS) { o[i] = excl; s_cnt[i] = excl; }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry_s = carry + warp_sums[nw - 1];
    __syncthreads();
  }
  if (threadIdx.x == 0) o[NS] = carry_s;
  for (int pr = threadIdx.x; pr < pairs; pr += blockDim.x) {
    int bucket;
    const int g = pr / p.T;
    if (pair_bucket(p, b, g, h, pr % p.T, bucket)) gr[atomicAdd(&s_cnt[bucket], 1)] = inv_entry(p, g, pr % p.T);
  }
  __syncthreads();                                   // scatter (global) visible to the block
  for (int sidx = threadIdx.x; sidx < NS; sidx += blockDim.x) {
    const int end = s_cnt[sidx];                     // cursor now points one past the bucket
    const int beg = o[sidx];
    for (int a = beg + 1; a < end; ++a) {
      const int32_t v = gr[a];
      int c = a - 1;
      while (c >= beg && gr[c] > v) { gr[c + 1] = gr[c]; --c; }
      gr[c + 1] = v;
    }
  }
  if (STAGED || p.slots != nullptr) {
    __syncthreads();
    const int total = carry_s;                         // pairs that landed in a bucket
    int32_t* sl_out = p.slots != nullptr ? p.slots + row * static_cast<int64_t>(pairs) : nullptr;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
      const int32_t v = gr[i];
      if (sl_out != nullptr) {
        gr_out[i] = v >> kSlotBits;
        sl_out[i] = v & ((1 << kSlotBits) - 1);
      } else {
        gr_out[i] = v;
      }
    }
  }
}

// ------------------------------------------------------------------------------------ dQ
struct BwdParams {
  const char* q; int64_t q_sb, q_sm, q_sh;
  const char* o; int64_t o_sb, o_sm, o_sh;
  const char* dO; int64_t do_sb, do_sm, do_sh;
  char* dq; int64_t dq_sb, dq_sm, dq_sh;
  char* dk; char* dv;                    // contiguous [B,N,H,D]
  const float* lse;                      // [B,H,M]
  float* delta;                          // [B,H,M]
  const int32_t* ids; int64_t i_sb, i_sg, i_sh, i_st;
  const int32_t* groups;                 // [B,H,MG*T]
  const int32_t* offsets;                // [B,H,NS+1]
  KVSrc kv;
  int B, H, T, block_size, chunk_size, causal, G, MG;
  int64_t M, NS;
  float scale, scale_log2;
  // dK/dV kernel only, pointer mode (selection_bwd.cu:1409-1527, bwd_common.cuh:64-121): K/V blocks
  // and the fp32 gradient scratch of a block are found through [H, MAXB] tables of byte addresses
  // (block-level, or chunk-level plus an in-chunk offset); a zero or out-of-range entry skips the block.
  struct Tables {
    int on;
    const int64_t *base_k, *base_v, *base_dk, *base_dv;
    int64_t base_sh, base_sb;
    int max_base;
    const int32_t* n_blocks_per_head;
    int64_t batch_kv_bytes, batch_dkv_bytes, in_chunk_kv_bytes, in_chunk_dkv_bytes;
    int blocks_per_chunk;
    int64_t s_bn, s_dbn;        // elements between tokens: K/V blocks, fp32 scratch
  } tab;
};

template <typename T, int D>
__global__ void __launch_bounds__(256) sel_bwd_dq_kernel(const BwdParams p) {
  constexpr int PITCH = D + 8;
  constexpr int ESZ = sizeof(T);
  constexpr int KK = D / 16;
  constexpr int DN = D / 8;
  extern __shared__ __align__(16) char smem[];

  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, t4 = lane & 3;
  const int rows_pad = (blockDim.x >> 5) * 16;
  const int64_t m0 = static_cast<int64_t>(g) * p.G;
  const int n_q = static_cast<int>(p.M - m0 < p.G ? p.M - m0 : p.G);
  const int q_chunk = static_cast<int>(m0 / p.chunk_size);

  T* tiles = reinterpret_cast<T*>(smem);                         // [2][2][64][PITCH]
  T* sQ = tiles + 4 * kTileRows * PITCH;                          // [rows_pad][PITCH]
  T* sdO = sQ + rows_pad * PITCH;
  float* s_lse = reinterpret_cast<float*>(sdO + rows_pad * PITCH);
  float* s_delta = s_lse + rows_pad;
  const SlotTable st = carve_slot_table(reinterpret_cast<char*>(s_delta + rows_pad), p.T);
  auto stageK = [&](int s) { return tiles + (s * 2) * kTileRows * PITCH; };
  auto stageV = [&](int s) { return tiles + (s * 2 + 1) * kTileRows * PITCH; };

  const int total = build_slot_table<ESZ>(st, p.kv, p.ids, b * p.i_sb + g * p.i_sg + h * p.i_sh, p.i_st,
                                          p.T, b, h, D, p.block_size, p.chunk_size, p.causal != 0, q_chunk);

  const char* q_base = p.q + (b * p.q_sb + m0 * p.q_sm + h * p.q_sh) * ESZ;
  const char* o_base = p.o + (b * p.o_sb + m0 * p.o_sm + h * p.o_sh) * ESZ;
  const char* do_base = p.dO + (b * p.do_sb + m0 * p.do_sm + h * p.do_sh) * ESZ;
  char* dq_base = p.dq + (b * p.dq_sb + m0 * p.dq_sm + h * p.dq_sh) * ESZ;
  const int64_t bhm = (static_cast<int64_t>(b) * p.H + h) * p.M + m0;

  // delta = sum_d O * dO (one warp per row), kept in shared memory and stored for dK/dV
  for (int r = warp; r < rows_pad; r += (blockDim.x >> 5)) {
    float acc = 0.f;
    if (r < n_q) {
      const T* orow = reinterpret_cast<const T*>(o_base + r * p.o_sm * ESZ);
      const T* drow = reinterpret_cast<const T*>(do_base + r * p.do_sm * ESZ);
      for (int d = lane * 2; d < D; d += 64) {
        const float2 a = unpack2<T>(*reinterpret_cast<const uint32_t*>(orow + d));
        const float2 c = unpack2<T>(*reinterpret_cast<const uint32_t*>(drow + d));
        acc += a.x * c.x + a.y * c.y;
      }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) {
      s_delta[r] = acc;
      s_lse[r] = r < n_q ? p.lse[bhm + r] * kLog2e : INFINITY;
      if (r < n_q) p.delta[bhm + r] = acc;
    }
  }

  if (total == 0) {
    for (int i = threadIdx.x; i < n_q * (D / 8); i += blockDim.x) {
      const int r = i / (D / 8), c = i % (D / 8);
      *reinterpret_cast<uint4*>(dq_base + r * p.dq_sm * ESZ + c * 16) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  const int64_t k_row_bytes = kv_row_bytes(p.kv, false, D, ESZ);
  const int64_t v_row_bytes = kv_row_bytes(p.kv, true, D, ESZ);
  const int ntiles = (total + kTileRows - 1) / kTileRows;

  issue_rows<T, D, PITCH>(sQ, q_base, p.q_sm * ESZ, n_q, rows_pad);
  issue_rows<T, D, PITCH>(sdO, do_base, p.do_sm * ESZ, n_q, rows_pad);
  issue_kv_tile<T, D, PITCH>(stageK(0), stageV(0), st, p.T, 0, total, k_row_bytes, v_row_bytes, p.q);
  cp_async_commit();

  float dq[DN][4];
#pragma unroll
  for (int n = 0; n < DN; ++n) { dq[n][0] = dq[n][1] = dq[n][2] = dq[n][3] = 0.f; }
  const bool warp_active = warp * 16 < n_q;
  const T* qa = sQ + (warp * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8;
  const T* da = sdO + (warp * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8;

  for (int i = 0; i < ntiles; ++i) {
    if (i + 1 < ntiles) {
      issue_kv_tile<T, D, PITCH>(stageK((i + 1) & 1), stageV((i + 1) & 1), st, p.T,
                                 (i + 1) * kTileRows, total, k_row_bytes, v_row_bytes, p.q);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (warp_active) {
      const T* sK = stageK(i & 1);
      const T* sV = stageV(i & 1);
      const int nvalid = min(kTileRows, total - i * kTileRows);
      const int nb_off = ((lane & 7) + ((lane >> 4) << 3)) * PITCH + ((lane >> 3) & 1) * 8;
      float s[8][4], dp[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f;
      }
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        uint32_t aq[4], ad[4];
        ldmatrix_x4(aq, qa + kk * 16);
        ldmatrix_x4(ad, da + kk * 16);
#pragma unroll
        for (int n16 = 0; n16 < 4; ++n16) {
          if (n16 * 16 < nvalid) {
            uint32_t bf[4];
            ldmatrix_x4(bf, sK + nb_off + n16 * 16 * PITCH + kk * 16);
            mma16816<T>(s[2 * n16], aq, bf[0], bf[1]);
            mma16816<T>(s[2 * n16 + 1], aq, bf[2], bf[3]);
            ldmatrix_x4(bf, sV + nb_off + n16 * 16 * PITCH + kk * 16);
            mma16816<T>(dp[2 * n16], ad, bf[0], bf[1]);
            mma16816<T>(dp[2 * n16 + 1], ad, bf[2], bf[3]);
          }
        }
      }
      const float lse0 = s_lse[warp * 16 + gid], lse1 = s_lse[warp * 16 + gid + 8];
      const float dl0 = s_delta[warp * 16 + gid], dl1 = s_delta[warp * 16 + gid + 8];
      uint32_t dsa[4][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        float ds[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = n * 8 + 2 * t4 + (e & 1);
          const float l = (e >> 1) ? lse1 : lse0;
          const float dl = (e >> 1) ? dl1 : dl0;
          const float pe = (col < nvalid) ? fast_exp2(s[n][e] * p.scale_log2 - l) : 0.f;
          ds[e] = pe * (dp[n][e] - dl) * p.scale;
        }
        dsa[n >> 1][(n & 1) * 2] = pack2<T>(ds[0], ds[1]);
        dsa[n >> 1][(n & 1) * 2 + 1] = pack2<T>(ds[2], ds[3]);
      }
      const T* kb = sK + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (lane >> 4) * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j * 16 < nvalid) {
#pragma unroll
          for (int d16 = 0; d16 < D / 16; ++d16) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, kb + j * 16 * PITCH + d16 * 16);
            mma16816<T>(dq[2 * d16], dsa[j], bf[0], bf[1]);
            mma16816<T>(dq[2 * d16 + 1], dsa[j], bf[2], bf[3]);
          }
        }
      }
    }
    __syncthreads();
  }

  if (warp_active) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = warp * 16 + gid + 8 * r;
      if (row < n_q) {
        char* drow = dq_base + row * p.dq_sm * ESZ;
#pragma unroll
        for (int n = 0; n < DN; ++n)
          *reinterpret_cast<uint32_t*>(drow + (n * 8 + 2 * t4) * ESZ) =
              pack2<T>(dq[n][2 * r], dq[n][2 * r + 1]);
      }
    }
  }
}

// --------------------------------------------------------------------------------- dK / dV
template <typename T, int D>
__global__ void __launch_bounds__(128) sel_bwd_dkv_kernel(const BwdParams p, int tiles_per_block) {
  constexpr int PITCH = D + 8;
  constexpr int ESZ = sizeof(T);
  constexpr int KK = D / 16;
  constexpr int DN = D / 8;
  constexpr int QT = 64;
  extern __shared__ __align__(16) char smem[];

  const int blk = blockIdx.x / tiles_per_block, kt = blockIdx.x % tiles_per_block;
  const int h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, t4 = lane & 3;

  T* sK = reinterpret_cast<T*>(smem);            // [64][PITCH]
  T* sV = sK + kTileRows * PITCH;
  T* sQd = sV + kTileRows * PITCH;               // [2][2][QT][PITCH]  (stage, Q|dO)
  float* s_lse = reinterpret_cast<float*>(sQd + 4 * QT * PITCH);   // [2][QT]
  float* s_delta = s_lse + 2 * QT;                                  // [2][QT]
  int* s_grp = reinterpret_cast<int*>(s_delta + 2 * QT);            // [kSortCap]
  int* s_tmp = s_grp + kSortCap;                                    // [kSortCap]
  auto stageQ = [&](int s) { return sQd + (s * 2) * QT * PITCH; };
  auto stageD = [&](int s) { return sQd + (s * 2 + 1) * QT * PITCH; };

  const int64_t t0 = static_cast<int64_t>(blk) * p.block_size;
  const int n_blk = p.tab.on ? p.block_size : static_cast<int>(min64(p.block_size, p.kv.n_tokens - t0));  // tokens that exist
  const int row_lo = kt * kTileRows;                        // first block row of this tile
  const int n_rows = max(0, min(kTileRows, n_blk - row_lo)); // rows this tile owns
  if (n_rows == 0) return;
  const int64_t tok0 = t0 + row_lo;
  char* dk_base = p.dk + ((static_cast<int64_t>(b) * p.kv.n_tokens + tok0) * p.H + h) * D * ESZ;
  char* dv_base = p.dv + ((static_cast<int64_t>(b) * p.kv.n_tokens + tok0) * p.H + h) * D * ESZ;
  const int64_t out_row_bytes = static_cast<int64_t>(p.H) * D * ESZ;

  const int64_t row = static_cast<int64_t>(b) * p.H + h;
  const int32_t* offs = p.offsets + row * (p.NS + 1);
  const int beg = offs[blk], n_ent = offs[blk + 1] - beg;
  const int32_t* bucket = p.groups + row * static_cast<int64_t>(p.MG) * p.T + beg;

  BlockRef br{nullptr, nullptr, 0};
  float* fdk = nullptr;
  float* fdv = nullptr;
  if (p.tab.on) {
    const auto& tb = p.tab;
    if (tb.n_blocks_per_head == nullptr || blk < tb.n_blocks_per_head[h]) {
      int64_t idx = blk, off_kv = 0, off_dkv = 0;
      if (tb.blocks_per_chunk > 0) {
        idx = blk / tb.blocks_per_chunk;
        const int64_t in_chunk = blk - idx * tb.blocks_per_chunk;
        off_kv = in_chunk * tb.in_chunk_kv_bytes;
        off_dkv = in_chunk * tb.in_chunk_dkv_bytes;
      }
      if (idx < tb.max_base) {
        const int64_t o = static_cast<int64_t>(h) * tb.base_sh + idx * tb.base_sb;
        const int64_t bk = tb.base_k[o], bv = tb.base_v[o], bdk = tb.base_dk[o], bdv = tb.base_dv[o];
        if (bk != 0 && bv != 0 && bdk != 0 && bdv != 0) {     // all four or nothing
          const int64_t okv = static_cast<int64_t>(b) * tb.batch_kv_bytes + off_kv;
          const int64_t odkv = static_cast<int64_t>(b) * tb.batch_dkv_bytes + off_dkv;
          br.k = reinterpret_cast<const char*>(static_cast<uintptr_t>(bk + okv));
          br.v = reinterpret_cast<const char*>(static_cast<uintptr_t>(bv + okv));
          br.n_vis = p.block_size;
          fdk = reinterpret_cast<float*>(static_cast<uintptr_t>(bdk + odkv)) + static_cast<int64_t>(row_lo) * tb.s_dbn;
          fdv = reinterpret_cast<float*>(static_cast<uintptr_t>(bdv + odkv)) + static_cast<int64_t>(row_lo) * tb.s_dbn;
        }
      }
    }
    if (n_ent == 0 || br.k == nullptr) return;      // the scratch of an untouched block is left as it is
  } else {
    br = resolve_block<ESZ>(p.kv, b, h, blk, D, p.block_size, 1, false, 0);
  }
  if (n_ent == 0 || br.k == nullptr) {
    for (int i = threadIdx.x; i < n_rows * (D / 8); i += blockDim.x) {
      const int r = i / (D / 8), c = i % (D / 8);
      *reinterpret_cast<uint4*>(dk_base + r * out_row_bytes + c * 16) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(dv_base + r * out_row_bytes + c * 16) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  // bucket -> ascending group order (rank sort; duplicates keep their arrival order)
  const bool sorted = n_ent <= kSortCap;
  if (sorted) {
    for (int i = threadIdx.x; i < n_ent; i += blockDim.x) s_tmp[i] = bucket[i];
    __syncthreads();
    for (int i = threadIdx.x; i < n_ent; i += blockDim.x) {
      const int v = s_tmp[i];
      int rank = 0;
      for (int j = 0; j < n_ent; ++j) {
        const int w = s_tmp[j];
        rank += (w < v) || (w == v && j < i);
      }
      s_grp[rank] = v;
    }
    __syncthreads();
  }
  auto entry = [&](int i) { return sorted ? s_grp[i] : bucket[i]; };

  const int spg = (p.G + QT - 1) / QT;      // query sub-tiles per group
  const int n_items = n_ent * spg;
  const int64_t k_row_bytes = p.tab.on ? p.tab.s_bn * ESZ : kv_row_bytes(p.kv, false, D, ESZ);
  const int64_t v_row_bytes = p.tab.on ? p.tab.s_bn * ESZ : kv_row_bytes(p.kv, true, D, ESZ);

  auto issue_item = [&](int it, int stg) {
    const int g = entry(it / spg), sub = it % spg;
    const int64_t m0 = static_cast<int64_t>(g) * p.G + sub * QT;
    int nq = static_cast<int>(min64(p.G, p.M - static_cast<int64_t>(g) * p.G)) - sub * QT;
    nq = max(0, min(QT, nq));
    issue_rows<T, D, PITCH>(stageQ(stg), p.q + (b * p.q_sb + m0 * p.q_sm + h * p.q_sh) * ESZ,
                            p.q_sm * ESZ, nq, QT);
    issue_rows<T, D, PITCH>(stageD(stg), p.dO + (b * p.do_sb + m0 * p.do_sm + h * p.do_sh) * ESZ,
                            p.do_sm * ESZ, nq, QT);
    if (threadIdx.x < QT) {
      const int r = threadIdx.x;
      const int64_t at = (static_cast<int64_t>(b) * p.H + h) * p.M + m0 + r;
      s_lse[stg * QT + r] = r < nq ? p.lse[at] * kLog2e : INFINITY;
      s_delta[stg * QT + r] = r < nq ? p.delta[at] : 0.f;
    }
  };

  issue_rows<T, D, PITCH>(sK, br.k + row_lo * k_row_bytes, k_row_bytes, n_rows, kTileRows);
  issue_rows<T, D, PITCH>(sV, br.v + row_lo * v_row_bytes, v_row_bytes, n_rows, kTileRows);
  issue_item(0, 0);
  cp_async_commit();

  float dk[DN][4], dv[DN][4];
#pragma unroll
  for (int n = 0; n < DN; ++n) {
    dk[n][0] = dk[n][1] = dk[n][2] = dk[n][3] = 0.f;
    dv[n][0] = dv[n][1] = dv[n][2] = dv[n][3] = 0.f;
  }
  const T* ka = sK + (warp * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8;
  const T* va = sV + (warp * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8;
  const int nb_off = ((lane & 7) + ((lane >> 4) << 3)) * PITCH + ((lane >> 3) & 1) * 8;
  const int tb_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (lane >> 4) * 8;
  const bool warp_active = warp * 16 < n_rows;

  for (int it = 0; it < n_items; ++it) {
    if (it + 1 < n_items) {
      issue_item(it + 1, (it + 1) & 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int g = entry(it / spg), sub = it % spg;
    int nq = static_cast<int>(min64(p.G, p.M - static_cast<int64_t>(g) * p.G)) - sub * QT;
    nq = max(0, min(QT, nq));
    // rows of this tile the group may see (causal: prefix of the block)
    int vis = n_blk;
    if (p.causal) {
      const int64_t qc = (static_cast<int64_t>(g) * p.G) / p.chunk_size;
      vis = static_cast<int>(min64(vis, (qc + 1) * p.chunk_size - t0));
    }
    const int nkv = max(0, min(kTileRows, vis - row_lo));
    if (warp_active && nq > 0 && warp * 16 < nkv) {
      const T* sQ = stageQ(it & 1);
      const T* sD = stageD(it & 1);
      const float* lse2 = s_lse + (it & 1) * QT;
      const float* dlt = s_delta + (it & 1) * QT;
      float st[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) { st[n][0] = st[n][1] = st[n][2] = st[n][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, ka + kk * 16);
#pragma unroll
        for (int n16 = 0; n16 < 4; ++n16) {
          if (n16 * 16 < nq) {
            uint32_t bf[4];
            ldmatrix_x4(bf, sQ + nb_off + n16 * 16 * PITCH + kk * 16);
            mma16816<T>(st[2 * n16], a, bf[0], bf[1]);
            mma16816<T>(st[2 * n16 + 1], a, bf[2], bf[3]);
          }
        }
      }
      uint32_t pa[4][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        float pe[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int krow = warp * 16 + gid + 8 * (e >> 1);
          const int col = n * 8 + 2 * t4 + (e & 1);
          pe[e] = (krow < nkv && col < nq) ? fast_exp2(st[n][e] * p.scale_log2 - lse2[col]) : 0.f;
        }
        pa[n >> 1][(n & 1) * 2] = pack2<T>(pe[0], pe[1]);
        pa[n >> 1][(n & 1) * 2 + 1] = pack2<T>(pe[2], pe[3]);
      }
      // dV += P^T dO
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j * 16 < nq) {
#pragma unroll
          for (int d16 = 0; d16 < D / 16; ++d16) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, sD + tb_off + j * 16 * PITCH + d16 * 16);
            mma16816<T>(dv[2 * d16], pa[j], bf[0], bf[1]);
            mma16816<T>(dv[2 * d16 + 1], pa[j], bf[2], bf[3]);
          }
        }
      }
      // dP^T = V dO^T
#pragma unroll
      for (int n = 0; n < 8; ++n) { st[n][0] = st[n][1] = st[n][2] = st[n][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, va + kk * 16);
#pragma unroll
        for (int n16 = 0; n16 < 4; ++n16) {
          if (n16 * 16 < nq) {
            uint32_t bf[4];
            ldmatrix_x4(bf, sD + nb_off + n16 * 16 * PITCH + kk * 16);
            mma16816<T>(st[2 * n16], a, bf[0], bf[1]);
            mma16816<T>(st[2 * n16 + 1], a, bf[2], bf[3]);
          }
        }
      }
      // dS^T = P^T (dP^T - delta) scale, packed back into the same A fragments
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int col = n * 8 + 2 * t4;
        const float d0 = dlt[col], d1 = dlt[col + 1];
        const float2 p01 = unpack2<T>(pa[n >> 1][(n & 1) * 2]);
        const float2 p23 = unpack2<T>(pa[n >> 1][(n & 1) * 2 + 1]);
        pa[n >> 1][(n & 1) * 2] =
            pack2<T>(p01.x * (st[n][0] - d0) * p.scale, p01.y * (st[n][1] - d1) * p.scale);
        pa[n >> 1][(n & 1) * 2 + 1] =
            pack2<T>(p23.x * (st[n][2] - d0) * p.scale, p23.y * (st[n][3] - d1) * p.scale);
      }
      // dK += dS^T Q
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j * 16 < nq) {
#pragma unroll
          for (int d16 = 0; d16 < D / 16; ++d16) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, sQ + tb_off + j * 16 * PITCH + d16 * 16);
            mma16816<T>(dk[2 * d16], pa[j], bf[0], bf[1]);
            mma16816<T>(dk[2 * d16 + 1], pa[j], bf[2], bf[3]);
          }
        }
      }
    }
    __syncthreads();
  }

  if (warp_active) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int krow = warp * 16 + gid + 8 * r;
      if (krow < n_rows && p.tab.on) {
        float* kr = fdk + static_cast<int64_t>(krow) * p.tab.s_dbn;
        float* vr = fdv + static_cast<int64_t>(krow) * p.tab.s_dbn;
#pragma unroll
        for (int n = 0; n < DN; ++n) {
          *reinterpret_cast<float2*>(kr + n * 8 + 2 * t4) = make_float2(dk[n][2 * r], dk[n][2 * r + 1]);
          *reinterpret_cast<float2*>(vr + n * 8 + 2 * t4) = make_float2(dv[n][2 * r], dv[n][2 * r + 1]);
        }
      } else if (krow < n_rows) {
        char* kr = dk_base + krow * out_row_bytes;
        char* vr = dv_base + krow * out_row_bytes;
#pragma unroll
        for (int n = 0; n < DN; ++n) {
          *reinterpret_cast<uint32_t*>(kr + (n * 8 + 2 * t4) * ESZ) = pack2<T>(dk[n][2 * r], dk[n][2 * r + 1]);
          *reinterpret_cast<uint32_t*>(vr + (n * 8 + 2 * t4) * ESZ) = pack2<T>(dv[n][2 * r], dv[n][2 * r + 1]);
        }
      }
    }
  }
}

size_t dq_smem(int rows_pad, int D, int T) {
  return static_cast<size_t>(4 * kTileRows + 2 * rows_pad) * (D + 8) * 2 + 2 * rows_pad * 4 +
         slot_table_bytes(T);
}
size_t dkv_smem(int D) {
  return static_cast<size_t>(2 * kTileRows + 4 * 64) * (D + 8) * 2 + 4 * 64 * 4 + 2 * kSortCap * 4;
}

template <typename T, int D>
int launch_dq(const BwdParams& p, cudaStream_t stream) {
  const int nw = cdiv(p.G, 16);
  const size_t smem_q = dq_smem(nw * 16, D, p.T);
  NSA_REQUIRE(smem_q <= 220 * 1024, NSA_ERR_UNSUPPORTED, "sel_bwd: T=%d needs too much shared memory", p.T);
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_bwd_dq_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(smem_q)));
  sel_bwd_dq_kernel<T, D><<<dim3(p.MG, p.H, p.B), nw * 32, smem_q, stream>>>(p);
  NSA_LAUNCH_OK("sel_bwd_dq_kernel");
  return NSA_OK;
}

template <typename T, int D>
int launch_dkv(const BwdParams& p, cudaStream_t stream) {
  const size_t smem_kv = dkv_smem(D);
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_bwd_dkv_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(smem_kv)));
  const int tpb = cdiv(p.block_size, kTileRows);
  const int64_t nblk = p.NS * tpb;
  NSA_REQUIRE(nblk <= 0x7fffffff, NSA_ERR_INVALID, "sel_bwd: too many K/V tiles");
  if (nblk > 0) {
    sel_bwd_dkv_kernel<T, D><<<dim3(static_cast<unsigned>(nblk), p.H, p.B), 128, smem_kv, stream>>>(p, tpb);
    NSA_LAUNCH_OK("sel_bwd_dkv_kernel");
  }
  return NSA_OK;
}

template <bool DQ>
int dispatch_bwd(const BwdParams& p, int dtype, int D, cudaStream_t s) {
  if (dtype == NSA_BF16) {
    if (D == 128) return DQ ? launch_dq<__nv_bfloat16, 128>(p, s) : launch_dkv<__nv_bfloat16, 128>(p, s);
    return DQ ? launch_dq<__nv_bfloat16, 64>(p, s) : launch_dkv<__nv_bfloat16, 64>(p, s);
  }
  if (D == 128) return DQ ? launch_dq<__half, 128>(p, s) : launch_dkv<__half, 128>(p, s);
  return DQ ? launch_dq<__half, 64>(p, s) : launch_dkv<__half, 64>(p, s);
}

int run_inverted_index(const IdxParams& ip, int32_t* groups, int32_t* offsets, int32_t* counts,
                       cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(ip.B) * ip.H;
  if (rows == 0) return NSA_OK;
  if (ip.NS == 0) {
    NSA_CUDA_OK(cudaMemsetAsync(offsets, 0, rows * sizeof(int32_t), stream));
    return NSA_OK;
  }
  const int64_t pairs = static_cast<int64_t>(ip.MG) * ip.T;
  if (ip.NS * 4 <= 160 * 1024 && pairs <= 0x7fffffff && rows <= 0x7fffffff) {
    const size_t smem_idx = static_cast<size_t>(ip.NS) * 4, smem_all = smem_idx + static_cast<size_t>(pairs) * 4;
    if (smem_all <= 200 * 1024) {
      NSA_CUDA_OK(cudaFuncSetAttribute(inv_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_all)));
      inv_fused_kernel<true><<<static_cast<unsigned>(rows), 1024, smem_all, stream>>>(ip, groups, offsets);
    } else {
      NSA_CUDA_OK(cudaFuncSetAttribute(inv_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_idx)));
      inv_fused_kernel<false><<<static_cast<unsigned>(rows), 1024, smem_idx, stream>>>(ip, groups, offsets);
    }
    NSA_LAUNCH_OK("inv_fused_kernel");
    return NSA_OK;
  }
  NSA_CUDA_OK(cudaMemsetAsync(counts, 0, rows * ip.NS * sizeof(int32_t), stream));
  const dim3 grid(static_cast<unsigned>(cdiv64(pairs, kIdxThreads)), ip.H, ip.B);
  if (pairs > 0) {
    inv_pass_kernel<false><<<grid, kIdxThreads, 0, stream>>>(ip, counts, groups);
    NSA_LAUNCH_OK("inv_pass_kernel<count>");
  }
  inv_scan_kernel<<<static_cast<unsigned>(rows), 1024, 0, stream>>>(counts, offsets, ip.NS);
  NSA_LAUNCH_OK("inv_scan_kernel");
  if (pairs > 0) {
    inv_pass_kernel<true><<<grid, kIdxThreads, 0, stream>>>(ip, counts, groups);
    NSA_LAUNCH_OK("inv_pass_kernel<scatter>");
    const int64_t n_buckets = rows * ip.NS;
    inv_sort_kernel<<<static_cast<unsigned>(cdiv64(n_buckets, 128)), 128, 0, stream>>>(offsets, groups, ip.NS, pairs,
                                                                                       n_buckets, ip.slots);
    NSA_LAUNCH_OK("inv_sort_kernel");
  }
  return NSA_OK;
}

}  // namespace

int check_strides16(const char* what, const void* ptr, const int64_t* stride, int n, int esz);
int try_launch_sel_bwd_dq_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* ids,
                             const int64_t* idx_stride, const void* out, const int64_t* out_stride, const float* lse,
                             const void* d_out, const int64_t* do_stride, void* dq, const int64_t* dq_stride,
                             float* delta, int B, int64_t M, int H, int D, int T, int block_size, int chunk_size,
                             int causal, int G, float scale, int dtype, cudaStream_t stream, bool* launched,
                             void* pds);
int try_launch_sel_bwd_dkv_pds_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* groups,
                                  const int32_t* slots, const int32_t* offsets, const void* pds, const void* d_out,
                                  const int64_t* do_stride, void* dk, void* dv, int B, int64_t M, int H, int D, int T,
                                  int block_size, int G, int dtype, int32_t* counter, cudaStream_t stream,
                                  bool* launched);
int try_launch_sel_bwd_dkv_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* groups,
                              const int32_t* offsets, const float* lse, const float* delta, const void* d_out,
                              const int64_t* do_stride, void* dk, void* dv, int B, int64_t M, int H, int D, int T,
                              int block_size, int chunk_size, int causal, int G, float scale, int dtype,
                              int32_t* counter, cudaStream_t stream, bool* launched);

}  // namespace nsa

using namespace nsa;

extern "C" size_t nsa_inverted_index_workspace_bytes(int32_t B, int32_t H, int64_t NS) {
  return align_up(static_cast<size_t>(B) * H * NS * sizeof(int32_t), 256);
}

extern "C" int nsa_inverted_index_slots(const int32_t* block_indices, const int64_t idx_stride[4],
                                        int32_t B, int32_t MG, int32_t H, int32_t T, int64_t NS,
                                        int32_t block_size, int32_t chunk_size, int32_t causal,
                                        int32_t group_size, int32_t* groups, int32_t* offsets, int32_t* slots,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  NSA_REQUIRE(B >= 0 && MG >= 0 && H >= 0 && T >= 0 && NS >= 0, NSA_ERR_INVALID, "inverted_index: negative size");
  NSA_REQUIRE(block_size > 0 && chunk_size > 0 && group_size > 0, NSA_ERR_INVALID, "inverted_index: sizes must be > 0");
  NSA_REQUIRE(H <= 65535 && B <= 65535, NSA_ERR_INVALID, "inverted_index: B and H must be <= 65535");
  NSA_REQUIRE(workspace_bytes >= nsa_inverted_index_workspace_bytes(B, H, NS), NSA_ERR_WORKSPACE,
              "inverted_index: workspace too small");
  if (B == 0 || H == 0) return NSA_OK;
  NSA_REQUIRE(block_indices && groups && offsets && (workspace || NS == 0), NSA_ERR_INVALID, "inverted_index: null pointer");
  NSA_REQUIRE(slots == nullptr || (T <= (1 << kSlotBits) && MG < (1 << (31 - kSlotBits))), NSA_ERR_UNSUPPORTED,
              "inverted_index: the slot output serves T <= %d and fewer than %d query groups", 1 << kSlotBits, 1 << (31 - kSlotBits));
  IdxParams ip{block_indices, idx_stride[0], idx_stride[1], idx_stride[2], idx_stride[3],
               B, MG, H, T, NS, block_size, chunk_size, causal, group_size, slots};
  return run_inverted_index(ip, groups, offsets, static_cast<int32_t*>(workspace),
                            static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_inverted_index(const int32_t* block_indices, const int64_t idx_stride[4],
                                  int32_t B, int32_t MG, int32_t H, int32_t T, int64_t NS,
                                  int32_t block_size, int32_t chunk_size, int32_t causal,
                                  int32_t group_size, int32_t* groups, int32_t* offsets,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  return nsa_inverted_index_slots(block_indices, idx_stride, B, MG, H, T, NS, block_size, chunk_size, causal, group_size,
                                  groups, offsets, nullptr, workspace, workspace_bytes, stream);
}

// workspace layout: delta f32 [B,H,M] | counts i32 [B,H,NS] | offsets i32 [B,H,NS+1] | groups i32 [B,H,MG*T]
static void bwd_ws_layout(int32_t B, int64_t M, int32_t H, int64_t NS, int64_t MG, int32_t T,
                          size_t off[5]) {
  off[0] = 0;
  off[1] = off[0] + align_up(static_cast<size_t>(B) * H * M * 4, 256);
  off[2] = off[1] + align_up(static_cast<size_t>(B) * H * NS * 4, 256);
  off[3] = off[2] + align_up(static_cast<size_t>(B) * H * (NS + 1) * 4, 256);
  off[4] = off[3] + align_up(static_cast<size_t>(B) * H * MG * T * 4, 256);
  off[5] = off[4] + 256;   // scheduling counter of the dK/dV kernel
}

extern "C" size_t nsa_sel_bwd_workspace_bytes(int32_t B, int64_t M, int32_t H, int64_t N, int32_t T,
                                              int32_t block_size, int32_t group_size) {
  if (block_size <= 0 || group_size <= 0) return 0;
  size_t off[6];
  bwd_ws_layout(B, M, H, cdiv64(N, block_size), cdiv64(M, group_size), T, off);
  return off[5];
}

static int bwd_common_checks(const char* op, int32_t B, int64_t M, int32_t H, int32_t D, int32_t T,
                             int32_t block_size, int32_t chunk_size, int32_t group_size, int32_t dtype,
                             const nsa_kv_source* kv, bool allow_ptr = false) {
  NSA_REQUIRE(B >= 0 && M >= 0 && H >= 0, NSA_ERR_INVALID, "%s: negative size", op);
  NSA_REQUIRE(group_size >= 1 && group_size <= 128, NSA_ERR_INVALID,
              "%s: group_size must be in [1,128], got %d", op, group_size);
  NSA_REQUIRE(block_size > 0 && chunk_size > 0 && T > 0, NSA_ERR_INVALID, "%s: block_size, chunk_size, T must be > 0", op);
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_F16, NSA_ERR_UNSUPPORTED,
              "%s: only bf16 and fp16 are built (dtype %d)", op, dtype);
  NSA_REQUIRE(D == 64 || D == 128, NSA_ERR_UNSUPPORTED, "%s: head dim %d not built (64, 128)", op, D);
  NSA_REQUIRE(kv != nullptr, NSA_ERR_INVALID, "%s: kv source is null", op);
  NSA_REQUIRE(B <= 65535 && H <= 65535, NSA_ERR_INVALID, "%s: B and H must be <= 65535", op);
  NSA_REQUIRE(kv->mode != NSA_KV_PTR || allow_ptr, NSA_ERR_UNSUPPORTED,
              "%s: per-slot pointer tables serve the forward and dQ; dK/dV takes block base tables (nsa_sel_bwd_dkv_ptr)", op);
  NSA_REQUIRE(kv->mode != NSA_KV_PAGED || B == 1, NSA_ERR_INVALID, "%s: paged K/V needs B == 1", op);
  NSA_REQUIRE(cdiv64(M, group_size) <= 0x7fffffff && cdiv64(kv->n_tokens, block_size) <= 0x7fffffff, NSA_ERR_INVALID,
              "%s: too many groups / blocks", op);
  return NSA_OK;
}

extern "C" size_t nsa_sel_bwd_pds_bytes(int32_t B, int64_t M, int32_t H, int32_t T, int32_t group_size) {
  if (group_size <= 0 || B <= 0 || H <= 0 || T <= 0 || M <= 0) return 0;
  return static_cast<size_t>(B) * cdiv64(M, group_size) * H * T * 16384;
}

extern "C" int nsa_sel_bwd_dq(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                              const int32_t* block_indices, const int64_t idx_stride[4],
                              const void* out, const int64_t out_stride[3], const float* lse,
                              const void* d_out, const int64_t do_stride[3], void* dq,
                              const int64_t dq_stride[3], float* delta, int32_t B, int64_t M, int32_t H,
                              int32_t D, int32_t T, int32_t block_size, int32_t chunk_size,
                              int32_t causal, int32_t group_size, float scale, int32_t dtype,
                              void* stream) {
  return nsa_sel_bwd_dq_pds(q, q_stride, kv, block_indices, idx_stride, out, out_stride, lse, d_out, do_stride, dq,
                            dq_stride, delta, B, M, H, D, T, block_size, chunk_size, causal, group_size, scale,
                            nullptr, 0, nullptr, dtype, stream);
}

extern "C" int nsa_sel_bwd_dq_pds(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                                  const int32_t* block_indices, const int64_t idx_stride[4],
                                  const void* out, const int64_t out_stride[3], const float* lse,
                                  const void* d_out, const int64_t do_stride[3], void* dq,
                                  const int64_t dq_stride[3], float* delta, int32_t B, int64_t M, int32_t H,
                                  int32_t D, int32_t T, int32_t block_size, int32_t chunk_size,
                                  int32_t causal, int32_t group_size, float scale, void* pds, size_t pds_bytes,
                                  int32_t* pds_written, int32_t dtype, void* stream) {
  if (pds_written != nullptr) *pds_written = 0;
  int rc;
  if ((rc = bwd_common_checks("sel_bwd_dq", B, M, H, D, T, block_size, chunk_size, group_size, dtype, kv, true))) return rc;
  if (B == 0 || H == 0 || M == 0) return NSA_OK;
  NSA_REQUIRE((block_indices || kv->mode == NSA_KV_PTR) && lse && delta, NSA_ERR_INVALID, "sel_bwd_dq: null pointer");
  const int esz = 2;
  if ((rc = check_strides16("q", q, q_stride, 3, esz))) return rc;
  if ((rc = check_strides16("out", out, out_stride, 3, esz))) return rc;
  if ((rc = check_strides16("d_out", d_out, do_stride, 3, esz))) return rc;
  if ((rc = check_strides16("dq", dq, dq_stride, 3, esz))) return rc;
  BwdParams p{};
  if ((rc = make_kvsrc(kv, D, esz, block_size, &p.kv))) return rc;
  {
    // the page geometry runs on the tcgen05 kernel; every other shape on the general one
    bool launched = false;
    // the P / dS tiles are written only when the caller wants to know that they were (pds_written),
    // the buffer holds every (group, head, slot) pair and the lists are short enough for the storing kernel (64 slots)
    void* tiles = (pds != nullptr && pds_written != nullptr && T <= 64 &&
                   pds_bytes >= nsa_sel_bwd_pds_bytes(B, M, H, T, group_size) && aligned16(pds)) ? pds : nullptr;
    rc = try_launch_sel_bwd_dq_tc(q, q_stride, kv, block_indices, idx_stride, out, out_stride, lse, d_out, do_stride,
                                  dq, dq_stride, delta, B, M, H, D, T, block_size, chunk_size, causal, group_size,
                                  scale, dtype, static_cast<cudaStream_t>(stream), &launched, tiles);
    if (rc) return rc;
    if (launched) {
      if (tiles != nullptr) *pds_written = 1;
      return NSA_OK;
    }
  }
  p.q = static_cast<const char*>(q); p.q_sb = q_stride[0]; p.q_sm = q_stride[1]; p.q_sh = q_stride[2];
  p.o = static_cast<const char*>(out); p.o_sb = out_stride[0]; p.o_sm = out_stride[1]; p.o_sh = out_stride[2];
  p.dO = static_cast<const char*>(d_out); p.do_sb = do_stride[0]; p.do_sm = do_stride[1]; p.do_sh = do_stride[2];
  p.dq = static_cast<char*>(dq); p.dq_sb = dq_stride[0]; p.dq_sm = dq_stride[1]; p.dq_sh = dq_stride[2];
  p.lse = lse; p.delta = delta;
  p.ids = block_indices; p.i_sb = idx_stride[0]; p.i_sg = idx_stride[1]; p.i_sh = idx_stride[2]; p.i_st = idx_stride[3];
  p.B = B; p.H = H; p.T = T; p.block_size = block_size; p.chunk_size = chunk_size; p.causal = causal;
  p.G = group_size; p.MG = static_cast<int>(cdiv64(M, group_size)); p.M = M;
  p.NS = cdiv64(kv->n_tokens, block_size);
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  return dispatch_bwd<true>(p, dtype, D, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_sel_bwd_dkv(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                               const int32_t* groups, const int32_t* offsets, const float* lse,
                               const float* delta, const void* d_out, const int64_t do_stride[3],
                               void* dk, void* dv, int32_t B, int64_t M, int32_t H, int32_t D, int32_t T,
                               int32_t block_size, int32_t chunk_size, int32_t causal,
                               int32_t group_size, float scale, void* workspace, size_t workspace_bytes,
                               int32_t dtype, void* stream) {
  return nsa_sel_bwd_dkv_pds(q, q_stride, kv, groups, offsets, nullptr, nullptr, 0, lse, delta, d_out, do_stride, dk, dv,
                             B, M, H, D, T, block_size, chunk_size, causal, group_size, scale, workspace,
                             workspace_bytes, dtype, stream);
}

extern "C" int nsa_sel_bwd_dkv_pds(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                                   const int32_t* groups, const int32_t* offsets, const int32_t* slots,
                                   const void* pds, size_t pds_bytes, const float* lse,
                                   const float* delta, const void* d_out, const int64_t do_stride[3],
                                   void* dk, void* dv, int32_t B, int64_t M, int32_t H, int32_t D, int32_t T,
                                   int32_t block_size, int32_t chunk_size, int32_t causal,
                                   int32_t group_size, float scale, void* workspace, size_t workspace_bytes,
                                   int32_t dtype, void* stream) {
  int rc;
  if ((rc = bwd_common_checks("sel_bwd_dkv", B, M, H, D, T, block_size, chunk_size, group_size, dtype, kv))) return rc;
  const int64_t N = kv->n_tokens;
  if (B == 0 || H == 0 || N == 0) return NSA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int esz = 2;
  NSA_REQUIRE(dk && dv && aligned16(dk) && aligned16(dv), NSA_ERR_LAYOUT, "sel_bwd_dkv: dk/dv must be 16-byte aligned");
  if (M == 0) {
    NSA_CUDA_OK(cudaMemsetAsync(dk, 0, static_cast<size_t>(B) * N * H * D * esz, s));
    NSA_CUDA_OK(cudaMemsetAsync(dv, 0, static_cast<size_t>(B) * N * H * D * esz, s));
    return NSA_OK;
  }
  NSA_REQUIRE(groups && offsets && lse && delta, NSA_ERR_INVALID, "sel_bwd_dkv: null pointer");
  if ((rc = check_strides16("q", q, q_stride, 3, esz))) return rc;
  if ((rc = check_strides16("d_out", d_out, do_stride, 3, esz))) return rc;
  BwdParams p{};
  if ((rc = make_kvsrc(kv, D, esz, block_size, &p.kv))) return rc;
  {
    bool launched = false;
    int32_t* counter = (workspace != nullptr && workspace_bytes >= 256) ? static_cast<int32_t*>(workspace) : nullptr;
    if (pds != nullptr && slots != nullptr) {
      // P and dS of every pair were stored by the dQ kernel: stream them instead of recomputing S and dP
      NSA_REQUIRE(pds_bytes >= nsa_sel_bwd_pds_bytes(B, M, H, T, group_size) && aligned16(pds), NSA_ERR_WORKSPACE,
                  "sel_bwd_dkv: the P/dS buffer is too small or misaligned");
      rc = try_launch_sel_bwd_dkv_pds_tc(q, q_stride, kv, groups, slots, offsets, pds, d_out, do_stride, dk, dv, B, M, H,
                                         D, T, block_size, group_size, dtype, counter, s, &launched);
      if (rc) return rc;
      if (launched) return NSA_OK;
      NSA_REQUIRE(false, NSA_ERR_UNSUPPORTED, "sel_bwd_dkv: the stored-probabilities kernel does not serve this call");
    }
    rc = try_launch_sel_bwd_dkv_tc(q, q_stride, kv, groups, offsets, lse, delta, d_out, do_stride, dk, dv, B, M, H, D,
                                   T, block_size, chunk_size, causal, group_size, scale, dtype, counter, s, &launched);
    if (rc) return rc;
    if (launched) return NSA_OK;
  }
  p.q = static_cast<const char*>(q); p.q_sb = q_stride[0]; p.q_sm = q_stride[1]; p.q_sh = q_stride[2];
  p.dO = static_cast<const char*>(d_out); p.do_sb = do_stride[0]; p.do_sm = do_stride[1]; p.do_sh = do_stride[2];
  p.dk = static_cast<char*>(dk); p.dv = static_cast<char*>(dv);
  p.lse = lse; p.delta = const_cast<float*>(delta);
  p.groups = groups; p.offsets = offsets;
  p.B = B; p.H = H; p.T = T; p.block_size = block_size; p.chunk_size = chunk_size; p.causal = causal;
  p.G = group_size; p.MG = static_cast<int>(cdiv64(M, group_size)); p.M = M; p.NS = cdiv64(N, block_size);
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  return dispatch_bwd<false>(p, dtype, D, s);
}

extern "C" int nsa_sel_bwd_dkv_ptr(const void* q, const int64_t q_stride[3], const int64_t* base_k,
                                   const int64_t* base_v, const int64_t* base_dk, const int64_t* base_dv,
                                   const int64_t base_stride[2], int32_t max_base,
                                   const int32_t* n_blocks_per_head, int64_t batch_stride_kv_bytes,
                                   int64_t batch_stride_dkv_bytes, int64_t stride_bn, int64_t stride_dbn,
                                   int32_t blocks_per_chunk, int64_t in_chunk_block_bytes_kv,
                                   int64_t in_chunk_block_bytes_dkv, const int32_t* groups,
                                   const int32_t* offsets, int64_t NS, const float* lse, const float* delta,
                                   const void* d_out, const int64_t do_stride[3], int32_t B, int64_t M,
                                   int32_t H, int32_t D, int32_t T, int32_t block_size, int32_t group_size,
                                   float scale, int32_t dtype, void* stream) {
  nsa_kv_source dummy{};
  dummy.mode = NSA_KV_DENSE;
  dummy.n_tokens = NS * block_size;
  int rc;
  if ((rc = bwd_common_checks("sel_bwd_dkv_ptr", B, M, H, D, T, block_size, 1, group_size, dtype, &dummy))) return rc;
  if (B == 0 || H == 0 || M == 0 || NS == 0) return NSA_OK;
  NSA_REQUIRE(base_k && base_v && base_dk && base_dv && base_stride, NSA_ERR_INVALID, "sel_bwd_dkv_ptr: null base table");
  NSA_REQUIRE(groups && offsets && lse && delta, NSA_ERR_INVALID, "sel_bwd_dkv_ptr: null pointer");
  NSA_REQUIRE(max_base > 0, NSA_ERR_INVALID, "sel_bwd_dkv_ptr: max_base must be > 0");
  NSA_REQUIRE(blocks_per_chunk >= 0, NSA_ERR_INVALID, "sel_bwd_dkv_ptr: blocks_per_chunk must be >= 0");
  NSA_REQUIRE(blocks_per_chunk == 0 || (in_chunk_block_bytes_kv > 0 && in_chunk_block_bytes_dkv > 0), NSA_ERR_INVALID,
              "sel_bwd_dkv_ptr: chunk-level bases need in_chunk_block_bytes_kv/dkv > 0");
  NSA_REQUIRE(stride_bn > 0 && (stride_bn * 2) % 16 == 0, NSA_ERR_LAYOUT,
              "sel_bwd_dkv_ptr: K/V token stride must be a positive multiple of 16 bytes");
  NSA_REQUIRE(stride_dbn >= D && stride_dbn % 2 == 0, NSA_ERR_LAYOUT,
              "sel_bwd_dkv_ptr: stride_dbn must be the fp32 scratch stride (>= D, even)");
  const int esz = 2;
  if ((rc = check_strides16("q", q, q_stride, 3, esz))) return rc;
  if ((rc = check_strides16("d_out", d_out, do_stride, 3, esz))) return rc;
  BwdParams p{};
  p.kv.mode = NSA_KV_DENSE;
  p.kv.n_tokens = NS * block_size;
  p.q = static_cast<const char*>(q); p.q_sb = q_stride[0]; p.q_sm = q_stride[1]; p.q_sh = q_stride[2];
  p.dO = static_cast<const char*>(d_out); p.do_sb = do_stride[0]; p.do_sm = do_stride[1]; p.do_sh = do_stride[2];
  p.lse = lse; p.delta = const_cast<float*>(delta);
  p.groups = groups; p.offsets = offsets;
  p.B = B; p.H = H; p.T = T; p.block_size = block_size; p.chunk_size = 1; p.causal = 0;
  p.G = group_size; p.MG = static_cast<int>(cdiv64(M, group_size)); p.M = M; p.NS = NS;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.tab.on = 1;
  p.tab.base_k = base_k; p.tab.base_v = base_v; p.tab.base_dk = base_dk; p.tab.base_dv = base_dv;
  p.tab.base_sh = base_stride[0]; p.tab.base_sb = base_stride[1]; p.tab.max_base = max_base;
  p.tab.n_blocks_per_head = n_blocks_per_head;
  p.tab.batch_kv_bytes = batch_stride_kv_bytes; p.tab.batch_dkv_bytes = batch_stride_dkv_bytes;
  p.tab.in_chunk_kv_bytes = in_chunk_block_bytes_kv; p.tab.in_chunk_dkv_bytes = in_chunk_block_bytes_dkv;
  p.tab.blocks_per_chunk = blocks_per_chunk;
  p.tab.s_bn = stride_bn; p.tab.s_dbn = stride_dbn;
  return dispatch_bwd<false>(p, dtype, D, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_sel_bwd(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                           const int32_t* block_indices, const int64_t idx_stride[4],
                           const void* out, const int64_t out_stride[3], const float* lse,
                           const void* d_out, const int64_t do_stride[3], void* dq,
                           const int64_t dq_stride[3], void* dk, void* dv, int32_t B, int64_t M,
                           int32_t H, int32_t D, int32_t T, int32_t block_size, int32_t chunk_size,
                           int32_t causal, int32_t group_size, float scale, void* workspace,
                           size_t workspace_bytes, int32_t dtype, void* stream) {
  int rc;
  if ((rc = bwd_common_checks("sel_bwd", B, M, H, D, T, block_size, chunk_size, group_size, dtype, kv))) return rc;
  const int64_t N = kv->n_tokens;
  const int64_t NS = cdiv64(N, block_size), MG = cdiv64(M, group_size);
  NSA_REQUIRE(workspace_bytes >= nsa_sel_bwd_workspace_bytes(B, M, H, N, T, block_size, group_size),
              NSA_ERR_WORKSPACE, "sel_bwd: workspace too small");
  if (B == 0 || H == 0) return NSA_OK;
  NSA_REQUIRE(workspace != nullptr, NSA_ERR_INVALID, "sel_bwd: workspace is null");
  size_t off[6];
  bwd_ws_layout(B, M, H, NS, MG, T, off);
  char* ws = static_cast<char*>(workspace);
  float* delta = reinterpret_cast<float*>(ws + off[0]);
  int32_t* counts = reinterpret_cast<int32_t*>(ws + off[1]);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + off[2]);
  int32_t* groups = reinterpret_cast<int32_t*>(ws + off[3]);
  if (M > 0) {
    NSA_REQUIRE(block_indices != nullptr, NSA_ERR_INVALID, "sel_bwd: block_indices is null");
    IdxParams ip{block_indices, idx_stride[0], idx_stride[1], idx_stride[2], idx_stride[3],
                 B, static_cast<int>(MG), H, T, NS, block_size, chunk_size, causal, group_size, nullptr};
    if ((rc = run_inverted_index(ip, groups, offsets, counts, static_cast<cudaStream_t>(stream)))) return rc;
    if ((rc = nsa_sel_bwd_dq(q, q_stride, kv, block_indices, idx_stride, out, out_stride, lse, d_out, do_stride,
                             dq, dq_stride, delta, B, M, H, D, T, block_size, chunk_size, causal, group_size,
                             scale, dtype, stream))) return rc;
  }
  return nsa_sel_bwd_dkv(q, q_stride, kv, groups, offsets, lse, delta, d_out, do_stride, dk, dv, B, M, H, D, T,
                         block_size, chunk_size, causal, group_size, scale, ws + off[4], 256, dtype, stream);
}
