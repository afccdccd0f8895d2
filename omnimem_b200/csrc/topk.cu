// Block-compressed key scoring and top-k block selection.
//   pool_rows_kernel   mean over runs of rows (key blocks / query groups), 16-byte loads
//   score_kernel       fp32 scores of pooled queries against pooled keys
//   select_kernel      per (b, group, h) row: top-k by (score desc, id asc) over packed
//                      64-bit keys, -1 padding; also merges per-shard candidate lists
#include "common.cuh"
#include "tc_common.cuh"

#include <mutex>

namespace nsa {

int device_status_address(int32_t** out);     // the sticky status word of the tensor-core kernels (sel_fwd_tc.cu)

namespace {

// ---------------------------------------------------------------------------------- pooling
// Mean over runs of `size` rows of x [B,N,H,D].  A thread owns one 16-byte column piece of a row of
// one head and walks the run's rows with kPoolUnroll loads in flight; the threads of a block cover
// `hc` neighbouring heads, so that a block reads CONTIGUOUS row pieces (whole rows when hc = H):
// reading one head's 256 bytes out of every row, one thread block per head, left the DRAM pages
// half used and capped these kernels near 0.55 of the copy bandwidth.  Sums are fp32, rows added in
// ascending order, one rounding to the input dtype.
struct PoolParams {
  const char* x; int64_t x_sb, x_sn, x_sh;
  char* out; int64_t o_sb, o_sn, o_sh;
  int64_t N;
  int D, size;
  int H;
  int hc, hsplit;          // heads per thread block, thread blocks per run (hsplit = ceil(H / hc))
  int vec_store;           // output rows are 16-byte addressable
};

constexpr int kPoolUnroll = 8;

template <typename T>
__device__ __forceinline__ void pool_rows_body(const PoolParams& p, int64_t unit, int b) {
  constexpr int VEC = 16 / sizeof(T);
  const int cpr = p.D / VEC;                                  // 16-byte pieces per head row
  const int64_t c = unit / p.hsplit;
  const int h0 = static_cast<int>(unit % p.hsplit) * p.hc;
  const int nh = p.H - h0 < p.hc ? p.H - h0 : p.hc;
  const int64_t n0 = c * p.size;
  const int n = static_cast<int>(p.N - n0 < p.size ? p.N - n0 : p.size);
  const float inv = 1.f / static_cast<float>(n);
  const int64_t row_bytes = p.x_sn * sizeof(T);
  for (int item = threadIdx.x; item < nh * cpr; item += blockDim.x) {
    const int h = h0 + item / cpr, col = item % cpr;
    const char* base = p.x + (b * p.x_sb + n0 * p.x_sn + h * p.x_sh) * sizeof(T) + col * 16;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (int r = 0; r < n; r += kPoolUnroll) {
      uint4 v[kPoolUnroll];
#pragma unroll
      for (int u = 0; u < kPoolUnroll; ++u)
        v[u] = r + u < n ? *reinterpret_cast<const uint4*>(base + (r + u) * row_bytes) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < kPoolUnroll; ++u) {
        if (r + u < n) {
          const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[i] += to_f32<T>(e[i]);
        }
      }
    }
    char* orow = p.out + (b * p.o_sb + c * p.o_sn + h * p.o_sh) * sizeof(T) + col * 16;
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int i = 0; i < VEC; ++i) oe[i] = from_f32<T>(acc[i] * inv);
    if (p.vec_store) {
      *reinterpret_cast<uint4*>(orow) = o;
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) reinterpret_cast<T*>(orow)[i] = oe[i];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) pool_rows_kernel(const PoolParams p) {
  chain_release();
  chain_wait();
  pool_rows_body<T>(p, blockIdx.x, blockIdx.z);
}

// The same pooling for tensors whose rows are contiguous over the heads (x_sh == D, x_sn == H * D):
// a thread block owns one run of rows for ALL heads and streams it through shared memory with bulk
// asynchronous copies (cp.async.bulk, kBulkStages stages of up to 16 KiB, whole rows each), so the
// bytes in flight are set by shared memory - about 45 KiB per thread block, four or five blocks per SM,
// enough blocks resident for a selection's 586 runs to start together - not
// by registers: with 16-byte register loads these kernels had about 85 KiB per SM in flight and
// stayed near 0.68 of the copy bandwidth.  Thread i owns 16-byte column piece i of the row, adds the
// rows in ascending order (fp32) and writes its piece of the pooled row.  A wait that gives up
// (bounded) raises the sticky device status word.
constexpr int kBulkStages = 3;
constexpr int kBulkStageBytes = 16 * 1024;

struct BulkPlan { int rows_per_stage; int threads; size_t smem; };

template <typename T>
__device__ __forceinline__ void pool_rows_bulk_body(const PoolParams& p, int64_t c, int b, int rows_per_stage,
                                                    uint8_t* stage0, uint64_t* full, volatile int* abort) {
  constexpr int VEC = 16 / sizeof(T);
  const int row_bytes = p.H * p.D * static_cast<int>(sizeof(T));
  const uint32_t stage_bytes = static_cast<uint32_t>(rows_per_stage) * row_bytes;
  const int64_t n0 = c * p.size;
  const int n = static_cast<int>(p.N - n0 < p.size ? p.N - n0 : p.size);
  const int chunks = (n + rows_per_stage - 1) / rows_per_stage;
  const char* src = p.x + (b * p.x_sb + n0 * p.x_sn) * sizeof(T);
  auto issue = [&](int i) {                              // thread 0: chunk i into stage i % kBulkStages
    const int s = i % kBulkStages;
    const int r0 = i * rows_per_stage;
    const uint32_t bytes = static_cast<uint32_t>((n - r0 < rows_per_stage ? n - r0 : rows_per_stage)) * row_bytes;
    tc::mbar_expect_tx(&full[s], bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(stage0 + static_cast<size_t>(s) * stage_bytes)), "l"(src + static_cast<int64_t>(r0) * row_bytes),
                   "r"(bytes), "r"(smem_u32(&full[s])) : "memory");
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < chunks && i < kBulkStages; ++i) issue(i);
  const int items = row_bytes / 16;
  float acc[2][VEC];                                      // up to two column pieces per thread
#pragma unroll
  for (int k = 0; k < 2; ++k)
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[k][i] = 0.f;
  bool ok = true;
  for (int i = 0; i < chunks; ++i) {
    const int s = i % kBulkStages;
    ok = tc::mbar_wait(&full[s], (i / kBulkStages) & 1, abort);
    if (!ok) break;
    const int rows = n - i * rows_per_stage < rows_per_stage ? n - i * rows_per_stage : rows_per_stage;
    const uint8_t* st = stage0 + static_cast<size_t>(s) * stage_bytes;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int item = threadIdx.x + k * blockDim.x;
      if (item < items) {
        for (int r = 0; r < rows; ++r) {
          const uint4 v = *reinterpret_cast<const uint4*>(st + r * row_bytes + item * 16);
          const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int q = 0; q < VEC; ++q) acc[k][q] += to_f32<T>(e[q]);
        }
      }
    }
    __syncthreads();                                      // the stage is consumed: refill it
    if (threadIdx.x == 0 && i + kBulkStages < chunks) issue(i + kBulkStages);
  }
  if (!ok) return;
  const float inv = 1.f / static_cast<float>(n);
  const int cpr = p.D / VEC;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int item = threadIdx.x + k * blockDim.x;
    if (item < items) {
      const int h = item / cpr, col = item % cpr;
      char* orow = p.out + (b * p.o_sb + c * p.o_sn + h * p.o_sh) * sizeof(T) + col * 16;
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int q = 0; q < VEC; ++q) oe[q] = from_f32<T>(acc[k][q] * inv);
      if (p.vec_store) {
        *reinterpret_cast<uint4*>(orow) = o;
      } else {
#pragma unroll
        for (int q = 0; q < VEC; ++q) reinterpret_cast<T*>(orow)[q] = oe[q];
      }
    }
  }
}

// One or two poolings per launch: thread blocks [0, units_a) serve a (rows_a rows per stage), the rest b.
template <typename T>
__global__ void __launch_bounds__(512) pool_rows_bulk_kernel(const PoolParams a, const PoolParams b, int64_t units_a,
                                                             int rows_a, int rows_b, int32_t* status) {
  extern __shared__ __align__(128) uint8_t s_bulk[];
  __shared__ uint64_t full[kBulkStages];
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kBulkStages; ++i) tc::mbar_init(&full[i], 1);
    tc::fence_barrier_init();
  }
  __syncthreads();
  chain_release();
  chain_wait();
  if (static_cast<int64_t>(blockIdx.x) < units_a) pool_rows_bulk_body<T>(a, blockIdx.x, blockIdx.z, rows_a, s_bulk, full, &s_abort);
  else pool_rows_bulk_body<T>(b, blockIdx.x - units_a, blockIdx.z, rows_b, s_bulk, full, &s_abort);
  if (threadIdx.x == 0 && s_abort) atomicExch(status, NSA_ERR_CUDA);
}

// Two poolings in one launch (the query groups and the key blocks of one selection): thread blocks
// [0, units_a) serve a, the rest b.
template <typename T>
__global__ void __launch_bounds__(256) pool_rows_pair_kernel(const PoolParams a, const PoolParams b, int64_t units_a) {
  chain_release();
  chain_wait();
  if (static_cast<int64_t>(blockIdx.x) < units_a) pool_rows_body<T>(a, blockIdx.x, blockIdx.z);
  else pool_rows_body<T>(b, blockIdx.x - units_a, blockIdx.z);
}

// ---------------------------------------------------------------------------------- scoring
struct ScoreParams {
  const char* q; int64_t q_sb, q_sg, q_sh;
  const char* k; int64_t k_sb, k_sc, k_sh;
  float* scores;          // [B,H,MG,NC]
  int MG, H, D;
  int64_t NC;
  float scale;
};

constexpr int kScoreCols = 64;
constexpr int kScoreRows = 32;

template <typename T>
__global__ void __launch_bounds__(256) score_kernel(const ScoreParams p) {
  extern __shared__ float s_f[];
  float* ks = s_f;                                   // [64][D+1]
  float* qs = s_f + kScoreCols * (p.D + 1);          // [32][D]
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * kScoreCols;
  const int h = blockIdx.y, b = blockIdx.z;
  const int ncol = static_cast<int>(p.NC - c0 < kScoreCols ? p.NC - c0 : kScoreCols);
  for (int i = threadIdx.x; i < kScoreCols * p.D; i += blockDim.x) {
    const int c = i / p.D, d = i - c * p.D;
    float v = 0.f;
    if (c < ncol)
      v = to_f32<T>(*reinterpret_cast<const T*>(p.k + (b * p.k_sb + (c0 + c) * p.k_sc + h * p.k_sh + d) * sizeof(T)));
    ks[c * (p.D + 1) + d] = v;
  }
  const int cl = threadIdx.x & 63, gq = threadIdx.x >> 6;   // 4 row groups of 8 rows
  float* out = p.scores + ((static_cast<int64_t>(b) * p.H + h) * p.MG) * p.NC + c0 + cl;
  for (int g0 = 0; g0 < p.MG; g0 += kScoreRows) {
    __syncthreads();
    const int nrow = min(kScoreRows, p.MG - g0);
    for (int i = threadIdx.x; i < kScoreRows * p.D; i += blockDim.x) {
      const int r = i / p.D, d = i - r * p.D;
      float v = 0.f;
      if (r < nrow)
        v = to_f32<T>(*reinterpret_cast<const T*>(p.q + (b * p.q_sb + (g0 + r) * p.q_sg + h * p.q_sh + d) * sizeof(T)));
      qs[i] = v;
    }
    __syncthreads();
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    const float* kr = ks + cl * (p.D + 1);
    const float* qr = qs + gq * 8 * p.D;
    for (int d = 0; d < p.D; ++d) {
      const float kv = kr[d];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(qr[i * p.D + d], kv, acc[i]);
    }
    if (cl < ncol) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int g = g0 + gq * 8 + i;
        if (g < p.MG) out[static_cast<int64_t>(g) * p.NC] = acc[i] * p.scale + 0.f;
      }
    }
  }
}

// 16-bit inputs: the same scores on mma.sync (products of bf16 / fp16 operands are exact in fp32,
// the accumulation is fp32), one thread block per (64 key blocks, 64 query rows, head, batch).
constexpr int kScoreMmaRows = 64;

template <typename T>
__global__ void __launch_bounds__(128) score_mma_kernel(const ScoreParams p) {
  chain_release();
  chain_wait();
  extern __shared__ __align__(16) char s_raw[];
  const int PITCH = p.D + 8;
  T* sK = reinterpret_cast<T*>(s_raw);                  // [64][PITCH]
  T* sQ = sK + kScoreCols * PITCH;                      // [64][PITCH]
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * kScoreCols;
  const int g0 = blockIdx.y * kScoreMmaRows;
  const int h = blockIdx.z % p.H, b = blockIdx.z / p.H;
  const int ncol = static_cast<int>(p.NC - c0 < kScoreCols ? p.NC - c0 : kScoreCols);
  const int nrow = min(kScoreMmaRows, p.MG - g0);
  const int cpr = p.D / 8;                              // 16-byte chunks per row
  for (int i = threadIdx.x; i < kScoreCols * cpr; i += blockDim.x) {
    const int r = i / cpr, cc = i - r * cpr;
    const char* ksrc = p.k + (b * p.k_sb + (c0 + r) * p.k_sc + h * p.k_sh) * 2 + cc * 16;
    const char* qsrc = p.q + (b * p.q_sb + (g0 + r) * p.q_sg + h * p.q_sh) * 2 + cc * 16;
    cp_async16(sK + r * PITCH + cc * 8, r < ncol ? ksrc : p.k, r < ncol ? 16 : 0);
    cp_async16(sQ + r * PITCH + cc * 8, r < nrow ? qsrc : p.q, r < nrow ? 16 : 0);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, t4 = lane & 3;
  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
  const T* qa = sQ + (warp * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8;
  const T* kb = sK + ((lane & 7) + ((lane >> 4) << 3)) * PITCH + ((lane >> 3) & 1) * 8;
  for (int kk = 0; kk < p.D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, qa + kk * 16);
#pragma unroll
    for (int n16 = 0; n16 < 4; ++n16) {
      uint32_t bf[4];
      ldmatrix_x4(bf, kb + n16 * 16 * PITCH + kk * 16);
      mma16816<T>(acc[2 * n16], a, bf[0], bf[1]);
      mma16816<T>(acc[2 * n16 + 1], a, bf[2], bf[3]);
    }
  }
  float* out = p.scores + ((static_cast<int64_t>(b) * p.H + h) * p.MG + g0) * p.NC + c0;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + gid + 8 * r;
    if (row < nrow) {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int col = n * 8 + 2 * t4;
        if (col < ncol) out[static_cast<int64_t>(row) * p.NC + col] = acc[n][2 * r] * p.scale + 0.f;
        if (col + 1 < ncol) out[static_cast<int64_t>(row) * p.NC + col + 1] = acc[n][2 * r + 1] * p.scale + 0.f;
      }
    }
  }
}

template <typename T>
int launch_score_mma(const ScoreParams& sp, int B, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(2 * kScoreCols) * (sp.D + 8) * sizeof(T);
  NSA_CUDA_OK(cudaFuncSetAttribute(score_mma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const dim3 grid(static_cast<unsigned>(cdiv64(sp.NC, kScoreCols)), cdiv(sp.MG, kScoreMmaRows), sp.H * B);
  NSA_CUDA_OK(launch_chained(kChainSmall, score_mma_kernel<T>, grid, dim3(128), smem, s, sp));
  NSA_LAUNCH_OK("score_mma_kernel");
  return NSA_OK;
}

// --------------------------------------------------------------------------------- selection
struct Mask {
  int block_size, chunk_size, chunk_size_k, G, q_off, ex_win, ex_sink;
  int causal, tf, prog;
  int q_half, k_half;
  int id_base, id_stride;
};

struct RowMask { int q_cid, q_rel; bool q_clean, do_excl; };

__device__ __forceinline__ RowMask make_row_mask(const Mask& m, int g) {
  RowMask r;
  r.q_cid = static_cast<int>((static_cast<int64_t>(g) * m.G) / m.chunk_size) + m.q_off;
  if (m.tf) {
    r.q_clean = r.q_cid < m.q_half;
    r.q_rel = r.q_clean ? r.q_cid : r.q_cid - m.q_half;
  } else {
    r.q_clean = true;
    r.q_rel = r.q_cid;
  }
  r.do_excl = m.prog ? (r.q_rel >= m.ex_sink + m.ex_win) : true;
  return r;
}

// Visibility of the key block with GLOBAL id `bid` for a query row.
__device__ __forceinline__ bool visible(const Mask& m, const RowMask& r, int bid) {
  // (32-bit division when the token index fits: the 64-bit one is a long emulated sequence)
  const int64_t tok = static_cast<int64_t>(bid) * m.block_size;
  const int k_cid = tok <= 0x7fffffff ? static_cast<int>(static_cast<uint32_t>(tok) / static_cast<uint32_t>(m.chunk_size_k))
                                      : static_cast<int>(tok / m.chunk_size_k);
  const bool k_clean = m.tf ? (k_cid < m.k_half) : true;
  const int k_rel = (m.tf && !k_clean) ? k_cid - m.k_half : k_cid;
  bool valid;
  if (m.tf) {
    valid = (r.q_clean && k_clean && k_rel <= r.q_rel) || (!r.q_clean && k_clean && k_rel < r.q_rel) ||
            (!r.q_clean && !k_clean && k_rel == r.q_rel);
  } else {
    valid = m.causal ? (k_cid <= r.q_cid) : true;
  }
  if (m.ex_sink > 0) {
    const bool sink_ok = !k_clean || k_rel >= m.ex_sink;
    valid = valid && (sink_ok || !r.do_excl);
  }
  if (m.ex_win > 0) {
    bool in_win;
    if (m.tf) {
      in_win = k_clean && k_rel >= r.q_rel - m.ex_win + 1;
    } else {
      in_win = k_cid >= r.q_cid - m.ex_win + 1;
      if (!m.causal) in_win = in_win && k_cid <= r.q_cid + m.ex_win - 1;
    }
    valid = valid && (!in_win || !r.do_excl);
  }
  return valid;
}

// The same rule without the teacher-forcing layout, as three comparisons per block: for one query
// row the visible blocks are those with lo <= id < hi that do not lie in [win_lo, win_hi) - the
// chunk conditions of visible() solved for the block id once per row.
struct RowBounds { int lo, hi, win_lo, win_hi; };

__device__ __forceinline__ int ceil_div_pos(int64_t a, int64_t b) {            // ceil(a / b) for a >= 0, clamped to int
  const int64_t q = (a + b - 1) / b;
  return q > 0x7fffffff ? 0x7fffffff : static_cast<int>(q);
}
__device__ __forceinline__ RowBounds make_row_bounds(const Mask& m, const RowMask& r) {
  RowBounds rb{0, 0x7fffffff, 0, 0};
  const int64_t ck = m.chunk_size_k, bs = m.block_size;
  if (m.causal) rb.hi = ceil_div_pos((static_cast<int64_t>(r.q_cid) + 1) * ck, bs);      // k_cid <= q_cid
  if (r.do_excl) {
    if (m.ex_sink > 0) rb.lo = ceil_div_pos(static_cast<int64_t>(m.ex_sink) * ck, bs);  // k_cid >= ex_sink
    if (m.ex_win > 0) {
      const int64_t first = static_cast<int64_t>(r.q_cid) - m.ex_win + 1;               // k_cid >= first is in the window
      rb.win_lo = first > 0 ? ceil_div_pos(first * ck, bs) : 0;
      rb.win_hi = m.causal ? 0x7fffffff : ceil_div_pos((static_cast<int64_t>(r.q_cid) + m.ex_win) * ck, bs);
      if (rb.win_hi < 0) rb.win_hi = 0;
    }
  }
  return rb;
}
__device__ __forceinline__ bool visible_in(const RowBounds& rb, int bid) {
  return bid >= rb.lo && bid < rb.hi && !(bid >= rb.win_lo && bid < rb.win_hi);
}

// (score, id) -> 64-bit key; a larger key is a better candidate: higher score first, then the
// lower id.  0 is reserved for "not a candidate".
__device__ __forceinline__ unsigned long long pack_key(float s, int id) {
  uint32_t u = __float_as_uint(s + 0.f);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  if (s != s) u = 1u;
  if (u == 0u) u = 1u;
  return (static_cast<unsigned long long>(u) << 32) | (0xffffffffu - static_cast<uint32_t>(id));
}
__device__ __forceinline__ float key_score(unsigned long long k) {
  uint32_t u = static_cast<uint32_t>(k >> 32);
  u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
  return __uint_as_float(u);
}
__device__ __forceinline__ int key_id(unsigned long long k) {
  return static_cast<int>(0xffffffffu - static_cast<uint32_t>(k & 0xffffffffu));
}

struct SelectParams {
  const float* scores;    // MASKED mode: [rows_bh][MG][NC]; MERGE mode: [R][rows][T]
  const int32_t* cand_ids;// MERGE mode only
  int64_t NC;             // candidates per row
  int MG, H;              // MASKED: row = (b*MG + g)*H + h
  int seg_len;            // MERGE: T of the inputs
  int64_t seg_stride;     // MERGE: rows*T
  int topk;
  int32_t* out_idx;       // [rows][topk]
  float* out_scores;      // may be null
  Mask mask;
  int seg_cols;           // MASKED, first stage of long rows: columns per segment (0 = the whole row);
  int n_seg;              //   warp w takes segment w % n_seg of row w / n_seg and writes its list to
                          //   out_idx / out_scores laid out [n_seg][rows][topk]
};

template <bool MERGE>
__global__ void __launch_bounds__(128) select_kernel(const SelectParams p) {
  extern __shared__ unsigned long long s_keys[];     // [NC] when it fits (flag below), else unused
  __shared__ unsigned long long s_red[4];
  const int64_t row = blockIdx.x;
  const bool in_smem = p.NC * 8 <= 64 * 1024;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;

  RowMask rm{};
  const float* srow;
  if (MERGE) {
    srow = p.scores + row * p.seg_len;
  } else {
    const int h = static_cast<int>(row % p.H);
    const int64_t bg = row / p.H;
    const int g = static_cast<int>(bg % p.MG);
    const int64_t b = bg / p.MG;
    rm = make_row_mask(p.mask, g);
    srow = p.scores + ((b * p.H + h) * p.MG + g) * p.NC;
  }
  auto key_at = [&](int64_t c) -> unsigned long long {
    if (MERGE) {
      const int64_t off = (c / p.seg_len) * p.seg_stride + (c % p.seg_len);
      const int id = p.cand_ids[row * p.seg_len + off];
      return id < 0 ? 0ull : pack_key(srow[off], id);
    }
    const int bid = p.mask.id_base + static_cast<int>(c) * p.mask.id_stride;
    return visible(p.mask, rm, bid) ? pack_key(srow[c], bid) : 0ull;
  };
  if (in_smem) {
    for (int64_t c = threadIdx.x; c < p.NC; c += blockDim.x) s_keys[c] = key_at(c);
    __syncthreads();
  }
  auto scan_below = [&](unsigned long long bound) {
    unsigned long long best = 0ull;
    for (int64_t c = threadIdx.x; c < p.NC; c += blockDim.x) {
      const unsigned long long k = in_smem ? s_keys[c] : key_at(c);
      if (k < bound && k > best) best = k;
    }
    return best;
  };

  unsigned long long local = scan_below(~0ull);
  int32_t* oi = p.out_idx + row * p.topk;
  float* os = p.out_scores ? p.out_scores + row * p.topk : nullptr;
  int r = 0;
  for (; r < p.topk; ++r) {
    unsigned long long best = local;
#pragma unroll
    for (int d = 16; d; d >>= 1) {
      const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, d);
      best = o > best ? o : best;
    }
    if (lane == 0) s_red[warp] = best;
    __syncthreads();
    best = s_red[0];
    for (int w = 1; w < nw; ++w) best = s_red[w] > best ? s_red[w] : best;
    __syncthreads();
    if (best == 0ull) break;
    if (threadIdx.x == 0) {
      oi[r] = key_id(best);
      if (os) os[r] = key_score(best);
    }
    if (local == best) local = scan_below(best);
  }
  for (int i = r + threadIdx.x; i < p.topk; i += blockDim.x) {
    oi[i] = -1;
    if (os) os[i] = -INFINITY;
  }
}

#ifdef NSA_SS_TRACE
// Debug build only: clock64 stamps of thread 0 of thread block (0,0,0) of the fused kernel.
__device__ long long g_trace_ss[16];
#define SS_TRACE(slot) do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) g_trace_ss[slot] = clock64(); } while (0)
#else
#define SS_TRACE(slot) do { } while (0)
#endif

// Bitonic sort of up to 64 keys held two per lane (element e = i * 32 + lane), largest first; with
// `both` false the second key of every lane is known to be 0 and only the first 32 are sorted.
__device__ __forceinline__ void warp_sort64_desc(unsigned long long& k0, unsigned long long& k1, bool both) {
  const int lane = threadIdx.x & 31;
  auto exchange = [&](unsigned long long& v, int e, int k, int j) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, j);
    const bool keep_max = ((e & j) == 0) == ((e & k) == 0);
    const bool other_larger = other > v;
    v = (keep_max == other_larger) ? other : v;
  };
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1)
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      exchange(k0, lane, k, j);
      if (both) exchange(k1, 32 + lane, k, j);
    }
  if (both) {
    // k = 64: every element sorts downwards; j = 32 pairs the lane's two keys
    const unsigned long long hi = k0 > k1 ? k0 : k1, lo = k0 > k1 ? k1 : k0;
    k0 = hi;
    k1 = lo;
#pragma unroll
    for (int j = 16; j > 0; j >>= 1) {
      exchange(k0, lane, 64, j);
      exchange(k1, 32 + lane, 64, j);
    }
  }
}

// Rows with at most 32*ITEMS candidates: one warp per row, no block-wide barrier.  Same keys and
// order as select_kernel.
//
// The selection proper: the warp's candidates as packed keys, ITEMS per lane (0 = no candidate);
// writes the best `topk` in order and pads with -1 / -inf.  `sorted` is the warp's [ITEMS][32]
// scratch in shared memory.
template <int ITEMS>
__device__ __forceinline__ void warp_take_topk(unsigned long long (&keys)[ITEMS], int topk, int32_t* oi, float* os,
                                               unsigned long long (*sorted)[32]) {
  const int lane = threadIdx.x & 31;
  if (ITEMS >= 2 && topk <= 16) {
    // Threshold first: the topk-th largest of the 32 lane maxima, tau, has at least topk keys at or
    // above it, so the row's top-k is among the keys >= tau - a few dozen of the 32 * ITEMS - which
    // are compacted and sorted across the lanes.  Exact; rows that leave more than 64 such keys (few
    // candidates spread over fewer than topk lanes) take the general path below.
    unsigned long long v = keys[0];
#pragma unroll
    for (int i = 1; i < ITEMS; ++i) v = keys[i] > v ? keys[i] : v;
    unsigned long long none = 0ull;
    warp_sort64_desc(v, none, false);
    const unsigned long long tau = __shfl_sync(0xffffffffu, v, topk - 1);
    unsigned long long* cand = &sorted[0][0];
    int total = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const bool in = keys[i] != 0ull && keys[i] >= tau;
      const uint32_t m = __ballot_sync(0xffffffffu, in);
      if (in) {
        const int pos = total + __popc(m & ((1u << lane) - 1u));
        if (pos < 64) cand[pos] = keys[i];
      }
      total += __popc(m);
    }
    __syncwarp();
    if (total <= 64) {
      unsigned long long k0 = lane < total ? cand[lane] : 0ull;
      unsigned long long k1 = lane + 32 < total ? cand[32 + lane] : 0ull;
      warp_sort64_desc(k0, k1, total > 32);
      if (lane < topk) {
        oi[lane] = k0 != 0ull ? key_id(k0) : -1;
        if (os) os[lane] = k0 != 0ull ? key_score(k0) : -INFINITY;
      }
      return;
    }
    __syncwarp();                                          // the scratch is reused below
  }
  // Each lane sorts its own keys once, largest first (bitonic network, all indices compile-time
  // constants, so the keys stay in registers), and parks the list in shared memory; a lane that
  // owns a round's winner then only steps to its next key.
#pragma unroll
  for (int k = 2; k <= ITEMS; k <<= 1)
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1)
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int l = i ^ j;
        if (l > i) {
          const unsigned long long x = keys[i], y = keys[l];
          const bool sw = ((i & k) == 0) ? (x < y) : (x > y);
          keys[i] = sw ? y : x;
          keys[l] = sw ? x : y;
        }
      }
#pragma unroll
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) sorted[i][lane] = keys[i];      // [rank][lane]: conflict-free for a warp
  // Per round: the best score half by one warp reduction; the lane that holds it owns the winner.
  // Only when several lanes hold the same score does a second reduction (over the id half) pick
  // the lowest id.  The owner writes the winner itself and steps to its next key, which it already
  // holds in a register; the key after that is fetched off the round's dependency chain.
  unsigned long long local = keys[0];
  unsigned long long ahead = ITEMS > 1 ? keys[ITEMS > 1 ? 1 : 0] : 0ull;
  int next = 2;
  int r = 0;
  for (; r < topk; ++r) {
    const uint32_t lhi = static_cast<uint32_t>(local >> 32), llo = static_cast<uint32_t>(local);
    const uint32_t bhi = __reduce_max_sync(0xffffffffu, lhi);
    if (bhi == 0u) break;                                  // the score half of a real key is never 0
    bool owner = lhi == bhi;
    const uint32_t holders = __ballot_sync(0xffffffffu, owner);
    if (holders & (holders - 1u)) {                        // a tie on the score: keys are unique, the id half decides
      const uint32_t blo = __reduce_max_sync(0xffffffffu, owner ? llo : 0u);
      owner = owner && llo == blo;
    }
    if (owner) {
      oi[r] = key_id(local);
      if (os) os[r] = key_score(local);
      local = ahead;
      ahead = next < ITEMS ? sorted[next < ITEMS ? next : 0][lane] : 0ull;
      ++next;
    }
  }
  for (int i = r + lane; i < topk; i += 32) {
    oi[i] = -1;
    if (os) os[i] = -INFINITY;
  }
}

// One warp selects one row (or one 1024-column segment of it): `srow` holds the row's scores (or the
// candidates' scores when merging lists), masked and packed into keys here.
template <int ITEMS, bool MERGE>
__device__ __forceinline__ void warp_select(const SelectParams& p, const float* srow, const RowMask& rm, int64_t NC,
                                            int64_t c_off, int64_t row, int32_t* oi, float* os,
                                            unsigned long long (*sorted)[32]) {
  const int lane = threadIdx.x & 31;
  // all loads first, unconditionally (clamped index), so that they are in flight together
  float vals[ITEMS];
  int cids[ITEMS];
  const int64_t last = NC - 1;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    int64_t c = lane + 32 * i;
    c = c < last ? c : last;
    if (MERGE) {
      const int seg = static_cast<int>(c) / p.seg_len;
      const int64_t off = static_cast<int64_t>(seg) * p.seg_stride + (static_cast<int>(c) - seg * p.seg_len);
      cids[i] = p.cand_ids[row * p.seg_len + off];
      vals[i] = srow[off];
    } else {
      cids[i] = 0;
      vals[i] = srow[c];
    }
  }
  unsigned long long keys[ITEMS];
  const RowBounds rb = MERGE ? RowBounds{0, 0, 0, 0} : make_row_bounds(p.mask, rm);   // the row's rules as id intervals
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int64_t c = lane + 32 * i;
    unsigned long long k = 0ull;
    if (c < NC) {
      if (MERGE) {
        k = cids[i] < 0 ? 0ull : pack_key(vals[i], cids[i]);
      } else {
        const int bid = p.mask.id_base + static_cast<int>(c_off + c) * p.mask.id_stride;
        const bool vis = p.mask.tf ? visible(p.mask, rm, bid) : visible_in(rb, bid);
        k = vis ? pack_key(vals[i], bid) : 0ull;
      }
    }
    keys[i] = k;
  }
  warp_take_topk<ITEMS>(keys, p.topk, oi, os, sorted);
}

template <int ITEMS, bool MERGE>
__global__ void __launch_bounds__(128) select_warp_kernel(const SelectParams p, int64_t rows) {
  chain_release();
  chain_wait();
  const int warp = threadIdx.x >> 5;
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  const int n_seg = (!MERGE && p.seg_cols > 0) ? p.n_seg : 1;
  if (unit >= rows * n_seg) return;
  const int64_t row = unit / n_seg;
  const int seg = static_cast<int>(unit - row * n_seg);
  const int64_t c_off = static_cast<int64_t>(seg) * p.seg_cols;          // 0 unless segmented
  const int64_t NC = n_seg > 1 ? (p.NC - c_off < p.seg_cols ? p.NC - c_off : p.seg_cols) : p.NC;
  RowMask rm{};
  const float* srow;
  if (MERGE) {
    srow = p.scores + row * p.seg_len;
  } else {
    const int h = static_cast<int>(row % p.H);
    const int64_t bg = row / p.H;
    const int g = static_cast<int>(bg % p.MG);
    const int64_t b = bg / p.MG;
    rm = make_row_mask(p.mask, g);
    srow = p.scores + ((b * p.H + h) * p.MG + g) * p.NC + c_off;
  }
  __shared__ unsigned long long s_sorted[4][ITEMS][32];
  const int64_t out_row = n_seg > 1 ? static_cast<int64_t>(seg) * rows + row : row;
  warp_select<ITEMS, MERGE>(p, srow, rm, NC, c_off, row, p.out_idx + out_row * p.topk,
                            p.out_scores ? p.out_scores + out_row * p.topk : nullptr, s_sorted[warp]);
}

// ------------------------------------------------------------------- fused scoring + selection
// For rows of at most kFusedNC key blocks, top-k up to kFusedTopk, 16-bit operands and D <= 128: one
// thread block per (batch, head, kRowTile pooled query rows).
//   load    every thread copies its 16-byte column of the head's pooled key rows into padded
//           shared-memory rows (cp.async, up to kKeysPerRound keys per round); the keys complete on
//           kKeyGroups barriers so that the products of the first keys run while the rest arrive
//   score   warp w multiplies key tile w (16 keys) with the query tile: m16n8k16 products with the
//           keys as the 16-row operand and the kRowTile query rows as the 8-column one, so that no
//           row of a product is padding; the products and their order over the head dimension are
//           those of score_mma_kernel - the scores carry the same bits - and each score is masked
//           and packed into its 64-bit key in shared memory on the spot
//   select  one warp per row sorts its lane's keys and takes the top-k (warp_take_topk)
// No score buffer in global memory, one launch instead of two.
constexpr int kRowTile = 8;
constexpr int kFusedNC = 1024;
constexpr int kFusedTopk = 64;
constexpr int kFusedD = 128;
constexpr int kKeysPerRound = 512;
constexpr int kKeyGroups = 4;
constexpr int kGroupKeys = kKeysPerRound / kKeyGroups;
constexpr int kFusedThreads = 1024;

// Shared-memory scratch of the selection (one [ITEMS][32] list of 64-bit keys per row); it overlays
// the key tile, which is dead by then, and sets the size of that region when the tile is smaller.
constexpr size_t score_select_scratch(int items) { return static_cast<size_t>(kRowTile) * items * 32 * 8; }


struct ScoreSelectParams {
  ScoreParams sc;          // q, k pooled + strides, MG, H, D, NC, scale (scores pointer unused)
  SelectParams sel;        // topk, out_idx, out_scores, mask (scores pointer unused)
};

// This thread's cp.async copies so far count as one pending arrival on `bar` (no extra count).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <typename T, int ITEMS>
__global__ void __launch_bounds__(kFusedThreads, 1) score_select_kernel(const ScoreSelectParams p, int32_t* status) {
  extern __shared__ __align__(128) char s_fused[];
  __shared__ uint64_t s_bar[kKeyGroups];
  __shared__ int s_abort;
  __shared__ RowMask s_rm[kRowTile];
  __shared__ RowBounds s_rb[kRowTile];
  const int D = p.sc.D, PITCH = D + 8;
  const int NC = static_cast<int>(p.sc.NC), NCP = ((NC + 15) & ~15) + 2, topk = p.sel.topk;
  T* sQ = reinterpret_cast<T*>(s_fused);                                 // [kRowTile][PITCH], rows >= nrow zero
  T* sK = sQ + kRowTile * PITCH;                                         // [kKeysPerRound][PITCH]; later the sort scratch
  const size_t tile_bytes = static_cast<size_t>(kKeysPerRound) * PITCH * sizeof(T);
  const size_t region = tile_bytes > score_select_scratch(ITEMS) ? tile_bytes : score_select_scratch(ITEMS);
  unsigned long long* sKey = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(sK) + region);   // [kRowTile][NCP]
  const int g0 = blockIdx.x * kRowTile;
  const int h = blockIdx.y, b = blockIdx.z;
  const int nrow = min(kRowTile, p.sc.MG - g0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, t4 = lane & 3;
  const int nwarp = kFusedThreads / 32;
  // ---- set-up that touches no input: barriers and the rows' mask constants
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < kKeyGroups; ++i) tc::mbar_init(&s_bar[i], kFusedThreads);
    tc::fence_barrier_init();
  }
  if (threadIdx.x < kRowTile) {
    const RowMask rm = make_row_mask(p.sel.mask, g0 + min(static_cast<int>(threadIdx.x), nrow - 1));
    s_rm[threadIdx.x] = rm;
    s_rb[threadIdx.x] = make_row_bounds(p.sel.mask, rm);
  }
  const int cpr = D / 8;                                                 // 16-byte chunks per row
  const int rpp = kFusedThreads / cpr;                                   // rows one pass of the block covers
  const int r0 = threadIdx.x / cpr, cc = threadIdx.x - r0 * cpr;
  __syncthreads();
  chain_release();
  chain_wait();
  SS_TRACE(0);
  volatile int* abort = &s_abort;
  uint32_t qf[kFusedD / 16][2];                                          // the query tile's fragments
  const int nkk = D / 16;
  bool ok = true;
  int round = 0;
  for (int k0 = 0; k0 < NC; k0 += kKeysPerRound, ++round) {
    const int nk = min(kKeysPerRound, NC - k0);
    const int nk16 = (nk + 15) & ~15;                                    // whole 16-key tiles, the tail zero-filled
    if (k0 > 0) __syncthreads();                                         // the previous round's keys are consumed
    if (k0 == 0 && r0 < kRowTile) {
      const bool real = r0 < nrow;
      const char* src = p.sc.q + (b * p.sc.q_sb + (g0 + (real ? r0 : 0)) * p.sc.q_sg + h * p.sc.q_sh) * 2 + cc * 16;
      cp_async16(sQ + r0 * PITCH + cc * 8, src, real ? 16 : 0);
    }
    {
      const char* kcol = p.sc.k + (b * p.sc.k_sb + static_cast<int64_t>(k0) * p.sc.k_sc + h * p.sc.k_sh) * 2 + cc * 16;
      const int64_t row_step = p.sc.k_sc * 2;
      T* dcol = sK + cc * 8;
#pragma unroll
      for (int gk = 0; gk < kKeyGroups; ++gk) {
        const int end = min((gk + 1) * kGroupKeys, nk16);
        for (int r = gk * kGroupKeys + r0; r < end; r += rpp) {
          const bool real = r < nk;
          cp_async16(dcol + r * PITCH, kcol + (real ? r : 0) * row_step, real ? 16 : 0);
        }
        cp_async_arrive(&s_bar[gk]);
      }
    }
    SS_TRACE(1 + 4 * round);
    for (int t = warp; t < nk16 / 16; t += nwarp) {                      // this warp's 16-key tiles
      ok = __all_sync(0xffffffffu, ok && tc::mbar_wait(&s_bar[(t * 16) / kGroupKeys], round & 1, abort));
      if (!ok) break;
      if (k0 == 0 && t == warp) {                                        // (the queries arrive with key group 0)
        if ((t * 16) / kGroupKeys != 0) ok = __all_sync(0xffffffffu, tc::mbar_wait(&s_bar[0], 0, abort));
        const T* qb = sQ + gid * PITCH + t4 * 2;
#pragma unroll
        for (int kk = 0; kk < kFusedD / 16; ++kk) {
          if (kk < nkk) {
            qf[kk][0] = *reinterpret_cast<const uint32_t*>(qb + kk * 16);
            qf[kk][1] = *reinterpret_cast<const uint32_t*>(qb + kk * 16 + 8);
          }
        }
      }
      SS_TRACE(2 + 4 * round);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const T* ka = sK + (t * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8;
#pragma unroll
      for (int kk = 0; kk < kFusedD / 16; ++kk) {
        if (kk < nkk) {
          uint32_t a[4];
          ldmatrix_x4(a, ka + kk * 16);
          mma16816<T>(acc, a, qf[kk][0], qf[kk][1]);
        }
      }
      SS_TRACE(3 + 4 * round);
      // acc[0..1]: key gid of the tile, query rows 2*t4 and 2*t4+1; acc[2..3]: key gid + 8
      const int c_lo = k0 + t * 16 + gid;
      const int n0 = 2 * t4;
      const RowBounds rb0 = s_rb[n0], rb1 = s_rb[n0 + 1];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c = c_lo + 8 * half;
        const int bid = p.sel.mask.id_base + c * p.sel.mask.id_stride;
        const float s0 = acc[2 * half] * p.sc.scale + 0.f, s1 = acc[2 * half + 1] * p.sc.scale + 0.f;
        bool v0, v1;
        if (p.sel.mask.tf) {
          v0 = visible(p.sel.mask, s_rm[n0], bid);
          v1 = visible(p.sel.mask, s_rm[n0 + 1], bid);
        } else {
          v0 = visible_in(rb0, bid);
          v1 = visible_in(rb1, bid);
        }
        const bool in = c < NC;
        sKey[n0 * NCP + c] = (in && v0) ? pack_key(s0, bid) : 0ull;
        sKey[(n0 + 1) * NCP + c] = (in && v1) ? pack_key(s1, bid) : 0ull;
      }
      SS_TRACE(4 + 4 * round);
    }
  }
  __syncthreads();                                                       // keys complete, key tile dead
  SS_TRACE(9);
  // ---- selection: warp r takes row r
  if (warp < nrow && !s_abort) {
    unsigned long long (*sorted)[32] = reinterpret_cast<unsigned long long (*)[32]>(sK) + warp * ITEMS;
    const int64_t row = (static_cast<int64_t>(b) * p.sc.MG + g0 + warp) * p.sc.H + h;
    const unsigned long long* krow = sKey + warp * NCP;
    unsigned long long keys[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int c = lane + 32 * i;
      keys[i] = c < NC ? krow[c] : 0ull;
    }
    warp_take_topk<ITEMS>(keys, topk, p.sel.out_idx + row * topk, p.sel.out_scores ? p.sel.out_scores + row * topk : nullptr, sorted);
  }
  SS_TRACE(10);
  if (threadIdx.x == 0 && s_abort) atomicExch(status, NSA_ERR_CUDA);
}

size_t score_select_smem(int D, int64_t NC) {
  const int items = NC <= 8 * 32 ? 8 : (NC <= 16 * 32 ? 16 : 32);
  const size_t tile = static_cast<size_t>(kKeysPerRound) * (D + 8) * 2;
  const size_t region = tile > score_select_scratch(items) ? tile : score_select_scratch(items);
  return static_cast<size_t>(kRowTile) * (D + 8) * 2 + region + static_cast<size_t>(kRowTile) * (((NC + 15) & ~15) + 2) * 8;
}

template <typename T>
int launch_score_select(const ScoreSelectParams& p, int B, cudaStream_t s) {
  const size_t smem = score_select_smem(p.sc.D, p.sc.NC);
  const dim3 grid(cdiv(p.sc.MG, kRowTile), p.sc.H, B);
  int32_t* status = nullptr;
  int rc;
  if ((rc = device_status_address(&status))) return rc;
  if (p.sc.NC <= 8 * 32) {
    NSA_CUDA_OK(cudaFuncSetAttribute(score_select_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    NSA_CUDA_OK(launch_chained(kChainSmall, score_select_kernel<T, 8>, grid, dim3(kFusedThreads), smem, s, p, status));
  } else if (p.sc.NC <= 16 * 32) {
    NSA_CUDA_OK(cudaFuncSetAttribute(score_select_kernel<T, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    NSA_CUDA_OK(launch_chained(kChainSmall, score_select_kernel<T, 16>, grid, dim3(kFusedThreads), smem, s, p, status));
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(score_select_kernel<T, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    NSA_CUDA_OK(launch_chained(kChainSmall, score_select_kernel<T, 32>, grid, dim3(kFusedThreads), smem, s, p, status));
  }
  NSA_LAUNCH_OK("score_select_kernel");
  return NSA_OK;
}

constexpr int kSegCols = 1024;       // candidates one warp sorts in registers
constexpr int kSegTopkMax = 64;      // largest top-k the two-stage selection of long rows is sized for

size_t segment_workspace_bytes(int64_t rows, int64_t NC) {
  if (NC <= kSegCols) return 0;
  return align_up(static_cast<size_t>(cdiv64(NC, kSegCols)) * rows * kSegTopkMax * 8, 256);
}

template <bool MERGE>
int launch_select(const SelectParams& sel, int64_t rows, cudaStream_t s, void* seg_ws = nullptr) {
  const unsigned blocks4 = static_cast<unsigned>(cdiv64(rows, 4));
  if (!MERGE && seg_ws != nullptr && sel.NC > kSegCols && sel.topk <= kSegTopkMax &&
      cdiv64(sel.NC, kSegCols) * rows <= 0x7fffffff) {
    // Long rows in two stages: one warp per (row, 1024-column segment) takes the segment's top-k
    // (same keys, same order), then the per-segment lists of a row are merged like per-shard
    // candidate lists.  Exact: the row's top-k is a subset of the union of the segments' top-k.
    const int n_seg = static_cast<int>(cdiv64(sel.NC, kSegCols));
    int32_t* cand_idx = static_cast<int32_t*>(seg_ws);
    float* cand_val = reinterpret_cast<float*>(cand_idx + static_cast<int64_t>(n_seg) * rows * sel.topk);
    SelectParams first = sel;
    first.seg_cols = kSegCols; first.n_seg = n_seg; first.out_idx = cand_idx; first.out_scores = cand_val;
    const unsigned blocks = static_cast<unsigned>(cdiv64(rows * n_seg, 4));
    NSA_CUDA_OK(launch_chained(kChainSmall, select_warp_kernel<32, false>, dim3(blocks), dim3(128), 0, s, first, rows));
    NSA_LAUNCH_OK("select kernel (segments)");
    SelectParams merge{};
    merge.scores = cand_val; merge.cand_ids = cand_idx; merge.NC = static_cast<int64_t>(n_seg) * sel.topk;
    merge.MG = 1; merge.H = 1; merge.seg_len = sel.topk; merge.seg_stride = rows * sel.topk; merge.topk = sel.topk;
    merge.out_idx = sel.out_idx; merge.out_scores = sel.out_scores;
    return launch_select<true>(merge, rows, s);
  }
  if (sel.NC <= 512) {
    NSA_CUDA_OK(launch_chained(kChainSmall, select_warp_kernel<16, MERGE>, dim3(blocks4), dim3(128), 0, s, sel, rows));
  } else if (sel.NC <= 1024) {
    NSA_CUDA_OK(launch_chained(kChainSmall, select_warp_kernel<32, MERGE>, dim3(blocks4), dim3(128), 0, s, sel, rows));
  } else {
    const size_t ksmem = sel.NC * 8 <= 64 * 1024 ? static_cast<size_t>(sel.NC) * 8 : 0;
    NSA_CUDA_OK(cudaFuncSetAttribute(select_kernel<MERGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    select_kernel<MERGE><<<static_cast<unsigned>(rows), 128, ksmem, s>>>(sel);
  }
  NSA_LAUNCH_OK("select kernel");
  return NSA_OK;
}

int fill_mask(const nsa_topk_mask* in, int MG, int64_t NC_global, Mask* m) {
  NSA_REQUIRE(in != nullptr, NSA_ERR_INVALID, "topk: mask is null");
  NSA_REQUIRE(in->block_size > 0 && in->chunk_size > 0 && in->chunk_size_k > 0 && in->q_group_size > 0,
              NSA_ERR_INVALID, "topk: block_size / chunk_size / chunk_size_k / q_group_size must be > 0");
  NSA_REQUIRE(in->ex_win >= 0 && in->ex_sink >= 0 && in->q_chunk_offset >= 0, NSA_ERR_INVALID,
              "topk: ex_win / ex_sink / q_chunk_offset must be >= 0");
  NSA_REQUIRE(!(in->tf_mask && in->q_chunk_offset != 0), NSA_ERR_INVALID,
              "topk: tf_mask assumes a full [clean|noisy] layout, q_chunk_offset must be 0");
  NSA_REQUIRE(in->id_stride >= 1 && in->id_base >= 0, NSA_ERR_INVALID, "topk: id_stride must be >= 1, id_base >= 0");
  m->block_size = in->block_size; m->chunk_size = in->chunk_size; m->chunk_size_k = in->chunk_size_k;
  m->G = in->q_group_size; m->q_off = in->q_chunk_offset; m->ex_win = in->ex_win; m->ex_sink = in->ex_sink;
  m->causal = in->causal; m->tf = in->tf_mask; m->prog = in->prog_excl;
  m->id_base = in->id_base; m->id_stride = in->id_stride;
  const int rows_per_chunk = in->chunk_size / in->q_group_size > 0 ? in->chunk_size / in->q_group_size : 1;
  m->q_half = in->tf_mask ? MG / (2 * rows_per_chunk) : 0;
  m->k_half = in->tf_mask ? static_cast<int>((NC_global * in->block_size) / (2 * static_cast<int64_t>(in->chunk_size_k))) : 0;
  return NSA_OK;
}

// The mask of a call over NC local columns.  The teacher-forcing layout splits the GLOBAL key
// blocks into a clean and a noisy half; a shard (id_stride > 1) does not know the global count
// (ragged shards would disagree on it), so that combination is rejected.
int fill_mask_checked(const nsa_topk_mask* in, int MG, int64_t NC, Mask* m) {
  NSA_REQUIRE(in != nullptr, NSA_ERR_INVALID, "topk: mask is null");
  NSA_REQUIRE(!(in->tf_mask && in->id_stride > 1), NSA_ERR_UNSUPPORTED,
              "topk: tf_mask cannot be combined with block-sharded ids (id_stride > 1)");
  return fill_mask(in, MG, NC, m);
}

// Heads per thread block: whole rows when there are enough runs to fill the GPU, otherwise the heads
// are split over several blocks (down to 512-byte pieces) so that short tensors still spread out.
void plan_pool(PoolParams* p, int64_t NB, int B, int esz) {
  int hc = p->H;
  const int min_hc = (512 + p->D * esz - 1) / (p->D * esz);
  while (hc > min_hc && NB * B * cdiv(p->H, hc) < 2 * 148) hc = cdiv(hc, 2);
  p->hc = hc;
  p->hsplit = cdiv(p->H, hc);
}
inline int pool_threads(const PoolParams& p, int esz) {
  const int items = p.hc * (p.D * esz / 16);
  const int t = (items + 31) / 32 * 32;
  return t < 32 ? 32 : (t > 256 ? 256 : t);
}

template <typename T>
int launch_pool(const PoolParams& p, int B, int64_t NB, cudaStream_t s) {
  const int64_t units = NB * p.hsplit;
  NSA_REQUIRE(units <= 0x7fffffff, NSA_ERR_INVALID, "pool_rows: too many runs");
  NSA_CUDA_OK(launch_chained(kChainSmall, pool_rows_kernel<T>, dim3(static_cast<unsigned>(units), 1, B),
                             dim3(pool_threads(p, sizeof(T))), 0, s, p));
  NSA_LAUNCH_OK("pool_rows_kernel");
  return NSA_OK;
}

// Whether the bulk-copy pooling kernel can serve p (rows contiguous over the heads, at most 16 KiB
// each, 16-byte aligned), and how it would be launched.
bool bulk_plan(const PoolParams& p, int B, int esz, BulkPlan* plan) {
  const int64_t row_bytes = static_cast<int64_t>(p.H) * p.D * esz;
  if (p.x_sh != p.D || p.x_sn != static_cast<int64_t>(p.H) * p.D) return false;
  if (row_bytes % 16 != 0 || row_bytes > 16 * 1024 || !aligned16(p.x) || (p.x_sb * esz) % 16 != 0) return false;
  (void)B;
  int rows = static_cast<int>(kBulkStageBytes / row_bytes);
  if (rows < 1) rows = 1;
  if (rows > p.size) rows = p.size;
  const int items = static_cast<int>(row_bytes / 16);
  int threads = (items + 31) / 32 * 32;
  if (threads > 512) threads = ((items + 1) / 2 + 31) / 32 * 32;
  plan->rows_per_stage = rows;
  plan->threads = threads;
  plan->smem = static_cast<size_t>(kBulkStages) * rows * row_bytes;
  return true;
}

template <typename T>
int launch_pool_bulk(const PoolParams& a, const BulkPlan& pa, int64_t units_a, const PoolParams& b, const BulkPlan& pb,
                     int64_t units_b, int B, cudaStream_t s) {
  const size_t smem = pa.smem > pb.smem ? pa.smem : pb.smem;
  const int threads = pa.threads > pb.threads ? pa.threads : pb.threads;
  int32_t* status = nullptr;
  int rc;
  if ((rc = device_status_address(&status))) return rc;
  NSA_REQUIRE(units_a + units_b <= 0x7fffffff, NSA_ERR_INVALID, "pool_rows: too many runs");
  NSA_CUDA_OK(cudaFuncSetAttribute(pool_rows_bulk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  NSA_CUDA_OK(launch_chained(kChainSmall, pool_rows_bulk_kernel<T>, dim3(static_cast<unsigned>(units_a + units_b), 1, B),
                             dim3(threads), smem, s, a, b, units_a, pa.rows_per_stage, pb.rows_per_stage, status));
  NSA_LAUNCH_OK("pool_rows_bulk_kernel");
  return NSA_OK;
}

int check_rows16(const char* what, const void* ptr, const int64_t* stride, int esz) {
  NSA_REQUIRE(ptr != nullptr, NSA_ERR_INVALID, "%s: null pointer", what);
  NSA_REQUIRE(aligned16(ptr), NSA_ERR_LAYOUT, "%s: base address must be 16-byte aligned", what);
  for (int i = 0; i < 3; ++i)
    NSA_REQUIRE((stride[i] * esz) % 16 == 0, NSA_ERR_LAYOUT, "%s: stride %d is not a multiple of 16 bytes", what, i);
  return NSA_OK;
}

int run_score_select(const void* qp, const int64_t* qs, const void* kp, const int64_t* ks, int B,
                     int MG, int H, int D, int64_t NC, int topk, float scale, const Mask& m,
                     int32_t* out_idx, float* out_scores, float* scores, int dtype, cudaStream_t s,
                     void* seg_ws = nullptr, bool allow_fused = true) {
  ScoreParams sp{static_cast<const char*>(qp), qs[0], qs[1], qs[2], static_cast<const char*>(kp),
                 ks[0], ks[1], ks[2], scores, MG, H, D, NC, scale};
  const size_t smem = (static_cast<size_t>(kScoreCols) * (D + 1) + static_cast<size_t>(kScoreRows) * D) * sizeof(float);
  const dim3 grid(static_cast<unsigned>(cdiv64(NC, kScoreCols)), H, B);
  // 16-bit operands with 16-byte addressable rows go to the mma kernel
  const bool mma_ok = dtype != NSA_F32 && D % 16 == 0 && D <= 256 && static_cast<int64_t>(H) * B <= 65535 &&
                      aligned16(qp) && aligned16(kp) && (qs[0] * 2) % 16 == 0 && (qs[1] * 2) % 16 == 0 &&
                      (qs[2] * 2) % 16 == 0 && (ks[0] * 2) % 16 == 0 && (ks[1] * 2) % 16 == 0 && (ks[2] * 2) % 16 == 0;
  // rows short enough to keep their scores in shared memory: scoring and selection in ONE kernel
  if (allow_fused && mma_ok && D <= kFusedD && NC <= kFusedNC && topk <= kFusedTopk &&
      score_select_smem(D, NC) <= 220 * 1024 && H <= 65535 && B <= 65535) {
    ScoreSelectParams fp{};
    fp.sc = sp;
    fp.sel.NC = NC; fp.sel.MG = MG; fp.sel.H = H; fp.sel.topk = topk; fp.sel.out_idx = out_idx;
    fp.sel.out_scores = out_scores; fp.sel.mask = m;
    return dtype == NSA_BF16 ? launch_score_select<__nv_bfloat16>(fp, B, s) : launch_score_select<__half>(fp, B, s);
  }
  if (mma_ok) {
    const int rc = dtype == NSA_BF16 ? launch_score_mma<__nv_bfloat16>(sp, B, s) : launch_score_mma<__half>(sp, B, s);
    if (rc) return rc;
  } else if (dtype == NSA_BF16) {
    NSA_CUDA_OK(cudaFuncSetAttribute(score_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    score_kernel<__nv_bfloat16><<<grid, 256, smem, s>>>(sp);
  } else if (dtype == NSA_F16) {
    NSA_CUDA_OK(cudaFuncSetAttribute(score_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    score_kernel<__half><<<grid, 256, smem, s>>>(sp);
  } else {
    NSA_CUDA_OK(cudaFuncSetAttribute(score_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    score_kernel<float><<<grid, 256, smem, s>>>(sp);
  }
  NSA_LAUNCH_OK("score_kernel");
  SelectParams sel{};
  sel.scores = scores; sel.cand_ids = nullptr; sel.NC = NC; sel.MG = MG; sel.H = H;
  sel.seg_len = 0; sel.seg_stride = 0; sel.topk = topk; sel.out_idx = out_idx; sel.out_scores = out_scores;
  sel.mask = m;
  return launch_select<false>(sel, static_cast<int64_t>(B) * MG * H, s, seg_ws);
}

__global__ void fill_empty_kernel(int32_t* __restrict__ out_idx, float* __restrict__ out_scores, int64_t n) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    out_idx[i] = -1;
    if (out_scores) out_scores[i] = -INFINITY;
  }
}

int fill_minus_one(int32_t* out_idx, float* out_scores, int64_t n, cudaStream_t s) {
  const int blocks = static_cast<int>(n / 256 + 1 < 1024 ? n / 256 + 1 : 1024);
  fill_empty_kernel<<<blocks, 256, 0, s>>>(out_idx, out_scores, n);
  NSA_LAUNCH_OK("fill_empty_kernel");
  return NSA_OK;
}

}  // namespace
}  // namespace nsa

using namespace nsa;

static int make_pool_params(const char* what, const void* x, const int64_t x_stride[3], void* out,
                            const int64_t out_stride[3], int32_t B, int64_t N, int32_t H, int32_t D, int32_t size,
                            int32_t dtype, PoolParams* p, int64_t* NB) {
  NSA_REQUIRE(B >= 0 && N >= 0 && H >= 0 && D > 0 && size > 0, NSA_ERR_INVALID, "%s: bad size", what);
  NSA_REQUIRE(dtype >= NSA_BF16 && dtype <= NSA_F32, NSA_ERR_UNSUPPORTED, "%s: unknown dtype %d", what, dtype);
  const int esz = dtype_size(dtype);
  NSA_REQUIRE((D * esz) % 16 == 0 && D * esz / 16 <= 128, NSA_ERR_UNSUPPORTED,
              "%s: head dim %d not supported (row must be a multiple of 16 bytes, <= 2 KiB)", what, D);
  *NB = cdiv64(N, size);
  if (B == 0 || N == 0 || H == 0) return NSA_OK;
  NSA_REQUIRE(B <= 65535 && H <= 65535, NSA_ERR_INVALID, "%s: B and H must be <= 65535", what);
  int rc;
  if ((rc = check_rows16(what, x, x_stride, esz))) return rc;
  NSA_REQUIRE(out != nullptr, NSA_ERR_INVALID, "%s: out is null", what);
  *p = PoolParams{static_cast<const char*>(x), x_stride[0], x_stride[1], x_stride[2],
                  static_cast<char*>(out), out_stride[0], out_stride[1], out_stride[2], N, D, size, H, H, 1, 0};
  p->vec_store = aligned16(out) && (out_stride[0] * esz) % 16 == 0 && (out_stride[1] * esz) % 16 == 0 &&
                 (out_stride[2] * esz) % 16 == 0;
  plan_pool(p, *NB, B, esz);
  return NSA_OK;
}

extern "C" int nsa_pool_rows(const void* x, const int64_t x_stride[3], void* out,
                             const int64_t out_stride[3], int32_t B, int64_t N, int32_t H, int32_t D,
                             int32_t size, int32_t dtype, void* stream) {
  PoolParams p{};
  int64_t NB = 0;
  int rc;
  if ((rc = make_pool_params("pool_rows x", x, x_stride, out, out_stride, B, N, H, D, size, dtype, &p, &NB))) return rc;
  if (B == 0 || N == 0 || H == 0) return NSA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  BulkPlan plan;
  if (bulk_plan(p, B, dtype_size(dtype), &plan)) {
    if (dtype == NSA_BF16) return launch_pool_bulk<__nv_bfloat16>(p, plan, NB, p, plan, 0, B, s);
    if (dtype == NSA_F16) return launch_pool_bulk<__half>(p, plan, NB, p, plan, 0, B, s);
    return launch_pool_bulk<float>(p, plan, NB, p, plan, 0, B, s);
  }
  if (dtype == NSA_BF16) return launch_pool<__nv_bfloat16>(p, B, NB, s);
  if (dtype == NSA_F16) return launch_pool<__half>(p, B, NB, s);
  return launch_pool<float>(p, B, NB, s);
}

// scores [B,H,MG,NC] fp32, then (rows longer than 1024 columns) the per-segment candidate lists
static size_t score_bytes(int32_t B, int32_t MG, int32_t H, int64_t NC) {
  return align_up(static_cast<size_t>(B) * MG * H * NC * sizeof(float), 256);
}
extern "C" size_t nsa_topk_workspace_bytes(int32_t B, int32_t MG, int32_t H, int64_t NC) {
  return score_bytes(B, MG, H, NC) + segment_workspace_bytes(static_cast<int64_t>(B) * MG * H, NC);
}

static int topk_common_checks(int32_t B, int32_t MG, int32_t H, int32_t D, int64_t NC, int32_t topk,
                              int32_t dtype, const int32_t* out_idx) {
  NSA_REQUIRE(B >= 0 && MG >= 0 && H >= 0 && NC >= 0, NSA_ERR_INVALID, "topk: negative size");
  NSA_REQUIRE(D >= 1 && D <= 256, NSA_ERR_INVALID, "topk: head dim must be in [1, 256], got %d", D);
  NSA_REQUIRE(topk >= 1, NSA_ERR_INVALID, "topk: topk must be >= 1, got %d", topk);
  NSA_REQUIRE(dtype >= NSA_BF16 && dtype <= NSA_F32, NSA_ERR_UNSUPPORTED, "topk: unknown dtype %d", dtype);
  NSA_REQUIRE(static_cast<int64_t>(B) <= 65535 && H <= 65535, NSA_ERR_INVALID, "topk: B and H must be <= 65535");
  NSA_REQUIRE(static_cast<int64_t>(B) * MG * H <= 0x7fffffff, NSA_ERR_INVALID, "topk: too many rows");
  NSA_REQUIRE(out_idx != nullptr || static_cast<int64_t>(B) * MG * H == 0, NSA_ERR_INVALID, "topk: out_idx is null");
  return NSA_OK;
}

extern "C" int nsa_topk(const void* q_pooled, const int64_t q_stride[3], const void* k_pooled,
                        const int64_t k_stride[3], int32_t B, int32_t MG, int32_t H, int32_t D,
                        int64_t NC, int32_t topk, float scale, const nsa_topk_mask* mask,
                        int32_t* out_idx, float* out_scores, void* workspace, size_t workspace_bytes,
                        int32_t dtype, void* stream) {
  int rc;
  if ((rc = topk_common_checks(B, MG, H, D, NC, topk, dtype, out_idx))) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t rows = static_cast<int64_t>(B) * MG * H;
  if (rows == 0) return NSA_OK;
  if (NC == 0) return fill_minus_one(out_idx, out_scores, rows * topk, s);
  NSA_REQUIRE(q_pooled && k_pooled, NSA_ERR_INVALID, "topk: null pointer");
  NSA_REQUIRE(workspace && workspace_bytes >= nsa_topk_workspace_bytes(B, MG, H, NC), NSA_ERR_WORKSPACE,
              "topk: workspace too small");
  Mask m;
  if ((rc = fill_mask_checked(mask, MG, NC, &m))) return rc;
  void* seg_ws = NC > kSegCols ? static_cast<char*>(workspace) + score_bytes(B, MG, H, NC) : nullptr;
  return run_score_select(q_pooled, q_stride, k_pooled, k_stride, B, MG, H, D, NC, topk, scale, m,
                          out_idx, out_scores, static_cast<float*>(workspace), dtype, s, seg_ws);
}

// Pooling of the raw keys, then scoring + selection (one kernel when a row's scores fit shared memory).
extern "C" int nsa_pool_score_topk(const void* q_pooled, const int64_t q_stride[3], const void* k,
                                   const int64_t k_stride[3], int32_t B, int32_t MG, int32_t H,
                                   int32_t D, int64_t N, int32_t topk, float scale,
                                   const nsa_topk_mask* mask, void* k_pooled_out, int32_t* out_idx,
                                   float* out_scores, void* workspace, size_t workspace_bytes,
                                   int32_t dtype, void* stream) {
  NSA_REQUIRE(mask != nullptr && mask->block_size > 0, NSA_ERR_INVALID, "pool_score_topk: mask / block_size");
  NSA_REQUIRE(N >= 0, NSA_ERR_INVALID, "pool_score_topk: N < 0");
  const int64_t NC = cdiv64(N, mask->block_size);
  int rc;
  if ((rc = topk_common_checks(B, MG, H, D, NC, topk, dtype, out_idx))) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t rows = static_cast<int64_t>(B) * MG * H;
  if (rows == 0 && (NC == 0 || !k_pooled_out)) return NSA_OK;
  NSA_REQUIRE(k_pooled_out != nullptr, NSA_ERR_INVALID, "pool_score_topk: k_pooled_out is null");
  const int64_t ps[3] = {NC * H * D, static_cast<int64_t>(H) * D, D};
  if (NC > 0) {
    if ((rc = nsa_pool_rows(k, k_stride, k_pooled_out, ps, B, N, H, D, mask->block_size, dtype, stream))) return rc;
  }
  if (rows == 0) return NSA_OK;
  if (NC == 0) return fill_minus_one(out_idx, out_scores, rows * topk, s);
  return nsa_topk(q_pooled, q_stride, k_pooled_out, ps, B, MG, H, D, NC, topk, scale, mask, out_idx,
                  out_scores, workspace, workspace_bytes, dtype, stream);
}

extern "C" int nsa_select_blocks(const void* q, const int64_t q_stride[3], const void* k,
                                 const int64_t k_stride[3], int32_t B, int64_t M, int32_t H, int32_t D,
                                 int64_t N, int32_t topk, float scale, const nsa_topk_mask* mask,
                                 void* q_pooled_out, void* k_pooled_out, int32_t* out_idx, float* out_scores,
                                 void* workspace, size_t workspace_bytes, int32_t dtype, void* stream) {
  NSA_REQUIRE(mask != nullptr && mask->q_group_size > 0 && mask->block_size > 0, NSA_ERR_INVALID,
              "select_blocks: mask / q_group_size / block_size");
  NSA_REQUIRE(M >= 0 && N >= 0 && cdiv64(M, mask->q_group_size) <= 0x7fffffff, NSA_ERR_INVALID, "select_blocks: bad M / N");
  const int32_t MG = static_cast<int32_t>(cdiv64(M, mask->q_group_size));
  const int64_t NC = cdiv64(N, mask->block_size);
  const int64_t qs[3] = {static_cast<int64_t>(MG) * H * D, static_cast<int64_t>(H) * D, D};
  const int64_t ps[3] = {NC * H * D, static_cast<int64_t>(H) * D, D};
  int rc;
  if ((rc = topk_common_checks(B, MG, H, D, NC, topk, dtype, out_idx))) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // both poolings in ONE launch: neither depends on the other
  PoolParams pq{}, pk{};
  int64_t nbq = 0, nbk = 0;
  const bool have_q = B > 0 && M > 0 && H > 0, have_k = B > 0 && N > 0 && H > 0;
  NSA_REQUIRE(!have_q || q_pooled_out, NSA_ERR_INVALID, "select_blocks: q_pooled_out is null");
  NSA_REQUIRE(!have_k || k_pooled_out, NSA_ERR_INVALID, "select_blocks: k_pooled_out is null");
  if (have_q && (rc = make_pool_params("select_blocks q", q, q_stride, q_pooled_out, qs, B, M, H, D, mask->q_group_size, dtype, &pq, &nbq))) return rc;
  if (have_k && (rc = make_pool_params("select_blocks k", k, k_stride, k_pooled_out, ps, B, N, H, D, mask->block_size, dtype, &pk, &nbk))) return rc;
  BulkPlan bq, bk;
  if (have_q && have_k && bulk_plan(pq, B, dtype_size(dtype), &bq) && bulk_plan(pk, B, dtype_size(dtype), &bk)) {
    // the long tensor first: its thread blocks fill the GPU while the short one's trail behind
    if (dtype == NSA_BF16) rc = launch_pool_bulk<__nv_bfloat16>(pk, bk, nbk, pq, bq, nbq, B, s);
    else if (dtype == NSA_F16) rc = launch_pool_bulk<__half>(pk, bk, nbk, pq, bq, nbq, B, s);
    else rc = launch_pool_bulk<float>(pk, bk, nbk, pq, bq, nbq, B, s);
    if (rc) return rc;
  } else if (have_q && have_k) {
    const int64_t ua = nbq * pq.hsplit, ub = nbk * pk.hsplit;
    NSA_REQUIRE(ua + ub <= 0x7fffffff, NSA_ERR_INVALID, "select_blocks: too many runs");
    const int esz = dtype_size(dtype);
    const int threads = pool_threads(pq, esz) > pool_threads(pk, esz) ? pool_threads(pq, esz) : pool_threads(pk, esz);
    const dim3 grid(static_cast<unsigned>(ua + ub), 1, B);
    if (dtype == NSA_BF16) NSA_CUDA_OK(launch_chained(kChainSmall, pool_rows_pair_kernel<__nv_bfloat16>, grid, dim3(threads), 0, s, pq, pk, ua));
    else if (dtype == NSA_F16) NSA_CUDA_OK(launch_chained(kChainSmall, pool_rows_pair_kernel<__half>, grid, dim3(threads), 0, s, pq, pk, ua));
    else NSA_CUDA_OK(launch_chained(kChainSmall, pool_rows_pair_kernel<float>, grid, dim3(threads), 0, s, pq, pk, ua));
    NSA_LAUNCH_OK("pool_rows_pair_kernel");
  } else if (have_q) {
    if ((rc = nsa_pool_rows(q, q_stride, q_pooled_out, qs, B, M, H, D, mask->q_group_size, dtype, stream))) return rc;
  } else if (have_k) {
    if ((rc = nsa_pool_rows(k, k_stride, k_pooled_out, ps, B, N, H, D, mask->block_size, dtype, stream))) return rc;
  }
  const int64_t rows = static_cast<int64_t>(B) * MG * H;
  if (rows == 0) return NSA_OK;
  if (NC == 0) return fill_minus_one(out_idx, out_scores, rows * topk, s);
  return nsa_topk(q_pooled_out, qs, k_pooled_out, ps, B, MG, H, D, NC, topk, scale, mask, out_idx, out_scores,
                  workspace, workspace_bytes, dtype, stream);
}

extern "C" int nsa_merge_candidates(const int32_t* idx, const float* scores, int32_t R, int64_t rows,
                                    int32_t T, int32_t topk, int32_t* out_idx, float* out_scores,
                                    void* stream) {
  NSA_REQUIRE(R >= 1 && rows >= 0 && T >= 1 && topk >= 1, NSA_ERR_INVALID, "merge_candidates: bad size");
  NSA_REQUIRE(rows <= 0x7fffffff, NSA_ERR_INVALID, "merge_candidates: too many rows");
  if (rows == 0) return NSA_OK;
  NSA_REQUIRE(idx && scores && out_idx, NSA_ERR_INVALID, "merge_candidates: null pointer");
  SelectParams sel{};
  sel.scores = scores; sel.cand_ids = idx; sel.NC = static_cast<int64_t>(R) * T; sel.MG = 1; sel.H = 1;
  sel.seg_len = T; sel.seg_stride = rows * T; sel.topk = topk; sel.out_idx = out_idx; sel.out_scores = out_scores;
  return launch_select<true>(sel, rows, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// Top-k for callers that must not allocate.
//
// nsa_topk needs a score buffer of B*MG*H*NC floats and asks its caller to supply it.  Some
// callers cannot: a serving process that hands the whole device to another allocator at start-up
// (a later cudaMalloc would fail or fragment its plan), a host runtime behind an FFI boundary that
// owns no device memory at all and only forwards pointers it was given, or a latency-critical loop
// whose memory plan is frozen once it starts.  For them the library carries its own score buffer:
// a fixed array in device global memory that is part of the loaded module, so it exists on every
// GPU that loads the library, from load until the process exits, and costs kStaticScratchBytes
// there whether or not this entry point is ever called.
namespace nsa {
constexpr size_t kStaticScratchFloats = static_cast<size_t>(1) << 20;          // 4 MiB
constexpr size_t kStaticScratchBytes = kStaticScratchFloats * sizeof(float);
static __device__ __align__(256) float g_topk_scratch[kStaticScratchFloats];

namespace {
// In host code `g_topk_scratch` is only a handle for the runtime, not an address a kernel can
// use; the device address is looked up once per device (with that device current) and cached.
int static_scratch_address(float** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static float* cached[kMaxDevices] = {};
  int dev = -1;
  NSA_CUDA_OK(cudaGetDevice(&dev));
  NSA_REQUIRE(dev >= 0 && dev < kMaxDevices, NSA_ERR_UNSUPPORTED, "topk_static_scratch: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    NSA_CUDA_OK(cudaGetSymbolAddress(&p, g_topk_scratch));
    NSA_REQUIRE(p != nullptr, NSA_ERR_CUDA, "topk_static_scratch: the scratch array has no device address");
    cached[dev] = static_cast<float*>(p);
  }
  *out = cached[dev];
  return NSA_OK;
}
}  // namespace
}  // namespace nsa

#ifdef NSA_SS_TRACE
extern "C" int nsa_debug_trace_ss(long long* out) {
  NSA_CUDA_OK(cudaMemcpyFromSymbol(out, nsa::g_trace_ss, sizeof(long long) * 16));
  return NSA_OK;
}
#endif

extern "C" size_t nsa_topk_static_scratch_max_scores(void) { return nsa::kStaticScratchFloats; }

extern "C" int nsa_topk_static_scratch(const void* q_pooled, const int64_t q_stride[3], const void* k_pooled,
                                       const int64_t k_stride[3], int32_t B, int32_t MG, int32_t H, int32_t D,
                                       int64_t NC, int32_t topk, float scale, const nsa_topk_mask* mask,
                                       int32_t* out_idx, float* out_scores, int32_t dtype, void* stream) {
  int rc;
  if ((rc = topk_common_checks(B, MG, H, D, NC, topk, dtype, out_idx))) return rc;
  const int64_t rows = static_cast<int64_t>(B) * MG * H;
  const int64_t need = rows * NC;
  NSA_REQUIRE(need <= static_cast<int64_t>(nsa::kStaticScratchFloats), NSA_ERR_WORKSPACE,
              "topk_static_scratch: B*MG*H*NC = %lld scores exceed the built-in scratch of %zu scores (%zu MiB); "
              "use nsa_topk with a caller-provided workspace for this size",
              static_cast<long long>(need), nsa::kStaticScratchFloats, nsa::kStaticScratchBytes >> 20);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) return NSA_OK;
  if (NC == 0) return fill_minus_one(out_idx, out_scores, rows * topk, s);
  NSA_REQUIRE(q_pooled && k_pooled, NSA_ERR_INVALID, "topk_static_scratch: null pointer");
  Mask m;
  if ((rc = fill_mask_checked(mask, MG, NC, &m))) return rc;
  float* scratch = nullptr;
  if ((rc = nsa::static_scratch_address(&scratch))) return rc;
  // Every score the selection reads is written by the scoring kernel of the same call, so nothing
  // in the array has to start at zero and whatever an earlier call left behind is never read.
  return run_score_select(q_pooled, q_stride, k_pooled, k_stride, B, MG, H, D, NC, topk, scale, m, out_idx,
                          out_scores, scratch, dtype, s, nullptr, /*allow_fused=*/false);
}
