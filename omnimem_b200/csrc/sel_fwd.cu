// Selection attention forward, general geometry (any block size, group size <= 128,
// D in {64, 128}, bf16 / fp16): one thread block per (batch, query group, head); each warp
// owns 16 query rows; selected tokens are packed into 64-row K/V tiles that stream through a
// two-stage cp.async ring; S = Q K^T and O += P V run on mma.sync m16n8k16 with fp32
// accumulation and an online softmax in the exp2 domain.
#include "sel_common.cuh"

namespace nsa {
namespace {

struct FwdParams {
  const char* q;
  int64_t q_sb, q_sm, q_sh;
  char* out;
  int64_t o_sb, o_sm, o_sh;
  float* lse;               // [B,H,M]
  const int32_t* ids;
  int64_t i_sb, i_sg, i_sh, i_st;
  KVSrc kv;
  int B, H, T, block_size, chunk_size, causal, G;
  int64_t M;
  float scale_log2;
};

template <typename T, int D>
__global__ void __launch_bounds__(256) sel_fwd_kernel(const FwdParams p) {
  constexpr int PITCH = D + 8;
  constexpr int ESZ = sizeof(T);
  constexpr int KK = D / 16;     // k-steps of S = Q K^T
  constexpr int DN = D / 8;      // n8 tiles of O
  extern __shared__ __align__(16) char smem[];

  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, t4 = lane & 3;
  const int64_t m0 = static_cast<int64_t>(g) * p.G;
  const int n_q = static_cast<int>(p.M - m0 < p.G ? p.M - m0 : p.G);
  const int q_chunk = static_cast<int>(m0 / p.chunk_size);

  T* tiles = reinterpret_cast<T*>(smem);                       // [2][2][64][PITCH]
  const SlotTable st = carve_slot_table(smem + 4 * kTileRows * PITCH * ESZ, p.T);
  auto stageK = [&](int s) { return tiles + (s * 2) * kTileRows * PITCH; };
  auto stageV = [&](int s) { return tiles + (s * 2 + 1) * kTileRows * PITCH; };

  const int total = build_slot_table<ESZ>(st, p.kv, p.ids, b * p.i_sb + g * p.i_sg + h * p.i_sh, p.i_st,
                                          p.T, b, h, D, p.block_size, p.chunk_size, p.causal != 0, q_chunk);

  char* out_row0 = p.out + (b * p.o_sb + m0 * p.o_sm + h * p.o_sh) * ESZ;
  float* lse_row0 = p.lse + (static_cast<int64_t>(b) * p.H + h) * p.M + m0;
  if (total == 0) {  // no visible key: O = 0, LSE = -inf
    for (int i = threadIdx.x; i < n_q * (D / 8); i += blockDim.x) {
      const int r = i / (D / 8), c = i % (D / 8);
      *reinterpret_cast<uint4*>(out_row0 + r * p.o_sm * ESZ + c * 16) = make_uint4(0, 0, 0, 0);
    }
    for (int r = threadIdx.x; r < n_q; r += blockDim.x) lse_row0[r] = -INFINITY;
    return;
  }

  const int64_t k_row_bytes = kv_row_bytes(p.kv, false, D, ESZ);
  const int64_t v_row_bytes = kv_row_bytes(p.kv, true, D, ESZ);
  const char* q_base = p.q + (b * p.q_sb + m0 * p.q_sm + h * p.q_sh) * ESZ;
  const int ntiles = (total + kTileRows - 1) / kTileRows;
  const int rows_pad = (blockDim.x >> 5) * 16;

  // Q goes through stage 1 (128 rows) while tile 0 lands in stage 0.
  issue_rows<T, D, PITCH>(stageK(1), q_base, p.q_sm * ESZ, n_q, rows_pad);
  cp_async_commit();
  issue_kv_tile<T, D, PITCH>(stageK(0), stageV(0), st, p.T, 0, total, k_row_bytes, v_row_bytes, p.q);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  uint32_t qf[KK][4];
  {
    const T* sQ = stageK(1) + (warp * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) ldmatrix_x4(qf[kk], sQ + kk * 16);
  }
  __syncthreads();

  float o[DN][4];
#pragma unroll
  for (int n = 0; n < DN; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m_i[2] = {-INFINITY, -INFINITY};
  float l_i[2] = {0.f, 0.f};
  const bool warp_active = warp * 16 < n_q;

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
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
      const T* kb = sK + ((lane & 7) + ((lane >> 4) << 3)) * PITCH + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
        for (int n16 = 0; n16 < 4; ++n16) {
          if (n16 * 16 < nvalid) {
            uint32_t bf[4];
            ldmatrix_x4(bf, kb + n16 * 16 * PITCH + kk * 16);
            mma16816<T>(s[2 * n16], qf[kk], bf[0], bf[1]);
            mma16816<T>(s[2 * n16 + 1], qf[kk], bf[2], bf[3]);
          }
        }
      }
      // mask + online softmax (rows gid and gid + 8), exp2 domain
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = n * 8 + 2 * t4 + (e & 1);
          const float v = (col < nvalid) ? s[n][e] * p.scale_log2 : -INFINITY;
          s[n][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_i[r], mx[r]);   // finite: every tile has a valid column
        const float corr = fast_exp2(m_i[r] - m_new);
        m_i[r] = m_new;
        l_i[r] *= corr;
#pragma unroll
        for (int n = 0; n < DN; ++n) { o[n][2 * r] *= corr; o[n][2 * r + 1] *= corr; }
      }
      uint32_t pa[4][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const float p0 = fast_exp2(s[n][0] - m_i[0]);
        const float p1 = fast_exp2(s[n][1] - m_i[0]);
        const float p2 = fast_exp2(s[n][2] - m_i[1]);
        const float p3 = fast_exp2(s[n][3] - m_i[1]);
        l_i[0] += p0 + p1;
        l_i[1] += p2 + p3;
        pa[n >> 1][(n & 1) * 2] = pack2<T>(p0, p1);
        pa[n >> 1][(n & 1) * 2 + 1] = pack2<T>(p2, p3);
      }
      const T* vb = sV + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (lane >> 4) * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j * 16 < nvalid) {
#pragma unroll
          for (int d16 = 0; d16 < D / 16; ++d16) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, vb + j * 16 * PITCH + d16 * 16);
            mma16816<T>(o[2 * d16], pa[j], bf[0], bf[1]);
            mma16816<T>(o[2 * d16 + 1], pa[j], bf[2], bf[3]);
          }
        }
      }
    }
    __syncthreads();
  }

  if (warp_active) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
      l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
      const int row = warp * 16 + gid + 8 * r;
      if (row < n_q) {
        const float inv = l_i[r] > 0.f ? 1.f / l_i[r] : 0.f;
        char* orow = out_row0 + row * p.o_sm * ESZ;
#pragma unroll
        for (int n = 0; n < DN; ++n)
          *reinterpret_cast<uint32_t*>(orow + (n * 8 + 2 * t4) * ESZ) =
              pack2<T>(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
        if (t4 == 0)
          lse_row0[row] = l_i[r] > 0.f ? (m_i[r] + log2f(l_i[r])) * kLn2 : -INFINITY;
      }
    }
  }
}

template <typename T, int D>
int launch(const FwdParams& p, int MG, cudaStream_t stream) {
  const int nw = cdiv(p.G, 16);
  const size_t smem = 4 * kTileRows * (D + 8) * sizeof(T) + slot_table_bytes(p.T);
  NSA_REQUIRE(smem <= 200 * 1024, NSA_ERR_UNSUPPORTED, "sel_fwd: T=%d needs too much shared memory", p.T);
  NSA_CUDA_OK(cudaFuncSetAttribute(sel_fwd_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(smem)));
  dim3 grid(MG, p.H, p.B);
  sel_fwd_kernel<T, D><<<grid, nw * 32, smem, stream>>>(p);
  NSA_LAUNCH_OK("sel_fwd_kernel");
  return NSA_OK;
}

}  // namespace

int try_launch_sel_fwd_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, const int32_t* ids,
                          const int64_t* idx_stride, void* out, const int64_t* out_stride, float* lse, int B,
                          int64_t M, int H, int D, int T, int block_size, int chunk_size, int causal, int G,
                          float scale, int dtype, int32_t* status, cudaStream_t stream, bool* launched);

int try_launch_sel_range_fwd_tc(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int first_block,
                                int n_blocks, void* out, const int64_t* out_stride, float* lse, int B, int64_t M,
                                int H, int D, int block_size, float scale, int dtype, int splits,
                                cudaStream_t stream, bool* launched);
int range_fwd_splits(int B, int64_t M, int H, int n_blocks);

int check_strides16(const char* what, const void* ptr, const int64_t* stride, int n, int esz) {
  NSA_REQUIRE(ptr != nullptr, NSA_ERR_INVALID, "%s: null pointer", what);
  NSA_REQUIRE(aligned16(ptr), NSA_ERR_LAYOUT, "%s: base address must be 16-byte aligned", what);
  for (int i = 0; i < n; ++i)
    NSA_REQUIRE((stride[i] * esz) % 16 == 0, NSA_ERR_LAYOUT,
                "%s: stride %d (%lld elements) is not a multiple of 16 bytes", what, i,
                static_cast<long long>(stride[i]));
  return NSA_OK;
}

int make_kvsrc(const nsa_kv_source* in, int D, int esz, int block_size, KVSrc* out) {
  NSA_REQUIRE(in != nullptr, NSA_ERR_INVALID, "kv source is null");
  NSA_REQUIRE(in->mode == NSA_KV_DENSE || in->mode == NSA_KV_PAGED || in->mode == NSA_KV_PTR, NSA_ERR_INVALID,
              "kv source: unknown mode %d", in->mode);
  NSA_REQUIRE(in->n_tokens >= 0, NSA_ERR_INVALID, "kv source: n_tokens < 0");
  out->mode = in->mode;
  out->k = static_cast<const char*>(in->k);
  out->v = static_cast<const char*>(in->v);
  out->n_tokens = in->n_tokens;
  out->block_table = in->block_table;
  out->max_blocks = in->max_blocks;
  out->page_tokens = in->page_tokens;
  out->ptr_k = in->ptr_k; out->ptr_v = in->ptr_v; out->ptr_sn = in->ptr_stride_n;
  out->k_sb = in->k_stride[0]; out->k_sn = in->k_stride[1]; out->k_sh = in->k_stride[2];
  out->v_sb = in->v_stride[0]; out->v_sn = in->v_stride[1]; out->v_sh = in->v_stride[2];
  if (in->mode == NSA_KV_PTR) {
    NSA_REQUIRE(in->ptr_k && in->ptr_v, NSA_ERR_INVALID, "pointer kv source: null table");
    NSA_REQUIRE((in->ptr_stride_n * esz) % 16 == 0 && in->ptr_stride_n >= D, NSA_ERR_LAYOUT,
                "pointer kv source: token stride must be >= D and a multiple of 16 bytes");
    return NSA_OK;
  }
  if (in->n_tokens == 0) return NSA_OK;
  if (in->mode == NSA_KV_DENSE) {
    int rc = check_strides16("k", in->k, in->k_stride, 3, esz);
    if (rc) return rc;
    rc = check_strides16("v", in->v, in->v_stride, 3, esz);
    if (rc) return rc;
  } else {
    NSA_REQUIRE(in->k && in->v && in->block_table, NSA_ERR_INVALID, "paged kv source: null pointer");
    NSA_REQUIRE(aligned16(in->k) && aligned16(in->v), NSA_ERR_LAYOUT, "page pools must be 16-byte aligned");
    NSA_REQUIRE(in->page_tokens == block_size, NSA_ERR_INVALID,
                "paged kv source: block_size (%d) must equal page_tokens (%d)", block_size, in->page_tokens);
    NSA_REQUIRE(in->max_blocks > 0, NSA_ERR_INVALID, "paged kv source: max_blocks must be > 0");
    NSA_REQUIRE((static_cast<int64_t>(D) * esz) % 16 == 0, NSA_ERR_LAYOUT, "page rows must be 16-byte multiples");
  }
  return NSA_OK;
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_sel_fwd(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                           const int32_t* block_indices, const int64_t idx_stride[4], void* out,
                           const int64_t out_stride[3], float* lse, int32_t B, int64_t M, int32_t H,
                           int32_t D, int32_t T, int32_t block_size, int32_t chunk_size,
                           int32_t causal, int32_t group_size, float scale, int32_t dtype,
                           void* stream) {
  NSA_REQUIRE(B >= 0 && M >= 0 && H >= 0, NSA_ERR_INVALID, "sel_fwd: negative size");
  NSA_REQUIRE(group_size >= 1 && group_size <= 128, NSA_ERR_INVALID,
              "sel_fwd: group_size must be in [1,128], got %d", group_size);
  NSA_REQUIRE(block_size > 0 && chunk_size > 0, NSA_ERR_INVALID, "sel_fwd: block_size and chunk_size must be > 0");
  NSA_REQUIRE(T > 0, NSA_ERR_INVALID, "sel_fwd: T must be > 0");
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_F16, NSA_ERR_UNSUPPORTED,
              "sel_fwd: only bf16 and fp16 are built (dtype %d)", dtype);
  NSA_REQUIRE(D == 64 || D == 128, NSA_ERR_UNSUPPORTED, "sel_fwd: head dim %d not built (64, 128)", D);
  if (B == 0 || M == 0 || H == 0) return NSA_OK;
  NSA_REQUIRE(static_cast<int64_t>(B) <= 65535 && H <= 65535, NSA_ERR_INVALID, "sel_fwd: B and H must be <= 65535");
  NSA_REQUIRE(kv && (kv->mode == NSA_KV_DENSE || B == 1), NSA_ERR_INVALID, "sel_fwd: paged K/V needs B == 1");
  NSA_REQUIRE((block_indices || kv->mode == NSA_KV_PTR) && lse, NSA_ERR_INVALID, "sel_fwd: null pointer");
  const int esz = 2;
  int rc = check_strides16("q", q, q_stride, 3, esz);
  if (rc) return rc;
  rc = check_strides16("out", out, out_stride, 3, esz);
  if (rc) return rc;
  FwdParams p;
  rc = make_kvsrc(kv, D, esz, block_size, &p.kv);
  if (rc) return rc;
  p.q = static_cast<const char*>(q);
  p.q_sb = q_stride[0]; p.q_sm = q_stride[1]; p.q_sh = q_stride[2];
  p.out = static_cast<char*>(out);
  p.o_sb = out_stride[0]; p.o_sm = out_stride[1]; p.o_sh = out_stride[2];
  p.lse = lse;
  p.ids = block_indices;
  p.i_sb = idx_stride[0]; p.i_sg = idx_stride[1]; p.i_sh = idx_stride[2]; p.i_st = idx_stride[3];
  p.B = B; p.H = H; p.T = T; p.block_size = block_size; p.chunk_size = chunk_size;
  p.causal = causal; p.G = group_size; p.M = M;
  p.scale_log2 = scale * kLog2e;
  const int64_t MG = cdiv64(M, group_size);
  NSA_REQUIRE(MG <= 0x7fffffff, NSA_ERR_INVALID, "sel_fwd: too many query groups");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    // the page geometry runs on the tcgen05 kernel; every other shape on the general one
    bool launched = false;
    rc = try_launch_sel_fwd_tc(q, q_stride, kv, block_indices, idx_stride, out, out_stride, lse, B, M, H, D, T,
                               block_size, chunk_size, causal, group_size, scale, dtype, nullptr, s, &launched);
    if (rc) return rc;
    if (launched) return NSA_OK;
  }
  if (dtype == NSA_BF16) {
    return D == 128 ? launch<__nv_bfloat16, 128>(p, static_cast<int>(MG), s)
                    : launch<__nv_bfloat16, 64>(p, static_cast<int>(MG), s);
  }
  return D == 128 ? launch<__half, 128>(p, static_cast<int>(MG), s)
                  : launch<__half, 64>(p, static_cast<int>(MG), s);
}

extern "C" size_t nsa_range_fwd_workspace_bytes(int32_t B, int64_t M, int32_t H, int32_t D, int32_t n_blocks) {
  if (B <= 0 || M <= 0 || H <= 0 || D <= 0 || n_blocks <= 0) return 0;
  const int splits = nsa::range_fwd_splits(B, M, H, n_blocks);
  if (splits == 1) return 0;
  const size_t outs = static_cast<size_t>(splits) * B * M * H * D * 2;
  return ((outs + 255) & ~static_cast<size_t>(255)) + static_cast<size_t>(splits) * B * H * M * 4;
}

extern "C" int nsa_range_fwd(const void* q, const int64_t* q_stride, const nsa_kv_source* kv, int32_t first_block,
                             int32_t n_blocks, void* out, const int64_t* out_stride, float* lse, int32_t B,
                             int64_t M, int32_t H, int32_t D, int32_t block_size, float scale, void* workspace,
                             size_t workspace_bytes, int32_t dtype, void* stream) {
  using namespace nsa;
  NSA_REQUIRE(q && kv && out && lse && q_stride && out_stride, NSA_ERR_INVALID, "range_fwd: null pointer");
  NSA_REQUIRE(first_block >= 0 && n_blocks >= 0, NSA_ERR_INVALID, "range_fwd: first_block %d, n_blocks %d",
              first_block, n_blocks);
  if (B == 0 || M == 0 || H == 0) return NSA_OK;
  NSA_REQUIRE(static_cast<int64_t>(B) <= 65535 && H <= 65535, NSA_ERR_INVALID, "range_fwd: B and H must be <= 65535");
  NSA_REQUIRE(kv->mode == NSA_KV_DENSE || B == 1, NSA_ERR_INVALID, "range_fwd: paged K/V needs B == 1");
  int rc = check_strides16("q", q, q_stride, 3, 2);
  if (rc) return rc;
  rc = check_strides16("out", out, out_stride, 3, 2);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // spans of the range on thread blocks of their own, when that fills the machine better and the
  // caller gave the room for their partial results (the merged output is written contiguous)
  int splits = n_blocks > 0 ? range_fwd_splits(B, M, H, n_blocks) : 1;
  const size_t outs_bytes = (static_cast<size_t>(splits) * B * M * H * D * 2 + 255) & ~static_cast<size_t>(255);
  const bool contiguous = out_stride[2] == D && out_stride[1] == static_cast<int64_t>(H) * D &&
                          (B == 1 || out_stride[0] == M * H * D);
  if (splits > 1 && (workspace == nullptr || !aligned16(workspace) || !contiguous || B * splits > 65535 ||
                     workspace_bytes < outs_bytes + static_cast<size_t>(splits) * B * H * M * 4))
    splits = 1;
  bool launched = false;
  if (splits > 1) {
    char* part_out = static_cast<char*>(workspace);
    float* part_lse = reinterpret_cast<float*>(part_out + outs_bytes);
    const int64_t part_stride[3] = {M * H * D, static_cast<int64_t>(H) * D, D};
    rc = try_launch_sel_range_fwd_tc(q, q_stride, kv, first_block, n_blocks, part_out, part_stride, part_lse, B, M, H,
                                     D, block_size, scale, dtype, splits, s, &launched);
    if (rc) return rc;
    if (launched) return nsa_merge_partials(part_out, part_lse, splits, B, M, H, D, out, lse, dtype, stream);
  }
  rc = try_launch_sel_range_fwd_tc(q, q_stride, kv, first_block, n_blocks, out, out_stride, lse, B, M, H, D,
                                   block_size, scale, dtype, 1, s, &launched);
  if (rc) return rc;
  NSA_REQUIRE(launched, NSA_ERR_UNSUPPORTED,
              "range_fwd: built for bf16, D = 128, 64-token blocks, H > 1, dense or paged K/V, at most 1024 blocks; "
              "list the blocks and call nsa_sel_fwd for anything else");
  return NSA_OK;
}
