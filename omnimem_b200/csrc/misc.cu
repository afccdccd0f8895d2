// Small kernels around the selection path: exact merge of attention partials computed over
// disjoint key sets (block-sharded KV) and the block id -> byte address table.
#include "common.cuh"

namespace nsa {
namespace {

constexpr int kMaxParts = 16;

// One thread per 16-byte chunk (8 elements) of an output row.
template <typename T>
__global__ void merge_partials_kernel(const char* __restrict__ outs, const float* __restrict__ lses,
                                      int R, int B, int64_t M, int H, int D, char* __restrict__ out,
                                      float* __restrict__ lse) {
  const int cpr = D / 8;
  const int64_t total = static_cast<int64_t>(B) * M * H * cpr;
  const int64_t part_elems = static_cast<int64_t>(B) * M * H * D;
  const int64_t part_rows = static_cast<int64_t>(B) * H * M;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % cpr);
    const int64_t row = i / cpr;                 // (b*M + m)*H + h
    const int h = static_cast<int>(row % H);
    const int64_t bm = row / H;
    const int64_t m = bm % M, b = bm / M;
    const int64_t lrow = (b * H + h) * M + m;
    float w[kMaxParts];
    float mx = -INFINITY;
    for (int r = 0; r < R; ++r) { w[r] = lses[r * part_rows + lrow]; mx = fmaxf(mx, w[r]); }
    float den = 0.f;
    for (int r = 0; r < R; ++r) { w[r] = (w[r] == -INFINITY) ? 0.f : __expf(w[r] - mx); den += w[r]; }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int r = 0; r < R; ++r) {
      if (w[r] == 0.f) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(outs + (r * part_elems + row * D) * sizeof(T) + cc * 16);
      const T* e8 = reinterpret_cast<const T*>(&v);
      const float wr = w[r] * inv;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += wr * to_f32<T>(e8[e]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < 8; ++e) oe[e] = from_f32<T>(acc[e]);
    *reinterpret_cast<uint4*>(out + row * D * sizeof(T) + cc * 16) = o;
    if (cc == 0) lse[lrow] = den > 0.f ? mx + logf(den) : -INFINITY;
  }
}

// The same merge over PACKED rows, for the row-split exchange of the block-sharded forward: a row
// holds the partial output of one query token for all heads (H*D elements) followed by its H
// log-sum-exps as fp32, padded to a multiple of 16 bytes; `parts` is [R][rows] such rows (what one rank receives from the all-to-all:
// its share of the rows from every rank), `merged` [rows] rows in the same format.
template <typename T>
__global__ void merge_packed_rows_kernel(const char* __restrict__ parts, int R, int64_t rows, int H, int D,
                                         int64_t row_bytes, char* __restrict__ merged) {
  const int cpr = D / 8;
  const int64_t total = rows * H * cpr;
  const int64_t part_bytes = rows * row_bytes;
  const int64_t lse_off = static_cast<int64_t>(H) * D * sizeof(T);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % cpr);
    const int64_t rh = i / cpr;
    const int h = static_cast<int>(rh % H);
    const int64_t row = rh / H;
    const char* base = parts + row * row_bytes;
    float w[kMaxParts];
    float mx = -INFINITY;
    for (int r = 0; r < R; ++r) {
      w[r] = *reinterpret_cast<const float*>(base + r * part_bytes + lse_off + h * 4);
      mx = fmaxf(mx, w[r]);
    }
    float den = 0.f;
    for (int r = 0; r < R; ++r) { w[r] = (w[r] == -INFINITY) ? 0.f : __expf(w[r] - mx); den += w[r]; }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int r = 0; r < R; ++r) {
      if (w[r] == 0.f) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(base + r * part_bytes + (static_cast<int64_t>(h) * D) * sizeof(T) + cc * 16);
      const T* e8 = reinterpret_cast<const T*>(&v);
      const float wr = w[r] * inv;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += wr * to_f32<T>(e8[e]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < 8; ++e) oe[e] = from_f32<T>(acc[e]);
    char* orow = merged + row * row_bytes;
    *reinterpret_cast<uint4*>(orow + (static_cast<int64_t>(h) * D) * sizeof(T) + cc * 16) = o;
    if (cc == 0) *reinterpret_cast<float*>(orow + lse_off + h * 4) = den > 0.f ? mx + logf(den) : -INFINITY;
  }
}

__global__ void build_ptr_table_kernel(const int32_t* __restrict__ ids, int64_t i_sb, int64_t i_sg,
                                       int64_t i_sh, int64_t i_st, const int64_t* __restrict__ base_k,
                                       const int64_t* __restrict__ base_v,
                                       const int32_t* __restrict__ n_blocks_per_head, int B, int MG,
                                       int H, int T, int max_chunks, int64_t batch_stride,
                                       int blocks_per_chunk, int64_t in_chunk_block_bytes,
                                       int64_t* __restrict__ ptr_k, int64_t* __restrict__ ptr_v) {
  const int64_t total = static_cast<int64_t>(B) * MG * H * T;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i % T);
    int64_t r = i / T;
    const int h = static_cast<int>(r % H); r /= H;
    const int g = static_cast<int>(r % MG);
    const int b = static_cast<int>(r / MG);
    const int32_t bid = ids[b * i_sb + g * i_sg + h * i_sh + t * i_st];
    int64_t ak = 0, av = 0;
    if (bid >= 0 && bid < n_blocks_per_head[h]) {
      const int cid = bid / blocks_per_chunk, loc = bid % blocks_per_chunk;
      if (cid < max_chunks) {
        const int64_t off = b * batch_stride + loc * in_chunk_block_bytes;
        const int64_t bk = base_k[static_cast<int64_t>(h) * max_chunks + cid];
        const int64_t bv = base_v[static_cast<int64_t>(h) * max_chunks + cid];
        // test the base before adding the offset so a zero base never becomes an address
        if (bk != 0) ak = bk + off;
        if (bv != 0) av = bv + off;
      }
    }
    ptr_k[i] = ak;
    ptr_v[i] = av;
  }
}

}  // namespace
}  // namespace nsa

using namespace nsa;

extern "C" int nsa_merge_partials(const void* outs, const float* lses, int32_t R, int32_t B, int64_t M,
                                  int32_t H, int32_t D, void* out, float* lse, int32_t dtype,
                                  void* stream) {
  NSA_REQUIRE(R >= 1 && R <= kMaxParts, NSA_ERR_INVALID, "merge_partials: R must be in [1,%d]", kMaxParts);
  NSA_REQUIRE(B >= 0 && M >= 0 && H >= 0 && D > 0 && D % 8 == 0, NSA_ERR_INVALID, "merge_partials: bad size");
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_F16, NSA_ERR_UNSUPPORTED, "merge_partials: bf16 / fp16 only");
  const int64_t total = static_cast<int64_t>(B) * M * H * (D / 8);
  if (total == 0) return NSA_OK;
  NSA_REQUIRE(outs && lses && out && lse && aligned16(outs) && aligned16(out), NSA_ERR_INVALID,
              "merge_partials: null or misaligned pointer");
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == NSA_BF16)
    merge_partials_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const char*>(outs), lses, R, B, M, H, D,
                                                                static_cast<char*>(out), lse);
  else
    merge_partials_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const char*>(outs), lses, R, B, M, H, D,
                                                         static_cast<char*>(out), lse);
  NSA_LAUNCH_OK("merge_partials_kernel");
  return NSA_OK;
}

extern "C" int nsa_merge_packed_rows(const void* parts, int32_t R, int64_t rows, int32_t H, int32_t D,
                                     void* merged, int32_t dtype, void* stream) {
  NSA_REQUIRE(R >= 1 && R <= kMaxParts, NSA_ERR_INVALID, "merge_packed_rows: R must be in [1,%d]", kMaxParts);
  NSA_REQUIRE(rows >= 0 && H > 0 && D > 0 && D % 8 == 0, NSA_ERR_INVALID, "merge_packed_rows: bad size");
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_F16, NSA_ERR_UNSUPPORTED, "merge_packed_rows: bf16 / fp16 only");
  const int64_t row_bytes = static_cast<int64_t>(align_up(static_cast<size_t>(H) * D * 2 + static_cast<size_t>(H) * 4, 16));
  const int64_t total = rows * H * (D / 8);
  if (total == 0) return NSA_OK;
  NSA_REQUIRE(parts && merged && aligned16(parts) && aligned16(merged), NSA_ERR_INVALID,
              "merge_packed_rows: null or misaligned pointer");
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == NSA_BF16)
    merge_packed_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const char*>(parts), R, rows, H, D, row_bytes,
                                                                   static_cast<char*>(merged));
  else
    merge_packed_rows_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const char*>(parts), R, rows, H, D, row_bytes,
                                                            static_cast<char*>(merged));
  NSA_LAUNCH_OK("merge_packed_rows_kernel");
  return NSA_OK;
}

namespace nsa {
namespace {
__global__ void local_block_ids_kernel(const int32_t* __restrict__ ids, int64_t n, int R, int r, int32_t* __restrict__ out) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int32_t id = ids[i];
    out[i] = (id >= 0 && id % R == r) ? id / R : -1;
  }
}
}  // namespace
}  // namespace nsa

extern "C" int nsa_local_block_ids(const int32_t* ids, int64_t n, int32_t R, int32_t r, int32_t* out, void* stream) {
  NSA_REQUIRE(R >= 1 && r >= 0 && r < R && n >= 0, NSA_ERR_INVALID, "local_block_ids: need 0 <= r < R and n >= 0");
  if (n == 0) return NSA_OK;
  NSA_REQUIRE(ids && out, NSA_ERR_INVALID, "local_block_ids: null pointer");
  const int blocks = static_cast<int>(n / 256 + 1 < 148 * 8 ? n / 256 + 1 : 148 * 8);
  nsa::local_block_ids_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(ids, n, R, r, out);
  NSA_LAUNCH_OK("local_block_ids_kernel");
  return NSA_OK;
}

extern "C" int nsa_build_ptr_table(const int32_t* block_indices, const int64_t idx_stride[4],
                                   const int64_t* base_k, const int64_t* base_v,
                                   const int32_t* n_blocks_per_head, int32_t B, int32_t MG, int32_t H,
                                   int32_t T, int32_t max_chunks, int64_t batch_stride,
                                   int32_t blocks_per_chunk, int64_t in_chunk_block_bytes,
                                   int64_t* ptr_k, int64_t* ptr_v, void* stream) {
  NSA_REQUIRE(B >= 0 && MG >= 0 && H >= 0 && T >= 0 && max_chunks >= 0, NSA_ERR_INVALID, "build_ptr_table: negative size");
  NSA_REQUIRE(blocks_per_chunk > 0, NSA_ERR_INVALID, "build_ptr_table: blocks_per_chunk must be > 0");
  const int64_t total = static_cast<int64_t>(B) * MG * H * T;
  if (total == 0) return NSA_OK;
  NSA_REQUIRE(block_indices && base_k && base_v && n_blocks_per_head && ptr_k && ptr_v, NSA_ERR_INVALID,
              "build_ptr_table: null pointer");
  const int blocks = static_cast<int>(total / 256 + 1 < 65535 ? total / 256 + 1 : 65535);
  build_ptr_table_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      block_indices, idx_stride[0], idx_stride[1], idx_stride[2], idx_stride[3], base_k, base_v,
      n_blocks_per_head, B, MG, H, T, max_chunks, batch_stride, blocks_per_chunk, in_chunk_block_bytes, ptr_k, ptr_v);
  NSA_LAUNCH_OK("build_ptr_table_kernel");
  return NSA_OK;
}
