// Shared device/host helpers of the sm_100a NSA selection kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdlib>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/omnimem_b200.h"

namespace nsa {

// ---- error reporting (thread local, never throws across the C boundary) -------------
void set_error(const char* fmt, ...);

#define NSA_REQUIRE(cond, code, ...)          \
  do {                                        \
    if (!(cond)) {                            \
      ::nsa::set_error(__VA_ARGS__);          \
      return (code);                          \
    }                                         \
  } while (0)

#define NSA_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess) {                                                          \
      ::nsa::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),        \
                       __FILE__, __LINE__);                                            \
      return NSA_ERR_CUDA;                                                             \
    }                                                                                  \
  } while (0)

#define NSA_LAUNCH_OK(name)                                                            \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess) {                                                          \
      ::nsa::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__));      \
      return NSA_ERR_CUDA;                                                             \
    }                                                                                  \
  } while (0)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
__host__ __device__ __forceinline__ constexpr int cdiv(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ constexpr int64_t cdiv64(int64_t a, int64_t b) {
  return (a + b - 1) / b;
}

inline int dtype_size(int dtype) { return dtype == NSA_F32 ? 4 : 2; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---- scalar conversions ------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float x) {
  return __float2half_rn(x);
}

// two fp32 -> packed pair of 16-bit floats (low half = a)
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

// ---- programmatic dependent launch --------------------------------------------------
// A kernel launched with launch_chained() may become resident while the kernel before it in the
// stream is still running: its thread blocks start as soon as every block of the predecessor has
// called chain_release() (or exited) and room is free, run whatever needs no result of the
// predecessor (barrier set-up, TMEM allocation, descriptor prefetch) and stop at chain_wait(),
// which returns when the predecessor has completed and its writes are visible.  Both
// instructions do nothing in a kernel launched the ordinary way.
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// OMNIMEM_B200_CHAINED_LAUNCH is a bit mask of the launch sites that use it (1: pooling, scoring and
// selection, 2: forward, 4: dQ, 8: dK/dV with its counter reset); 0 launches everything the ordinary way.
constexpr int kChainSmall = 1, kChainFwd = 2, kChainDq = 4, kChainDkv = 8;
inline int chained_launch_mask() {
  static const int mask = [] {
    const char* e = getenv("OMNIMEM_B200_CHAINED_LAUNCH");
    return e != nullptr ? atoi(e) : 15;
  }();
  return mask;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(int site, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (chained_launch_mask() & site) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- async copies, ldmatrix, mma.sync -----------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte global -> shared copy; src_bytes < 16 zero-fills the remainder (0 = all zeros)
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

// D(16x8,f32) += A(16x16) * B(16x8), 16-bit operands
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4],
                                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                 uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// ---- K/V block resolution shared by forward and backward ----------------------------------
// Device copy of nsa_kv_source with strides widened once on the host.
struct KVSrc {
  int mode;
  const char* k;
  const char* v;
  int64_t k_sb, k_sn, k_sh;   // element strides (dense)
  int64_t v_sb, v_sn, v_sh;
  int64_t n_tokens;
  const int32_t* block_table;
  int max_blocks;
  int page_tokens;
  const int64_t* ptr_k;
  const int64_t* ptr_v;
  int64_t ptr_sn;
};

// bytes between consecutive tokens of a block
__device__ __forceinline__ int64_t kv_row_bytes(const KVSrc& kv, bool is_v, int D, int esz) {
  if (kv.mode == NSA_KV_DENSE) return (is_v ? kv.v_sn : kv.k_sn) * esz;
  if (kv.mode == NSA_KV_PTR) return kv.ptr_sn * esz;
  return static_cast<int64_t>(D) * esz;
}

struct BlockRef {
  const char* k;     // first token of the block (nullptr: nothing to read)
  const char* v;
  int n_vis;         // visible tokens (prefix of the block)
};

// Resolves selected block `bid` of (b, h) for a query group whose chunk id is q_chunk.
// Mirrors the reference accessors: negative / out-of-range ids and blocks entirely in a later
// chunk are skipped, the last block is clipped to the tokens that exist, and under the causal
// rule only the prefix that lies in chunks <= q_chunk is visible.
template <int ESZ>
__device__ __forceinline__ BlockRef resolve_block(const KVSrc& kv, int b, int h, int bid, int D,
                                                  int block_size, int chunk_size, bool causal,
                                                  int q_chunk) {
  BlockRef r{nullptr, nullptr, 0};
  if (bid < 0) return r;
  const int64_t t0 = static_cast<int64_t>(bid) * block_size;
  if (t0 >= kv.n_tokens) return r;
  int64_t n = kv.n_tokens - t0;
  if (n > block_size) n = block_size;
  if (causal) {
    if (t0 / chunk_size > q_chunk) return r;
    const int64_t lim = static_cast<int64_t>(q_chunk + 1) * chunk_size - t0;
    if (lim < n) n = lim;
    if (n <= 0) return r;
  }
  if (kv.mode == NSA_KV_DENSE) {
    r.k = kv.k + (b * kv.k_sb + t0 * kv.k_sn + h * kv.k_sh) * ESZ;
    r.v = kv.v + (b * kv.v_sb + t0 * kv.v_sn + h * kv.v_sh) * ESZ;
  } else {
    if (bid >= kv.max_blocks) return r;
    const int page = kv.block_table[static_cast<int64_t>(h) * kv.max_blocks + bid];
    if (page < 0) return r;
    const int64_t off = static_cast<int64_t>(page) * kv.page_tokens * D * ESZ;
    r.k = kv.k + off;
    r.v = kv.v + off;
  }
  r.n_vis = static_cast<int>(n);
  return r;
}

int make_kvsrc(const nsa_kv_source* in, int D, int esz, int block_size, KVSrc* out);

}  // namespace nsa
