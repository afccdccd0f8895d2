// Three-branch gate + sum that consumes the selection output:
//     g = clamp(g_logits, -10, 10);  (g_cmp, g_slc, g_swa) = sigmoid(g)  or  softmax(g)
//     x = g_cmp * o_cmp + g_slc * o_slc + g_swa * o_swa          (a skipped branch drops its term)
// (models/transformers/causal_wan_nsa_model.py:378-386 and 541-546), forward and backward, each one
// pass over the [B, M, H, D] tensors: HBM-bound, 16-byte accesses, one thread per 8 elements, the
// lanes that share a row reduce the three dot products sum_d(dx * o_i) with shuffles.
#include "common.cuh"

namespace nsa {
namespace {

struct GateParams {
  const char* g;        // [rows, 3] logits
  const char* o[3];     // [rows, D] each, nullptr = branch skipped
  const char* dx;       // backward only
  char* x;              // forward only
  char* d_o[3];         // backward: gradients of the branches (nullptr = skipped)
  char* dg;             // backward: [rows, 3] gradient of the logits
  int64_t rows;
  int D, softmax;
};

template <typename T>
__device__ __forceinline__ void gates_of_row(const GateParams& p, int64_t row, float (&s)[3], bool (&inside)[3]) {
  float z[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const float raw = to_f32<T>(reinterpret_cast<const T*>(p.g)[row * 3 + i]);
    inside[i] = raw >= -10.f && raw <= 10.f;       // clamp passes the gradient on the closed interval
    z[i] = fminf(fmaxf(raw, -10.f), 10.f);
  }
  if (p.softmax) {
    const float m = fmaxf(z[0], fmaxf(z[1], z[2]));
    const float e0 = expf(z[0] - m), e1 = expf(z[1] - m), e2 = expf(z[2] - m);
    const float inv = 1.f / (e0 + e1 + e2);
    s[0] = e0 * inv; s[1] = e1 * inv; s[2] = e2 * inv;
  } else {
#pragma unroll
    for (int i = 0; i < 3; ++i) s[i] = 1.f / (1.f + expf(-z[i]));
  }
}

// One thread per 16-byte chunk of a row; gates are rounded to T before the product, as the
// reference's tensors are (g has the activations' dtype).
template <typename T>
__global__ void gate_combine_fwd_kernel(const GateParams p) {
  const uint32_t cpr = static_cast<uint32_t>(p.D / 8);
  const int64_t total = p.rows * cpr;
  {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    // rows * cpr fits 32 bits for every launch the host makes (checked there): 32-bit division
    const uint32_t iu = static_cast<uint32_t>(i);
    const int64_t row = iu / cpr;
    const int cc = static_cast<int>(iu - static_cast<uint32_t>(row) * cpr);
    float s[3];
    bool inside[3];
    gates_of_row<T>(p, row, s, inside);
    // every product and every partial sum is rounded to T, left to right, as the eager expression does
    float acc[8];
    bool first = true;
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      if (p.o[b] == nullptr) continue;
      const float gb = to_f32<T>(from_f32<T>(s[b]));
      const uint4 v = *reinterpret_cast<const uint4*>(p.o[b] + (row * p.D) * sizeof(T) + cc * 16);
      const T* e8 = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float prod = to_f32<T>(from_f32<T>(gb * to_f32<T>(e8[e])));
        acc[e] = first ? prod : to_f32<T>(from_f32<T>(acc[e] + prod));
      }
      first = false;
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < 8; ++e) oe[e] = from_f32<T>(acc[e]);
    *reinterpret_cast<uint4*>(p.x + (row * p.D) * sizeof(T) + cc * 16) = o;
  }
}

// LPR = lanes per row (D / 8): 8, 16 or 32.  d_o_i = g_i dx;  t_i = sum_d dx o_i;
// sigmoid: dg_i = t_i s_i (1 - s_i);  softmax: dg_i = s_i (t_i - sum_j s_j t_j);  zero outside the clamp.
template <typename T, int LPR>
__global__ void gate_combine_bwd_kernel(const GateParams p) {
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = gthread / LPR;
  const int cc = static_cast<int>(gthread % LPR);
  const bool live = row < p.rows;
  float s[3] = {0.f, 0.f, 0.f};
  bool inside[3] = {false, false, false};
  float t[3] = {0.f, 0.f, 0.f};
  if (live) {
    gates_of_row<T>(p, row, s, inside);
    const uint4 dv = *reinterpret_cast<const uint4*>(p.dx + (row * p.D) * sizeof(T) + cc * 16);
    const T* d8 = reinterpret_cast<const T*>(&dv);
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      if (p.o[b] == nullptr) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(p.o[b] + (row * p.D) * sizeof(T) + cc * 16);
      const T* e8 = reinterpret_cast<const T*>(&v);
      const float gb = to_f32<T>(from_f32<T>(s[b]));
      uint4 w;
      T* we = reinterpret_cast<T*>(&w);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float dxe = to_f32<T>(d8[e]);
        t[b] += dxe * to_f32<T>(e8[e]);
        we[e] = from_f32<T>(gb * dxe);
      }
      if (p.d_o[b] != nullptr) *reinterpret_cast<uint4*>(p.d_o[b] + (row * p.D) * sizeof(T) + cc * 16) = w;
    }
  }
#pragma unroll
  for (int d = LPR / 2; d >= 1; d >>= 1) {
#pragma unroll
    for (int b = 0; b < 3; ++b) t[b] += __shfl_xor_sync(0xffffffffu, t[b], d);
  }
  if (live && cc == 0 && p.dg != nullptr) {
    float dg[3];
    if (p.softmax) {
      const float dot = s[0] * t[0] + s[1] * t[1] + s[2] * t[2];
#pragma unroll
      for (int b = 0; b < 3; ++b) dg[b] = s[b] * (t[b] - dot);
    } else {
#pragma unroll
      for (int b = 0; b < 3; ++b) dg[b] = t[b] * s[b] * (1.f - s[b]);
    }
#pragma unroll
    for (int b = 0; b < 3; ++b)
      reinterpret_cast<T*>(p.dg)[row * 3 + b] = from_f32<T>(inside[b] ? dg[b] : 0.f);
  }
}

int check_common(const char* what, const void* g, const void* o_cmp, const void* o_slc, const void* o_swa,
                 int64_t rows, int D, int dtype) {
  NSA_REQUIRE(g != nullptr, NSA_ERR_INVALID, "%s: gate logits are null", what);
  NSA_REQUIRE(o_cmp != nullptr || o_slc != nullptr || o_swa != nullptr, NSA_ERR_INVALID, "%s: all three branches are null", what);
  NSA_REQUIRE(rows >= 0 && D > 0 && D % 8 == 0, NSA_ERR_UNSUPPORTED, "%s: head dim %d must be a positive multiple of 8", what, D);
  NSA_REQUIRE(dtype == NSA_BF16 || dtype == NSA_F16, NSA_ERR_UNSUPPORTED, "%s: dtype %d (bf16 and fp16 only)", what, dtype);
  const void* ptrs[3] = {o_cmp, o_slc, o_swa};
  for (int i = 0; i < 3; ++i)
    NSA_REQUIRE(ptrs[i] == nullptr || aligned16(ptrs[i]), NSA_ERR_LAYOUT, "%s: branch %d is not 16-byte aligned", what, i);
  return NSA_OK;
}

}  // namespace
}  // namespace nsa

using namespace nsa;

extern "C" int nsa_gate_combine(const void* g_logits, const void* o_cmp, const void* o_slc, const void* o_swa,
                                void* x, int64_t rows, int32_t D, int32_t softmax, int32_t dtype, void* stream) {
  int rc;
  if ((rc = check_common("gate_combine", g_logits, o_cmp, o_slc, o_swa, rows, D, dtype))) return rc;
  NSA_REQUIRE(x != nullptr && aligned16(x), NSA_ERR_LAYOUT, "gate_combine: output must be non-null and 16-byte aligned");
  if (rows == 0) return NSA_OK;
  GateParams p{};
  p.g = static_cast<const char*>(g_logits);
  p.o[0] = static_cast<const char*>(o_cmp); p.o[1] = static_cast<const char*>(o_slc); p.o[2] = static_cast<const char*>(o_swa);
  p.x = static_cast<char*>(x); p.rows = rows; p.D = D; p.softmax = softmax;
  const int64_t total = rows * (D / 8);
  NSA_REQUIRE(total <= 0xffffffffll, NSA_ERR_INVALID, "gate_combine: too many rows");
  const unsigned blocks = static_cast<unsigned>(cdiv64(total, 256));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == NSA_BF16) gate_combine_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p);
  else gate_combine_fwd_kernel<__half><<<blocks, 256, 0, s>>>(p);
  NSA_LAUNCH_OK("gate_combine_fwd_kernel");
  return NSA_OK;
}

extern "C" int nsa_gate_combine_bwd(const void* g_logits, const void* o_cmp, const void* o_slc, const void* o_swa,
                                    const void* dx, void* d_g_logits, void* d_o_cmp, void* d_o_slc, void* d_o_swa,
                                    int64_t rows, int32_t D, int32_t softmax, int32_t dtype, void* stream) {
  int rc;
  if ((rc = check_common("gate_combine_bwd", g_logits, o_cmp, o_slc, o_swa, rows, D, dtype))) return rc;
  NSA_REQUIRE(dx != nullptr && aligned16(dx), NSA_ERR_LAYOUT, "gate_combine_bwd: dx must be non-null and 16-byte aligned");
  NSA_REQUIRE(D == 64 || D == 128 || D == 256, NSA_ERR_UNSUPPORTED, "gate_combine_bwd: head dim %d (64, 128 or 256)", D);
  void* outs[3] = {d_o_cmp, d_o_slc, d_o_swa};
  for (int i = 0; i < 3; ++i)
    NSA_REQUIRE(outs[i] == nullptr || aligned16(outs[i]), NSA_ERR_LAYOUT, "gate_combine_bwd: gradient %d is not 16-byte aligned", i);
  if (rows == 0) return NSA_OK;
  GateParams p{};
  p.g = static_cast<const char*>(g_logits);
  p.o[0] = static_cast<const char*>(o_cmp); p.o[1] = static_cast<const char*>(o_slc); p.o[2] = static_cast<const char*>(o_swa);
  p.dx = static_cast<const char*>(dx);
  for (int i = 0; i < 3; ++i) p.d_o[i] = static_cast<char*>(outs[i]);
  p.dg = static_cast<char*>(d_g_logits);
  p.rows = rows; p.D = D; p.softmax = softmax;
  const int lpr = D / 8;
  const unsigned blocks = static_cast<unsigned>(cdiv64(rows * lpr, 256));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define NSA_GATE_BWD(T)                                                                   \
  do {                                                                                    \
    if (lpr == 8) gate_combine_bwd_kernel<T, 8><<<blocks, 256, 0, s>>>(p);                \
    else if (lpr == 16) gate_combine_bwd_kernel<T, 16><<<blocks, 256, 0, s>>>(p);         \
    else gate_combine_bwd_kernel<T, 32><<<blocks, 256, 0, s>>>(p);                        \
  } while (0)
  if (dtype == NSA_BF16) NSA_GATE_BWD(__nv_bfloat16);
  else NSA_GATE_BWD(__half);
#undef NSA_GATE_BWD
  NSA_LAUNCH_OK("gate_combine_bwd_kernel");
  return NSA_OK;
}
