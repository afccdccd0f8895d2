// Tile machinery shared by the selection forward and backward kernels (legacy-MMA path used
// for every geometry; the tcgen05 kernel covers the 64/64/128 bf16 case).
//
// A (b, group, h) row attends to the visible tokens of its T selected blocks.  The kernels
// pack those tokens, in slot order, into 64-row tiles (a tile may hold several short blocks
// or part of a long one), so tiles are always full except the last one, whatever the block
// size.
#pragma once

#include "common.cuh"

namespace nsa {

constexpr int kTileRows = 64;

// Slot table in shared memory: per selected slot the K/V base address of its block and the
// running count of visible tokens before it.
struct SlotTable {
  const char** kptr;
  const char** vptr;
  int* cum;          // [T+1]
};

__host__ __device__ inline size_t slot_table_bytes(int T) {
  return static_cast<size_t>(T) * 16 + (static_cast<size_t>(T) + 1 + 3) / 4 * 16;
}

__device__ __forceinline__ SlotTable carve_slot_table(char* base, int T) {
  SlotTable s;
  s.kptr = reinterpret_cast<const char**>(base);
  s.vptr = reinterpret_cast<const char**>(base + static_cast<size_t>(T) * 8);
  s.cum = reinterpret_cast<int*>(base + static_cast<size_t>(T) * 16);
  return s;
}

// Fills the slot table for row (b, g, h); every thread of the block must call it.  Returns the
// number of packed rows (sum of visible tokens).  Ends with a __syncthreads().
// `ids_off` is the element offset of slot 0 of the row inside block_indices (and, in pointer
// mode, inside the two address tables, which share its layout).
template <int ESZ>
__device__ __forceinline__ int build_slot_table(const SlotTable& st, const KVSrc& kv,
                                                const int32_t* ids, int64_t ids_off, int64_t ids_st,
                                                int T, int b, int h, int D, int block_size,
                                                int chunk_size, bool causal, int q_chunk) {
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    BlockRef r{nullptr, nullptr, 0};
    if (kv.mode == NSA_KV_PTR) {
      const int64_t ak = kv.ptr_k[ids_off + t * ids_st], av = kv.ptr_v[ids_off + t * ids_st];
      if (ak != 0 && av != 0) {
        r.k = reinterpret_cast<const char*>(static_cast<uintptr_t>(ak));
        r.v = reinterpret_cast<const char*>(static_cast<uintptr_t>(av));
        r.n_vis = block_size;
      }
    } else {
      r = resolve_block<ESZ>(kv, b, h, ids[ids_off + t * ids_st], D, block_size, chunk_size, causal, q_chunk);
    }
    st.kptr[t] = r.k;
    st.vptr[t] = r.v;
    st.cum[t + 1] = r.n_vis;   // turned into a running sum below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    st.cum[0] = 0;
    for (int t = 0; t < T; ++t) {
      acc += st.cum[t + 1];
      st.cum[t + 1] = acc;
    }
  }
  __syncthreads();
  return st.cum[T];
}

// Slot that holds packed row pr (cum[t] <= pr < cum[t+1]); pr < cum[T] required.
__device__ __forceinline__ int find_slot(const int* cum, int T, int pr) {
  int lo = 0, hi = T;  // answer in [lo, hi)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cum[mid] <= pr) lo = mid; else hi = mid;
  }
  return lo;
}

// Issues the cp.async copies of packed rows [row0, row0+64) of K and V into a stage
// (layout [64][PITCH] each).  Rows past `total` are zero-filled.
template <typename T, int D, int PITCH>
__device__ __forceinline__ void issue_kv_tile(T* sK, T* sV, const SlotTable& st, int nslots,
                                              int row0, int total, int64_t k_row_bytes,
                                              int64_t v_row_bytes, const void* dummy) {
  constexpr int CPR = D * static_cast<int>(sizeof(T)) / 16;  // 16-byte chunks per row
  for (int c = threadIdx.x; c < kTileRows * CPR; c += blockDim.x) {
    const int r = c / CPR;
    const int cc = c - r * CPR;
    const int pr = row0 + r;
    T* dk = sK + r * PITCH + cc * (16 / static_cast<int>(sizeof(T)));
    T* dv = sV + r * PITCH + cc * (16 / static_cast<int>(sizeof(T)));
    if (pr < total) {
      const int t = find_slot(st.cum, nslots, pr);
      const int64_t tok = pr - st.cum[t];
      cp_async16(dk, st.kptr[t] + tok * k_row_bytes + cc * 16, 16);
      cp_async16(dv, st.vptr[t] + tok * v_row_bytes + cc * 16, 16);
    } else {
      cp_async16(dk, dummy, 0);
      cp_async16(dv, dummy, 0);
    }
  }
}

// Copies `rows` rows of a [rows][D] strided matrix into shared memory [rows_pad][PITCH];
// rows in [rows, rows_pad) are zero-filled.
template <typename T, int D, int PITCH>
__device__ __forceinline__ void issue_rows(T* dst, const char* src, int64_t row_bytes, int rows,
                                           int rows_pad) {
  constexpr int CPR = D * static_cast<int>(sizeof(T)) / 16;
  for (int c = threadIdx.x; c < rows_pad * CPR; c += blockDim.x) {
    const int r = c / CPR;
    const int cc = c - r * CPR;
    T* d = dst + r * PITCH + cc * (16 / static_cast<int>(sizeof(T)));
    if (r < rows) cp_async16(d, src + r * row_bytes + cc * 16, 16);
    else cp_async16(d, src, 0);
  }
}

}  // namespace nsa
