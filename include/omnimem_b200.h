/*
 * omnimem_b200 - C ABI of the B200 (sm_100a) NSA selection path.
 *
 * Every function takes raw device pointers, sizes, element strides and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), launches on that stream, never synchronises,
 * never allocates device memory and never throws: it returns 0 on success or a negative
 * nsa_status, and nsa_last_error() then returns a human-readable message (thread local).
 * Scratch memory is owned by the caller: each *_workspace_bytes() function says how much
 * a call needs; pass a device buffer of at least that size (256-byte aligned).
 *
 * Tensors follow the reference operator layouts: q/out [B,M,H,D], k/v [B,N,H,D],
 * block_indices int32 [B,MG,H,T], lse float [B,H,M] (natural log).  Strides are in
 * elements; the innermost (D) stride must be 1 and every row must start on a 16-byte
 * boundary (the host wrapper copies a tensor that does not satisfy this).
 *
 * Each declaration cites the reference interface it replaces, as
 * path:line inside the reference project (src/omnimem/nsa/cuda_backend/csrc/...).
 */
#ifndef OMNIMEM_B200_H_
#define OMNIMEM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum nsa_status {
  NSA_OK = 0,
  NSA_ERR_INVALID = -1,     /* bad argument (shape, range, null pointer) */
  NSA_ERR_LAYOUT = -2,      /* stride / alignment the kernels cannot address */
  NSA_ERR_UNSUPPORTED = -3, /* dtype / head dim / size outside the built kernels */
  NSA_ERR_WORKSPACE = -4,   /* workspace too small */
  NSA_ERR_CUDA = -5,        /* a CUDA runtime call or launch failed */
  NSA_ERR_EXHAUSTED = -6    /* page pool has no free page */
} nsa_status;

typedef enum nsa_dtype { NSA_BF16 = 0, NSA_F16 = 1, NSA_F32 = 2 } nsa_dtype;

/* Where the selection kernels find the K/V tokens of block `bid` of head h. */
typedef enum nsa_kv_mode {
  NSA_KV_DENSE = 0, /* k/v [B,N,H,D] with element strides (common.cuh:158-190 DenseKV)   */
  NSA_KV_PAGED = 1, /* fixed-page pool + int32 block table [H][max_blocks] -> page or -1;
                       the B200-native replacement of the int64 pointer tables.  Whole pages
                       are read: the rows of a partly filled page behind the block's last
                       token get probability 0, but must hold finite values (0 x NaN = NaN
                       in the P V and dS K products) - zero the pool once at allocation   */
  NSA_KV_PTR = 2    /* int64 byte-address tables [B,MG,H,T] laid out like block_indices, 0 =
                       skip, whole blocks only (common.cuh:193-215 PtrKV); block_indices is
                       ignored by the forward in this mode                                */
} nsa_kv_mode;

typedef struct nsa_kv_source {
  int32_t mode;              /* nsa_kv_mode */
  const void* k;             /* dense: k base; paged: K page pool base */
  const void* v;             /* dense: v base; paged: V page pool base */
  int64_t k_stride[3];       /* dense: element strides of (b, n, h); paged: unused */
  int64_t v_stride[3];
  int64_t n_tokens;          /* N: tokens that exist (last block may be partial) */
  const int32_t* block_table;/* paged: [H][max_blocks] page id or -1 (not resident) */
  int32_t max_blocks;        /* paged: row length of block_table */
  int32_t page_tokens;       /* paged: tokens per page (== block_size); page = [page_tokens][D] */
  const int64_t* ptr_k;      /* ptr: K block addresses, element strides = idx_stride */
  const int64_t* ptr_v;      /* ptr: V block addresses */
  int64_t ptr_stride_n;      /* ptr: elements between consecutive tokens of a block */
  int64_t num_pages;         /* paged: pages in the pool (0 = unknown) */
} nsa_kv_source;

/* Visibility rules of the top-k (topk.cu:16-97 TopkMask / visible()). */
typedef struct nsa_topk_mask {
  int32_t block_size;     /* tokens per key block */
  int32_t chunk_size;     /* query chunk length, in query TOKENS (rows * q_group_size) */
  int32_t chunk_size_k;   /* key chunk length in tokens */
  int32_t q_group_size;   /* tokens one pooled query row stands for (1: rows are tokens) */
  int32_t q_chunk_offset; /* added to every query chunk id */
  int32_t ex_win;
  int32_t ex_sink;
  int32_t causal;
  int32_t tf_mask;
  int32_t prog_excl;
  int32_t id_base;        /* global block id of local column c is id_base + c*id_stride */
  int32_t id_stride;      /* (block-sharded KV: rank r of R owns ids r, r+R, ...)        */
} nsa_topk_mask;

const char* nsa_last_error(void);
/* Library version string; also a cheap "does the library load" probe. */
const char* nsa_version(void);

/* Reads and clears the sticky device-side status word: 0, or a negative nsa_status when a
 * kernel gave up on a bounded wait (its outputs are then undefined).  Synchronises with the
 * device; meant for tests and debugging, not for the hot path. */
int nsa_device_status(int32_t* value);

/* Mean over runs of `size` rows of dim 1: x [B,N,H,D] -> out [B,ceil(N/size),H,D], fp32
 * accumulation, rounded to the input dtype; a short last run averages the rows that exist.
 * Replaces the torch expressions k.view(b, s//bs, bs, n, d).mean(2)
 * (models/transformers/causal_wan_nsa_model.py:408-409,481,487) and the query-group
 * pooling of nsa/ops/index_topk.py:72-79. */
int nsa_pool_rows(const void* x, const int64_t x_stride[3], void* out, const int64_t out_stride[3],
                  int32_t B, int64_t N, int32_t H, int32_t D, int32_t size, int32_t dtype,
                  void* stream);

/* Top-k block selection.  q_pooled [B,MG,H,D], k_pooled [B,NC,H,D] ->
 * out_idx int32 [B,MG,H,topk] (contiguous), visible blocks by (score desc, id asc), -1 in
 * unused slots; out_scores (may be NULL) float [B,MG,H,topk], -inf in unused slots.
 * Replaces topk_cuda (topk.cu:664-808; schema bindings.cpp `topk`). */
size_t nsa_topk_workspace_bytes(int32_t B, int32_t MG, int32_t H, int64_t NC);
int nsa_topk(const void* q_pooled, const int64_t q_stride[3], const void* k_pooled,
             const int64_t k_stride[3], int32_t B, int32_t MG, int32_t H, int32_t D, int64_t NC,
             int32_t topk, float scale, const nsa_topk_mask* mask, int32_t* out_idx,
             float* out_scores, void* workspace, size_t workspace_bytes, int32_t dtype,
             void* stream);

/* nsa_topk without a caller-provided workspace, for callers that cannot allocate device
 * memory: a process whose device memory was all handed to another allocator when it started,
 * a host runtime behind an FFI boundary that owns no device memory and only forwards the
 * pointers it is given, or a loop whose memory plan is frozen.  The score buffer is a fixed
 * 4 MiB array inside the library's device image (present on every GPU that loads the library,
 * until the process exits).  It holds nsa_topk_static_scratch_max_scores() = 1,048,576 scores:
 * a call with B*MG*H*NC above that returns NSA_ERR_WORKSPACE and launches nothing.
 * The call makes no cudaMalloc / cudaFree and calls no allocating library routine.  Its first
 * call on each device looks up the array's device address (cudaGetSymbolAddress) with that
 * device current; make that first call before any stream capture begins.  All calls on a
 * device share the one array: calls whose kernels overlap on the GPU (different streams) race
 * on it and must be serialised by the caller; nothing in it needs clearing between calls,
 * because every score that is read was written earlier in the same call.
 * No counterpart in the reference (its top-k allocates its buffers through torch). */
size_t nsa_topk_static_scratch_max_scores(void);
int nsa_topk_static_scratch(const void* q_pooled, const int64_t q_stride[3], const void* k_pooled,
                            const int64_t k_stride[3], int32_t B, int32_t MG, int32_t H, int32_t D,
                            int64_t NC, int32_t topk, float scale, const nsa_topk_mask* mask,
                            int32_t* out_idx, float* out_scores, int32_t dtype, void* stream);

/* Block-compressed key scoring from the RAW keys: pools k [B,N,H,D] block by block (each key is
 * read exactly once, streamed through shared memory with bulk asynchronous copies; the pooled
 * keys go to k_pooled_out [B,NC,H,D] contiguous, which must not be NULL), then scores and selects
 * as nsa_topk does: for 16-bit operands, D <= 128, NC <= 1024 and topk <= 64 in ONE kernel that
 * keeps a row's scores in shared memory (no score buffer in global memory), otherwise as a scoring
 * and a selection kernel.  Same outputs, bit for bit, as nsa_pool_rows + nsa_topk.
 * Replaces pooling + topk_cuda of the two citations above (the score tile + merge of
 * topk.cu:296-439). */
int nsa_pool_score_topk(const void* q_pooled, const int64_t q_stride[3], const void* k,
                        const int64_t k_stride[3], int32_t B, int32_t MG, int32_t H, int32_t D,
                        int64_t N, int32_t topk, float scale, const nsa_topk_mask* mask,
                        void* k_pooled_out, int32_t* out_idx, float* out_scores, void* workspace,
                        size_t workspace_bytes, int32_t dtype, void* stream);

/* The whole block selection from the RAW tensors: pools the keys k [B,N,H,D] in blocks of
 * mask->block_size and the queries q [B,M,H,D] in groups of mask->q_group_size (-> q_pooled_out
 * [B,MG,H,D] contiguous, MG = ceil(M / q_group_size)) in ONE launch, then scores and selects as
 * nsa_topk does; the kernels follow one another as programmatic dependents.
 * Workspace: nsa_topk_workspace_bytes(B, MG, H, ceil(N / mask->block_size)).
 * Replaces, in one call, the query-group pooling of nsa/ops/index_topk.py:72-79, the key pooling
 * of models/transformers/causal_wan_nsa_model.py:408-409 and topk_cuda (topk.cu:664-808). */
int nsa_select_blocks(const void* q, const int64_t q_stride[3], const void* k,
                      const int64_t k_stride[3], int32_t B, int64_t M, int32_t H, int32_t D, int64_t N,
                      int32_t topk, float scale, const nsa_topk_mask* mask, void* q_pooled_out,
                      void* k_pooled_out, int32_t* out_idx, float* out_scores, void* workspace,
                      size_t workspace_bytes, int32_t dtype, void* stream);

/* Block-sharded memories (block b on rank b mod R as local block b / R): the ids a rank attends
 * itself, out[i] = ids[i] / R where ids[i] >= 0 and ids[i] mod R == r, else -1.  No counterpart in
 * the reference (it has no multi-GPU mode for this path). */
int nsa_local_block_ids(const int32_t* ids, int64_t n, int32_t R, int32_t r, int32_t* out, void* stream);

/* Merge R candidate lists (idx/scores [R][rows][T], global ids) into the global top-k with
 * the same order rule.  New for block-sharded KV; the order rule is topk.cu:100-102 and the
 * packed-key merge it mirrors is topk.cu:442-471. */
int nsa_merge_candidates(const int32_t* idx, const float* scores, int32_t R, int64_t rows,
                         int32_t T, int32_t topk, int32_t* out_idx, float* out_scores,
                         void* stream);

/* Selection attention forward: out [B,M,H,D] (q dtype) and lse float [B,H,M].
 * Rows with no visible key give out = 0, lse = -inf.
 * Replaces sel_fwd_cuda (selection_fwd.cu:934-966) and, with NSA_KV_PAGED,
 * sel_fwd_ptr_cuda (selection_fwd.cu:968-992). */
int nsa_sel_fwd(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                const int32_t* block_indices, const int64_t idx_stride[4], void* out,
                const int64_t out_stride[3], float* lse, int32_t B, int64_t M, int32_t H,
                int32_t D, int32_t T, int32_t block_size, int32_t chunk_size, int32_t causal,
                int32_t group_size, float scale, int32_t dtype, void* stream);

/* Attention of every query over ONE contiguous range of KV blocks, [first_block, first_block +
 * n_blocks) clipped to kv->n_tokens, not causal: out [B,M,H,D] and lse float [B,H,M], the same
 * results as nsa_sel_fwd with every query group listing exactly those blocks (blocks without a
 * page are skipped; an empty range gives out = 0, lse = -inf).  Because the list is shared, the
 * kernel works on 128 query rows per thread block instead of one group.  Built for bf16, D = 128,
 * block_size = 64, H > 1, dense or paged K/V, n_blocks <= 1024: NSA_ERR_UNSUPPORTED otherwise
 * (list the blocks and call nsa_sel_fwd).
 * A long range over few query tiles is cut into spans that run on thread blocks of their own and
 * are joined by nsa_merge_partials, when `workspace` (nsa_range_fwd_workspace_bytes, 0 when no cut
 * pays) is given and `out` is contiguous; without it the call runs uncut.
 * Serves the layer's compressed and sliding-window branches, which the reference runs through
 * its dense attention() (models/transformers/causal_wan_nsa_model.py:506-508). */
size_t nsa_range_fwd_workspace_bytes(int32_t B, int64_t M, int32_t H, int32_t D, int32_t n_blocks);
int nsa_range_fwd(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                  int32_t first_block, int32_t n_blocks, void* out, const int64_t out_stride[3],
                  float* lse, int32_t B, int64_t M, int32_t H, int32_t D, int32_t block_size,
                  float scale, void* workspace, size_t workspace_bytes, int32_t dtype, void* stream);

/* Inverted (block -> query groups) CSR index: groups int32 [B,H,MG*T], offsets int32
 * [B,H,NS+1]; pairs that are negative, out of range or causally invisible are dropped.
 * Replaces build_inverted_index_impl (inverted_index.cu:106-178). */
size_t nsa_inverted_index_workspace_bytes(int32_t B, int32_t H, int64_t NS);
int nsa_inverted_index(const int32_t* block_indices, const int64_t idx_stride[4], int32_t B,
                       int32_t MG, int32_t H, int32_t T, int64_t NS, int32_t block_size,
                       int32_t chunk_size, int32_t causal, int32_t group_size, int32_t* groups,
                       int32_t* offsets, void* workspace, size_t workspace_bytes, void* stream);

/* Selection attention backward: dq (q dtype, q layout), dk/dv (k dtype, contiguous
 * [B,N,H,D]); dk/dv of every token are written (zero where no group selected it), with no
 * atomics: one thread block owns each dK/dV tile and walks its bucket of query groups in
 * ascending group order, so results are bit-reproducible.
 * Replaces sel_bwd_cuda (selection_bwd.cu:1329-1407). */
size_t nsa_sel_bwd_workspace_bytes(int32_t B, int64_t M, int32_t H, int64_t N, int32_t T,
                                   int32_t block_size, int32_t group_size);
int nsa_sel_bwd(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                const int32_t* block_indices, const int64_t idx_stride[4], const void* out,
                const int64_t out_stride[3], const float* lse, const void* d_out,
                const int64_t do_stride[3], void* dq, const int64_t dq_stride[3], void* dk,
                void* dv, int32_t B, int64_t M, int32_t H, int32_t D, int32_t T,
                int32_t block_size, int32_t chunk_size, int32_t causal, int32_t group_size,
                float scale, void* workspace, size_t workspace_bytes, int32_t dtype,
                void* stream);

/* The two halves of nsa_sel_bwd as separate calls (the inverted index is built with
 * nsa_inverted_index in between).  nsa_sel_bwd_dq also writes delta = sum_d(out * d_out),
 * float [B,H,M], which nsa_sel_bwd_dkv reads together with the CSR index.  nsa_sel_bwd_dkv
 * takes a 256-byte device workspace (the work counter of its persistent thread blocks).
 * Replace sel_bwd_dq_*_kernel (selection_bwd.cu:310-912) and sel_bwd_dkv_mma_kernel
 * (selection_bwd.cu:916-1044). */
int nsa_sel_bwd_dq(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                   const int32_t* block_indices, const int64_t idx_stride[4], const void* out,
                   const int64_t out_stride[3], const float* lse, const void* d_out,
                   const int64_t do_stride[3], void* dq, const int64_t dq_stride[3], float* delta,
                   int32_t B, int64_t M, int32_t H, int32_t D, int32_t T, int32_t block_size,
                   int32_t chunk_size, int32_t causal, int32_t group_size, float scale,
                   int32_t dtype, void* stream);
int nsa_sel_bwd_dkv(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                    const int32_t* groups, const int32_t* offsets, const float* lse,
                    const float* delta, const void* d_out, const int64_t do_stride[3], void* dk,
                    void* dv, int32_t B, int64_t M, int32_t H, int32_t D, int32_t T,
                    int32_t block_size, int32_t chunk_size, int32_t causal, int32_t group_size,
                    float scale, void* workspace, size_t workspace_bytes, int32_t dtype,
                    void* stream);

/* The backward with P and dS computed ONCE.  The reference's backward computes S = Q K^T,
 * dP = dO V^T and the exponentials in its dQ kernels and again in its dK/dV kernel
 * (selection_bwd.cu:310-912 and :916-1044); here the dQ call can store P and dS of every (query
 * group, head, selected slot) pair - bf16, 2 x 8 KiB per pair, nsa_sel_bwd_pds_bytes() in all
 * (B * MG * H * T * 16 KiB: 233 MB for 74 groups x 12 heads x 16 slots) - and the dK/dV call then
 * only streams those tiles with the Q / dO rows into its two products.  Sequence:
 *   nsa_inverted_index_slots  - nsa_inverted_index plus `slots` int32 [B,H,MG*T]: the position of
 *                               every bucket entry in its group's id list (T <= 256, MG < 2^23);
 *                               buckets are ordered by (group, slot)
 *   nsa_sel_bwd_dq_pds        - nsa_sel_bwd_dq; *pds_written (host) = 1 when the tiles were written
 *                               (bf16, D = 128, 64-token blocks, 16 <= group_size <= 64, T <= 64, H > 1,
 *                               dense or paged K/V, pds large enough), else 0 and `pds` is untouched
 *   nsa_sel_bwd_dkv_pds       - nsa_sel_bwd_dkv; with slots and pds non-NULL (only after
 *                               *pds_written == 1) it takes the tiles, with NULL it recomputes.
 * dK / dV keep their fixed summation order (ascending group, then slot): bit-reproducible. */
size_t nsa_sel_bwd_pds_bytes(int32_t B, int64_t M, int32_t H, int32_t T, int32_t group_size);
int nsa_inverted_index_slots(const int32_t* block_indices, const int64_t idx_stride[4], int32_t B,
                             int32_t MG, int32_t H, int32_t T, int64_t NS, int32_t block_size,
                             int32_t chunk_size, int32_t causal, int32_t group_size,
                             int32_t* groups, int32_t* offsets, int32_t* slots, void* workspace,
                             size_t workspace_bytes, void* stream);
int nsa_sel_bwd_dq_pds(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                       const int32_t* block_indices, const int64_t idx_stride[4], const void* out,
                       const int64_t out_stride[3], const float* lse, const void* d_out,
                       const int64_t do_stride[3], void* dq, const int64_t dq_stride[3],
                       float* delta, int32_t B, int64_t M, int32_t H, int32_t D, int32_t T,
                       int32_t block_size, int32_t chunk_size, int32_t causal, int32_t group_size,
                       float scale, void* pds, size_t pds_bytes, int32_t* pds_written,
                       int32_t dtype, void* stream);
int nsa_sel_bwd_dkv_pds(const void* q, const int64_t q_stride[3], const nsa_kv_source* kv,
                        const int32_t* groups, const int32_t* offsets, const int32_t* slots,
                        const void* pds, size_t pds_bytes, const float* lse, const float* delta,
                        const void* d_out, const int64_t do_stride[3], void* dk, void* dv,
                        int32_t B, int64_t M, int32_t H, int32_t D, int32_t T, int32_t block_size,
                        int32_t chunk_size, int32_t causal, int32_t group_size, float scale,
                        void* workspace, size_t workspace_bytes, int32_t dtype, void* stream);

/* dK/dV of the pointer path (sel_bwd_ptr_cuda, selection_bwd.cu:1409-1527; accessor
 * bwd_common.cuh:64-121).  The K/V block with id `bid` of head h and its fp32 gradient scratch are
 * found through four [H, MAXB] tables of int64 byte addresses (element strides base_stride[0..1]):
 * block-level (blocks_per_chunk = 0: entry bid) or chunk-level (entry bid / blocks_per_chunk plus
 * (bid % blocks_per_chunk) * in_chunk_block_bytes_*); batch b adds b * batch_stride_*_bytes.
 * A block whose id is >= n_blocks_per_head[h] (table may be NULL), whose entry is >= max_base or
 * whose four addresses are not all non-zero is skipped.  Every block with a non-empty bucket gets
 * its [block_size, D] fp32 tiles WRITTEN (token stride stride_dbn floats); other scratch is left
 * untouched.  groups / offsets are nsa_inverted_index's output for NS blocks, chunk_size 1,
 * causal 0 (the pointer path carries no token ids).  dQ of the pointer path is nsa_sel_bwd_dq
 * with an NSA_KV_PTR source. */
int nsa_sel_bwd_dkv_ptr(const void* q, const int64_t q_stride[3], const int64_t* base_k,
                        const int64_t* base_v, const int64_t* base_dk, const int64_t* base_dv,
                        const int64_t base_stride[2], int32_t max_base,
                        const int32_t* n_blocks_per_head, int64_t batch_stride_kv_bytes,
                        int64_t batch_stride_dkv_bytes, int64_t stride_bn, int64_t stride_dbn,
                        int32_t blocks_per_chunk, int64_t in_chunk_block_bytes_kv,
                        int64_t in_chunk_block_bytes_dkv, const int32_t* groups,
                        const int32_t* offsets, int64_t NS, const float* lse, const float* delta,
                        const void* d_out, const int64_t do_stride[3], int32_t B, int64_t M,
                        int32_t H, int32_t D, int32_t T, int32_t block_size, int32_t group_size,
                        float scale, int32_t dtype, void* stream);

/* Merge R attention partials over disjoint key sets: outs [R][B,M,H,D] (dtype),
 * lses float [R][B,H,M] -> out, lse.  O = sum_r exp(lse_r - lse) O_r.  New for
 * block-sharded KV (no counterpart: the reference never splits one row's keys). */
int nsa_merge_partials(const void* outs, const float* lses, int32_t R, int32_t B, int64_t M,
                       int32_t H, int32_t D, void* out, float* lse, int32_t dtype, void* stream);

/* nsa_merge_partials over packed rows, for a row-split exchange: a row is the partial output of
 * one query token for all heads (H*D elements of `dtype`) followed by its H log-sum-exps (fp32),
 * H*D*2 + H*4 bytes rounded up to a multiple of 16.  parts [R][rows] rows (a rank's share of the rows, one copy
 * from every rank) -> merged [rows] rows of the same format.  New for block-sharded KV. */
int nsa_merge_packed_rows(const void* parts, int32_t R, int64_t rows, int32_t H, int32_t D, void* merged,
                          int32_t dtype, void* stream);

/* Three-branch gate + sum that consumes the selection output
 * (models/transformers/causal_wan_nsa_model.py:378-386, 541-546):
 *   g = clamp(g_logits, -10, 10); (g_cmp, g_slc, g_swa) = sigmoid(g) (softmax = 0) or softmax over
 *   the three logits (softmax = 1); x = g_cmp*o_cmp + g_slc*o_slc + g_swa*o_swa.
 * g_logits [rows, 3], branches and x [rows, D] contiguous in `dtype` (bf16 / fp16), rows = B*M*H;
 * a NULL branch is skipped (the reference's skip_module), its gate still takes part in the softmax.
 * Products and partial sums are rounded to `dtype` left to right, as the eager expression does. */
int nsa_gate_combine(const void* g_logits, const void* o_cmp, const void* o_slc, const void* o_swa,
                     void* x, int64_t rows, int32_t D, int32_t softmax, int32_t dtype, void* stream);
/* Backward of nsa_gate_combine: d_o_i = g_i * dx (NULL = not wanted), d_g_logits [rows, 3]
 * (zero where a logit lies outside [-10, 10]).  D = 64, 128 or 256. */
int nsa_gate_combine_bwd(const void* g_logits, const void* o_cmp, const void* o_slc,
                         const void* o_swa, const void* dx, void* d_g_logits, void* d_o_cmp,
                         void* d_o_slc, void* d_o_swa, int64_t rows, int32_t D, int32_t softmax,
                         int32_t dtype, void* stream);

/* Block id -> int64 byte address tables, same contract as build_ptr_table_cuda
 * (ptr_table.cu:59-127): 0 for id < 0, id >= n_blocks_per_head[h], chunk >= max_chunks or a
 * zero chunk base. */
int nsa_build_ptr_table(const int32_t* block_indices, const int64_t idx_stride[4],
                        const int64_t* base_k, const int64_t* base_v,
                        const int32_t* n_blocks_per_head, int32_t B, int32_t MG, int32_t H,
                        int32_t T, int32_t max_chunks, int64_t batch_stride,
                        int32_t blocks_per_chunk, int64_t in_chunk_block_bytes, int64_t* ptr_k,
                        int64_t* ptr_v, void* stream);

/* ---- fixed-page block KV cache ----------------------------------------------------
 * Pool: k_pool / v_pool [num_pages][page_tokens][D]; a page holds one (head, block); block j
 * = tokens [j*page_tokens, (j+1)*page_tokens).  block_table int32 [H][max_blocks] -> page or
 * -1; page_owner int32 [num_pages] -> key h*max_blocks + bid or -1 (free); page_stamp int64
 * [num_pages] = epoch of last use (the LRU clock); k_pooled / v_pooled [H][max_blocks][D]
 * hold the mean key / value of EVERY block ever appended (evicted blocks stay candidates of
 * the top-k, as in the reference, and come back from the host tier when selected).
 * `status` is a device int32 the kernels set to a negative nsa_status on a device-detected
 * problem (pool exhausted); the host reads it when it chooses to.  Data-dependent counts
 * stay on the device (n_dev pointers), so no call needs a host synchronisation. */

/* Append S new tokens (k_new/v_new [S,H,D]; kv_stride = element strides of (s, h)) at
 * absolute token position pos0 <= n_tokens, the number of tokens the cache holds before the call
 * (pos0 < n_tokens rewrites tokens in place; the blocks it touches must be resident or receive a
 * page whose rows outside the rewritten range already hold the block's data).  A touched block
 * that has no page takes
 * new_pages[h*n_touched_blocks + j] (device int32; e.g. fresh page ids or the victims list).
 * Writes the tokens with 16-byte stores, stamps the pages with `epoch`, and recomputes the
 * pooled key / value of every touched block over the tokens it now holds (v_pooled may be
 * NULL).  Replaces MMCache.update_cache, chunk-per-head branch (models/cache.py:478-502), the
 * pooled-cache append of models/transformers/causal_wan_nsa_model.py:479-504, and
 * block_range_kernel (block_kv_range.cu:13-37). */
int nsa_cache_append(const void* k_new, const void* v_new, const int64_t kv_stride[2], int64_t S,
                     int64_t pos0, int64_t n_tokens, int32_t H, int32_t D, void* k_pool, void* v_pool,
                     int32_t page_tokens, int32_t* block_table, int32_t max_blocks,
                     const int32_t* new_pages, int32_t n_touched_blocks, int32_t* page_owner,
                     int64_t* page_stamp, int64_t epoch, void* k_pooled, void* v_pooled,
                     int32_t* status, int32_t dtype, void* stream);

/* Rotary embedding of a chunk of keys in the reordered token order (f h w fs hs ws) of the
 * pooling windows (causal_reorder_rope_apply, models/transformers/causal_wan_nsa_model.py:72-105).
 * freqs_* are complex128 tables (re, im pairs of float64; rope_params, wan_model.py:37-43):
 * freqs_f [frames, c_f], freqs_h [rows, c_h], freqs_w [columns, c_w], c_f + c_h + c_w = D / 2
 * (the reference's split: c_f = D/2 - 2*(D/2/3), c_h = c_w = D/2/3). */
typedef struct nsa_rope {
  const void* freqs_f;
  const void* freqs_h;
  const void* freqs_w;
  int32_t c_f, c_h, c_w;
  int32_t grid_h, grid_w;          /* latent rows / columns of a frame */
  int32_t pool_f, pool_h, pool_w;  /* pooling window of the token order (1, 1, 1 = plain f h w order) */
  int32_t start_frame;             /* frame index of the chunk's first frame */
} nsa_rope;

/* nsa_cache_append with the rotary embedding applied to the new keys on their way into the pages
 * (float64 products, rounded float64 -> float32 -> dtype like the reference), so the un-roped
 * keys are read once and the roped ones never exist outside the cache; the pooled keys are those
 * of the roped keys.  S must be whole groups of pool_f frames.  Replaces
 * causal_reorder_rope_apply + update_cache + the pooled-cache append
 * (causal_wan_nsa_model.py:72-105, 479-504; cache.py:478-502). */
int nsa_cache_append_rope(const void* k_new, const void* v_new, const int64_t kv_stride[2], int64_t S,
                          int64_t pos0, int64_t n_tokens, int32_t H, int32_t D, void* k_pool, void* v_pool,
                          int32_t page_tokens, int32_t* block_table, int32_t max_blocks,
                          const int32_t* new_pages, int32_t n_touched_blocks, int32_t* page_owner,
                          int64_t* page_stamp, int64_t epoch, void* k_pooled, void* v_pooled,
                          int32_t* status, int32_t dtype, const nsa_rope* rope, void* stream);

/* The same rotary embedding for a chunk of queries: x [S,H,D] (x_stride = element strides of (s, h))
 * -> out [S,H,D] contiguous, float64 products rounded like the reference.  Replaces
 * causal_reorder_rope_apply on the query side (causal_wan_nsa_model.py:72-105, 463-466). */
int nsa_rope_apply(const void* x, const int64_t x_stride[2], int64_t S, int32_t H, int32_t D, void* out,
                   int32_t dtype, const nsa_rope* rope, void* stream);

/* Selected (head, block) pairs of a flattened [B,MG,H,T] id table -> strictly ascending
 * unique keys (cid*H + h)*bpc + loc (cid = bid / bpc, loc = bid % bpc): out_unique[0] = count
 * (may exceed cap), out_unique[1..cap] keys.  `stamp` is a persistent int32 [H*max_blocks]
 * scratch of the cache; epoch32 >= 1 must differ from call to call.  With a block_table
 * (needs bpc == max_blocks, so key = h*max_blocks + bid): resident pages among the keys get
 * page_stamp = epoch (the LRU touch) and out_missing (may be NULL) receives, in the same
 * format, the keys whose block has no page; `counters` (device int64 [4], may be NULL) then
 * receives counters[0] += keys found resident (LRU hits), counters[1] += keys without a page
 * (misses) - the hit / miss counts of MMCache (models/cache.py:156-163, 673-699, 713-716).
 * Replaces dedup_run (block_kv_dedup.cu:16-120; block_kv_ops.h:26-31) and the host LRU touch
 * loop of nsa/ops/selection/padded_ptr/wrapper.py:253-362. */
size_t nsa_cache_dedup_workspace_bytes(int64_t n_keys);
int nsa_cache_dedup_touch(const int32_t* block_indices, int64_t n_entries, int32_t H, int32_t T,
                          int32_t max_blocks, int32_t bpc, int32_t* stamp, int32_t epoch32,
                          const int32_t* block_table, int64_t* page_stamp, int64_t epoch,
                          int32_t* out_unique, int32_t* out_missing, int32_t cap, int64_t* counters,
                          void* workspace, size_t workspace_bytes, void* stream);

/* n pages to (re)use: free pages first (ascending page id), then the least recently used owned
 * pages, ascending (stamp, page): owner's block id below protect_from_bid and not stamped with
 * the current epoch.  n = *n_dev when n_dev != NULL
 * (clamped to cap), else the host value n.  Sets *status = NSA_ERR_EXHAUSTED and pads with
 * -1 when fewer pages qualify.  Replaces the OrderedDict pop of
 * MMCache.lru_touch_per_head (models/cache.py:673-699). */
int nsa_cache_select_victims(const int32_t* page_owner, const int64_t* page_stamp,
                             int32_t num_pages, int32_t max_blocks, int32_t protect_from_bid,
                             int64_t epoch, int32_t n, const int32_t* n_dev, int32_t cap,
                             int32_t* victims, int32_t* status, void* stream);

/* Move pages between the pool and the host tier (pinned, device-mapped memory; the slot of
 * key is host_k/host_v + key*page_bytes) and publish AFTER the copy of the page is complete:
 *   direction 0 (evict): pages[i] -> slot of its owner; then block_table[owner] = -1 and the
 *                        page is free (host_k == NULL drops the data instead of saving it);
 *   direction 1 (fetch): slot of keys[1+i] -> pages[i]; then block_table[key] = page,
 *                        owner and stamp set.  keys is a count-first list as written by
 *                        nsa_cache_dedup_touch (out_missing).
 *   direction 2 (stage): write-behind eviction, first half - pages[i] -> slot i of a STAGING buffer in
 *                        device memory (passed as host_k / host_v), its owner -> keys[i] (written; -1 =
 *                        nothing staged); tables updated as by an evict, so the page is free at once;
 *   direction 3 (drain): second half, meant for a stream of its own - staging slot i (passed as
 *                        k_pool / v_pool) -> the host slot of keys[i]; a fetch of those keys must be
 *                        ordered after it (pages and the tables are not used).
 * n = *n_dev when n_dev != NULL (grid sized by cap), else n.  `counters` (device int64 [4], may
 * be NULL): counters[2] += pages evicted, counters[3] += pages fetched (bytes moved = pages x
 * 2 x page_bytes).
 * Replaces gather_publish_clear (block_kv_gather.cu:13-45) and the copies of
 * MMCache.flush_offload (models/cache.py:1032-1142). */
int nsa_cache_move_pages(int32_t direction, const int32_t* pages, const int32_t* keys, int32_t n,
                         const int32_t* n_dev, int32_t cap, void* k_pool, void* v_pool,
                         int64_t page_bytes, void* host_k, void* host_v, int32_t* block_table,
                         int32_t* page_owner, int64_t* page_stamp, int64_t epoch, int64_t* counters,
                         void* stream);

/* The reference's K1 and K2 entry points with their own contracts (block_kv_ops.h:12-24):
 * desc int64 SoA [src_k|src_v|dst_k|dst_v|pub_k|pub_v] x n_fetch then clear x n_clear;
 * *ctas_launched = n_fetch + ceil(n_clear/256).  K3 (dedup_run) is nsa_cache_dedup_touch with
 * block_table = NULL. */
int nsa_gather_publish_clear(const int64_t* desc, int64_t n_fetch, int64_t n_clear,
                             int64_t block_bytes, int32_t wide, int32_t num_warps,
                             int64_t* ctas_launched, void* stream);
int nsa_block_range(int64_t* table, int32_t* n_valid, int32_t H, int64_t MB, int64_t first_bid,
                    int64_t n_blocks, int64_t k_base, int64_t v_base, int64_t head_stride_bytes,
                    int64_t block_bytes, int64_t n_valid_value, int32_t write_k, int32_t write_v,
                    int32_t clear, void* stream);

/* Measurement aid (no counterpart in the reference): one thread block per SM pulls the whole buffer
 * `passes` times into shared memory with 16 KiB bulk copies, three per stage, four stages - the
 * streaming dK/dV kernel's copy shape with nothing computed.  The caller times the launch; bytes
 * moved = floor(bytes / 49152) * 49152 * passes.  bench.py quotes the rate over an L2-resident and
 * over an HBM-resident buffer as that kernel's delivery rooflines. */
int nsa_probe_bulk_stream(const void* buf, size_t bytes, int32_t passes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OMNIMEM_B200_H_ */
