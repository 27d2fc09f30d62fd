/*
 * sparta_b200.h -- C ABI of the B200 (sm_100a) block-sparse operator library.
 *
 * The reference (microsoft/SparTA) has no C ABI on this path: its native code is reached through
 * pycuda function handles captured in Python closures.  Each entry point below names the
 * reference closure / kernel it replaces (paths are relative to the reference project root).
 *
 * Conventions
 *   - every function returns an int status: 0 = ok, < 0 = argument problem found on the host before
 *     anything was launched, > 0 = a CUDA runtime error code (cudaError_t) from a launch;
 *   - nothing throws, nothing calls exit();
 *   - every pointer is a DEVICE pointer unless its name starts with h_;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - no function allocates device memory: scratch is passed in, its size comes from the matching
 *     *_workspace_bytes() query;
 *   - block counts that depend on the mask (nnz) are always read from device memory by the kernels,
 *     so no call needs a host synchronisation;
 *   - index packing follows the reference: BCSR entry = (block_row << 16) | block_col,
 *     BCSC entry = (block_col << 16) | block_row, and when both formats are built the BCSC entry is a
 *     64-bit word whose upper half holds the position of the block in BCSR order
 *     (sparta/tesa/templates/block_compressed.cu.j2:151,163-166).  Unlike the reference, entries
 *     inside a block row (column) are always in ascending column (row) order.
 */
#ifndef SPARTA_B200_H_
#define SPARTA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPARTA_B200_VERSION 100

/* status codes (< 0: host-side argument errors) */
#define SPARTA_OK 0
#define SPARTA_ERR_BAD_ARG (-1)      /* null pointer, non-positive size, unknown enum value        */
#define SPARTA_ERR_SHAPE (-2)        /* sizes not divisible by the block / tile sizes, or too large */
#define SPARTA_ERR_UNSUPPORTED (-3)  /* valid request that no prebuilt kernel covers                */
#define SPARTA_ERR_WORKSPACE (-4)    /* workspace missing or too small                              */
#define SPARTA_ERR_ALIGN (-5)        /* pointer or leading dimension not aligned as required        */
#define SPARTA_ERR_DRIVER (-6)       /* CUDA driver entry point (tensor-map encode) unavailable     */
#define SPARTA_ERR_DEVICE_STATUS (-7)/* a kernel reported a bounded wait that ran out              */

/* element types of the floating-point operands */
#define SPARTA_F32 0
#define SPARTA_F16 1
#define SPARTA_BF16 2

/* matmul kernel families ("_impl" in the reference's config dictionaries) */
#define SPARTA_IMPL_AUTO 0    /* pick from the tile table                                  */
#define SPARTA_IMPL_SIMT 1    /* fp32-accumulating FMA kernel, every dtype / layout        */
#define SPARTA_IMPL_TCGEN05 2 /* tcgen05 + TMEM + TMA kernel, fp16 / bf16, selected layouts */

/* library version (SPARTA_B200_VERSION of the build). */
int sparta_version(void);

/* human-readable text for a status code returned by any function of this header. */
const char* sparta_status_string(int status);

/* ---------------------------------------------------------------------------------------------
 * Dense mask -> block-compressed indexes.
 * Replaces BCSFunctionContext.build_indexes / _build_BCSR_indexes / _build_BCSC_indexes
 * (sparta/tesa/block_compressed.py:242-309) and the kernels bcs_index_1 / bcs_index_2
 * (sparta/tesa/templates/block_compressed.cu.j2:67-170) together with the torch.cumsum and the
 * .item() host synchronisation between them.
 *
 * mask      uint8 [n_masks, H, W]; a block is kept when any of its BH x BW bytes is non-zero.
 * row_ptr   int32 [n_masks, H/BH + 1]      (written when want_bcsr)
 * bcsr_idx  int32 [n_masks, idx_capacity]  (written when want_bcsr; first nnz entries valid)
 * col_ptr   int32 [n_masks, W/BW + 1]      (written when want_bcsc)
 * bcsc_idx  int32 [n_masks, idx_capacity] when only want_bcsc, int64 when both are requested
 * nnz       int32 [n_masks]  number of kept blocks
 * uniform   int32 [n_masks] or NULL; set to 1 when every kept block is completely non-zero
 *           (element masks then equal block masks), else 0
 * h_nnz     host (pinned) int32 [n_masks] or NULL; when given, an async copy of nnz is queued
 * idx_capacity  entries available per mask in the idx arrays; (H/BH)*(W/BW) always suffices
 * workspace sparta_bcs_build_workspace_bytes() bytes; it must be zero-filled once after allocation
 *           and is left zero-filled by every call that completes.
 */
size_t sparta_bcs_build_workspace_bytes(int n_masks, int H, int W, int BH, int BW);

int sparta_bcs_build(const uint8_t* mask, int n_masks, int H, int W, int BH, int BW,
                     int want_bcsr, int want_bcsc,
                     int32_t* row_ptr, int32_t* bcsr_idx, int32_t* col_ptr, void* bcsc_idx,
                     int64_t idx_capacity, int32_t* nnz, int32_t* uniform, int32_t* h_nnz,
                     void* workspace, size_t workspace_bytes, void* stream);

/* Index build without a caller-supplied workspace (no counterpart in the reference, which allocates
 * freely with torch).  For callers that cannot allocate device memory -- a serving loop with a memory
 * pool frozen after start-up, a plug-in whose host framework forbids cudaMalloc on its threads, a mask
 * update issued while another thread holds the allocator lock.  Same arguments and results as
 * sparta_bcs_build minus workspace / h_nnz; the scratch is a fixed SPARTA_BCS_STATIC_SCRATCH_BYTES array
 * inside the library, one per device.  Requests whose sparta_bcs_build_workspace_bytes() exceeds it
 * return SPARTA_ERR_WORKSPACE.  The first call on a device resolves the array's address: make it before
 * any stream capture.  Calls on one device share the array: do not let two of them overlap on the GPU. */
#define SPARTA_BCS_STATIC_SCRATCH_BYTES (1 << 20)

int sparta_bcs_build_static(const uint8_t* mask, int n_masks, int H, int W, int BH, int BW,
                            int want_bcsr, int want_bcsc,
                            int32_t* row_ptr, int32_t* bcsr_idx, int32_t* col_ptr, void* bcsc_idx,
                            int64_t idx_capacity, int32_t* nnz, int32_t* uniform, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Dense <-> compressed values.
 * Replaces BCSFunctionContext.convert / inverse (sparta/tesa/block_compressed.py:311-358) and
 * dense_to_bcs_val / bcs_val_to_dense (sparta/tesa/templates/block_compressed.cu.j2:172-220).
 * The reference handles fp32 only; here elem_bytes may be 1, 2 or 4 (masks, half types, fp32).
 *
 * dense   [batch, H, W] elements            vals  [batch, val_stride_blocks * BH * BW] elements
 * idx     packed block indexes (BCSR or BCSC packing, see is_bcsr; 64-bit entries when idx_is_64 --
 *         only the low 32 bits are used here, values always live at the loop position)
 * nnz     device int32: number of blocks to move
 * val_stride_blocks  blocks per batch element in `vals` (>= nnz)
 * sparta_bcs_scatter zero-fills `dense` first, like the reference's torch.zeros.
 */
int sparta_bcs_gather(const void* dense, void* vals, const void* idx, const int32_t* nnz,
                      int batch, int H, int W, int BH, int BW, int elem_bytes, int is_bcsr,
                      int idx_is_64, int64_t val_stride_blocks, int64_t grid_blocks_hint,
                      void* stream);

int sparta_bcs_scatter(const void* vals, void* dense, const void* idx, const int32_t* nnz,
                       int batch, int H, int W, int BH, int BW, int elem_bytes, int is_bcsr,
                       int idx_is_64, int64_t val_stride_blocks, int64_t grid_blocks_hint,
                       void* stream);

/* Row sums ([batch, H]) and column sums ([batch, W]) of compressed values stored in BCSR order.
 * Replaces BCSFunctionContext.row_sum / col_sum (sparta/tesa/block_compressed.py:360-403) and
 * bcsr_val_sum_row / bcsr_val_sum_col (block_compressed.cu.j2:222-288).  `out` is fully written.
 * idx is the BCSR index array (int32). */
int sparta_bcs_sum(const void* vals, void* out, const int32_t* row_ptr, const int32_t* bcsr_idx,
                   const int32_t* nnz, int batch, int H, int W, int BH, int BW, int dtype,
                   int axis_is_row, int64_t val_stride_blocks, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Block-sparse matrix multiplication  C = op(A) * op(B) (+ bias).
 * Replaces the launch closures SparseMatMulKernel.update_func builds
 * (sparta/specializer/kernels/matmul.py:151-188) and the kernels
 * sparta_sparse_matmul_{sdd,dsd,dds}.cuh.j2 / openai_sparse_matmul_{sdd,dsd,dds}.cuh.j2
 * (sparta/specializer/kernels/templates/).  Mode letters describe A, B, C in that order
 * (matmul.py:60-84): sdd = A sparse, dsd = B sparse, dds = C sparse.
 *
 * Dense operands:  A is [batch, M, K] (trans_a: [batch, K, M]); B is [batch, K, N]
 * (trans_b: [batch, N, K]); C is [batch, M, N]; bias is [batch, N] or NULL.
 * The sparse operand is stored either dense-shaped (compressed = 0) or as
 * [batch, val_stride_blocks * block elements] in index order, each block row-major in its stored
 * orientation (compressed = 1).  Sparse block shape of the stored tensor (Appendix of matmul.py:53-97):
 *   sdd: BM x BK (trans_a: BK x BM, BCSC, ptr = col_ptr);   dsd: trans_b ? BN x BK (BCSR) : BK x BN (BCSC);
 *   dds: BM x BN (BCSR; ptr unused).
 * ptr / idx / nnz   index arrays from sparta_bcs_build; idx_is_64 selects the 64-bit BCSC form whose
 *                   upper half is the value position.
 * n_index_sets      1 = every batch element shares one mask (the reference), or == batch for one
 *                   mask per batch element; ptr_stride / idx_stride are the per-set strides in entries.
 * val_stride_blocks blocks per batch element in the compressed tensor.
 * For dds with compressed = 0 the dense C is zero-filled first (matmul.py:171).
 * impl              SPARTA_IMPL_*; AUTO uses the tile table.  grid_blocks_hint bounds the dds grid
 *                   (pass idx_capacity or the host's nnz if known; <= 0 lets the library choose).
 * SPARTA_IMPL_TCGEN05 covers, for fp16 / bf16 (fp32 accumulation):
 *   dsd  trans_a = 0, compressed = 1, BM = 128, BK = BN = 32, M % 128 == 0, K <= 8192, one index set:
 *        trans_b = 1 with the 32-bit BCSR (the SparseLinear weight layout) or trans_b = 0 with the BCSC,
 *        32- or 64-bit (its input gradient);
 *   sdd  trans_b = 1, compressed = 1, BM = BK = 32, BN = 128, N % 128 == 0, K <= 8192, one index set:
 *        trans_a = 0 with the 32-bit BCSR or trans_a = 1 with the BCSC, 32- or 64-bit;
 *   dds  either trans_a, either trans_b, 32-bit BCSR, BM = BN = 32, BK = 64, M % 128 == 0, N <= 32768,
 *        compressed or dense output, one index set or one per batch element;
 * and returns SPARTA_ERR_UNSUPPORTED otherwise.  SPARTA_IMPL_SIMT (and AUTO outside that coverage)
 * takes every mode, transposition and dtype with CTA tiles 4 .. 64 per dimension.
 */
typedef struct sparta_bsmm_args {
  const void* A;
  const void* B;
  const void* bias;
  void* C;
  const int32_t* ptr;
  const void* idx;
  const int32_t* nnz;
  int32_t batch, M, K, N;
  int32_t BM, BK, BN;
  int32_t trans_a, trans_b, compressed, idx_is_64;
  int32_t dtype, impl;
  int32_t n_index_sets;
  int64_t ptr_stride, idx_stride, val_stride_blocks, grid_blocks_hint;
} sparta_bsmm_args;

int sparta_bsmm_sdd(const sparta_bsmm_args* args, void* stream);
int sparta_bsmm_dsd(const sparta_bsmm_args* args, void* stream);
int sparta_bsmm_dds(const sparta_bsmm_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Masked softmax over the kept blocks of every row, y = softmax(x * scale) on unmasked elements.
 * Replaces the closures of SparseSoftmaxForwardKernel / SparseSoftmaxBackwardKernel.update_func
 * (sparta/specializer/kernels/softmax.py:64-89,115-141) and
 * sparta_sparse_softmax_{forward,backward}.cuh.j2.  `scale` is 1/temperature, as the reference
 * passes it (sparta/specializer/funtional/batch_softmax.py:19).
 * x, y, (dy, dx): [batch, H, W] (compressed = 0) or [batch, val_stride_blocks*BH*BW] (compressed = 1);
 * mask: uint8 in the same layout as x (one copy, shared by the batch) or NULL = every element of
 * a kept block takes part.  Masked elements and, for compressed = 0, dropped blocks are written 0.
 * With compressed = 0 the output is zero-filled before the kernel runs, so it must not alias an input
 * (SPARTA_ERR_BAD_ARG); compressed tensors may be processed in place.
 */
int sparta_softmax_fwd(const void* x, void* y, const int32_t* row_ptr, const int32_t* bcsr_idx,
                       const int32_t* nnz, const uint8_t* mask, float scale, int batch, int H, int W,
                       int BH, int BW, int compressed, int dtype, int64_t val_stride_blocks,
                       void* stream);

int sparta_softmax_bwd(const void* dy, const void* y, void* dx, const int32_t* row_ptr,
                       const int32_t* bcsr_idx, const int32_t* nnz, const uint8_t* mask, float scale,
                       int batch, int H, int W, int BH, int BW, int compressed, int dtype,
                       int64_t val_stride_blocks, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Fused sparse attention forward  O = softmax(mask(Q K^T * scale)) V  over kept blocks only.
 * Replaces the three launches of SparseAttention.forward
 * (sparta/specializer/operators/sparse_attention.py:76-80): dds(Q,K^T) -> sparse softmax -> sdd(P,V);
 * the score tensor is never written to global memory.
 * Q: [heads, Nt, D]; K, V: [heads, Ns, D]; O: [heads, Nt, D]; fp16 or bf16; D in {64, 128}.
 * row_ptr / bcsr_idx / nnz: BCSR of the [Nt, Ns] mask with BLK x BLK blocks (BLK = 64), shared by
 * every head.  mask: the dense uint8 [Nt, Ns] mask for element-level masking inside kept blocks, or
 * NULL when kept blocks are completely non-zero.  lse: optional fp32 [heads, Nt] log-sum-exp output.
 * status: optional device int32[4]; a bounded wait that runs out stores a non-zero code there.
 */
size_t sparta_attn_fwd_workspace_bytes(int heads, int Nt, int Ns, int D, int BLK);

int sparta_attn_fwd(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                    const int32_t* bcsr_idx, const int32_t* nnz, const uint8_t* mask, float scale,
                    int heads, int Nt, int Ns, int D, int BLK, int dtype, float* lse,
                    int32_t* status, void* workspace, size_t workspace_bytes, void* stream);

/* The same forward with the all-gather of the outputs fused into it, for heads sharded over the GPUs of one
 * box (no counterpart in the reference, which has no multi-GPU code; the configuration "sharded by
 * batch x head with outputs all-gathered over NVLink" ends in this exchange).  copies[0 .. n_copies-1] are
 * device addresses -- normally in peers' memory, mapped into this process (symmetric memory, IPC) -- laid
 * out like O: every output tile is stored to O and, from shared memory with bulk tensor stores, to each
 * copy, so the transfer over NVLink overlaps the remaining tiles' compute and no separate collective pass
 * reads O again.  The copies are complete when the kernel is; peers learn of it by whatever barrier the
 * caller uses between ranks.  Covered: D = 128 with Nt a multiple of 256 (SPARTA_ERR_UNSUPPORTED
 * otherwise: gather with a collective instead); n_copies <= SPARTA_ATTN_MAX_COPIES. */
#define SPARTA_ATTN_MAX_COPIES 7
int sparta_attn_fwd_gather(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                           const int32_t* bcsr_idx, const int32_t* nnz, const uint8_t* mask, float scale,
                           int heads, int Nt, int Ns, int D, int BLK, int dtype, float* lse,
                           int32_t* status, void* const* copies, int n_copies, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Tile table: what sparta.nn.tune searches over in the reference
 * (sparta/specializer/kernels/look_up_tables/sparta_matmul_lut.csv, sparta/nn/module_tuner.py:169)
 * becomes a fixed list of prebuilt kernels.  op: 0 sdd, 1 dsd, 2 dds, 3 softmax, 4 attention.
 * Fills up to max_entries records and returns the number of records available (>= 0). */
typedef struct sparta_tile_entry {
  int32_t op, dtype, impl;
  int32_t block_m, block_k, block_n; /* CTA tile = BCSR block sizes it accepts */
  int32_t trans_a, trans_b, compressed; /* -1 = any */
} sparta_tile_entry;

int sparta_tile_table(int op, int dtype, sparta_tile_entry* out_entries, int max_entries);

/* Status words of the tcgen05 kernels on the current device: all zero unless a bounded wait (on an
 * mbarrier) ran out, in which case the kernel stopped early and its output is invalid.  Word 0:
 * a producer (TMA-issuing) warp gave up, 1: an MMA-issuing warp, 2: the wait for the accumulator before
 * the epilogue (in the fused attention: the P.V issuer), 3: the warps between the two (the dsd kernel's
 * activation converters, the attention kernel's softmax warps).  Synchronises the device and clears the
 * words.
 * No counterpart in the reference, whose kernels contain no waits. */
int sparta_last_status(int32_t h_out[4]);

/* Whether the running device can execute this library's kernels (compute capability 10.x). */
int sparta_device_supported(int device);

#ifdef __cplusplus
}
#endif
#endif /* SPARTA_B200_H_ */
