// Internal parameter block shared by the block-sparse matmul kernels.
#pragma once

#include "common.cuh"

namespace sparta {

enum BsmmMode { MODE_SDD = 0, MODE_DSD = 1, MODE_DDS = 2 };

struct BsmmParams {
  const void* A;
  const void* B;
  const void* bias;
  void* C;
  const int32_t* ptr;
  const void* idx;
  const int32_t* nnz;
  int mode;
  int batch, M, K, N;
  int BM, BK, BN;
  int trans_a, trans_b, compressed, idx_is_64;
  int dtype;
  int n_index_sets;
  long long ptr_stride, idx_stride, val_stride_blocks, grid_blocks_hint;
};

// FMA kernels: bsmm_simt takes every layout (and hands the SparseLinear layout with small square
// blocks to the register-tiled dsd kernel).  Return a status code of sparta_b200.h.
int bsmm_simt(const BsmmParams& p, cudaStream_t st);
bool dsd_fma_supported(const BsmmParams& p);
int dsd_fma_launch(const BsmmParams& p, cudaStream_t st);

// tcgen05 kernels: return SPARTA_ERR_UNSUPPORTED when the configuration is outside their coverage.
bool dsd_tc_supported(const BsmmParams& p);
int dsd_tc_launch(const BsmmParams& p, cudaStream_t st);
bool dds_tc_supported(const BsmmParams& p);
int dds_tc_launch(const BsmmParams& p, cudaStream_t st);
inline bool bsmm_tc_supported(const BsmmParams& p) { return dsd_tc_supported(p) || dds_tc_supported(p); }
inline int bsmm_tc(const BsmmParams& p, cudaStream_t st) {
  return p.mode == MODE_DDS ? dds_tc_launch(p, st) : dsd_tc_launch(p, st);
}

// fused attention with two Q tiles per CTA (attn_tc2.cu): query lengths that are a multiple of 256
bool attn_tc2_supported(int Nt);
bool kv_exceeds_l2(int heads, int Ns, int D);
int attn_tc2_launch(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                    const int32_t* bcsr_idx, const uint8_t* mask, float scale_log2, int heads, int Nt, int Ns,
                    int D, int dtype, float* lse, int32_t* status, void* const* copies, int n_copies, cudaStream_t st);

// fused attention for head dim 64 with one K block per step and four CTAs per SM (attn_tc64.cu)
int attn_tc64_launch(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                     const int32_t* bcsr_idx, const uint8_t* mask, float scale_log2, int heads, int Nt, int Ns,
                     int dtype, float* lse, int32_t* status, cudaStream_t st);

// whether the tcgen05 matmul / fused attention kernels are compiled into this build
bool bsmm_tc_available();
bool attn_tc_available();

}  // namespace sparta
