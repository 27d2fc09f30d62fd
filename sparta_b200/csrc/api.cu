// C-ABI entry points that validate arguments and pick a kernel family.
#include "bsmm.cuh"

using namespace sparta;

extern "C" int sparta_version(void) { return SPARTA_B200_VERSION; }

extern "C" const char* sparta_status_string(int status) {
  switch (status) {
    case SPARTA_OK: return "ok";
    case SPARTA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unknown enum)";
    case SPARTA_ERR_SHAPE: return "shape not divisible by the block sizes or beyond the index packing limits";
    case SPARTA_ERR_UNSUPPORTED: return "no prebuilt kernel covers this configuration";
    case SPARTA_ERR_WORKSPACE: return "workspace missing or too small";
    case SPARTA_ERR_ALIGN: return "pointer or leading dimension not aligned as required";
    case SPARTA_ERR_DRIVER: return "CUDA driver entry point for tensor maps unavailable";
    case SPARTA_ERR_DEVICE_STATUS: return "a kernel reported a bounded wait that ran out";
    default:
      return status > 0 ? cudaGetErrorString(static_cast<cudaError_t>(status)) : "unknown status";
  }
}

extern "C" int sparta_device_supported(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) return 0;
  return major == 10;
}

static int bsmm_entry(int mode, const sparta_bsmm_args* a, void* stream) {
  if (!a || !a->A || !a->B || !a->C || !a->idx || !a->nnz) return SPARTA_ERR_BAD_ARG;
  if (mode != MODE_DDS && !a->ptr) return SPARTA_ERR_BAD_ARG;
  if (a->batch <= 0 || a->M <= 0 || a->K <= 0 || a->N <= 0) return SPARTA_ERR_BAD_ARG;
  if (a->BM <= 0 || a->BK <= 0 || a->BN <= 0) return SPARTA_ERR_BAD_ARG;
  if (a->dtype < SPARTA_F32 || a->dtype > SPARTA_BF16) return SPARTA_ERR_BAD_ARG;
  if (a->M % a->BM || a->K % a->BK || a->N % a->BN) return SPARTA_ERR_SHAPE;
  if (a->n_index_sets != 1 && a->n_index_sets != a->batch) return SPARTA_ERR_BAD_ARG;
  if (a->compressed && a->val_stride_blocks < 0) return SPARTA_ERR_BAD_ARG;
  if (mode == MODE_DDS && a->idx_is_64) return SPARTA_ERR_UNSUPPORTED;  // dds walks the BCSR array

  BsmmParams p;
  p.A = a->A; p.B = a->B; p.bias = a->bias; p.C = a->C;
  p.ptr = a->ptr; p.idx = a->idx; p.nnz = a->nnz;
  p.mode = mode;
  p.batch = a->batch; p.M = a->M; p.K = a->K; p.N = a->N;
  p.BM = a->BM; p.BK = a->BK; p.BN = a->BN;
  p.trans_a = a->trans_a != 0; p.trans_b = a->trans_b != 0;
  p.compressed = a->compressed != 0; p.idx_is_64 = a->idx_is_64 != 0;
  p.dtype = a->dtype;
  p.n_index_sets = a->n_index_sets;
  p.ptr_stride = a->ptr_stride; p.idx_stride = a->idx_stride;
  p.val_stride_blocks = a->val_stride_blocks; p.grid_blocks_hint = a->grid_blocks_hint;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mode == MODE_DDS && !p.compressed) {
    const size_t esz = p.dtype == SPARTA_F32 ? 4 : 2;
    cudaError_t e = cudaMemsetAsync(p.C, 0, (size_t)p.batch * p.M * p.N * esz, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  switch (a->impl) {
    case SPARTA_IMPL_AUTO:
      if (bsmm_tc_supported(p)) return bsmm_tc(p, st);
      return bsmm_simt(p, st);
    case SPARTA_IMPL_SIMT:
      return bsmm_simt(p, st);
    case SPARTA_IMPL_TCGEN05:
      if (!bsmm_tc_supported(p)) return SPARTA_ERR_UNSUPPORTED;
      return bsmm_tc(p, st);
    default:
      return SPARTA_ERR_BAD_ARG;
  }
}

extern "C" int sparta_bsmm_sdd(const sparta_bsmm_args* args, void* stream) {
  return bsmm_entry(MODE_SDD, args, stream);
}
extern "C" int sparta_bsmm_dsd(const sparta_bsmm_args* args, void* stream) {
  return bsmm_entry(MODE_DSD, args, stream);
}
extern "C" int sparta_bsmm_dds(const sparta_bsmm_args* args, void* stream) {
  return bsmm_entry(MODE_DDS, args, stream);
}

// ---- tile table -------------------------------------------------------------------------------
namespace {
const int kSimtSizes[] = {8, 16, 32, 64};
}

extern "C" int sparta_tile_table(int op, int dtype, sparta_tile_entry* out, int max_entries) {
  if (op < 0 || op > 4 || dtype < SPARTA_F32 || dtype > SPARTA_BF16) return SPARTA_ERR_BAD_ARG;
  int n = 0;
  auto emit = [&](sparta_tile_entry e) {
    if (out && n < max_entries) out[n] = e;
    ++n;
  };
  if (op <= 2) {
    // tcgen05 entries first: they are the preferred choice where they apply
    if (dtype != SPARTA_F32 && bsmm_tc_available()) {
      if (op == 0) emit({op, dtype, SPARTA_IMPL_TCGEN05, 32, 32, 128, -1, 1, 1});
      if (op == 1) emit({op, dtype, SPARTA_IMPL_TCGEN05, 128, 32, 32, 0, -1, 1});
      if (op == 2) emit({op, dtype, SPARTA_IMPL_TCGEN05, 32, 64, 32, -1, -1, -1});
    }
    for (int bm : kSimtSizes)
      for (int bk : kSimtSizes)
        for (int bn : kSimtSizes) emit({op, dtype, SPARTA_IMPL_SIMT, bm, bk, bn, -1, -1, -1});
  } else if (op == 3) {
    const int hs[] = {8, 16, 32, 64, 128}, ws[] = {16, 32, 64, 128};
    for (int h : hs)
      for (int w : ws) emit({op, dtype, SPARTA_IMPL_SIMT, h, 0, w, -1, -1, -1});
  } else {
    if (dtype != SPARTA_F32 && attn_tc_available()) emit({op, dtype, SPARTA_IMPL_TCGEN05, 64, 64, 64, 0, 1, 1});
  }
  return n;
}
