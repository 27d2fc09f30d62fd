// Dense <-> block-compressed value movement and compressed row / column sums.
//
// Replaces dense_to_bcs_val / bcs_val_to_dense / bcsr_val_sum_row / bcsr_val_sum_col
// (sparta/tesa/templates/block_compressed.cu.j2:172-288).  The block count is read from device
// memory and the grid walks blocks with a stride, so no launch depends on a host copy of nnz.
#include "common.cuh"

namespace sparta {
namespace {

struct MoveParams {
  const uint8_t* src;
  uint8_t* dst;
  const void* idx;
  const int32_t* nnz;
  int H, W, BH, BW, elem_bytes, is_bcsr, idx_is_64;
  long long val_stride_blocks;
};

__device__ __forceinline__ void decode(const MoveParams& p, int t, int& by, int& bx) {
  int v = p.idx_is_64 ? (int)(reinterpret_cast<const long long*>(p.idx)[t] & 0xffffffffll)
                      : reinterpret_cast<const int32_t*>(p.idx)[t];
  if (p.is_bcsr) { by = v >> 16; bx = v & 0xffff; }
  else { bx = v >> 16; by = v & 0xffff; }
}

// VEC = bytes moved per thread per step (16, 8, 4, 2 or 1); GATHER: dense -> vals, else vals -> dense
template <int VEC, bool GATHER>
__global__ void __launch_bounds__(256) bcs_move_kernel(MoveParams p) {
  // never walk past the value buffer: an index build whose capacity was too small reports the full count
  const int nnz = p.val_stride_blocks > 0 ? (int)min((long long)*p.nnz, p.val_stride_blocks) : *p.nnz;
  const size_t row_bytes = (size_t)p.BW * p.elem_bytes;        // bytes of one block row
  const size_t blk_bytes = row_bytes * p.BH;
  const int vec_per_row = (int)(row_bytes / VEC);
  const int vec_per_blk = vec_per_row * p.BH;
  const uint8_t* dense_c = (GATHER ? p.src : p.dst) + (size_t)blockIdx.y * p.H * p.W * p.elem_bytes;
  const uint8_t* vals_c = (GATHER ? p.dst : p.src) + (size_t)blockIdx.y * p.val_stride_blocks * blk_bytes;
  uint8_t* dense = const_cast<uint8_t*>(dense_c);
  uint8_t* vals = const_cast<uint8_t*>(vals_c);
  for (int t = blockIdx.x; t < nnz; t += gridDim.x) {
    int by, bx;
    decode(p, t, by, bx);
    uint8_t* d0 = dense + ((size_t)by * p.BH * p.W + (size_t)bx * p.BW) * p.elem_bytes;
    uint8_t* v0 = vals + (size_t)t * blk_bytes;
    for (int i = threadIdx.x; i < vec_per_blk; i += blockDim.x) {
      const int y = i / vec_per_row, x = i - y * vec_per_row;
      uint8_t* dp = d0 + (size_t)y * p.W * p.elem_bytes + (size_t)x * VEC;
      uint8_t* vp = v0 + (size_t)i * VEC;
      if constexpr (VEC == 16) {
        if (GATHER) *reinterpret_cast<uint4*>(vp) = __ldg(reinterpret_cast<const uint4*>(dp));
        else *reinterpret_cast<uint4*>(dp) = __ldg(reinterpret_cast<const uint4*>(vp));
      } else if constexpr (VEC == 8) {
        if (GATHER) *reinterpret_cast<uint2*>(vp) = __ldg(reinterpret_cast<const uint2*>(dp));
        else *reinterpret_cast<uint2*>(dp) = __ldg(reinterpret_cast<const uint2*>(vp));
      } else if constexpr (VEC == 4) {
        if (GATHER) *reinterpret_cast<uint32_t*>(vp) = __ldg(reinterpret_cast<const uint32_t*>(dp));
        else *reinterpret_cast<uint32_t*>(dp) = __ldg(reinterpret_cast<const uint32_t*>(vp));
      } else if constexpr (VEC == 2) {
        if (GATHER) *reinterpret_cast<uint16_t*>(vp) = __ldg(reinterpret_cast<const uint16_t*>(dp));
        else *reinterpret_cast<uint16_t*>(dp) = __ldg(reinterpret_cast<const uint16_t*>(vp));
      } else {
        if (GATHER) *vp = __ldg(dp);
        else *dp = __ldg(vp);
      }
    }
  }
}

template <bool GATHER>
int launch_move(const void* src, void* dst, const void* idx, const int32_t* nnz, int batch, int H,
                int W, int BH, int BW, int elem_bytes, int is_bcsr, int idx_is_64,
                int64_t val_stride_blocks, int64_t grid_hint, void* stream) {
  if (!src || !dst || !idx || !nnz || batch <= 0 || H <= 0 || W <= 0) return SPARTA_ERR_BAD_ARG;
  if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return SPARTA_ERR_BAD_ARG;
  if (!valid_bcs_block(BH) || !valid_bcs_block(BW) || H % BH || W % BW) return SPARTA_ERR_SHAPE;
  if (val_stride_blocks < 0 || batch > 65535) return SPARTA_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!GATHER) {
    cudaError_t e = cudaMemsetAsync(dst, 0, (size_t)batch * H * W * elem_bytes, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  MoveParams p{static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), idx, nnz, H, W, BH, BW,
               elem_bytes, is_bcsr, idx_is_64, (long long)val_stride_blocks};
  // widest vector that divides a block row and keeps every access aligned
  const size_t row_bytes = (size_t)BW * elem_bytes, ld_bytes = (size_t)W * elem_bytes;
  int vec = 16;
  while (vec > 1 && (row_bytes % vec || ld_bytes % vec || !aligned(src, vec) || !aligned(dst, vec) ||
                     ((size_t)H * ld_bytes) % vec))
    vec >>= 1;
  if (vec < elem_bytes) return SPARTA_ERR_ALIGN;
  long long gx = grid_hint > 0 ? grid_hint : (long long)(H / BH) * (W / BW);
  const long long cap = (long long)kNumSMs * 16;
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  dim3 grid((unsigned)gx, batch), block(256);
  switch (vec) {
    case 16: bcs_move_kernel<16, GATHER><<<grid, block, 0, st>>>(p); break;
    case 8: bcs_move_kernel<8, GATHER><<<grid, block, 0, st>>>(p); break;
    case 4: bcs_move_kernel<4, GATHER><<<grid, block, 0, st>>>(p); break;
    case 2: bcs_move_kernel<2, GATHER><<<grid, block, 0, st>>>(p); break;
    default: bcs_move_kernel<1, GATHER><<<grid, block, 0, st>>>(p); break;
  }
  return launch_status();
}

// One warp per output element group: row sums -> out[batch, H], column sums -> out[batch, W].
template <typename T, bool ROW>
__global__ void __launch_bounds__(256) bcs_sum_kernel(const T* vals, T* out, const int32_t* row_ptr,
                                                      const int32_t* idx, const int32_t* nnz_p, int H,
                                                      int W, int BH, int BW, long long val_stride_blocks) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int n_out = ROW ? H : W;
  if (warp >= n_out) return;
  const T* v = vals + (size_t)blockIdx.y * val_stride_blocks * BH * BW;
  float acc = 0.f;
  if (ROW) {
    const int br = warp / BH, y = warp % BH;
    const int t0 = row_ptr[br], t1 = row_ptr[br + 1];
    const int n = (t1 - t0) * BW;
    for (int j = lane; j < n; j += 32) {
      const int t = t0 + j / BW, x = j % BW;
      acc += to_float(v[((size_t)t * BH + y) * BW + x]);
    }
  } else {
    // column sums walk every kept block and keep those of this block column
    const int bc = warp / BW, x = warp % BW;
    const int nnz = val_stride_blocks > 0 ? (int)min((long long)*nnz_p, val_stride_blocks) : *nnz_p;
    for (int t = 0; t < nnz; ++t) {
      if ((idx[t] & 0xffff) != bc) continue;
      for (int y = lane; y < BH; y += 32) acc += to_float(v[((size_t)t * BH + y) * BW + x]);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[(size_t)blockIdx.y * n_out + warp] = from_float<T>(acc);
}

template <typename T>
int launch_sum(const void* vals, void* out, const int32_t* row_ptr, const int32_t* idx,
               const int32_t* nnz, int batch, int H, int W, int BH, int BW, int axis_is_row,
               int64_t vsb, cudaStream_t st) {
  const int n_out = axis_is_row ? H : W;
  dim3 grid((n_out * 32 + 255) / 256, batch), block(256);
  if (axis_is_row)
    bcs_sum_kernel<T, true><<<grid, block, 0, st>>>(static_cast<const T*>(vals), static_cast<T*>(out),
                                                    row_ptr, idx, nnz, H, W, BH, BW, vsb);
  else
    bcs_sum_kernel<T, false><<<grid, block, 0, st>>>(static_cast<const T*>(vals), static_cast<T*>(out),
                                                     row_ptr, idx, nnz, H, W, BH, BW, vsb);
  return launch_status();
}

}  // namespace
}  // namespace sparta

using namespace sparta;

extern "C" int sparta_bcs_gather(const void* dense, void* vals, const void* idx, const int32_t* nnz,
                                 int batch, int H, int W, int BH, int BW, int elem_bytes, int is_bcsr,
                                 int idx_is_64, int64_t val_stride_blocks, int64_t grid_blocks_hint,
                                 void* stream) {
  return launch_move<true>(dense, vals, idx, nnz, batch, H, W, BH, BW, elem_bytes, is_bcsr, idx_is_64,
                           val_stride_blocks, grid_blocks_hint, stream);
}

extern "C" int sparta_bcs_scatter(const void* vals, void* dense, const void* idx, const int32_t* nnz,
                                  int batch, int H, int W, int BH, int BW, int elem_bytes, int is_bcsr,
                                  int idx_is_64, int64_t val_stride_blocks, int64_t grid_blocks_hint,
                                  void* stream) {
  return launch_move<false>(vals, dense, idx, nnz, batch, H, W, BH, BW, elem_bytes, is_bcsr, idx_is_64,
                            val_stride_blocks, grid_blocks_hint, stream);
}

extern "C" int sparta_bcs_sum(const void* vals, void* out, const int32_t* row_ptr,
                              const int32_t* bcsr_idx, const int32_t* nnz, int batch, int H, int W,
                              int BH, int BW, int dtype, int axis_is_row, int64_t val_stride_blocks,
                              void* stream) {
  if (!vals || !out || !row_ptr || !bcsr_idx || !nnz || batch <= 0) return SPARTA_ERR_BAD_ARG;
  if (!valid_bcs_block(BH) || !valid_bcs_block(BW) || H % BH || W % BW) return SPARTA_ERR_SHAPE;
  if (batch > 65535 || val_stride_blocks < 0) return SPARTA_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SPARTA_F32:
      return launch_sum<float>(vals, out, row_ptr, bcsr_idx, nnz, batch, H, W, BH, BW, axis_is_row,
                               val_stride_blocks, st);
    case SPARTA_F16:
      return launch_sum<__half>(vals, out, row_ptr, bcsr_idx, nnz, batch, H, W, BH, BW, axis_is_row,
                                val_stride_blocks, st);
    case SPARTA_BF16:
      return launch_sum<__nv_bfloat16>(vals, out, row_ptr, bcsr_idx, nnz, batch, H, W, BH, BW,
                                       axis_is_row, val_stride_blocks, st);
    default:
      return SPARTA_ERR_BAD_ARG;
  }
}
