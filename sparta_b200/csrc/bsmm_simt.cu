// Block-sparse matmul, FMA path: every mode (sdd / dsd / dds), transposition, compressed or
// dense-shaped sparse operand, fp32 / fp16 / bf16 storage with fp32 accumulation, CTA tiles from
// 8 to 64 per dimension.  This is the full-coverage kernel; the tcgen05 kernels take the large
// half-precision configurations.
//
// Replaces sparta_sparse_matmul_{sdd,dsd,dds}.cuh.j2 and openai_sparse_matmul_{sdd,dsd,dds}.cuh.j2
// (sparta/specializer/kernels/templates/).  As in the reference the CTA tile (BM, BK, BN) equals the
// block size of the sparse operand in its two dimensions (sparta/specializer/kernels/matmul.py:53-97).
#include "bsmm.cuh"

namespace sparta {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxTile = 64;

struct Operand {   // where the current K-chunk of an operand tile lives
  const void* base;
  long long s_outer;  // stride (elements) along M (for A) or N (for B)
  long long s_k;      // stride along K
};

template <typename T>
__device__ __forceinline__ void stage_tile(float* smem, const Operand& op, int outer, int tk, int ld) {
  // smem[kk * ld + o] = tile(o, kk); consecutive threads follow the unit-stride dimension
  const T* g = static_cast<const T*>(op.base);
  const int total = outer * tk;
  if (op.s_k == 1) {
    for (int i = threadIdx.x; i < total; i += kThreads) {
      const int o = i / tk, kk = i - o * tk;
      smem[kk * ld + o] = to_float(g[(long long)o * op.s_outer + kk]);
    }
  } else {
    for (int i = threadIdx.x; i < total; i += kThreads) {
      const int kk = i / outer, o = i - kk * outer;
      smem[kk * ld + o] = to_float(g[(long long)o * op.s_outer + (long long)kk * op.s_k]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) bsmm_simt_kernel(BsmmParams p) {
  __shared__ float As[kMaxTile * (kMaxTile + 1)];
  __shared__ float Bs[kMaxTile * (kMaxTile + 1)];
  const int tm = p.BM, tn = p.BN, tk = p.BK;
  const int lda = tm + 1, ldb = tn + 1;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;

  const int set = p.n_index_sets > 1 ? (p.mode == MODE_DDS ? blockIdx.y : blockIdx.z) : 0;
  const int32_t* ptr = p.ptr ? p.ptr + (long long)set * p.ptr_stride : nullptr;
  const int32_t* idx32 = reinterpret_cast<const int32_t*>(p.idx) + (long long)set * p.idx_stride;
  const long long* idx64 = reinterpret_cast<const long long*>(p.idx) + (long long)set * p.idx_stride;
  const int nnz = p.nnz[set];
  const int batch_id = p.mode == MODE_DDS ? blockIdx.y : blockIdx.z;

  const T* A = static_cast<const T*>(p.A);
  const T* B = static_cast<const T*>(p.B);
  T* C = static_cast<T*>(p.C);
  const long long vstride = p.val_stride_blocks;  // blocks per batch element of the compressed tensor

  // batch offsets
  const bool a_comp = p.mode == MODE_SDD && p.compressed;
  const bool b_comp = p.mode == MODE_DSD && p.compressed;
  const bool c_comp = p.mode == MODE_DDS && p.compressed;
  A += a_comp ? (long long)batch_id * vstride * tm * tk : (long long)batch_id * p.M * p.K;
  B += b_comp ? (long long)batch_id * vstride * tn * tk : (long long)batch_id * p.K * p.N;
  C += c_comp ? (long long)batch_id * vstride * tm * tn : (long long)batch_id * p.M * p.N;
  const T* bias = p.bias ? static_cast<const T*>(p.bias) + (long long)batch_id * p.N : nullptr;

  // dense-operand strides
  const long long a_sm = p.trans_a ? 1 : p.K, a_sk = p.trans_a ? p.M : 1;
  const long long b_sn = p.trans_b ? p.K : 1, b_sk = p.trans_b ? 1 : p.N;

  const int out_first = p.mode == MODE_DDS ? blockIdx.x : 0;
  const int out_step = p.mode == MODE_DDS ? gridDim.x : 1;
  // dds: never past the compressed output buffer (an index build with too small a capacity reports the full count)
  const int out_last = p.mode == MODE_DDS ? ((c_comp && vstride > 0 && nnz > vstride) ? (int)vstride : nnz) : 1;

  for (int ob = out_first; ob < out_last; ob += out_step) {
    int by, bx, c_pos = ob;
    int chunk0, chunk1;
    if (p.mode == MODE_DDS) {
      int v;
      if (p.idx_is_64) { long long w = idx64[ob]; v = (int)(w & 0xffffffffll); c_pos = (int)(w >> 32); }
      else v = idx32[ob];
      by = v >> 16; bx = v & 0xffff;
      chunk0 = 0; chunk1 = p.K / tk;
    } else {
      by = blockIdx.y; bx = blockIdx.x;
      const int line = p.mode == MODE_SDD ? by : bx;
      chunk0 = ptr[line]; chunk1 = ptr[line + 1];
    }

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int t = chunk0; t < chunk1; ++t) {
      int kb = t, pos = t;
      if (p.mode != MODE_DDS) {
        if (p.idx_is_64) { long long w = idx64[t]; kb = (int)(w & 0xffff); pos = (int)(w >> 32); }
        else kb = idx32[t] & 0xffff;
      }
      const long long k0 = (long long)kb * tk;
      Operand oa, obp;
      if (a_comp) {
        // stored block: BM x BK rows (or BK x BM when trans_a), row-major
        oa.base = A + (long long)pos * tm * tk;
        oa.s_outer = p.trans_a ? 1 : tk;
        oa.s_k = p.trans_a ? tm : 1;
      } else {
        oa.base = A + (long long)by * tm * a_sm + k0 * a_sk;
        oa.s_outer = a_sm; oa.s_k = a_sk;
      }
      if (b_comp) {
        // stored block: BN x BK (trans_b) or BK x BN, row-major
        obp.base = B + (long long)pos * tn * tk;
        obp.s_outer = p.trans_b ? tk : 1;
        obp.s_k = p.trans_b ? 1 : tn;
      } else {
        obp.base = B + (long long)bx * tn * b_sn + k0 * b_sk;
        obp.s_outer = b_sn; obp.s_k = b_sk;
      }
      __syncthreads();
      stage_tile<T>(As, oa, tm, tk, lda);
      stage_tile<T>(Bs, obp, tn, tk, ldb);
      __syncthreads();
#pragma unroll 4
      for (int kk = 0; kk < tk; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = (ty + 16 * i < tm) ? As[kk * lda + ty + 16 * i] : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = (tx + 16 * j < tn) ? Bs[kk * ldb + tx + 16 * j] : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    }

    // epilogue
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = ty + 16 * i;
      if (m >= tm) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = tx + 16 * j;
        if (n >= tn) continue;
        float v = acc[i][j];
        if (bias) v += to_float(bias[(long long)bx * tn + n]);
        if (c_comp)
          C[((long long)c_pos * tm + m) * tn + n] = from_float<T>(v);
        else
          C[((long long)by * tm + m) * p.N + (long long)bx * tn + n] = from_float<T>(v);
      }
    }
  }
}

template <typename T>
int launch(const BsmmParams& p, cudaStream_t st) {
  dim3 grid;
  if (p.mode == MODE_DDS) {
    long long gx = p.grid_blocks_hint > 0 ? p.grid_blocks_hint : (long long)(p.M / p.BM) * (p.N / p.BN);
    const long long cap = 65535ll * 8;
    if (gx > cap) gx = cap;
    grid = dim3((unsigned)gx, p.batch, 1);
  } else {
    grid = dim3(p.N / p.BN, p.M / p.BM, p.batch);
  }
  bsmm_simt_kernel<T><<<grid, kThreads, 0, st>>>(p);
  return launch_status();
}

}  // namespace

int bsmm_simt(const BsmmParams& p, cudaStream_t st) {
  if (dsd_fma_supported(p)) return dsd_fma_launch(p, st);
  if (p.BM > kMaxTile || p.BN > kMaxTile || p.BK > kMaxTile) return SPARTA_ERR_UNSUPPORTED;
  if (p.BM < 4 || p.BN < 4 || p.BK < 4) return SPARTA_ERR_UNSUPPORTED;
  if (p.batch > 65535 || p.M / p.BM > 65535) return SPARTA_ERR_SHAPE;
  switch (p.dtype) {
    case SPARTA_F32: return launch<float>(p, st);
    case SPARTA_F16: return launch<__half>(p, st);
    case SPARTA_BF16: return launch<__nv_bfloat16>(p, st);
    default: return SPARTA_ERR_BAD_ARG;
  }
}

}  // namespace sparta
