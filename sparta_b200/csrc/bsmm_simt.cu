// Block-sparse matmul, FMA path: every mode (sdd / dsd / dds), transposition, compressed or
// dense-shaped sparse operand, fp32 / fp16 / bf16 storage with fp32 accumulation, CTA tiles from
// 8 to 64 per dimension.  This is the full-coverage kernel; the tcgen05 kernels take the large
// half-precision configurations.
//
// Replaces sparta_sparse_matmul_{sdd,dsd,dds}.cuh.j2 and openai_sparse_matmul_{sdd,dsd,dds}.cuh.j2
// (sparta/specializer/kernels/templates/).  As in the reference the CTA tile (BM, BK, BN) equals the
// block size of the sparse operand in its two dimensions (sparta/specializer/kernels/matmul.py:53-97).
#include <cstring>

#include "bsmm.cuh"

namespace sparta {
namespace {

constexpr int kMaxTile = 64;
// A thread computes R x R outputs (R = 4, 2 or 1, chosen so that a CTA has at least 64 threads where the tile
// allows it: a 32 x 32 tile is 64 threads of 4 x 4, a 64 x 64 tile 256 threads); its R rows and R columns are
// contiguous, so that one vector read of shared memory fetches them: 2 reads per 16 multiply-adds for R = 4.
// (A fixed 16 x 16 grid of threads with 4 x 4 outputs each, as before, spent three quarters of its multiply-adds
// on padding for 32 x 32 tiles.)  Shared memory is sized by the tile, so small tiles put many CTAs on an SM.

struct Operand {   // where the current K-chunk of an operand tile lives
  const void* base;
  long long s_outer;  // stride (elements) along M (for A) or N (for B)
  long long s_k;      // stride along K
};

// four consecutive elements as fp32 (16-byte aligned for fp32, 8-byte for the 16-bit types)
template <typename T>
__device__ __forceinline__ float4 load4(const T* src) {
  if constexpr (sizeof(T) == 4) {
    return *reinterpret_cast<const float4*>(src);
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    T e[4];
    memcpy(e, &raw, 8);
    return make_float4(to_float(e[0]), to_float(e[1]), to_float(e[2]), to_float(e[3]));
  }
}

// smem[kk * ld + o] = tile(o, kk) for an outer x tk tile (sizes are powers of two >= 4).  With `vec` (aligned
// operand) a thread moves four elements of the operand's unit-stride dimension at a time and has four such loads
// in flight before it stores the first: a CTA may be as small as 64 threads, and one scalar load per loop turn
// left a lone CTA (a nearly empty mask) waiting out the memory latency sixteen times per tile.
template <typename T>
__device__ __forceinline__ void stage_tile(float* smem, const Operand& op, int outer, int tk, int ld, int outer_shift,
                                           int tk_shift, bool vec) {
  const T* g = static_cast<const T*>(op.base);
  const int total = outer * tk;
  const int nt = blockDim.x;
  if (vec) {
    const int nvec = total >> 2;
    const bool k_unit = op.s_k == 1;  // else the outer dimension has unit stride
    const int vshift = (k_unit ? tk_shift : outer_shift) - 2, vmask = (1 << vshift) - 1;
    const long long line_stride = k_unit ? op.s_outer : op.s_k;
    for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * nt) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * nt;
        if (i < nvec) v[u] = load4<T>(g + (long long)(i >> vshift) * line_stride + ((i & vmask) << 2));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * nt;
        if (i < nvec) {
          const int line = i >> vshift, q = (i & vmask) << 2;
          if (k_unit) {  // line = o, q = first of four kk
            float* d = smem + q * ld + line;
            d[0] = v[u].x; d[ld] = v[u].y; d[2 * ld] = v[u].z; d[3 * ld] = v[u].w;
          } else {       // line = kk, q = first of four o
            *reinterpret_cast<float4*>(smem + line * ld + q) = v[u];
          }
        }
      }
    }
    return;
  }
  if (op.s_k == 1) {
    for (int i = threadIdx.x; i < total; i += nt) {
      const int o = i >> tk_shift, kk = i & (tk - 1);
      smem[kk * ld + o] = to_float(g[(long long)o * op.s_outer + kk]);
    }
  } else {
    for (int i = threadIdx.x; i < total; i += nt) {
      const int kk = i >> outer_shift, o = i & (outer - 1);
      smem[kk * ld + o] = to_float(g[(long long)o * op.s_outer + (long long)kk * op.s_k]);
    }
  }
}

template <int R>
__device__ __forceinline__ void load_frag(const float* src, float (&out)[R]) {  // R contiguous floats, R * 4-byte aligned
  if constexpr (R == 4) {
    const float4 v = *reinterpret_cast<const float4*>(src);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else if constexpr (R == 2) {
    const float2 v = *reinterpret_cast<const float2*>(src);
    out[0] = v.x; out[1] = v.y;
  } else {
    out[0] = src[0];
  }
}

template <typename T, int R>
__global__ void __launch_bounds__(256) bsmm_simt_kernel(BsmmParams p) {
  extern __shared__ __align__(16) float simt_smem[];
  const int tm = p.BM, tn = p.BN, tk = p.BK;
  const int lda = tm + 4, ldb = tn + 4;  // rows stay 16-byte aligned for the vector reads
  float* As = simt_smem;
  float* Bs = simt_smem + tk * lda;
  const int tm_shift = __ffs(tm) - 1, tn_shift = __ffs(tn) - 1, tk_shift = __ffs(tk) - 1;
  // vector staging needs 16-byte (8-byte for 16-bit types) aligned rows: aligned bases and dimensions that are
  // multiples of four elements (tile sizes are; the operands' leading dimensions are multiples of the tiles)
  const bool vec = ((reinterpret_cast<uintptr_t>(p.A) | reinterpret_cast<uintptr_t>(p.B)) & 15) == 0;
  const bool vec_c = (reinterpret_cast<uintptr_t>(p.C) & 15) == 0;
  const int cols = tn / R;  // threads along N
  const int ty = threadIdx.x / cols, tx = threadIdx.x - ty * cols;

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

    float acc[R][R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int j = 0; j < R; ++j) acc[i][j] = 0.f;

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
      stage_tile<T>(As, oa, tm, tk, lda, tm_shift, tk_shift, vec);
      stage_tile<T>(Bs, obp, tn, tk, ldb, tn_shift, tk_shift, vec);
      __syncthreads();
      const float* ap = As + ty * R;
      const float* bp = Bs + tx * R;
#pragma unroll 4
      for (int kk = 0; kk < tk; ++kk) {
        float a[R], b[R];
        load_frag<R>(ap + kk * lda, a);
        load_frag<R>(bp + kk * ldb, b);
#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
          for (int j = 0; j < R; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    }

    // epilogue
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int m = ty * R + i;
      T* crow = c_comp ? C + ((long long)c_pos * tm + m) * tn + tx * R
                       : C + ((long long)by * tm + m) * p.N + (long long)bx * tn + tx * R;
      alignas(16) T out[R];
#pragma unroll
      for (int j = 0; j < R; ++j) {
        float v = acc[i][j];
        if (bias) v += to_float(bias[(long long)bx * tn + tx * R + j]);
        out[j] = from_float<T>(v);
      }
      if (R > 1 && vec_c) {  // the thread's R outputs of a row as one store
        if constexpr (R * sizeof(T) == 16) *reinterpret_cast<uint4*>(crow) = *reinterpret_cast<const uint4*>(out);
        else if constexpr (R * sizeof(T) == 8) *reinterpret_cast<uint2*>(crow) = *reinterpret_cast<const uint2*>(out);
        else if constexpr (R * sizeof(T) == 4) *reinterpret_cast<uint32_t*>(crow) = *reinterpret_cast<const uint32_t*>(out);
      } else {
#pragma unroll
        for (int j = 0; j < R; ++j) crow[j] = out[j];
      }
    }
  }
}

template <typename T>
int launch(const BsmmParams& p, cudaStream_t st) {
  const int outputs = p.BM * p.BN;
  const int r = outputs >= 1024 ? 4 : (outputs >= 256 ? 2 : 1);  // outputs per thread and dimension
  const int threads = outputs / (r * r);                           // 64 .. 256 (16 for a 4 x 4 tile)
  const size_t smem = (size_t)p.BK * (p.BM + 4 + p.BN + 4) * sizeof(float);  // at most 34 KB
  dim3 grid;
  if (p.mode == MODE_DDS) {
    long long gx = p.grid_blocks_hint > 0 ? p.grid_blocks_hint : (long long)(p.M / p.BM) * (p.N / p.BN);
    const long long cap = 65535ll * 8;
    if (gx > cap) gx = cap;
    grid = dim3((unsigned)gx, p.batch, 1);
  } else {
    grid = dim3(p.N / p.BN, p.M / p.BM, p.batch);
  }
  if (r == 4) bsmm_simt_kernel<T, 4><<<grid, threads, smem, st>>>(p);
  else if (r == 2) bsmm_simt_kernel<T, 2><<<grid, threads, smem, st>>>(p);
  else bsmm_simt_kernel<T, 1><<<grid, threads, smem, st>>>(p);
  return launch_status();
}

}  // namespace

int bsmm_simt(const BsmmParams& p, cudaStream_t st) {
  if (dsd_fma_supported(p)) return dsd_fma_launch(p, st);
  if (p.BM > kMaxTile || p.BN > kMaxTile || p.BK > kMaxTile) return SPARTA_ERR_UNSUPPORTED;
  if (p.BM < 4 || p.BN < 4 || p.BK < 4) return SPARTA_ERR_UNSUPPORTED;
  if ((p.BM & (p.BM - 1)) || (p.BN & (p.BN - 1)) || (p.BK & (p.BK - 1))) return SPARTA_ERR_UNSUPPORTED;  // powers of two
  if (p.batch > 65535 || p.M / p.BM > 65535) return SPARTA_ERR_SHAPE;
  switch (p.dtype) {
    case SPARTA_F32: return launch<float>(p, st);
    case SPARTA_F16: return launch<__half>(p, st);
    case SPARTA_BF16: return launch<__nv_bfloat16>(p, st);
    default: return SPARTA_ERR_BAD_ARG;
  }
}

}  // namespace sparta
