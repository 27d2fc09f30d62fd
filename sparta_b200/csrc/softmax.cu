// Masked softmax over the kept blocks of each row, one warp per matrix row.  softmax_kernel: one online
// (max, sum) pass followed by one write pass, so x is read from HBM once (the second read hits L1/L2);
// softmax_fwd_vec_kernel: the forward pass with the row held in registers (16-byte accesses).
//
// Replaces sparta_sparse_softmax_forward.cuh.j2 / sparta_sparse_softmax_backward.cuh.j2
// (sparta/specializer/kernels/templates/): three global passes plus a per-thread index list there.
#include <type_traits>

#include "common.cuh"

namespace sparta {
namespace {

struct SmParams {
  const void* x;      // fwd: x      bwd: dy
  const void* y_in;   // bwd: y
  void* out;          // fwd: y      bwd: dx
  const int32_t* row_ptr;
  const int32_t* idx;
  const int32_t* nnz;
  const uint8_t* mask;
  float scale;
  int H, W, BH, BW, compressed;
  long long val_stride_blocks;
};

// element offset of (block t, row y inside the block, column x inside the block)
__device__ __forceinline__ long long elem_off(const SmParams& p, int t, int row, int y, int x) {
  if (p.compressed) return ((long long)t * p.BH + y) * p.BW + x;
  return (long long)row * p.W + (long long)(p.idx[t] & 0xffff) * p.BW + x;
}

template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(256) softmax_kernel(SmParams p) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= p.H) return;
  const long long bstride = p.compressed ? p.val_stride_blocks * p.BH * p.BW : (long long)p.H * p.W;
  const T* x = static_cast<const T*>(p.x) + (long long)blockIdx.y * bstride;
  T* out = static_cast<T*>(p.out) + (long long)blockIdx.y * bstride;
  const int br = row / p.BH, y = row - br * p.BH;
  const int t0 = p.row_ptr[br], t1 = p.row_ptr[br + 1];
  const int n = (t1 - t0) * p.BW;
  const int shift = __ffs(p.BW) - 1;  // BW is a power of two

  if (!BACKWARD) {
    float m = -INFINITY, s = 0.f;
    for (int j = lane; j < n; j += 32) {
      const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
      if (p.mask && !p.mask[o]) continue;
      const float v = to_float(x[o]) * p.scale;
      if (v > m) { s = s * expf(m - v) + 1.f; m = v; }
      else s += expf(v - m);
    }
    const float mw = warp_max(m);
    s = (m == -INFINITY) ? 0.f : s * expf(m - mw);
    s = warp_sum(s);
    const float inv = s > 0.f ? 1.f / s : 0.f;
    for (int j = lane; j < n; j += 32) {
      const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
      float r = 0.f;
      if (!p.mask || p.mask[o]) r = expf(to_float(x[o]) * p.scale - mw) * inv;
      out[o] = from_float<T>(r);
    }
  } else {
    const T* yv = static_cast<const T*>(p.y_in) + (long long)blockIdx.y * bstride;
    float dot = 0.f;
    for (int j = lane; j < n; j += 32) {
      const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
      if (p.mask && !p.mask[o]) continue;
      dot += to_float(x[o]) * to_float(yv[o]);
    }
    dot = warp_sum(dot);
    for (int j = lane; j < n; j += 32) {
      const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
      float r = 0.f;
      if (!p.mask || p.mask[o]) {
        const float yy = to_float(yv[o]);
        r = (to_float(x[o]) * yy - yy * dot) * p.scale;
      }
      out[o] = from_float<T>(r);
    }
  }
}

// Forward pass with 16-byte accesses for rows that fit in registers: a lane holds up to kVecs vectors of
// the row (2048 sixteen-bit or 1024 fp32 values per row), all requested before the first is used, so
// x is read once and every value is exponentiated once (ex2 on values pre-scaled by log2 e).  Longer
// rows take the scalar two-pass path of softmax_kernel inside the same launch.  The host checks the
// alignment this needs (block width a multiple of the vector, 16-byte aligned bases and rows).
constexpr int kVecs = 8;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two 16-bit values at a time: a register of the row vector holds a pair, and the pair forms of max,
// multiply and conversion keep the instruction count per value low (element-wise access to the packed
// registers cost a byte-permute per value and made the kernel issue-bound at 24 instructions per value).
template <typename T> struct Pair;
template <> struct Pair<__half> {
  using P = __half2;
  static __device__ __forceinline__ float2 unpack(P v) { return __half22float2(v); }
  static __device__ __forceinline__ P pack(float a, float b) { return __floats2half2_rn(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
  using P = __nv_bfloat162;
  static __device__ __forceinline__ float2 unpack(P v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ P pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
};

template <typename T>
__device__ __forceinline__ void softmax_row_in_registers(const SmParams& p, uint4 (&raw)[kVecs], const uint32_t (&off)[kVecs],
                                                         int n, int lane, T* out);

template <typename T>
__global__ void __launch_bounds__(128, 9) softmax_fwd_vec_kernel(SmParams p) {
  constexpr int E = 16 / sizeof(T);
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= p.H) return;
  const long long bstride = p.compressed ? p.val_stride_blocks * p.BH * p.BW : (long long)p.H * p.W;
  const T* x = static_cast<const T*>(p.x) + (long long)blockIdx.y * bstride;
  T* out = static_cast<T*>(p.out) + (long long)blockIdx.y * bstride;
  const int br = row / p.BH, y = row - br * p.BH;
  const int t0 = p.row_ptr[br], t1 = p.row_ptr[br + 1];
  const int n = (t1 - t0) * p.BW;
  const int shift = __ffs(p.BW) - 1;  // BW is a power of two
  const int nv = n / E;
  if (nv > 32 * kVecs) {  // row too long for the registers: scalar path (warp-uniform branch)
    float m = -INFINITY, s = 0.f;
    for (int j = lane; j < n; j += 32) {
      const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
      if (p.mask && !p.mask[o]) continue;
      const float v = to_float(x[o]) * p.scale;
      if (v > m) { s = s * expf(m - v) + 1.f; m = v; }
      else s += expf(v - m);
    }
    const float mw = warp_max(m);
    s = (m == -INFINITY) ? 0.f : s * expf(m - mw);
    s = warp_sum(s);
    const float inv = s > 0.f ? 1.f / s : 0.f;
    for (int j = lane; j < n; j += 32) {
      const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
      float r = 0.f;
      if (!p.mask || p.mask[o]) r = expf(to_float(x[o]) * p.scale - mw) * inv;
      out[o] = from_float<T>(r);
    }
    return;
  }
  uint32_t off[kVecs];  // within one batch slice (the host checks that a slice has fewer than 2^32 elements)
  uint4 raw[kVecs];  // the row's values stay packed in their own type: 32 registers, so four CTAs fit an SM
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int j = (lane + 32 * i) * E;
    if (j < n) {
      off[i] = static_cast<uint32_t>(elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1)));
      raw[i] = *reinterpret_cast<const uint4*>(x + off[i]);
    }
  }
  softmax_row_in_registers<T>(p, raw, off, n, lane, out);
}

// The row's values are in raw[] (vector i of a lane = elements (lane + 32 i) E .. + E - 1 of the kept row, at
// element offset off[i] of the tensors): maximum, probabilities, sum, normalise, store.
template <typename T>
__device__ __forceinline__ void softmax_row_in_registers(const SmParams& p, uint4 (&raw)[kVecs], const uint32_t (&off)[kVecs],
                                                         int n, int lane, T* out) {
  constexpr int E = 16 / sizeof(T);
  const float scale2 = p.scale * 1.4426950408889634f;
  // pass 1: maximum; masked elements become -inf in place, so the later passes need no mask
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    if ((lane + 32 * i) * E < n) {
      T* e = reinterpret_cast<T*>(&raw[i]);
      if (p.mask) {
        unsigned long long mk;  // E mask bytes
        if (E == 8) mk = *reinterpret_cast<const unsigned long long*>(p.mask + off[i]);
        else mk = *reinterpret_cast<const unsigned int*>(p.mask + off[i]);
#pragma unroll
        for (int k = 0; k < E; ++k)
          if (!((mk >> (8 * k)) & 0xffull)) e[k] = from_float<T>(-INFINITY);
      }
      if constexpr (sizeof(T) == 2) {
        using PT = typename Pair<T>::P;
        const PT* h = reinterpret_cast<const PT*>(&raw[i]);
        const PT mm = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));  // exact in any precision
        const float2 f = Pair<T>::unpack(mm);
        m = fmaxf(m, fmaxf(f.x, f.y));
      } else {
#pragma unroll
        for (int k = 0; k < E; ++k) m = fmaxf(m, to_float(e[k]));
      }
    }
  }
  const float mw = warp_max(m) * scale2;                // scale > 0
  const float sub = mw > -INFINITY ? mw : 0.f;          // a fully masked row: every value is -inf, every probability 0
  // pass 2: unnormalised probabilities, stored back in the row's own type; the sum takes the fp32 values
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    if ((lane + 32 * i) * E < n) {
      if constexpr (sizeof(T) == 2) {
        using PT = typename Pair<T>::P;
        PT* h = reinterpret_cast<PT*>(&raw[i]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = Pair<T>::unpack(h[k]);
          const float p0 = ex2_approx(fmaf(f.x, scale2, -sub)), p1 = ex2_approx(fmaf(f.y, scale2, -sub));
          s += p0 + p1;
          h[k] = Pair<T>::pack(p0, p1);
        }
      } else {
        T* e = reinterpret_cast<T*>(&raw[i]);
#pragma unroll
        for (int k = 0; k < E; ++k) {
          const float pe = ex2_approx(fmaf(to_float(e[k]), scale2, -sub));
          s += pe;
          e[k] = from_float<T>(pe);
        }
      }
    }
  }
  s = warp_sum(s);
  const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    if ((lane + 32 * i) * E < n) {
      if constexpr (sizeof(T) == 2) {
        // fp16: 1 / sum lies in [1 / 2048, 1], exact enough in the row's own type: one multiply per pair
        using PT = typename Pair<T>::P;
        PT* h = reinterpret_cast<PT*>(&raw[i]);
        if constexpr (std::is_same<T, __half>::value) {
          const PT inv2 = Pair<T>::pack(inv, inv);
#pragma unroll
          for (int k = 0; k < 4; ++k) h[k] = __hmul2(h[k], inv2);
        } else {  // bf16 keeps only eight bits: multiply in fp32
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = Pair<T>::unpack(h[k]);
            h[k] = Pair<T>::pack(f.x * inv, f.y * inv);
          }
        }
      } else {
        T* e = reinterpret_cast<T*>(&raw[i]);
#pragma unroll
        for (int k = 0; k < E; ++k) e[k] = from_float<T>(to_float(e[k]) * inv);
      }
      *reinterpret_cast<uint4*>(out + off[i]) = raw[i];
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Forward pass with the loads staged through shared memory.  In the kernel above a row's loads occupy the
// registers that later hold the row, so a warp alternates between waiting for its loads and storing, and
// the bytes an SM keeps in flight are bounded by its register file.  Here a warp owns up to kRingRows
// rows of one block row (every kRingWarps-th row of its CTA's share) and a private ring in shared memory; it issues the asynchronous copies
// (cp.async, 16 bytes per lane) of the rows up to `slots - 1` ahead of the one it computes, so about
// 100 KB per SM are in flight whatever the warps are doing.  Measured on 1.35 GB of compressed fp16 scores
// (rows of 2.5 KB): 16 rows per warp with a 12 KB ring and four CTAs per SM 0.274 ms, 8 rows 0.250 ms, 8 rows with
// an 8 KB ring and five CTAs 0.238 ms (the register-resident kernel above: 0.349 ms).  A lane copies, reads back and stores the
// same 16-byte vectors, so the ring needs no barrier: its own wait_group orders the copy before the read,
// and the read's register dependency orders it before the slot is refilled.  The offsets of a row are
// those of the warp's first row plus a row step.  Used when block rows have at least 16 rows.
// ---------------------------------------------------------------------------------------------------
constexpr int kRingRows = 8;             // rows per warp at most; a CTA takes kRingWarps x rows consecutive rows of a block row
constexpr int kRingBytes = 8 * 1024;     // ring capacity per warp
constexpr int kRingWarps = 4;            // warps per CTA: 32 KB of shared memory, five CTAs per SM (96 registers)
constexpr int kRingMaxSlots = 8;

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// at most `pending` of this thread's copy groups may still be in flight
__device__ __forceinline__ void cp_async_wait_pending(int pending) {
  switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}

// Softmax of one row that sits in shared memory as nv 16-byte vectors (vector v = elements v E .. of the kept
// row, at element offset off_of(v) of the tensors); every lane touches only its own vectors.
template <typename T, typename OffsetOf>
__device__ __forceinline__ void softmax_row_in_shared(const SmParams& p, uint8_t* slot, int nv, int lane, T* out,
                                                      OffsetOf off_of) {
  constexpr int E = 16 / sizeof(T);
  const float scale2 = p.scale * 1.4426950408889634f;
  uint4* vecs = reinterpret_cast<uint4*>(slot);
  float m = -INFINITY;
  for (int v = lane; v < nv; v += 32) {
    uint4 raw = vecs[v];
    T* e = reinterpret_cast<T*>(&raw);
    if (p.mask) {
      const uint32_t o = off_of(v);
      unsigned long long mk;
      if (E == 8) mk = *reinterpret_cast<const unsigned long long*>(p.mask + o);
      else mk = *reinterpret_cast<const unsigned int*>(p.mask + o);
#pragma unroll
      for (int k = 0; k < E; ++k)
        if (!((mk >> (8 * k)) & 0xffull)) e[k] = from_float<T>(-INFINITY);
      vecs[v] = raw;
    }
#pragma unroll
    for (int k = 0; k < E; ++k) m = fmaxf(m, to_float(e[k]));
  }
  const float mw = warp_max(m) * scale2;
  const float sub = mw > -INFINITY ? mw : 0.f;
  float sum = 0.f;
  for (int v = lane; v < nv; v += 32) {
    uint4 raw = vecs[v];
    T* e = reinterpret_cast<T*>(&raw);
    float pe[E];
#pragma unroll
    for (int k = 0; k < E; ++k) {
      pe[k] = ex2_approx(fmaf(to_float(e[k]), scale2, -sub));
      sum += pe[k];
    }
    // the unnormalised probabilities go back into the slot in the row's own type, as in the register path
#pragma unroll
    for (int k = 0; k < E; ++k) e[k] = from_float<T>(pe[k]);
    vecs[v] = raw;
  }
  sum = warp_sum(sum);
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  for (int v = lane; v < nv; v += 32) {
    uint4 raw = vecs[v];
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int k = 0; k < E; ++k) e[k] = from_float<T>(to_float(e[k]) * inv);
    *reinterpret_cast<uint4*>(out + off_of(v)) = raw;
  }
}

template <typename T>
__global__ void __launch_bounds__(kRingWarps * 32, 5) softmax_fwd_ring_kernel(SmParams p) {
  constexpr int E = 16 / sizeof(T);
  extern __shared__ __align__(16) uint8_t ring_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the warps of a CTA interleave: together they read kRingWarps consecutive rows (one contiguous piece of every
  // block of the block row) at a time, which keeps the DRAM accesses of a CTA next to each other
  const int rows_w = min(kRingRows, p.BH / kRingWarps);
  const int row0 = blockIdx.x * kRingWarps * rows_w + warp;
  if (row0 >= p.H) return;
  const long long bstride = p.compressed ? p.val_stride_blocks * p.BH * p.BW : (long long)p.H * p.W;
  const T* x = static_cast<const T*>(p.x) + (long long)blockIdx.y * bstride;
  T* out = static_cast<T*>(p.out) + (long long)blockIdx.y * bstride;
  const int br = row0 / p.BH, y0 = row0 - br * p.BH;
  const int t0 = p.row_ptr[br], t1 = p.row_ptr[br + 1];
  const int n = (t1 - t0) * p.BW;
  const int shift = __ffs(p.BW) - 1;
  const int nv = n / E;
  if (nv * 16 > kRingBytes) {  // rows too long for the ring: the scalar two-pass path, row by row
    for (int k = 0; k < rows_w; ++k) {
      const int row = row0 + k * kRingWarps, y = y0 + k * kRingWarps;
      float m = -INFINITY, sum = 0.f;
      for (int j = lane; j < n; j += 32) {
        const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
        if (p.mask && !p.mask[o]) continue;
        const float v = to_float(x[o]) * p.scale;
        if (v > m) { sum = sum * expf(m - v) + 1.f; m = v; }
        else sum += expf(v - m);
      }
      const float mw = warp_max(m);
      sum = (m == -INFINITY) ? 0.f : sum * expf(m - mw);
      sum = warp_sum(sum);
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      for (int j = lane; j < n; j += 32) {
        const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
        float r = 0.f;
        if (!p.mask || p.mask[o]) r = expf(to_float(x[o]) * p.scale - mw) * inv;
        out[o] = from_float<T>(r);
      }
    }
    return;
  }
  if (n == 0) return;
  // offsets of the warp's first row; row k adds k row steps
  uint32_t off0[kVecs];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int j = (lane + 32 * i) * E;
    off0[i] = j < n ? static_cast<uint32_t>(elem_off(p, t0 + (j >> shift), row0, y0, j & (p.BW - 1))) : 0u;
  }
  const uint32_t row_step = (p.compressed ? p.BW : p.W) * kRingWarps;
  const int row_bytes = nv * 16;  // at most the ring's capacity
  int slots = kRingBytes / row_bytes;
  if (slots > kRingMaxSlots) slots = kRingMaxSlots;
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(ring_smem)) + warp * kRingBytes;
  const uint8_t* ring_ptr = ring_smem + warp * kRingBytes;

  auto issue = [&](int k) {  // copies of row k (none beyond the warp's rows), always one group
    if (k < rows_w) {
      const uint32_t dst = ring + (k % slots) * row_bytes;
#pragma unroll
      for (int i = 0; i < kVecs; ++i) {
        const int v = lane + 32 * i;
        if (v < nv) cp_async_16(dst + v * 16, x + off0[i] + k * row_step);
      }
    }
    cp_async_commit();
  };
  if (nv > 32 * kVecs) {
    // Rows longer than the registers hold (up to the ring's capacity) stay in shared memory: the same pipeline,
    // with the three passes reading and rewriting the row's slot.  A lane owns vectors lane, lane + 32, ...
    const uint32_t step = p.compressed ? p.BW : p.W;
    auto vec_off = [&](int v, int k) -> uint32_t {
      const int j = v * E;
      return static_cast<uint32_t>(elem_off(p, t0 + (j >> shift), row0, y0, j & (p.BW - 1))) + k * kRingWarps * step;
    };
    auto issue_long = [&](int k) {
      if (k < rows_w) {
        const uint32_t dst = ring + (k % slots) * row_bytes;
        for (int v = lane; v < nv; v += 32) cp_async_16(dst + v * 16, x + vec_off(v, k));
      }
      cp_async_commit();
    };
    for (int k = 0; k < slots - 1; ++k) issue_long(k);
    for (int k = 0; k < rows_w; ++k) {
      issue_long(k + slots - 1);
      cp_async_wait_pending(slots - 1);
      softmax_row_in_shared<T>(p, const_cast<uint8_t*>(ring_ptr) + (k % slots) * row_bytes, nv, lane, out,
                               [&](int v) { return vec_off(v, k); });
    }
    return;
  }
  for (int k = 0; k < slots - 1; ++k) issue(k);
  for (int k = 0; k < rows_w; ++k) {
    issue(k + slots - 1);            // into the slot read in the previous iteration
    cp_async_wait_pending(slots - 1);  // row k has landed
    const uint8_t* src = ring_ptr + (k % slots) * row_bytes;
    uint4 raw[kVecs];
    uint32_t off[kVecs];
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const int v = lane + 32 * i;
      off[i] = off0[i] + k * row_step;
      if (v < nv) raw[i] = *reinterpret_cast<const uint4*>(src + v * 16);
    }
    softmax_row_in_registers<T>(p, raw, off, n, lane, out);
  }
}

// ---------------------------------------------------------------------------------------------------
// Backward pass through the same kind of ring: dx = y (dy - sum(dy y)) / T per row.  A slot holds the row of
// dy followed by the row of y; both are read back into registers (64 of them), the dot product and the
// result are formed in fp32, and dx is stored from registers.  Rows beyond the registers' 4 KB are processed
// in the slot itself (up to 8 KB each); longer ones take scalar passes.  Masked elements: y is zeroed where the element mask is, which zeroes their terms and results.
// ---------------------------------------------------------------------------------------------------
constexpr int kBwdRingBytes = 16 * 1024;  // per warp: 64 KB per CTA, three CTAs per SM

template <typename T>
__global__ void __launch_bounds__(kRingWarps * 32, 3) softmax_bwd_ring_kernel(SmParams p) {
  constexpr int E = 16 / sizeof(T);
  extern __shared__ __align__(16) uint8_t ring_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_w = min(kRingRows, p.BH / kRingWarps);
  const int row0 = blockIdx.x * kRingWarps * rows_w + warp;
  if (row0 >= p.H) return;
  const long long bstride = p.compressed ? p.val_stride_blocks * p.BH * p.BW : (long long)p.H * p.W;
  const T* dy = static_cast<const T*>(p.x) + (long long)blockIdx.y * bstride;
  const T* yv = static_cast<const T*>(p.y_in) + (long long)blockIdx.y * bstride;
  T* out = static_cast<T*>(p.out) + (long long)blockIdx.y * bstride;
  const int br = row0 / p.BH, y0 = row0 - br * p.BH;
  const int t0 = p.row_ptr[br], t1 = p.row_ptr[br + 1];
  const int n = (t1 - t0) * p.BW;
  const int shift = __ffs(p.BW) - 1;
  const int nv = n / E;
  const int row_bytes = nv * 16;
  if (2 * row_bytes > kBwdRingBytes) {  // rows too long for the ring: scalar passes, row by row
    for (int k = 0; k < rows_w; ++k) {
      const int row = row0 + k * kRingWarps, y = y0 + k * kRingWarps;
      float dot = 0.f;
      for (int j = lane; j < n; j += 32) {
        const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
        if (p.mask && !p.mask[o]) continue;
        dot += to_float(dy[o]) * to_float(yv[o]);
      }
      dot = warp_sum(dot);
      for (int j = lane; j < n; j += 32) {
        const long long o = elem_off(p, t0 + (j >> shift), row, y, j & (p.BW - 1));
        float r = 0.f;
        if (!p.mask || p.mask[o]) {
          const float yy = to_float(yv[o]);
          r = (to_float(dy[o]) * yy - yy * dot) * p.scale;
        }
        out[o] = from_float<T>(r);
      }
    }
    return;
  }
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(ring_smem)) + warp * kBwdRingBytes;
  const uint8_t* ring_ptr = ring_smem + warp * kBwdRingBytes;
  int slots = kBwdRingBytes / (2 * row_bytes);
  if (slots > kRingMaxSlots) slots = kRingMaxSlots;
  if (nv > 32 * kVecs) {
    // rows longer than the registers hold (up to half the ring each): the same pipeline, two passes over the slot
    const uint32_t step = p.compressed ? p.BW : p.W;
    auto vec_off = [&](int v, int k) -> uint32_t {
      const int j = v * E;
      return static_cast<uint32_t>(elem_off(p, t0 + (j >> shift), row0, y0, j & (p.BW - 1))) + k * kRingWarps * step;
    };
    auto issue_long = [&](int k) {
      if (k < rows_w) {
        const uint32_t dst = ring + (k % slots) * (2 * row_bytes);
        for (int v = lane; v < nv; v += 32) {
          const uint32_t o = vec_off(v, k);
          cp_async_16(dst + v * 16, dy + o);
          cp_async_16(dst + row_bytes + v * 16, yv + o);
        }
      }
      cp_async_commit();
    };
    for (int k = 0; k < slots - 1; ++k) issue_long(k);
    for (int k = 0; k < rows_w; ++k) {
      issue_long(k + slots - 1);
      cp_async_wait_pending(slots - 1);
      uint8_t* slot = const_cast<uint8_t*>(ring_ptr) + (k % slots) * (2 * row_bytes);
      const uint4* gv = reinterpret_cast<const uint4*>(slot);
      uint4* yvec = reinterpret_cast<uint4*>(slot + row_bytes);
      float dot = 0.f;
      for (int v = lane; v < nv; v += 32) {
        const uint4 g = gv[v];
        uint4 yy = yvec[v];
        if (p.mask) {
          const uint32_t o = vec_off(v, k);
          unsigned long long mk;
          if (E == 8) mk = *reinterpret_cast<const unsigned long long*>(p.mask + o);
          else mk = *reinterpret_cast<const unsigned int*>(p.mask + o);
          T* e = reinterpret_cast<T*>(&yy);
#pragma unroll
          for (int q = 0; q < E; ++q)
            if (!((mk >> (8 * q)) & 0xffull)) e[q] = from_float<T>(0.f);
          yvec[v] = yy;
        }
        const T* a = reinterpret_cast<const T*>(&g);
        const T* b = reinterpret_cast<const T*>(&yy);
#pragma unroll
        for (int q = 0; q < E; ++q) dot = fmaf(to_float(a[q]), to_float(b[q]), dot);
      }
      dot = warp_sum(dot);
      for (int v = lane; v < nv; v += 32) {
        uint4 g = gv[v];
        const uint4 yy = yvec[v];
        T* a = reinterpret_cast<T*>(&g);
        const T* b = reinterpret_cast<const T*>(&yy);
#pragma unroll
        for (int q = 0; q < E; ++q) {
          const float yq = to_float(b[q]);
          a[q] = from_float<T>((to_float(a[q]) * yq - yq * dot) * p.scale);
        }
        *reinterpret_cast<uint4*>(out + vec_off(v, k)) = g;
      }
    }
    return;
  }
  if (n == 0) return;
  uint32_t off0[kVecs];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) {
    const int j = (lane + 32 * i) * E;
    off0[i] = j < n ? static_cast<uint32_t>(elem_off(p, t0 + (j >> shift), row0, y0, j & (p.BW - 1))) : 0u;
  }
  const uint32_t row_step = (p.compressed ? p.BW : p.W) * kRingWarps;

  auto issue = [&](int k) {
    if (k < rows_w) {
      const uint32_t dst = ring + (k % slots) * (2 * row_bytes);
#pragma unroll
      for (int i = 0; i < kVecs; ++i) {
        const int v = lane + 32 * i;
        if (v < nv) {
          cp_async_16(dst + v * 16, dy + off0[i] + k * row_step);
          cp_async_16(dst + row_bytes + v * 16, yv + off0[i] + k * row_step);
        }
      }
    }
    cp_async_commit();
  };
  for (int k = 0; k < slots - 1; ++k) issue(k);
  for (int k = 0; k < rows_w; ++k) {
    issue(k + slots - 1);
    cp_async_wait_pending(slots - 1);
    const uint8_t* src = ring_ptr + (k % slots) * (2 * row_bytes);
    uint4 g[kVecs], yy[kVecs];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const int v = lane + 32 * i;
      if (v < nv) {
        g[i] = *reinterpret_cast<const uint4*>(src + v * 16);
        yy[i] = *reinterpret_cast<const uint4*>(src + row_bytes + v * 16);
        if (p.mask) {
          const uint32_t o = off0[i] + k * row_step;
          unsigned long long mk;
          if (E == 8) mk = *reinterpret_cast<const unsigned long long*>(p.mask + o);
          else mk = *reinterpret_cast<const unsigned int*>(p.mask + o);
          T* e = reinterpret_cast<T*>(&yy[i]);
#pragma unroll
          for (int q = 0; q < E; ++q)
            if (!((mk >> (8 * q)) & 0xffull)) e[q] = from_float<T>(0.f);
        }
        const T* a = reinterpret_cast<const T*>(&g[i]);
        const T* b = reinterpret_cast<const T*>(&yy[i]);
#pragma unroll
        for (int q = 0; q < E; ++q) dot = fmaf(to_float(a[q]), to_float(b[q]), dot);
      }
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < kVecs; ++i) {
      const int v = lane + 32 * i;
      if (v < nv) {
        T* a = reinterpret_cast<T*>(&g[i]);
        const T* b = reinterpret_cast<const T*>(&yy[i]);
#pragma unroll
        for (int q = 0; q < E; ++q) {
          const float yq = to_float(b[q]);
          a[q] = from_float<T>((to_float(a[q]) * yq - yq * dot) * p.scale);
        }
        *reinterpret_cast<uint4*>(out + off0[i] + k * row_step) = g[i];
      }
    }
  }
}

// whether the 16-byte path applies: block width and row pitch multiples of the vector, aligned bases
bool vec_ok(const SmParams& p, int dtype) {
  const int esz = dtype == SPARTA_F32 ? 4 : 2, E = 16 / esz;
  if (p.BW % E || !(p.scale > 0.f)) return false;  // the kernel scales the row maximum after taking it
  if ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.y_in)) & 15) return false;
  if (p.mask && (reinterpret_cast<uintptr_t>(p.mask) & 7)) return false;
  const long long bstride = p.compressed ? p.val_stride_blocks * p.BH * p.BW : (long long)p.H * p.W;
  if (bstride % E || bstride >= (1ll << 32)) return false;
  if (!p.compressed && p.W % E) return false;
  return true;
}

template <bool BACKWARD>
int launch(const SmParams& p, int batch, int dtype, cudaStream_t st) {
  dim3 grid((p.H + 7) / 8, batch), block(256);
  if (!BACKWARD && vec_ok(p, dtype) && p.BH >= 4 * kRingWarps) {
    const int rows_cta = kRingWarps * (kRingRows < p.BH / kRingWarps ? kRingRows : p.BH / kRingWarps);
    const dim3 grid(p.H / rows_cta, batch), block(kRingWarps * 32);
    constexpr int kSmem = kRingWarps * kRingBytes;
    static SmemAttrOnce attr_f, attr_h, attr_b;
    switch (dtype) {
      case SPARTA_F32:
        if (cudaError_t e = attr_f.ensure(softmax_fwd_ring_kernel<float>, kSmem); e != cudaSuccess) return (int)e;
        softmax_fwd_ring_kernel<float><<<grid, block, kSmem, st>>>(p);
        break;
      case SPARTA_F16:
        if (cudaError_t e = attr_h.ensure(softmax_fwd_ring_kernel<__half>, kSmem); e != cudaSuccess) return (int)e;
        softmax_fwd_ring_kernel<__half><<<grid, block, kSmem, st>>>(p);
        break;
      case SPARTA_BF16:
        if (cudaError_t e = attr_b.ensure(softmax_fwd_ring_kernel<__nv_bfloat16>, kSmem); e != cudaSuccess) return (int)e;
        softmax_fwd_ring_kernel<__nv_bfloat16><<<grid, block, kSmem, st>>>(p);
        break;
      default: return SPARTA_ERR_BAD_ARG;
    }
    return launch_status();
  }
  if (BACKWARD && vec_ok(p, dtype) && p.BH >= 4 * kRingWarps) {
    const int rows_cta = kRingWarps * (kRingRows < p.BH / kRingWarps ? kRingRows : p.BH / kRingWarps);
    const dim3 grid(p.H / rows_cta, batch), block(kRingWarps * 32);
    constexpr int kSmem = kRingWarps * kBwdRingBytes;
    static SmemAttrOnce attr_f, attr_h, attr_b;
    switch (dtype) {
      case SPARTA_F32:
        if (cudaError_t e = attr_f.ensure(softmax_bwd_ring_kernel<float>, kSmem); e != cudaSuccess) return (int)e;
        softmax_bwd_ring_kernel<float><<<grid, block, kSmem, st>>>(p);
        break;
      case SPARTA_F16:
        if (cudaError_t e = attr_h.ensure(softmax_bwd_ring_kernel<__half>, kSmem); e != cudaSuccess) return (int)e;
        softmax_bwd_ring_kernel<__half><<<grid, block, kSmem, st>>>(p);
        break;
      case SPARTA_BF16:
        if (cudaError_t e = attr_b.ensure(softmax_bwd_ring_kernel<__nv_bfloat16>, kSmem); e != cudaSuccess) return (int)e;
        softmax_bwd_ring_kernel<__nv_bfloat16><<<grid, block, kSmem, st>>>(p);
        break;
      default: return SPARTA_ERR_BAD_ARG;
    }
    return launch_status();
  }
  if (!BACKWARD && vec_ok(p, dtype)) {
    const dim3 grid((p.H + 3) / 4, batch), block(128);  // four rows per CTA measured 5 % faster than eight
    switch (dtype) {
      case SPARTA_F32: softmax_fwd_vec_kernel<float><<<grid, block, 0, st>>>(p); break;
      case SPARTA_F16: softmax_fwd_vec_kernel<__half><<<grid, block, 0, st>>>(p); break;
      case SPARTA_BF16: softmax_fwd_vec_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(p); break;
      default: return SPARTA_ERR_BAD_ARG;
    }
    return launch_status();
  }
  switch (dtype) {
    case SPARTA_F32: softmax_kernel<float, BACKWARD><<<grid, block, 0, st>>>(p); break;
    case SPARTA_F16: softmax_kernel<__half, BACKWARD><<<grid, block, 0, st>>>(p); break;
    case SPARTA_BF16: softmax_kernel<__nv_bfloat16, BACKWARD><<<grid, block, 0, st>>>(p); break;
    default: return SPARTA_ERR_BAD_ARG;
  }
  return launch_status();
}

int check(const void* a, const void* b, const int32_t* row_ptr, const int32_t* idx, const int32_t* nnz,
          int batch, int H, int W, int BH, int BW, int compressed, int64_t vsb) {
  if (!a || !b || !row_ptr || !idx || !nnz || batch <= 0 || H <= 0 || W <= 0) return SPARTA_ERR_BAD_ARG;
  if (!valid_bcs_block(BH) || !valid_bcs_block(BW) || H % BH || W % BW) return SPARTA_ERR_SHAPE;
  if (batch > 65535) return SPARTA_ERR_SHAPE;
  if (compressed && vsb < 0) return SPARTA_ERR_BAD_ARG;
  return SPARTA_OK;
}

}  // namespace
}  // namespace sparta

using namespace sparta;

extern "C" int sparta_softmax_fwd(const void* x, void* y, const int32_t* row_ptr,
                                  const int32_t* bcsr_idx, const int32_t* nnz, const uint8_t* mask,
                                  float scale, int batch, int H, int W, int BH, int BW, int compressed,
                                  int dtype, int64_t val_stride_blocks, void* stream) {
  int rc = check(x, y, row_ptr, bcsr_idx, nnz, batch, H, W, BH, BW, compressed, val_stride_blocks);
  if (rc != SPARTA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!compressed && x == y) return SPARTA_ERR_BAD_ARG;  // the zero fill below would wipe the input
  if (!compressed) {  // dropped blocks of the dense-shaped output must read 0
    const size_t esz = dtype == SPARTA_F32 ? 4 : 2;
    cudaError_t e = cudaMemsetAsync(y, 0, (size_t)batch * H * W * esz, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  SmParams p{x, nullptr, y, row_ptr, bcsr_idx, nnz, mask, scale, H, W, BH, BW, compressed,
             (long long)val_stride_blocks};
  return launch<false>(p, batch, dtype, st);
}

extern "C" int sparta_softmax_bwd(const void* dy, const void* y, void* dx, const int32_t* row_ptr,
                                  const int32_t* bcsr_idx, const int32_t* nnz, const uint8_t* mask,
                                  float scale, int batch, int H, int W, int BH, int BW, int compressed,
                                  int dtype, int64_t val_stride_blocks, void* stream) {
  int rc = check(dy, dx, row_ptr, bcsr_idx, nnz, batch, H, W, BH, BW, compressed, val_stride_blocks);
  if (rc != SPARTA_OK) return rc;
  if (!y) return SPARTA_ERR_BAD_ARG;
  if (!compressed && (dx == dy || dx == y)) return SPARTA_ERR_BAD_ARG;  // the zero fill below would wipe an input
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!compressed) {
    const size_t esz = dtype == SPARTA_F32 ? 4 : 2;
    cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)batch * H * W * esz, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  SmParams p{dy, y, dx, row_ptr, bcsr_idx, nnz, mask, scale, H, W, BH, BW, compressed,
             (long long)val_stride_blocks};
  return launch<true>(p, batch, dtype, st);
}
