// dsd on the FMA units for the SparseLinear layout with small square blocks (8, 16 or 32), any dtype
// with fp32 accumulation: C[m, n] = sum over kept K-blocks k of row-block n of X[m, k-block] . W_block^T.
//
// The generic FMA kernel gives every (row tile, block row) its own CTA and stages both operands
// through shared memory with two barriers per K-block; with 8 x 8 blocks that is 64 x 8 outputs and
// eight multiply-adds per thread between barriers.  Here a thread owns one token row and 64 output
// columns (a panel of 64 / B block rows of W) in registers, and a CTA owns 128 (or 64) such rows, each
// shared by two threads that take alternate K-blocks and add their partial sums at the end (twice the
// warps for the same loads: with one thread per row an SM would hold only three or four warps):
//   * the prologue turns the BCSR rows of the panel into kmask[k] (which block rows keep K-block k) and
//     wpos[k][l] (where that block sits in the value array), so the main loop has no index search;
//   * K is walked in chunks of 64 values.  A chunk's activations (rows x 64) and its kept W blocks
//     (at most 64 x 64 values, each block in a fixed slot) are brought into shared memory with
//     cp.async, three stages deep, so the loads of the next two chunks overlap the multiply-adds of this
//     one (a chunk's arithmetic is shorter than the latency of its loads);
//   * a thread reads its own activations with conflict-free vector loads (padded rows) and the weights
//     with broadcast loads; the block-row loop is unrolled so that the accumulators stay in registers.
//
// Replaces sparta_sparse_matmul_dsd.cuh.j2 for these configurations (the reference covers 8 x 8 masks
// with 16 x 16 or larger tiles, sparta/specializer/kernels/matmul.py:53-97).
#include <type_traits>

#include "bsmm.cuh"

namespace sparta {
namespace {

constexpr int kPanelCols = 64;   // output columns per thread
constexpr int kMaxKbFma = 1024;  // K-blocks the schedule can hold

template <typename T, int N>
__device__ __forceinline__ void load_floats(const T* src, float (&out)[N]) {
  // N values starting at a 16-byte aligned address, as fp32
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const float4 v = *(reinterpret_cast<const float4*>(src) + i);
      out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < N / 8; ++i) {
      const uint4 v = *(reinterpret_cast<const uint4*>(src) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        T lo, hi;
        const uint16_t l16 = static_cast<uint16_t>(w[j] & 0xffffu), h16 = static_cast<uint16_t>(w[j] >> 16);
        memcpy(&lo, &l16, 2);
        memcpy(&hi, &h16, 2);
        out[8 * i + 2 * j] = to_float(lo);
        out[8 * i + 2 * j + 1] = to_float(hi);
      }
    }
  }
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gsrc)
               : "memory");
}

constexpr int kChunkK = 64;  // K values per chunk

template <int TM, typename T>
struct FmaSmem {
  static constexpr int kXRow = kChunkK * (int)sizeof(T) + 16;  // padded row: conflict-free 16-byte reads, one row per lane
  static constexpr int kXBytes = TM * kXRow;
  static constexpr int kWBytes = kChunkK * kPanelCols * (int)sizeof(T);  // (64 / B)^2 slots of B x B values
  static constexpr int kStage = kXBytes + kWBytes;
  static constexpr int kStages = 3;  // chunks in flight: one being used, two on their way
  static constexpr int kTotal = kStages * kStage;
};

template <int B, int TM, typename T>
__global__ void __launch_bounds__(2 * TM) bsmm_dsd_fma_kernel(BsmmParams p) {
  constexpr int NT = 2 * TM;          // threads: two per row
  constexpr int P = kPanelCols / B;   // block rows of W per panel
  constexpr int KC = kChunkK / B;     // K-blocks per chunk
  using S = FmaSmem<TM, T>;
  extern __shared__ __align__(16) uint8_t stage_mem[];
  __shared__ uint32_t kmask[kMaxKbFma];
  __shared__ uint16_t wpos[kMaxKbFma * P];
  __shared__ uint16_t clist[kMaxKbFma * B / kChunkK + 1];  // chunks of K in which the panel keeps a block, ascending
  __shared__ int s_range[2];
  __shared__ int s_nchunks;

  const int panel = blockIdx.x, m0 = blockIdx.y * TM, batch = blockIdx.z;
  const int Nb = p.N / B, Kb = p.K / B;
  const int nb0 = panel * P, nb_end = min(nb0 + P, Nb);
  if (threadIdx.x == 0) {
    s_range[0] = p.ptr[nb0];
    s_range[1] = p.ptr[nb_end];
  }
  for (int k = threadIdx.x; k < Kb; k += NT) kmask[k] = 0;
  __syncthreads();
  const int e0 = s_range[0];
  const int32_t* idx = static_cast<const int32_t*>(p.idx);
  for (int e = e0 + threadIdx.x; e < s_range[1]; e += NT) {
    const int v = __ldg(idx + e);
    const int k = v & 0xffff, l = (v >> 16) - nb0;
    if (k < Kb && l >= 0 && l < P) {  // caller-provided indexes never address shared memory unchecked
      atomicOr(&kmask[k], 1u << l);
      wpos[k * P + l] = static_cast<uint16_t>(e - e0);
    }
  }
  __syncthreads();

  // Only the chunks of K in which this panel keeps a block are fetched and walked: with few blocks left, reading
  // every activation chunk for every panel was most of the time (and all of it for a panel without blocks).
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x, all = p.K / kChunkK;
    int n = 0;
    for (int c0 = 0; c0 < all; c0 += 32) {
      const int c = c0 + lane;
      uint32_t any = 0;
      if (c < all)
        for (int kc = 0; kc < KC; ++kc) any |= kmask[c * KC + kc];
      const unsigned bal = __ballot_sync(0xffffffffu, any != 0);
      if (any) clist[n + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>(c);
      n += __popc(bal);
    }
    if (lane == 0) s_nchunks = n;
  }
  __syncthreads();

  const T* xtile = static_cast<const T*>(p.A) + ((long long)batch * p.M + m0) * p.K;
  const T* wbase = static_cast<const T*>(p.B) + ((long long)batch * p.val_stride_blocks + e0) * (B * B);
  const int n_chunks = s_nchunks;

  // staging: every thread copies the same 16-byte piece of successive rows / block slots, so the
  // index arithmetic is done once
  constexpr int XP = kChunkK * (int)sizeof(T) / 16;  // 16-byte pieces per row
  constexpr int SP = B * B * (int)sizeof(T) / 16;    // pieces per block slot
  constexpr int WP = S::kWBytes / 16;
  static_assert(NT % XP == 0 && (TM * XP) % NT == 0 && WP % NT == 0, "whole passes over the pieces");
  const int x_r0 = threadIdx.x / XP, x_q = threadIdx.x % XP;
  const uint8_t* x_src0 = reinterpret_cast<const uint8_t*>(xtile + (long long)x_r0 * p.K) + x_q * 16;
  const long long x_step = (long long)(NT / XP) * p.K * (long long)sizeof(T);
  auto issue = [&](int ci, int buf) {  // ci: position in clist
    const int c = clist[ci];
    uint8_t* xs = stage_mem + buf * S::kStage;
    uint8_t* ws = xs + S::kXBytes;
    const uint8_t* src = x_src0 + (long long)c * kChunkK * sizeof(T);
    uint8_t* dst = xs + x_r0 * S::kXRow + x_q * 16;
#pragma unroll
    for (int it = 0; it < TM * XP / NT; ++it) {
      cp_async_16(dst, src);
      src += x_step;
      dst += (NT / XP) * S::kXRow;
    }
#pragma unroll
    for (int it = 0; it < WP / NT; ++it) {
      const int i = threadIdx.x + it * NT;
      const int slot = i / SP, within = i % SP;  // powers of two
      const int kc = slot / P, l = slot % P;
      const int k = c * KC + kc;
      if ((kmask[k] >> l) & 1u)
        cp_async_16(ws + i * 16, reinterpret_cast<const uint8_t*>(wbase + (long long)wpos[k * P + l] * (B * B)) + within * 16);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[kPanelCols];
#pragma unroll
  for (int j = 0; j < kPanelCols; ++j) acc[j] = 0.f;

  // every iteration commits exactly one group (an empty one past the end), so "all but the newest
  // kStages - 2 groups are complete" always means that chunk c has landed
  for (int c = 0; c < S::kStages - 1; ++c) {
    if (c < n_chunks) issue(c, c);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int c = 0; c < n_chunks; ++c) {
    asm volatile("cp.async.wait_group %0;" ::"n"(S::kStages - 2) : "memory");
    __syncthreads();  // chunk c is visible to everyone, and everyone is done with the stage refilled below
    if (c + S::kStages - 1 < n_chunks) issue(c + S::kStages - 1, (c + S::kStages - 1) % S::kStages);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const uint8_t* xs = stage_mem + (c % S::kStages) * S::kStage;
    const uint8_t* ws = xs + S::kXBytes;
    const T* xrow = reinterpret_cast<const T*>(xs + (threadIdx.x % TM) * S::kXRow);
    const int chunk = clist[c];
#pragma unroll 1
    for (int kc = threadIdx.x / TM; kc < KC; kc += 2) {  // the two threads of a row take alternate K-blocks
      const uint32_t m = kmask[chunk * KC + kc];  // the same for every thread of the CTA
      if (!m) continue;
      float x[B];
      load_floats<T, B>(xrow + kc * B, x);
#pragma unroll
      for (int l = 0; l < P; ++l) {
        if (!((m >> l) & 1u)) continue;
        const T* wb = reinterpret_cast<const T*>(ws) + (kc * P + l) * (B * B);  // stored [n][k], row-major
        // four outputs at a time: their multiply-add chains are independent, so one is always ready to issue
        // (a single chain of B dependent multiply-adds per output left the FMA pipe waiting on its own latency)
        constexpr int KV = 16 / (int)sizeof(T);  // values per 16-byte vector
#pragma unroll
        for (int n = 0; n < B; n += 4) {
          float s0 = acc[l * B + n], s1 = acc[l * B + n + 1], s2 = acc[l * B + n + 2], s3 = acc[l * B + n + 3];
#pragma unroll
          for (int k0 = 0; k0 < B; k0 += KV) {
            float w0[KV], w1[KV], w2[KV], w3[KV];
            load_floats<T, KV>(wb + (n + 0) * B + k0, w0);
            load_floats<T, KV>(wb + (n + 1) * B + k0, w1);
            load_floats<T, KV>(wb + (n + 2) * B + k0, w2);
            load_floats<T, KV>(wb + (n + 3) * B + k0, w3);
#pragma unroll
            for (int kk = 0; kk < KV; ++kk) {
              s0 = fmaf(x[k0 + kk], w0[kk], s0);
              s1 = fmaf(x[k0 + kk], w1[kk], s1);
              s2 = fmaf(x[k0 + kk], w2[kk], s2);
              s3 = fmaf(x[k0 + kk], w3[kk], s3);
            }
          }
          acc[l * B + n] = s0; acc[l * B + n + 1] = s1; acc[l * B + n + 2] = s2; acc[l * B + n + 3] = s3;
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // all copies have landed and all reads of the staging memory are done

  // the second thread of every row hands its partial sums over through the (now idle) staging memory
  float* red = reinterpret_cast<float*>(stage_mem);
  static_assert(S::kTotal >= TM * (kPanelCols + 1) * 4, "staging memory holds the partial sums");
  if (threadIdx.x >= TM) {
#pragma unroll
    for (int j = 0; j < kPanelCols; ++j) red[j * TM + (threadIdx.x - TM)] = acc[j];
  }
  __syncthreads();
  if (threadIdx.x >= TM) return;
#pragma unroll
  for (int j = 0; j < kPanelCols; ++j) acc[j] += red[j * TM + threadIdx.x];

  // epilogue: + bias, convert, 16-byte stores along the row
  const int row = m0 + threadIdx.x;
  const int n0 = nb0 * B;
  const int n_cols = (nb_end - nb0) * B;
  const T* bias = p.bias ? static_cast<const T*>(p.bias) + (long long)batch * p.N + n0 : nullptr;
  T* crow = static_cast<T*>(p.C) + ((long long)batch * p.M + row) * p.N + n0;
  constexpr int kVec = 16 / sizeof(T);
#pragma unroll
  for (int j0 = 0; j0 < kPanelCols; j0 += kVec) {
    if (j0 < n_cols) {
      alignas(16) T out[kVec];
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        float v = acc[j0 + j];
        if (bias) v += to_float(bias[j0 + j]);
        out[j] = from_float<T>(v);
      }
      *reinterpret_cast<uint4*>(crow + j0) = *reinterpret_cast<const uint4*>(out);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// 32 x 32 blocks: the same staging and schedule, with the multiply-adds tiled over registers in both
// directions.  In the kernel above a thread owns one row and reads every weight value it needs from shared
// memory for a single multiply-add: one 16-byte shared-memory read per four multiply-adds, which is what the
// shared-memory pipe delivers at best, so the FMA pipe idled two thirds of the time.  Here a thread owns
// 8 rows x (4 + 4) columns -- four columns in each of the panel's two block rows of W -- and per step of four
// K values (eight for 16-bit types) reads 8 row pieces of X and 2 x 4 row pieces of W for 256 (512) multiply-adds:
// one read per 16 (32).  Threads 0-127 and 128-255 share the kept blocks of a chunk between them; a warp
// is 4 row groups x 8 column groups, so that every quarter warp reads one X address (broadcast) and eight W
// rows whose 16-byte pieces are stored swizzled (piece q of row n at q ^ (n / 4)): no bank conflicts.
// ---------------------------------------------------------------------------------------------------
// fp32: two stages and two CTAs per SM (102 KB each, 128 registers) measured 20 % faster than three stages and one
// CTA (522 against 651 us on the dense 3072 x 768 x 4096 product); the 16-bit types need more registers for the
// conversions and keep three stages, one CTA by registers.
// Row tiles of 64 (128 threads, 67 KB, three CTAs per SM in fp32) serve token counts that are no multiple of 128;
// where both apply the 128-row tile is faster even for small grids (notebook workload, 384 CTAs: 204 against
// 235 us; dense grid point 531 against 624 us).
template <typename T, int TM>
struct Fma32Cfg {
  static constexpr int kStages = sizeof(T) == 4 ? 2 : 3;
  static constexpr int kCtas = TM == 64 ? 3 : (sizeof(T) == 4 ? 2 : 1);
};

template <typename T, int TM>
__global__ void __launch_bounds__(2 * TM, Fma32Cfg<T, TM>::kCtas) bsmm_dsd_fma32_kernel(BsmmParams p) {
  constexpr int B = 32, NT = 2 * TM, P = 2, KC = 2;
  constexpr int kSt = Fma32Cfg<T, TM>::kStages;
  constexpr int KV = 16 / (int)sizeof(T);     // values per 16-byte piece
  constexpr int RP = B / KV;                  // pieces per block row (8 for fp32, 4 for 16-bit types)
  using S = FmaSmem<TM, T>;
  extern __shared__ __align__(16) uint8_t stage_mem[];
  __shared__ uint32_t kmask[kMaxKbFma];
  __shared__ uint16_t wpos[kMaxKbFma * P];
  __shared__ uint16_t clist[kMaxKbFma * B / kChunkK + 1];
  __shared__ int s_range[2];
  __shared__ int s_nchunks;

  const int panel = blockIdx.x, m0 = blockIdx.y * TM, batch = blockIdx.z;
  const int Nb = p.N / B, Kb = p.K / B;
  const int nb0 = panel * P, nb_end = min(nb0 + P, Nb);
  if (threadIdx.x == 0) {
    s_range[0] = p.ptr[nb0];
    s_range[1] = p.ptr[nb_end];
  }
  for (int k = threadIdx.x; k < Kb + (Kb & 1); k += NT) kmask[k] = 0;
  __syncthreads();
  const int e0 = s_range[0];
  const int32_t* idx = static_cast<const int32_t*>(p.idx);
  for (int e = e0 + threadIdx.x; e < s_range[1]; e += NT) {
    const int v = __ldg(idx + e);
    const int k = v & 0xffff, l = (v >> 16) - nb0;
    if (k < Kb && l >= 0 && l < P) {  // caller-provided indexes never address shared memory unchecked
      atomicOr(&kmask[k], 1u << l);
      wpos[k * P + l] = static_cast<uint16_t>(e - e0);
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x, all = p.K / kChunkK;
    int n = 0;
    for (int c0 = 0; c0 < all; c0 += 32) {
      const int c = c0 + lane;
      const uint32_t any = c < all ? (kmask[c * KC] | kmask[c * KC + 1]) : 0u;
      const unsigned bal = __ballot_sync(0xffffffffu, any != 0);
      if (any) clist[n + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>(c);
      n += __popc(bal);
    }
    if (lane == 0) s_nchunks = n;
  }
  __syncthreads();
  const int n_chunks = s_nchunks;

  const T* xtile = static_cast<const T*>(p.A) + ((long long)batch * p.M + m0) * p.K;
  const T* wbase = static_cast<const T*>(p.B) + ((long long)batch * p.val_stride_blocks + e0) * (B * B);
  constexpr int XP = kChunkK * (int)sizeof(T) / 16;
  constexpr int SP = B * B * (int)sizeof(T) / 16;
  constexpr int WP = S::kWBytes / 16;
  static_assert(NT % XP == 0 && (TM * XP) % NT == 0 && WP % NT == 0, "whole passes over the pieces");
  const int x_r0 = threadIdx.x / XP, x_q = threadIdx.x % XP;
  const uint8_t* x_src0 = reinterpret_cast<const uint8_t*>(xtile + (long long)x_r0 * p.K) + x_q * 16;
  const long long x_step = (long long)(NT / XP) * p.K * (long long)sizeof(T);
  auto issue = [&](int ci, int buf) {
    const int c = clist[ci];
    uint8_t* xs = stage_mem + buf * S::kStage;
    uint8_t* ws = xs + S::kXBytes;
    const uint8_t* src = x_src0 + (long long)c * kChunkK * sizeof(T);
    uint8_t* dst = xs + x_r0 * S::kXRow + x_q * 16;
#pragma unroll
    for (int it = 0; it < TM * XP / NT; ++it) {
      cp_async_16(dst, src);
      src += x_step;
      dst += (NT / XP) * S::kXRow;
    }
#pragma unroll
    for (int it = 0; it < WP / NT; ++it) {
      const int i = threadIdx.x + it * NT;
      const int slot = i / SP, within = i % SP;
      const int kc = slot / P, l = slot % P;
      const int k = c * KC + kc;
      if ((kmask[k] >> l) & 1u) {
        const int n = within / RP, q = within % RP;
        cp_async_16(ws + (slot * SP + n * RP + (q ^ ((n >> 2) & (RP - 1)))) * 16,
                    reinterpret_cast<const uint8_t*>(wbase + (long long)wpos[k * P + l] * (B * B)) + within * 16);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int g = threadIdx.x / TM, t = threadIdx.x % TM, ty = t >> 3, tx = t & 7;
  float acc[P][8][4];
#pragma unroll
  for (int l = 0; l < P; ++l)
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[l][i][c] = 0.f;

  for (int c = 0; c < kSt - 1; ++c) {
    if (c < n_chunks) issue(c, c);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int c = 0; c < n_chunks; ++c) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kSt - 2) : "memory");
    __syncthreads();
    if (c + kSt - 1 < n_chunks) issue(c + kSt - 1, (c + kSt - 1) % kSt);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    // The chunk's kept (K-block, block row) products -- at most four -- are dealt out alternately to the two thread
    // groups (whichever group computes a product, the partial sums are added at the end), starting with a
    // different group every chunk: with one K-block per group, a chunk whose two K-blocks keep different numbers
    // of blocks left one group waiting at the next barrier.
    const int chunk = clist[c];
    const uint32_t bits = (kmask[chunk * KC] & 3u) | ((kmask[chunk * KC + 1] & 3u) << 2);  // bit kc * 2 + l
    const uint8_t* xs = stage_mem + (c % kSt) * S::kStage;
    const uint8_t* ws = xs + S::kXBytes;
    int turn = c + g;  // the product is this group's when `turn` is even
#pragma unroll
    for (int pi = 0; pi < KC * P; ++pi) {
      if (!((bits >> pi) & 1u)) continue;
      if ((turn++) & 1) continue;
      const int kc = pi >> 1, l = pi & 1;  // compile-time after unrolling: acc[l] stays in registers
      const T* xrow = reinterpret_cast<const T*>(xs + (ty * 8) * S::kXRow) + kc * B;
      const uint8_t* wb = ws + (kc * P + l) * (SP * 16);
#pragma unroll 1
      for (int q = 0; q < RP; ++q) {
        float x[8][KV];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          load_floats<T, KV>(reinterpret_cast<const T*>(reinterpret_cast<const uint8_t*>(xrow) + i * S::kXRow) + q * KV, x[i]);
        float w[4][KV];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
          load_floats<T, KV>(reinterpret_cast<const T*>(wb + ((tx * 4 + cc) * RP + (q ^ (tx & (RP - 1)))) * 16), w[cc]);
#pragma unroll
        for (int kk = 0; kk < KV; ++kk)
#pragma unroll
          for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) acc[l][i][cc] = fmaf(x[i][kk], w[cc][kk], acc[l][i][cc]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // the second group hands its partial sums over through the (now idle) staging memory: [value][thread]
  float* red = reinterpret_cast<float*>(stage_mem);
  static_assert(kSt * S::kStage >= TM * 64 * 4, "staging memory holds the partial sums");
  if (g == 1) {
#pragma unroll
    for (int l = 0; l < P; ++l)
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[((l * 8 + i) * 4 + c) * TM + t] = acc[l][i][c];
  }
  __syncthreads();
  if (g == 1) return;
#pragma unroll
  for (int l = 0; l < P; ++l)
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[l][i][c] += red[((l * 8 + i) * 4 + c) * TM + t];

  // epilogue: + bias, convert; the eight threads of a row group write 32 consecutive columns of a row
  const T* bias = p.bias ? static_cast<const T*>(p.bias) + (long long)batch * p.N : nullptr;
#pragma unroll
  for (int l = 0; l < P; ++l) {
    if (nb0 + l >= nb_end) continue;
    const int col = (nb0 + l) * B + tx * 4;
    float bv[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias) {
#pragma unroll
      for (int c = 0; c < 4; ++c) bv[c] = to_float(bias[col + c]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      T* dst = static_cast<T*>(p.C) + ((long long)batch * p.M + m0 + ty * 8 + i) * p.N + col;
      alignas(16) T out[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) out[c] = from_float<T>(acc[l][i][c] + bv[c]);
      if constexpr (sizeof(T) == 4) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(out);
      else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(out);
    }
  }
}

template <typename T, int TM>
int launch_fma32_tm(const BsmmParams& p, cudaStream_t st) {
  using S = FmaSmem<TM, T>;
  auto kern = bsmm_dsd_fma32_kernel<T, TM>;
  static SmemAttrOnce attr;
  constexpr int kSmem = Fma32Cfg<T, TM>::kStages * S::kStage;
  if (cudaError_t e = attr.ensure(kern, kSmem); e != cudaSuccess) return static_cast<int>(e);
  const int panels = (p.N / 32 + 1) / 2;
  kern<<<dim3(panels, p.M / TM, p.batch), 2 * TM, kSmem, st>>>(p);
  return launch_status();
}

template <typename T>
int launch_fma32(const BsmmParams& p, cudaStream_t st) {
  if (p.M % 128 == 0) return launch_fma32_tm<T, 128>(p, st);
  return launch_fma32_tm<T, 64>(p, st);
}

template <int B, int TM, typename T>
int launch_tm(const BsmmParams& p, int panels, cudaStream_t st) {
  using S = FmaSmem<TM, T>;
  auto kern = bsmm_dsd_fma_kernel<B, TM, T>;
  static SmemAttrOnce attr;
  if (cudaError_t e = attr.ensure(kern, S::kTotal); e != cudaSuccess) return static_cast<int>(e);
  kern<<<dim3(panels, p.M / TM, p.batch), 2 * TM, S::kTotal, st>>>(p);
  return launch_status();
}

template <int B, typename T>
int launch_b(const BsmmParams& p, cudaStream_t st) {
  const int P = kPanelCols / B;
  const int panels = (p.N / B + P - 1) / P;
  if (p.M % 128 == 0 && (long long)panels * (p.M / 128) * p.batch >= kNumSMs / 2)
    return launch_tm<B, 128, T>(p, panels, st);
  return launch_tm<B, 64, T>(p, panels, st);
}

template <typename T>
int launch_t(const BsmmParams& p, cudaStream_t st) {
  switch (p.BN) {
    case 8: return launch_b<8, T>(p, st);
    case 16: return launch_b<16, T>(p, st);
    case 32: return launch_fma32<T>(p, st);  // M is a multiple of 64 (dsd_fma_supported)
    default: return SPARTA_ERR_UNSUPPORTED;
  }
}

}  // namespace

bool dsd_fma_supported(const BsmmParams& p) {
  if (p.mode != MODE_DSD || !p.trans_b || p.trans_a || !p.compressed || p.idx_is_64) return false;
  if (p.BN != p.BK || (p.BN != 8 && p.BN != 16 && p.BN != 32)) return false;
  if (p.M % 64 || p.K % kChunkK || p.N % p.BN) return false;
  if (p.K / p.BK > kMaxKbFma || p.n_index_sets != 1 || p.val_stride_blocks <= 0 || !p.ptr) return false;
  if (p.batch > 65535 || p.M / 64 > 65535) return false;
  if (!aligned(p.A, 16) || !aligned(p.B, 16) || !aligned(p.C, 16)) return false;
  if (p.bias && !aligned(p.bias, 4)) return false;
  return true;
}

int dsd_fma_launch(const BsmmParams& p, cudaStream_t st) {
  switch (p.dtype) {
    case SPARTA_F32: return launch_t<float>(p, st);
    case SPARTA_F16: return launch_t<__half>(p, st);
    case SPARTA_BF16: return launch_t<__nv_bfloat16>(p, st);
    default: return SPARTA_ERR_BAD_ARG;
  }
}

}  // namespace sparta
