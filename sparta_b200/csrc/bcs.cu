// Dense uint8 mask -> BCSR / BCSC / BCSRC block indexes in ONE launch.
//
// Phase 1 (every CTA): warps stream strips of the mask (BH rows x a 512-byte column segment) with
// 16-byte loads, OR-reduce each BH x BW block in registers and store one occupancy byte per block.
// Phase 2 (the last CTA of each mask to finish, found with an atomic ticket -- no spinning): counts
// per block row, a block-wide prefix sum into row_ptr and an ordered compaction into the packed
// index array, so entries come out in ascending column order within a row.
//
// Replaces bcs_index_1 / bcs_index_2 + torch.cumsum + .item()
// (sparta/tesa/templates/block_compressed.cu.j2:67-170, sparta/tesa/block_compressed.py:242-309).
#include "common.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct BcsParams {
  const uint8_t* mask;
  int n_masks, H, W, BH, BW, R, Cn;
  int want_bcsr, want_bcsc;
  int32_t* row_ptr;
  int32_t* bcsr_idx;
  int32_t* col_ptr;
  void* bcsc_idx;
  long long idx_capacity;
  int32_t* nnz;
  int32_t* uniform;
  uint8_t* occ;        // [n_masks, R, Cn]  bit0 = block kept, bit1 = block has a zero byte
  int32_t* rank;       // [n_masks, R, Cn]  BCSR position of kept blocks (only when both formats)
  unsigned* counters;  // [n_masks] tickets, zero between calls
  int seg_w;           // bytes of one mask row a warp covers per unit
  int segs;            // units per block row
  int units_per_mask;
  int bw_shift;        // log2(BW)
  int32_t* status;     // device status words (TMA path: a bounded wait that ran out sets word 0)
};

// 0x80 in every byte of w that is zero
__device__ __forceinline__ uint32_t zero_bytes(uint32_t w) {
  return (w - 0x01010101u) & ~w & 0x80808080u;
}

// In-place inclusive scan of p[1..n] (p[0] must be 0) by one CTA of up to 1024 threads: every thread sums a
// chunk, the chunk sums are scanned with shuffles inside each warp and the warp totals through shared memory
// (two barriers in all; s_part needs one word per warp).
__device__ void block_scan_inplace(int32_t* p, int n, int32_t* s_part) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nt = blockDim.x;
  const int chunk = (n + nt - 1) / nt;
  const int lo = min(n, tid * chunk), hi = min(n, lo + chunk);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += p[i + 1];
  int incl = sum;  // inclusive scan of the chunk sums within the warp
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += v;
  }
  if (lane == 31) s_part[warp] = incl;
  __syncthreads();
  int run = incl - sum;  // exclusive prefix of this thread's chunk
  for (int w = 0; w < warp; ++w) run += s_part[w];
  for (int i = lo; i < hi; ++i) {
    run += p[i + 1];
    p[i + 1] = run;
  }
  __syncthreads();
}

constexpr int kOccSmem = 16384;  // blocks of one mask held in shared memory by the compaction phase
constexpr int kPtrSmem = 2048;   // block rows / columns whose pointer array fits in shared memory

// Counts, prefix sum and ordered compaction for mask b, run by the whole (last) CTA.
// SMEM: occupancy bytes and the pointer array live in shared memory; otherwise in global memory.
template <bool SMEM>
__device__ void phase2(const BcsParams& p, int b, const uint8_t* occ, int32_t* s_ptr, int32_t* s_part,
                       int* s_nonuniform) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int R = p.R, Cn = p.Cn;
  auto occ_at = [&](size_t i) -> int { return SMEM ? occ[i] : __ldcg(&occ[i]); };
  int32_t* rank = p.rank ? p.rank + (size_t)b * R * Cn : nullptr;
  int nonuni = 0;
  if (p.want_bcsr) {
    int32_t* g_row_ptr = p.row_ptr + (size_t)b * (R + 1);
    int32_t* row_ptr = SMEM ? s_ptr : g_row_ptr;
    int32_t* out = p.bcsr_idx + (size_t)b * p.idx_capacity;
    if (threadIdx.x == 0) row_ptr[0] = 0;
    for (int r = warp; r < R; r += nwarp) {
      int cnt = 0;
      for (int c0 = 0; c0 < Cn; c0 += 32) {  // whole warps, so that every lane takes part in the ballot
        const int o = c0 + lane < Cn ? occ_at((size_t)r * Cn + c0 + lane) : 0;
        cnt += __popc(__ballot_sync(0xffffffffu, o & 1));
        nonuni |= o & 2;
      }
      if (lane == 0) row_ptr[r + 1] = cnt;
    }
    __syncthreads();
    block_scan_inplace(row_ptr, R, s_part);
    if (SMEM)
      for (int r = threadIdx.x; r <= R; r += blockDim.x) g_row_ptr[r] = row_ptr[r];
    for (int r = warp; r < R; r += nwarp) {
      int off = row_ptr[r];
      for (int c0 = 0; c0 < Cn; c0 += 32) {
        const int c = c0 + lane;
        const int f = (c < Cn) ? (occ_at((size_t)r * Cn + c) & 1) : 0;
        const unsigned bal = __ballot_sync(0xffffffffu, f);
        if (f) {
          const int pos = off + __popc(bal & ((1u << lane) - 1u));
          if (pos < p.idx_capacity) out[pos] = (r << 16) | c;
          if (rank) rank[(size_t)r * Cn + c] = pos;
        }
        off += __popc(bal);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) p.nnz[b] = row_ptr[R];
    __syncthreads();
  }
  if (p.want_bcsc) {
    int32_t* g_col_ptr = p.col_ptr + (size_t)b * (Cn + 1);
    int32_t* col_ptr = SMEM ? s_ptr : g_col_ptr;
    if (threadIdx.x == 0) col_ptr[0] = 0;
    for (int c = threadIdx.x; c < Cn; c += blockDim.x) {
      int cnt = 0;
      for (int r = 0; r < R; ++r) {
        const int o = occ_at((size_t)r * Cn + c);
        cnt += o & 1;
        nonuni |= o & 2;
      }
      col_ptr[c + 1] = cnt;
    }
    __syncthreads();
    block_scan_inplace(col_ptr, Cn, s_part);
    if (SMEM)
      for (int c = threadIdx.x; c <= Cn; c += blockDim.x) g_col_ptr[c] = col_ptr[c];
    const bool both = p.want_bcsr != 0;
    int32_t* out32 = reinterpret_cast<int32_t*>(p.bcsc_idx) + (size_t)b * p.idx_capacity;
    long long* out64 = reinterpret_cast<long long*>(p.bcsc_idx) + (size_t)b * p.idx_capacity;
    for (int c = threadIdx.x; c < Cn; c += blockDim.x) {
      int pos = col_ptr[c];
      for (int r = 0; r < R; ++r) {
        if (occ_at((size_t)r * Cn + c) & 1) {
          if (pos < p.idx_capacity) {
            if (both)
              out64[pos] = ((long long)rank[(size_t)r * Cn + c] << 32) | (long long)((c << 16) | r);
            else
              out32[pos] = (c << 16) | r;
          }
          ++pos;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0 && !p.want_bcsr) p.nnz[b] = col_ptr[Cn];
  }
  if (nonuni) *s_nonuniform = 1;  // benign race: every writer stores 1
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.uniform) p.uniform[b] = *s_nonuniform ? 0 : 1;
    p.counters[b] = 0;  // leave the ticket ready for the next call
  }
}

template <int VW>
__global__ void __launch_bounds__(kThreads, 4) bcs_build_kernel(BcsParams p) {
  constexpr int NWORD = VW / 4;
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint8_t* mask = p.mask + (size_t)b * p.H * p.W;
  uint8_t* occ = p.occ + (size_t)b * p.R * p.Cn;

  // ---------------- phase 1: block occupancy ----------------
  const int nwarps = gridDim.x * kWarps;
  for (int u = blockIdx.x * kWarps + warp; u < p.units_per_mask; u += nwarps) {
    const int r = u / p.segs;
    const int col0 = (u - r * p.segs) * p.seg_w;
    uint32_t any[NWORD], zer[NWORD];
#pragma unroll
    for (int i = 0; i < NWORD; ++i) any[i] = zer[i] = 0;
    const uint8_t* row0 = mask + (size_t)r * p.BH * p.W;
    for (int c = col0 + lane * VW; c < col0 + p.seg_w; c += 32 * VW) {
      if (c < p.W) {
        const uint8_t* src = row0 + c;
        if constexpr (VW == 16) {
          const uint4* q = reinterpret_cast<const uint4*>(src);
          const size_t pitch = (size_t)p.W / 16;
          int y = 0;
          for (; y + 8 <= p.BH; y += 8) {  // eight 16-byte loads in flight per lane
            uint4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __ldg(q + (size_t)(y + i) * pitch);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              any[0] |= v[i].x; any[1] |= v[i].y; any[2] |= v[i].z; any[3] |= v[i].w;
              zer[0] |= zero_bytes(v[i].x); zer[1] |= zero_bytes(v[i].y);
              zer[2] |= zero_bytes(v[i].z); zer[3] |= zero_bytes(v[i].w);
            }
          }
          for (; y < p.BH; y += 4) {  // BH = 4 (or the tail of 12, 20, ...: not reachable, BH is 2^n)
            uint4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = __ldg(q + (size_t)(y + i) * pitch);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              any[0] |= v[i].x; any[1] |= v[i].y; any[2] |= v[i].z; any[3] |= v[i].w;
              zer[0] |= zero_bytes(v[i].x); zer[1] |= zero_bytes(v[i].y);
              zer[2] |= zero_bytes(v[i].z); zer[3] |= zero_bytes(v[i].w);
            }
          }
        } else {
          for (int y = 0; y < p.BH; y += 4) {  // BH is a multiple of 4: four loads in flight
            uint32_t v0 = __ldg(reinterpret_cast<const uint32_t*>(src + (size_t)(y + 0) * p.W));
            uint32_t v1 = __ldg(reinterpret_cast<const uint32_t*>(src + (size_t)(y + 1) * p.W));
            uint32_t v2 = __ldg(reinterpret_cast<const uint32_t*>(src + (size_t)(y + 2) * p.W));
            uint32_t v3 = __ldg(reinterpret_cast<const uint32_t*>(src + (size_t)(y + 3) * p.W));
            any[0] |= v0 | v1 | v2 | v3;
            zer[0] |= zero_bytes(v0) | zero_bytes(v1) | zero_bytes(v2) | zero_bytes(v3);
          }
        }
      }
    }
    const int c_lane = col0 + lane * VW;  // first column of this lane's (first) chunk
    if (p.BW >= VW) {
      uint32_t a = 0, z = 0;
#pragma unroll
      for (int i = 0; i < NWORD; ++i) { a |= any[i]; z |= zer[i]; }
      const int g = min(32, p.BW / VW);  // lanes per block
      for (int off = 1; off < g; off <<= 1) {
        a |= __shfl_xor_sync(0xffffffffu, a, off);
        z |= __shfl_xor_sync(0xffffffffu, z, off);
      }
      const int cb = c_lane / p.BW;
      if ((lane & (g - 1)) == 0 && cb < p.Cn)
        occ[(size_t)r * p.Cn + cb] = a ? (z ? 3 : 1) : 0;
    } else {
      // several blocks per lane (VW == 16, BW in {4, 8})
      const int words_per_block = p.BW / 4;
      for (int w = 0; w < NWORD; w += words_per_block) {
        uint32_t a = any[w], z = zer[w];
        if (words_per_block == 2 && w + 1 < NWORD) { a |= any[w + 1]; z |= zer[w + 1]; }
        const int cb = (c_lane + w * 4) / p.BW;
        if (cb < p.Cn) occ[(size_t)r * p.Cn + cb] = a ? (z ? 3 : 1) : 0;
      }
    }
  }

  // ---------------- ticket: is this the last CTA of mask b? ----------------
  __shared__ int s_last;
  __shared__ int32_t s_part[kThreads];
  __shared__ int s_nonuniform;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned ticket = atomicAdd(&p.counters[b], 1u);
    s_last = (ticket == gridDim.x - 1);
    s_nonuniform = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // ---------------- phase 2: scan + ordered compaction ----------------
  // Small block grids (the usual case) are first copied into shared memory with one round of wide
  // loads, so the counting / scanning / compaction below never waits on L2 again.
  __shared__ __align__(16) uint8_t s_occ[kOccSmem];
  __shared__ int32_t s_ptr[kPtrSmem + 1];
  const int R = p.R, Cn = p.Cn;
  const bool fast = (size_t)R * Cn <= kOccSmem && R <= kPtrSmem && Cn <= kPtrSmem &&
                    (((size_t)b * R * Cn) % 16 == 0);
  if (fast) {
    const int n16 = (R * Cn + 15) / 16;
    for (int i = threadIdx.x; i < n16; i += kThreads)
      reinterpret_cast<uint4*>(s_occ)[i] = __ldcg(reinterpret_cast<const uint4*>(occ) + i);
    __syncthreads();
    phase2<true>(p, b, s_occ, s_ptr, s_part, &s_nonuniform);
  } else {
    phase2<false>(p, b, occ, nullptr, s_part, &s_nonuniform);
  }
}

// ---------------------------------------------------------------------------------------------------
// Phase 1 through TMA.  The mask is described to the TMA unit as rows of 32-bit words, so one bulk
// tensor copy can fetch a tile of 4 rows x 1 KB (four contiguous kilobytes of DRAM pages instead of many
// short row pieces).  Each warp runs its own pipeline: three 4 KB shared-memory slots, each guarded by
// its own mbarrier, so 12 KB per warp (192 KB per SM with sixteen warps) are in flight without holding
// them in registers.  A lane owns the 16-byte chunks `lane` and `lane + 32` of the 64 chunks of a
// kilobyte, reduces them over the rows of a block row (BH / 4 tiles), writes the occupancy bytes and
// lets lane 0 re-arm the slot with the tile three steps ahead.  Phase 2 is shared with the load-based
// kernel.  Used when the row pitch is a multiple of 16 bytes.
// ---------------------------------------------------------------------------------------------------
constexpr int kTmaThreads = 256;
constexpr int kTmaWarps = kTmaThreads / 32;
constexpr int kTmaSlots = 3;
constexpr int kTileRows = 4, kTileCols = 1024;
constexpr int kTileBytes = kTileRows * kTileCols;
constexpr int kTmaSmem = kTmaWarps * kTmaSlots * kTileBytes + 256 + 1024;

// `any` / `zer`: OR of the words / of the zero-byte flags of one 16-byte column chunk over the rows of
// a block row; col is the chunk's first mask column.
__device__ __forceinline__ void emit_blocks(const BcsParams& p, uint8_t* occ_row, const uint32_t (&any)[4],
                                            const uint32_t (&zer)[4], int col, int lane) {
  if (p.BW >= 16) {
    uint32_t a = any[0] | any[1] | any[2] | any[3], z = zer[0] | zer[1] | zer[2] | zer[3];
    const int g = p.BW >> 4;  // lanes per block: 1 .. 16, a power of two
    for (int off = 1; off < g; off <<= 1) {
      a |= __shfl_xor_sync(0xffffffffu, a, off);
      z |= __shfl_xor_sync(0xffffffffu, z, off);
    }
    const int cb = col >> p.bw_shift;
    if ((lane & (g - 1)) == 0 && cb < p.Cn) occ_row[cb] = a ? (z ? 3 : 1) : 0;
  } else if (p.BW == 8) {
    const int cb = col >> 3;
    if (cb < p.Cn) occ_row[cb] = (any[0] | any[1]) ? ((zer[0] | zer[1]) ? 3 : 1) : 0;
    if (cb + 1 < p.Cn) occ_row[cb + 1] = (any[2] | any[3]) ? ((zer[2] | zer[3]) ? 3 : 1) : 0;
  } else {
    const int cb = col >> 2;
#pragma unroll
    for (int w = 0; w < 4; ++w)
      if (cb + w < p.Cn) occ_row[cb + w] = any[w] ? (zer[w] ? 3 : 1) : 0;
  }
}

__global__ void __launch_bounds__(kTmaThreads, 2)
bcs_build_tma_kernel(const __grid_constant__ CUtensorMap tm, BcsParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTmaWarps * kTmaSlots * kTileBytes);
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* occ = p.occ + (size_t)b * p.R * p.Cn;
  uint8_t* ring = smem + warp * kTmaSlots * kTileBytes;
  uint64_t* bar = bars + warp * kTmaSlots;

  // a unit = one block row (BH rows) x 1024 columns = BH / 4 tiles
  const int tiles_per_unit = p.BH / kTileRows;
  const int segs = (p.W + kTileCols - 1) / kTileCols;
  const int units = p.R * segs;
  // each warp takes a contiguous run of units
  const int wid = blockIdx.x * kTmaWarps + warp, nw = gridDim.x * kTmaWarps;
  const int u0 = (int)((long long)units * wid / nw);
  const int n_units = (int)((long long)units * (wid + 1) / nw) - u0;
  const int n_tiles = n_units * tiles_per_unit;

  if (lane == 0) {
    for (int s = 0; s < kTmaSlots; ++s) tc::mbar_init(&bar[s], 1);
    tc::fence_mbar_init();
  }
  __syncwarp();
  // cursors over (block row, segment, tile of the unit), advanced without divisions: one for the
  // producer lane (three tiles ahead) and one for the consumer
  struct Cursor { int br, sg, sub; };
  auto advance = [&](Cursor& c) {
    if (++c.sub == tiles_per_unit) {
      c.sub = 0;
      if (++c.sg == segs) { c.sg = 0; ++c.br; }
    }
  };
  Cursor pc = {u0 / segs, u0 % segs, 0}, cc = pc;
  int ps = 0;  // slot the producer fills next
  auto issue = [&]() {
    tc::mbar_arrive_expect_tx(&bar[ps], kTileBytes);
    // x in 32-bit words: a multiple of 256 words, so the copy starts on a 1 KB boundary of the row
    tc::tma_load_2d(ring + ps * kTileBytes, &tm, pc.sg * (kTileCols / 4), b * p.H + pc.br * p.BH + pc.sub * kTileRows,
                    &bar[ps]);
    advance(pc);
    ps = (ps == kTmaSlots - 1) ? 0 : ps + 1;
  };
  if (lane == 0)
    for (int t = 0; t < min(kTmaSlots, n_tiles); ++t) issue();

  uint32_t any0[4] = {0, 0, 0, 0}, zer0[4] = {0, 0, 0, 0}, any1[4] = {0, 0, 0, 0}, zer1[4] = {0, 0, 0, 0};
  int s = 0;
  uint32_t parity = 0;
  bool failed = false;  // a bounded wait gave up: tiles of this warp may still be in flight
  for (int t = 0; t < n_tiles; ++t) {
    if (!tc::mbar_wait_warp(&bar[s], parity)) {
      if (lane == 0 && p.status) atomicExch(&p.status[0], 1);
      failed = true;
      break;
    }
    const uint4* tile = reinterpret_cast<const uint4*>(ring + s * kTileBytes);
#pragma unroll
    for (int r = 0; r < kTileRows; ++r) {
      const uint4 v = tile[r * 64 + lane], w = tile[r * 64 + 32 + lane];
      any0[0] |= v.x; any0[1] |= v.y; any0[2] |= v.z; any0[3] |= v.w;
      zer0[0] |= zero_bytes(v.x); zer0[1] |= zero_bytes(v.y); zer0[2] |= zero_bytes(v.z); zer0[3] |= zero_bytes(v.w);
      any1[0] |= w.x; any1[1] |= w.y; any1[2] |= w.z; any1[3] |= w.w;
      zer1[0] |= zero_bytes(w.x); zer1[1] |= zero_bytes(w.y); zer1[2] |= zero_bytes(w.z); zer1[3] |= zero_bytes(w.w);
    }
    __syncwarp();  // every lane has read the slot before it is re-armed
    if (lane == 0 && t + kTmaSlots < n_tiles) issue();
    if (cc.sub == tiles_per_unit - 1) {
      uint8_t* occ_row = occ + (size_t)cc.br * p.Cn;
      const int col = cc.sg * kTileCols + lane * 16;
      emit_blocks(p, occ_row, any0, zer0, col, lane);
      emit_blocks(p, occ_row, any1, zer1, col + 512, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) any0[i] = zer0[i] = any1[i] = zer1[i] = 0;
    }
    advance(cc);
    if (++s == kTmaSlots) { s = 0; parity ^= 1; }
  }

  // ---------------- ticket + phase 2 (as in the load-based kernel) ----------------
  __shared__ int s_last;
  __shared__ int32_t s_part[256];
  __shared__ int s_nonuniform;
  tc::sync_and_drain(failed);
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned ticket = atomicAdd(&p.counters[b], 1u);
    s_last = (ticket == gridDim.x - 1);
    s_nonuniform = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the tile ring is idle now: reuse it for the occupancy bytes and the pointer array
  uint8_t* s_occ = smem;
  int32_t* s_ptr = reinterpret_cast<int32_t*>(smem + kOccSmem);
  const int R = p.R, Cn = p.Cn;
  const bool fast = (size_t)R * Cn <= kOccSmem && R <= kPtrSmem && Cn <= kPtrSmem &&
                    (((size_t)b * R * Cn) % 16 == 0);
  if (fast) {
    const int n16 = (R * Cn + 15) / 16;
    for (int i = threadIdx.x; i < n16; i += blockDim.x)
      reinterpret_cast<uint4*>(s_occ)[i] = __ldcg(reinterpret_cast<const uint4*>(occ) + i);
    __syncthreads();
    phase2<true>(p, b, s_occ, s_ptr, s_part, &s_nonuniform);
  } else {
    phase2<false>(p, b, occ, nullptr, s_part, &s_nonuniform);
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace
}  // namespace sparta

using namespace sparta;

extern "C" size_t sparta_bcs_build_workspace_bytes(int n_masks, int H, int W, int BH, int BW) {
  if (n_masks <= 0 || H <= 0 || W <= 0 || BH <= 0 || BW <= 0) return 0;
  const size_t blocks = (size_t)n_masks * (H / BH) * (W / BW);
  // occupancy bytes + BCSR ranks (int32) + tickets
  return align_up(blocks, 256) + align_up(blocks * 4, 256) + align_up((size_t)n_masks * 4, 256);
}

extern "C" int sparta_bcs_build(const uint8_t* mask, int n_masks, int H, int W, int BH, int BW,
                                int want_bcsr, int want_bcsc, int32_t* row_ptr, int32_t* bcsr_idx,
                                int32_t* col_ptr, void* bcsc_idx, int64_t idx_capacity, int32_t* nnz,
                                int32_t* uniform, int32_t* h_nnz, void* workspace,
                                size_t workspace_bytes, void* stream) {
  if (!mask || !nnz || n_masks <= 0 || H <= 0 || W <= 0) return SPARTA_ERR_BAD_ARG;
  if (!want_bcsr && !want_bcsc) return SPARTA_ERR_BAD_ARG;
  if (want_bcsr && (!row_ptr || !bcsr_idx)) return SPARTA_ERR_BAD_ARG;
  if (want_bcsc && (!col_ptr || !bcsc_idx)) return SPARTA_ERR_BAD_ARG;
  if (!valid_bcs_block(BH) || !valid_bcs_block(BW)) return SPARTA_ERR_SHAPE;
  if (H % BH || W % BW) return SPARTA_ERR_SHAPE;
  const int R = H / BH, Cn = W / BW;
  if (R > 32767 || Cn > 65535 || idx_capacity <= 0) return SPARTA_ERR_SHAPE;  // 16-bit packing
  if (n_masks > 65535) return SPARTA_ERR_SHAPE;
  if (!workspace || workspace_bytes < sparta_bcs_build_workspace_bytes(n_masks, H, W, BH, BW))
    return SPARTA_ERR_WORKSPACE;
  if (!aligned(workspace, 256) || !aligned(mask, 4)) return SPARTA_ERR_ALIGN;

  const size_t blocks = (size_t)n_masks * R * Cn;
  BcsParams p;
  p.mask = mask;
  p.n_masks = n_masks; p.H = H; p.W = W; p.BH = BH; p.BW = BW; p.R = R; p.Cn = Cn;
  p.want_bcsr = want_bcsr; p.want_bcsc = want_bcsc;
  p.row_ptr = row_ptr; p.bcsr_idx = bcsr_idx; p.col_ptr = col_ptr; p.bcsc_idx = bcsc_idx;
  p.idx_capacity = idx_capacity;
  p.nnz = nnz; p.uniform = uniform;
  p.status = nullptr;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.occ = ws;
  p.rank = (want_bcsr && want_bcsc) ? reinterpret_cast<int32_t*>(ws + align_up(blocks, 256)) : nullptr;
  p.counters = reinterpret_cast<unsigned*>(ws + align_up(blocks, 256) + align_up(blocks * 4, 256));

  const bool vec16 = (W % 16 == 0) && aligned(mask, 16);
  const int vw = vec16 ? 16 : 4;
  p.seg_w = (32 * vw > BW) ? 32 * vw : BW;
  p.segs = (W + p.seg_w - 1) / p.seg_w;
  p.units_per_mask = R * p.segs;
  p.bw_shift = 0;
  while ((1 << p.bw_shift) < BW) ++p.bw_shift;

  // spread the units of all masks over the warps resident at once (148 SMs x 4 CTAs x 8 warps), so
  // the grid is a single wave
  const long long total_units = (long long)n_masks * p.units_per_mask;
  const long long warp_slots = (long long)kNumSMs * 4 * kWarps;
  const int units_per_warp = (int)((total_units + warp_slots - 1) / warp_slots);
  int ctas = (p.units_per_mask + kWarps * units_per_warp - 1) / (kWarps * units_per_warp);
  if (ctas < 1) ctas = 1;
  dim3 grid(ctas, n_masks), block(kThreads);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  bool launched = false;
  if (vec16 && (long long)n_masks * H <= 0x7fffffffll && tc::encode_tiled_fn() != nullptr) {
    // TMA streaming path: two CTAs of eight warps per SM, every warp with its own three-slot pipeline
    CUtensorMap tm;
    const uint64_t dims[2] = {(uint64_t)W / 4, (uint64_t)n_masks * H};  // rows of 32-bit words
    const uint64_t strides[1] = {(uint64_t)W};
    const uint32_t box[2] = {kTileCols / 4, kTileRows};
    if (tc::make_tensor_map(&tm, mask, tc::kTensorMapU32, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE) ==
        SPARTA_OK) {
      static SmemAttrOnce attr;
      if (cudaError_t e = attr.ensure(bcs_build_tma_kernel, kTmaSmem); e != cudaSuccess) return static_cast<int>(e);
      const int units = R * ((W + kTileCols - 1) / kTileCols);
      int per_mask = (2 * kNumSMs) / n_masks;                       // fill the 296 CTA slots once
      const int by_units = (units + kTmaWarps - 1) / kTmaWarps;     // at least one unit per warp
      if (per_mask > by_units) per_mask = by_units;
      if (per_mask < 1) per_mask = 1;
      p.status = tc::device_status_ptr();
      bcs_build_tma_kernel<<<dim3(per_mask, n_masks), kTmaThreads, kTmaSmem, st>>>(tm, p);
      launched = true;
    }
  }
  if (!launched) {
    if (vec16)
      bcs_build_kernel<16><<<grid, block, 0, st>>>(p);
    else
      bcs_build_kernel<4><<<grid, block, 0, st>>>(p);
  }
  int rc = launch_status();
  if (rc != SPARTA_OK) return rc;
  if (h_nnz) {
    cudaError_t e = cudaMemcpyAsync(h_nnz, nnz, sizeof(int32_t) * n_masks, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return SPARTA_OK;
}

// ---------------------------------------------------------------------------------------------------
// Index build for callers that cannot allocate device memory.
//
// sparta_bcs_build() needs a workspace from its caller.  Some callers have no way to get one: a
// serving loop whose memory pool is frozen after start-up, a plug-in running under a host framework
// that forbids cudaMalloc on its threads (the call synchronises the device and can fail once memory
// is fragmented), or a mask update issued from a callback while another thread holds the framework's
// allocator lock.  For them the scratch lives in the library image itself: a fixed array in device
// global memory that every GPU loading this library carries until the process exits.
//
// Limits and rules
//   * the array is SPARTA_BCS_STATIC_SCRATCH_BYTES (1 MiB) per device; a mask set whose
//     sparta_bcs_build_workspace_bytes() is larger is refused with SPARTA_ERR_WORKSPACE
//     (1 MiB covers e.g. 32 masks of 2048 x 2048 or one mask of 8192 x 8192 at 32 x 32 blocks);
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress) with that
//     device current; make that first call before starting any stream capture;
//   * all calls on a device share the one array and it keeps whatever the previous call left, so the
//     ticket words are cleared on the stream before each launch; two calls that may run on the GPU at
//     the same time (different streams, different host threads) race on it -- serialise them;
//   * nothing here calls cudaMalloc, cudaFree or any allocating routine.
// ---------------------------------------------------------------------------------------------------
#include <mutex>

namespace {

static __device__ __align__(256) unsigned char g_bcs_static_scratch[SPARTA_BCS_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the static scratch on the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel may use, hence the symbol lookup (once per device).
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return SPARTA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_bcs_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (!p) return SPARTA_ERR_DRIVER;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return SPARTA_OK;
}

}  // namespace

extern "C" int sparta_bcs_build_static(const uint8_t* mask, int n_masks, int H, int W, int BH, int BW,
                                       int want_bcsr, int want_bcsc, int32_t* row_ptr, int32_t* bcsr_idx,
                                       int32_t* col_ptr, void* bcsc_idx, int64_t idx_capacity, int32_t* nnz,
                                       int32_t* uniform, void* stream) {
  if (n_masks <= 0 || H <= 0 || W <= 0) return SPARTA_ERR_BAD_ARG;
  if (!valid_bcs_block(BH) || !valid_bcs_block(BW) || H % BH || W % BW) return SPARTA_ERR_SHAPE;
  const size_t need = sparta_bcs_build_workspace_bytes(n_masks, H, W, BH, BW);
  if (need == 0 || need > (size_t)SPARTA_BCS_STATIC_SCRATCH_BYTES) return SPARTA_ERR_WORKSPACE;
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != SPARTA_OK) return rc;
  // the ticket words sit at the end of the workspace layout and must read zero when the kernel starts
  const size_t blocks = (size_t)n_masks * (H / BH) * (W / BW);
  const size_t ticket_off = align_up(blocks, 256) + align_up(blocks * 4, 256);
  cudaError_t e = cudaMemsetAsync(static_cast<unsigned char*>(scratch) + ticket_off, 0,
                                  align_up((size_t)n_masks * 4, 256), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return sparta_bcs_build(mask, n_masks, H, W, BH, BW, want_bcsr, want_bcsc, row_ptr, bcsr_idx, col_ptr,
                          bcsc_idx, idx_capacity, nnz, uniform, nullptr, scratch, need, stream);
}
