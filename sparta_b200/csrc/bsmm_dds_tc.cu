// Output-sparse (dds) block matmul on tcgen05 / TMEM / TMA, fp16 / bf16, 32 x 32 output blocks:
//   C_block(m, n) = A[m-block rows, :] . op(B)[:, n-block cols]  (+ bias)   for every kept block.
//
// Small-N tensor-core instructions carry a fixed cost (a 128 x 32 x 16 MMA takes about as long as a
// 128 x 128 x 16 one), so kept blocks are not computed one by one.  A CTA owns 128 consecutive rows
// (four block rows) and a GROUP of up to eight block columns picked from those in which at least one
// of the four block rows keeps a block; it runs the full-K contraction as M128 x N(32 * columns) MMAs
// with the B operand GATHERED column block by column block through TMA, and its epilogue writes only
// the kept 32 x 32 blocks (compressed BCSR order or dense).  At 90 % block sparsity about two thirds of
// the block columns of a row tile are skipped entirely.
//   warp 4    producer: A tile [128, 64] by coordinate (four [64, 32] boxes when A is stored [K, M]), B tiles
//             [32, 64] of the group's columns
//   warp 5    one thread issues four tcgen05.mma per 64-wide K chunk and commits
//   warps 0-3 epilogue: warp w holds block row w of the tile (TMEM lanes 32w .. 32w+31)
// Replaces sparta_sparse_matmul_dds.cuh.j2 / openai_sparse_matmul_dds.cuh.j2 for these layouts.
#include <type_traits>

#include "bsmm.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

using namespace tc;

constexpr int kBlk = 32;          // output block edge
constexpr int kTileM = 128;       // rows per CTA (four block rows)
constexpr int kGroup = 8;         // block columns per CTA
constexpr int kChunkK = 64;       // K elements per pipeline stage (128 bytes)
constexpr int kABytes = kTileM * kChunkK * 2;         // 16 KB
constexpr int kBBlockBytes = kBlk * kChunkK * 2;      // 4 KB per gathered column block
constexpr int kStageBytes = kABytes + kGroup * kBBlockBytes;  // 48 KB
constexpr int kMaxNb = 1024;      // block columns (N <= 32768)
constexpr int kThreads = 192;
// STAGES = 4 (197 KB, one CTA per SM) for long K; STAGES = 2 (101 KB, two CTAs per SM, so that the
// prologue and epilogue of one overlap the main loop of the other) when K has at most two chunks.
constexpr int smem_bytes(int stages) {
  return stages * kStageBytes + kMaxNb /* column masks */ + kMaxNb * 2 /* column list */ +
         512 /* barriers, positions */ + 1024 /* align */;
}

struct DdsTcParams {
  const int32_t* row_ptr;
  const int32_t* idx;
  const void* bias;
  void* C;
  int M, N, K, Nb;
  int compressed, trans_b;
  int n_index_sets;
  long long ptr_stride, idx_stride, val_stride_blocks;
  int32_t* status;
};

template <int FMT, int STAGES, bool LOOP, bool TA>
__global__ void __launch_bounds__(kThreads, STAGES == 2 ? 2 : 1)
bsmm_dds_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   DdsTcParams p) {
  using T = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* cmask = smem + STAGES * kStageBytes;                      // [Nb] 4 presence bits per column
  uint16_t* clist = reinterpret_cast<uint16_t*>(cmask + kMaxNb);      // needed columns, ascending
  uint8_t* ctl = reinterpret_cast<uint8_t*>(clist + kMaxNb);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctl);              // [STAGES]
  uint64_t* empty_bar = full_bar + STAGES;                           // [STAGES]
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_bar + 1);
  int* s_count = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_range = s_count + 1;                                         // [2]
  int* s_pos = s_range + 2;                                           // [4][kGroup] BCSR position or -1

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = blockIdx.x, tile = blockIdx.y, batch = blockIdx.z;
  const int mb0 = tile * 4;
  const int set = p.n_index_sets > 1 ? batch : 0;
  const int32_t* row_ptr = p.row_ptr + (long long)set * p.ptr_stride;
  const int32_t* idx = p.idx + (long long)set * p.idx_stride;

  // ---- which block columns does this row tile need? (uniform across the CTA, no tensor memory yet) ----
  if (threadIdx.x == 0) {
    s_range[0] = row_ptr[mb0];
    s_range[1] = row_ptr[mb0 + 4];
  }
  for (int c = threadIdx.x; c < p.Nb; c += kThreads) cmask[c] = 0;
  __syncthreads();
  for (int e = s_range[0] + threadIdx.x; e < s_range[1]; e += kThreads) {
    const int v = __ldg(idx + e);
    const int c = v & 0xffff, r = (v >> 16) - mb0;
    if (c < p.Nb && r >= 0 && r < 4)  // index arrays come from the caller: never index shared memory with them unchecked
      atomicOr(reinterpret_cast<unsigned int*>(cmask + (c & ~3)), (1u << r) << (8 * (c & 3)));
  }
  __syncthreads();
  if (warp == 0) {
    int n = 0;
    for (int base = 0; base < p.Nb; base += 32) {
      const int c = base + lane;
      const int m = c < p.Nb ? cmask[c] : 0;
      const unsigned bal = __ballot_sync(0xffffffffu, m != 0);
      if (m) clist[n + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>(c);
      n += __popc(bal);
    }
    if (lane == 0) *s_count = n;
  }
  __syncthreads();
  const int ncols_total = *s_count;
  if (group * kGroup >= ncols_total) return;  // nothing for this CTA: leave before any barrier / TMEM use
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    fence_mbar_init();
  }
  if (warp == 4 && lane == 0) {
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 5) tmem_alloc<256>(tmem_holder);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const int nchunks = p.K / kChunkK;

  // A CTA takes the groups blockIdx.x, blockIdx.x + gridDim.x, ... of its row tile one after the other:
  // the union of needed columns, the barriers and the tensor memory are set up once.  The pipeline
  // barriers keep their phases across groups (cc counts chunks since the start); a CTA-wide barrier
  // separates the groups, so the accumulator and s_pos are free when the next group starts.
  bool failed = false;  // a bounded wait of this thread gave up
  int cc0 = 0;          // chunks issued by the groups before this one
  for (int it = 0, g = group; g * kGroup < ncols_total; g += gridDim.x, ++it, cc0 += nchunks) {
  const int c_first = g * kGroup;
  const int ncols = min(kGroup, ncols_total - c_first);
  if (warp == 4) {
    // ------------------------------ producer ------------------------------
    const int col = lane < ncols ? clist[c_first + lane] : 0;
    bool ok = true;
    for (int c = 0; c < nchunks; ++c) {
      const int cc = LOOP ? cc0 + c : c, s = cc % STAGES;
      if (!mbar_wait(&empty_bar[s], ((cc / STAGES) & 1) ^ 1)) { ok = false; break; }
      uint8_t* st = stages + s * kStageBytes;
      if (lane == 0) {
        mbar_arrive_expect_tx(&full_bar[s], kABytes + ncols * kBBlockBytes);
        if constexpr (!TA) tma_load_2d(st, &tm_a, c * kChunkK, batch * p.M + tile * kTileM, &full_bar[s]);
      }
      if constexpr (TA) {  // A stored [K, M]: the tile's four block rows, 32 rows contiguous per K row
        if (lane >= 16 && lane < 20)
          tma_load_2d(st + (lane - 16) * kBBlockBytes, &tm_a, tile * kTileM + (lane - 16) * kBlk, batch * p.K + c * kChunkK,
                      &full_bar[s]);
      }
      if (lane < ncols) {
        uint8_t* dst = st + kABytes + lane * kBBlockBytes;
        if (p.trans_b) tma_load_2d(dst, &tm_b, c * kChunkK, batch * p.N + col * kBlk, &full_bar[s]);
        else tma_load_2d(dst, &tm_b, col * kBlk, batch * p.K + c * kChunkK, &full_bar[s]);
      }
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[0], 1);
  } else if (warp == 5) {
    // ------------------------------ MMA issue ------------------------------
    // A: K-major, 128-byte swizzle.  B: K-major 128-byte swizzle when stored [N, K]; MN-major 64-byte
    // swizzle when stored [K, N] (32 columns contiguous per K row, column blocks 4 KB apart).
    // A stored [K, M] is the mirror of B stored [K, N]: MN-major, block rows 4 KB apart.
    const uint64_t a_hi = TA ? make_smem_desc(0, kBBlockBytes, 512, SW_64B) : make_smem_desc(0, 16, 1024, SW_128B);
    constexpr uint32_t a_step = TA ? (16u * 64u) >> 4 : 2u;
    const uint64_t b_hi = p.trans_b ? make_smem_desc(0, 16, 1024, SW_128B)
                                    : make_smem_desc(0, kBBlockBytes, 512, SW_64B);
    const uint32_t b_step = p.trans_b ? 2u : (16u * 64u) >> 4;  // 16 K elements, in 16-byte units
    const uint32_t idesc = make_idesc_f16(kTileM, kBlk * ncols, FMT, TA ? 1 : 0, p.trans_b ? 0 : 1);
    const uint32_t base = smem_u32(stages) >> 4;
    bool ok = true;
    for (int c = 0; c < nchunks; ++c) {
      const int cc = LOOP ? cc0 + c : c, s = cc % STAGES;
      if (!mbar_wait(&full_bar[s], (cc / STAGES) & 1)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t a_lo = base + ((s * kStageBytes) >> 4);
        const uint32_t b_lo = a_lo + (kABytes >> 4);
#pragma unroll
        for (int kk = 0; kk < kChunkK / 16; ++kk)
          umma_ss(tmem_base, a_hi | (a_lo + a_step * kk), b_hi | (b_lo + b_step * kk), idesc, (c | kk) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[1], 1);
    if (lane == 0) umma_commit(accum_bar);
  } else {
    // ------------------------------ epilogue: kept blocks only ------------------------------
    // BCSR positions of the kept blocks of this group (for the compressed output), found by the four
    // epilogue warps while the loads and MMAs of the group run
    for (int i = threadIdx.x; i < 4 * kGroup; i += 128) s_pos[i] = -1;
    named_barrier_sync(1, 128);
    for (int e = s_range[0] + threadIdx.x; e < s_range[1]; e += 128) {
      const int v = __ldg(idx + e);
      const int c = v & 0xffff, r = (v >> 16) - mb0;
      if (r < 0 || r >= 4) continue;
      for (int l = 0; l < ncols; ++l)
        if (clist[c_first + l] == c) s_pos[r * kGroup + l] = e;
    }
    named_barrier_sync(1, 128);
    if (!mbar_wait_warp(accum_bar, LOOP ? (it & 1) : 0)) {
      failed = true;
      if (lane == 0) atomicExch(&p.status[2], 1);
    } else {
      tc_fence_after_sync();
      const T* bias = p.bias ? static_cast<const T*>(p.bias) + (long long)batch * p.N : nullptr;
      T* C = static_cast<T*>(p.C);
      for (int l = 0; l < ncols; ++l) {
        const int pos = s_pos[warp * kGroup + l];
        if (pos < 0) continue;  // warp-uniform: block (mb0 + warp, column l) is not kept
        const int col = clist[c_first + l];
        uint32_t r[32];
        tmem_ld_x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + l * kBlk, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float v0 = __uint_as_float(r[2 * j]), v1 = __uint_as_float(r[2 * j + 1]);
          if (bias) {
            v0 += to_float(__ldg(bias + col * kBlk + 2 * j));
            v1 += to_float(__ldg(bias + col * kBlk + 2 * j + 1));
          }
          if constexpr (FMT == 0) {
            const __half2 h = __floats2half2_rn(v0, v1);
            packed[j] = *reinterpret_cast<const uint32_t*>(&h);
          } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            packed[j] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        T* dst_row;
        if (p.compressed)
          dst_row = C + ((long long)batch * p.val_stride_blocks + pos) * (kBlk * kBlk) + lane * kBlk;
        else
          dst_row = C + ((long long)batch * p.M + (mb0 + warp) * kBlk + lane) * p.N + col * kBlk;
        uint4* dst = reinterpret_cast<uint4*>(dst_row);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
    }
  }
  if constexpr (!LOOP) break;  // launched with one CTA per group
  tc_fence_before_sync();
  if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }  // a wait gave up somewhere: stop here
  tc_fence_after_sync();
  }  // groups
  tc_fence_before_sync();
  sync_and_drain(failed);
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc<256>(tmem_base);
  }
}

template <int FMT, int STAGES, bool TA>
int launch_dds(const BsmmParams& p, cudaStream_t st) {
  CUtensorMap tm_a, tm_b;
  if (TA) {
    const uint64_t dims[2] = {(uint64_t)p.M, (uint64_t)p.batch * p.K};
    const uint64_t strides[1] = {(uint64_t)p.M * 2};
    const uint32_t box[2] = {kBlk, kChunkK};
    int rc = make_tensor_map(&tm_a, p.A, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != SPARTA_OK) return rc;
  } else {
    const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.batch * p.M};
    const uint64_t strides[1] = {(uint64_t)p.K * 2};
    const uint32_t box[2] = {kChunkK, kTileM};
    int rc = make_tensor_map(&tm_a, p.A, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  if (p.trans_b) {
    const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.batch * p.N};
    const uint64_t strides[1] = {(uint64_t)p.K * 2};
    const uint32_t box[2] = {kChunkK, kBlk};
    int rc = make_tensor_map(&tm_b, p.B, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  } else {
    const uint64_t dims[2] = {(uint64_t)p.N, (uint64_t)p.batch * p.K};
    const uint64_t strides[1] = {(uint64_t)p.N * 2};
    const uint32_t box[2] = {kBlk, kChunkK};
    int rc = make_tensor_map(&tm_b, p.B, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != SPARTA_OK) return rc;
  }
  DdsTcParams q;
  q.row_ptr = p.ptr;
  q.idx = static_cast<const int32_t*>(p.idx);
  q.bias = p.bias;
  q.C = p.C;
  q.M = p.M; q.N = p.N; q.K = p.K; q.Nb = p.N / kBlk;
  q.compressed = p.compressed; q.trans_b = p.trans_b;
  q.n_index_sets = p.n_index_sets;
  q.ptr_stride = p.ptr_stride; q.idx_stride = p.idx_stride; q.val_stride_blocks = p.val_stride_blocks;
  q.status = device_status_ptr();
  if (!q.status) return SPARTA_ERR_DRIVER;
  constexpr int kSmem = smem_bytes(STAGES);
  static SmemAttrOnce attr_one, attr_loop;
  if (cudaError_t e = attr_one.ensure(bsmm_dds_tc_kernel<FMT, STAGES, false, TA>, kSmem); e != cudaSuccess)
    return static_cast<int>(e);
  if (cudaError_t e = attr_loop.ensure(bsmm_dds_tc_kernel<FMT, STAGES, true, TA>, kSmem); e != cudaSuccess)
    return static_cast<int>(e);
  // CTAs per row tile: every group its own CTA when there are few row tiles; with many (batched masks)
  // most groups of a tile are empty, and a few CTAs per tile loop over the groups instead, aiming at
  // about two CTAs per resident slot
  constexpr long long kCtasPerSlot = 2;
  const int n_groups = (q.Nb + kGroup - 1) / kGroup;
  const long long tiles = (long long)(p.M / kTileM) * p.batch;
  long long per_tile = (kCtasPerSlot * 2 * kNumSMs + tiles - 1) / tiles;
  if (per_tile < 1) per_tile = 1;
  if (per_tile >= n_groups) {
    dim3 grid(n_groups, p.M / kTileM, p.batch);
    bsmm_dds_tc_kernel<FMT, STAGES, false, TA><<<grid, kThreads, kSmem, st>>>(tm_a, tm_b, q);
  } else {
    dim3 grid((unsigned)per_tile, p.M / kTileM, p.batch);
    bsmm_dds_tc_kernel<FMT, STAGES, true, TA><<<grid, kThreads, kSmem, st>>>(tm_a, tm_b, q);
  }
  return launch_status();
}

}  // namespace

bool dds_tc_supported(const BsmmParams& p) {
  if (p.mode != MODE_DDS || p.idx_is_64 || !p.ptr) return false;
  if (p.dtype != SPARTA_F16 && p.dtype != SPARTA_BF16) return false;
  if (p.BM != kBlk || p.BN != kBlk || p.BK != kChunkK) return false;
  if (p.M % kTileM || p.N % kBlk || p.K % kChunkK || p.N / kBlk > kMaxNb) return false;
  if (p.n_index_sets != 1 && p.n_index_sets != p.batch) return false;
  if ((long long)p.batch * p.M > 0x7fffffffll || (long long)p.batch * p.N > 0x7fffffffll ||
      (long long)p.batch * p.K > 0x7fffffffll || p.batch > 65535 || p.M / kTileM > 65535)
    return false;
  if (!aligned(p.A, 16) || !aligned(p.B, 16) || !aligned(p.C, 16) || (p.K * 2) % 16 || (p.N * 2) % 16 || (p.M * 2) % 16) return false;
  return true;
}

int dds_tc_launch(const BsmmParams& p, cudaStream_t st) {
  const bool h = p.dtype == SPARTA_F16;
  if (p.K <= 2 * kChunkK) {
    if (p.trans_a) return h ? launch_dds<0, 2, true>(p, st) : launch_dds<1, 2, true>(p, st);
    return h ? launch_dds<0, 2, false>(p, st) : launch_dds<1, 2, false>(p, st);
  }
  if (p.trans_a) return h ? launch_dds<0, 4, true>(p, st) : launch_dds<1, 4, true>(p, st);
  return h ? launch_dds<0, 4, false>(p, st) : launch_dds<1, 4, false>(p, st);
}

}  // namespace sparta
