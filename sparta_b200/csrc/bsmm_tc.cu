// Block-sparse matmul on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), fp16 / bf16.
//
// dsd, B stored [N, K] as BCSR 32 x 32 blocks (the SparseLinear weight layout):
//   C[m, n] = sum over kept K-blocks k of row-block n:  X[m, k-block] . W_block(n, k)^T   (+ bias)
//
// One CTA owns 128 token rows x a panel of NP block columns (NP * 32 output features), i.e. NP fp32
// accumulators of 128 x 32 in tensor memory.  It walks the K-blocks that ANY row-block of the panel
// keeps, in ascending order (an NP-way merge of the sorted BCSR rows done by the producer warp), so
// each 128 x 32 tile of X is staged once per panel and shared by every W block of that K-block.
//   warp 4    producer: merge + TMA loads (X tile by coordinate, W blocks gathered by BCSR position)
//   warp 5    one thread issues tcgen05.mma (M128 N32 K16, two per W block) and commits
//   warps 0-3 epilogue: tcgen05.ld -> + bias -> fp16 / bf16 -> global
// Every mbarrier wait is bounded; a wait that runs out sets a status word and the CTA winds down.
//
// Replaces sparta_sparse_matmul_dsd.cuh.j2 / openai_sparse_matmul_dsd.cuh.j2 for this layout.
#include <cstdlib>

#include "bsmm.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

using namespace tc;

constexpr int kBlk = 32;            // BCSR block edge (K and N)
constexpr int kTileM = 128;         // token rows per CTA
constexpr int kStages = 4;
constexpr int kXBytes = kTileM * kBlk * 2;   // 8 KB: 128 rows x 64 B
constexpr int kWBytes = kBlk * kBlk * 2;     // 2 KB
constexpr int kMaxRowBlocks = 512;  // K-blocks per W row-block held in shared memory
constexpr int kThreads = 192;

struct DsdTcParams {
  const int32_t* row_ptr;
  const int32_t* idx;
  const void* bias;
  void* C;
  int M, N, Kb, Nb;
  long long val_stride_blocks;
  int32_t* status;
};

template <int NP>
struct SmemLayout {
  static constexpr int kStageBytes = kXBytes + NP * kWBytes;
  static constexpr int kIdxBytes = NP * kMaxRowBlocks * 2;
  static constexpr int kTotal = kStages * kStageBytes + kIdxBytes + 1024 /* barriers etc. */ + 1024 /* align */;
};

template <int NP, int FMT>
__global__ void __launch_bounds__(kThreads, 1)
bsmm_dsd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   DsdTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = SmemLayout<NP>;
  uint8_t* stage_base = smem;
  uint16_t* s_idx = reinterpret_cast<uint16_t*>(smem + kStages * L::kStageBytes);
  uint8_t* ctl = smem + kStages * L::kStageBytes + L::kIdxBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctl);            // [kStages]
  uint64_t* empty_bar = full_bar + kStages;                         // [kStages]
  uint64_t* accum_bar = empty_bar + kStages;                        // [1]
  uint32_t* stage_mask = reinterpret_cast<uint32_t*>(accum_bar + 1);  // [kStages]
  uint32_t* tmem_holder = stage_mask + kStages;
  uint32_t* s_written = tmem_holder + 1;
  int* s_row_len = reinterpret_cast<int*>(s_written + 1);           // [NP]
  int* s_row_start = s_row_len + NP;                                // [NP]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int panel = blockIdx.x, m0 = blockIdx.y * kTileM, batch = blockIdx.z;
  constexpr uint32_t kTmemCols = NP * kBlk;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 2);
    fence_mbar_init();
    *s_written = 0;
  }
  if (warp == 4 && lane == 0) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
  }
  if (warp == 5) tmem_alloc<kTmemCols>(tmem_holder);
  // stage the BCSR rows of this panel (column numbers only) in shared memory
  if (threadIdx.x < NP) {
    const int nb = panel * NP + threadIdx.x;
    int start = 0, len = 0;
    if (nb < p.Nb) {
      start = p.row_ptr[nb];
      len = p.row_ptr[nb + 1] - start;
    }
    s_row_start[threadIdx.x] = start;
    s_row_len[threadIdx.x] = len;
  }
  __syncthreads();
  for (int l = 0; l < NP; ++l) {
    const int start = s_row_start[l], len = s_row_len[l];
    for (int j = threadIdx.x; j < len; j += kThreads)
      s_idx[l * kMaxRowBlocks + j] = static_cast<uint16_t>(p.idx[start + j] & 0xffff);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 4) {
    // ------------------------------ producer ------------------------------
    int cur = 0;
    const int len = lane < NP ? s_row_len[lane] : 0;
    const int vbase = lane < NP ? s_row_start[lane] : 0;
    const uint16_t* my = s_idx + (lane < NP ? lane : 0) * kMaxRowBlocks;
    int kcur = cur < len ? my[cur] : 0x7fffffff;
    int stage = 0;
    uint32_t phase = 0;
    while (true) {
      int kmin = kcur;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
      const bool last = (kmin == 0x7fffffff);
      const uint32_t active = __ballot_sync(0xffffffffu, !last && kcur == kmin);
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&empty_bar[stage], phase ^ 1) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        if (lane == 0) atomicExch(&p.status[0], 1);
        break;
      }
      uint8_t* st = stage_base + stage * L::kStageBytes;
      if (last) {
        if (lane == 0) {
          stage_mask[stage] = 0x80000000u;
          mbar_arrive(&full_bar[stage]);
        }
        break;
      }
      if (lane == 0) {
        stage_mask[stage] = active;
        mbar_arrive_expect_tx(&full_bar[stage], kXBytes + __popc(active) * kWBytes);
        tma_load_2d(st, &tm_x, kmin * kBlk, batch * p.M + m0, &full_bar[stage]);
      }
      __syncwarp();
      if ((active >> lane) & 1u) {
        const long long blk = (long long)batch * p.val_stride_blocks + vbase + cur;
        tma_load_2d(st + kXBytes + lane * kWBytes, &tm_w, 0, (int)(blk * kBlk), &full_bar[stage]);
        ++cur;
        kcur = cur < len ? my[cur] : 0x7fffffff;
      }
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issue ------------------------------
    constexpr uint32_t idesc = make_idesc_f16(kTileM, kBlk, FMT, 0, 0);
    uint32_t written = 0;
    int stage = 0;
    uint32_t phase = 0;
    while (true) {
      if (!mbar_wait(&full_bar[stage], phase)) {
        if (lane == 0) atomicExch(&p.status[1], 1);
        break;
      }
      const uint32_t mask = stage_mask[stage];
      if (mask & 0x80000000u) break;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(stage_base + stage * L::kStageBytes);
        uint32_t m = mask;
        while (m) {
          const int l = __ffs(m) - 1;
          m &= m - 1;
          const uint32_t b_addr = a_addr + kXBytes + l * kWBytes;
          const uint32_t acc = (written >> l) & 1u;
#pragma unroll
          for (int kk = 0; kk < kBlk / 16; ++kk) {
            const uint64_t a_desc = make_smem_desc(a_addr + kk * 32, 16, 512, SW_64B);
            const uint64_t b_desc = make_smem_desc(b_addr + kk * 32, 16, 512, SW_64B);
            umma_ss(tmem_base + l * kBlk, a_desc, b_desc, idesc, acc | (kk > 0 ? 1u : 0u));
          }
        }
        umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
      }
      __syncwarp();
      written |= mask;
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
    if (lane == 0) {
      *s_written = written;
      umma_commit(accum_bar);
      mbar_arrive(accum_bar);
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    using T = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
    if (!mbar_wait(accum_bar, 0)) {
      if (lane == 0) atomicExch(&p.status[2], 1);
    } else {
      tc_fence_after_sync();
      const uint32_t written = *s_written;
      const int row = m0 + warp * 32 + lane;
      T* crow = static_cast<T*>(p.C) + ((long long)batch * p.M + row) * p.N;
      const T* bias = p.bias ? static_cast<const T*>(p.bias) + (long long)batch * p.N : nullptr;
      for (int l = 0; l < NP; ++l) {
        const int nb = panel * NP + l;
        if (nb >= p.Nb) break;
        uint32_t r[32];
        if ((written >> l) & 1u) {
          tmem_ld_x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + l * kBlk, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float v0 = __uint_as_float(r[2 * j]), v1 = __uint_as_float(r[2 * j + 1]);
          if (bias) {
            v0 += to_float(__ldg(bias + nb * kBlk + 2 * j));
            v1 += to_float(__ldg(bias + nb * kBlk + 2 * j + 1));
          }
          if constexpr (FMT == 0) {
            __half2 h = __floats2half2_rn(v0, v1);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        uint4* dst = reinterpret_cast<uint4*>(crow + nb * kBlk);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

template <int NP, int FMT>
int launch_dsd(const BsmmParams& p, cudaStream_t st) {
  using L = SmemLayout<NP>;
  CUtensorMap tm_x, tm_w;
  {
    const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.batch * p.M};
    const uint64_t strides[1] = {(uint64_t)p.K * 2};
    const uint32_t box[2] = {kBlk, kTileM};
    int rc = make_tensor_map(&tm_x, p.A, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != SPARTA_OK) return rc;
  }
  {
    const uint64_t dims[2] = {kBlk, (uint64_t)p.batch * p.val_stride_blocks * kBlk};
    const uint64_t strides[1] = {kBlk * 2};
    const uint32_t box[2] = {kBlk, kBlk};
    int rc = make_tensor_map(&tm_w, p.B, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != SPARTA_OK) return rc;
  }
  DsdTcParams q;
  q.row_ptr = p.ptr;
  q.idx = static_cast<const int32_t*>(p.idx);
  q.bias = p.bias;
  q.C = p.C;
  q.M = p.M; q.N = p.N; q.Kb = p.K / kBlk; q.Nb = p.N / kBlk;
  q.val_stride_blocks = p.val_stride_blocks;
  q.status = device_status_ptr();
  if (!q.status) return SPARTA_ERR_DRIVER;
  auto kern = bsmm_dsd_tc_kernel<NP, FMT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  dim3 grid((q.Nb + NP - 1) / NP, p.M / kTileM, p.batch);
  kern<<<grid, kThreads, L::kTotal, st>>>(tm_x, tm_w, q);
  return launch_status();
}

int panel_width() {
  static int np = [] {
    const char* e = std::getenv("SPARTA_TC_PANEL");
    const int v = e ? std::atoi(e) : 16;
    return v == 8 ? 8 : 16;
  }();
  return np;
}

}  // namespace

bool bsmm_tc_available() { return true; }

bool bsmm_tc_supported(const BsmmParams& p) {
  if (p.mode != MODE_DSD || !p.trans_b || p.trans_a || !p.compressed || p.idx_is_64) return false;
  if (p.dtype != SPARTA_F16 && p.dtype != SPARTA_BF16) return false;
  if (p.BM != kTileM || p.BK != kBlk || p.BN != kBlk) return false;
  if (p.M % kTileM || p.K % kBlk || p.N % kBlk) return false;
  if (p.K / kBlk > kMaxRowBlocks || p.n_index_sets != 1 || p.val_stride_blocks <= 0) return false;
  if ((long long)p.batch * p.val_stride_blocks * kBlk > 0x7fffffffll) return false;
  if ((long long)p.batch * p.M > 0x7fffffffll || p.batch > 65535 || p.M / kTileM > 65535) return false;
  if (!aligned(p.A, 16) || !aligned(p.B, 16) || !aligned(p.C, 16)) return false;
  return true;
}

int bsmm_tc(const BsmmParams& p, cudaStream_t st) {
  const int fmt = p.dtype == SPARTA_F16 ? 0 : 1;
  if (panel_width() == 8) return fmt == 0 ? launch_dsd<8, 0>(p, st) : launch_dsd<8, 1>(p, st);
  return fmt == 0 ? launch_dsd<16, 0>(p, st) : launch_dsd<16, 1>(p, st);
}

}  // namespace sparta
