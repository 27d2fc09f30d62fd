// Block-sparse matmul on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), fp16 / bf16.
//
// dsd, B stored [N, K] as BCSR 32 x 32 blocks (the SparseLinear weight layout):
//   C[m, n] = sum over kept K-blocks k of row-block n:  X[m, k-block] . W_block(n, k)^T   (+ bias)
//
// Why the activations go through tensor memory.  With both operands in shared memory a
// tcgen05.mma M128 N32 K16 reads 4 KB of A and 1 KB of B; at 128 B per cycle that is 40 cycles for
// 16 cycles of math, so 32-wide blocks cannot pass 40 % of the tensor peak however they are issued.
// With A in tensor memory only the 1 KB of B crosses the shared-memory port and the same instruction
// runs at its 16-cycle rate (measured: four issuing threads, 16.2 cycles per MMA).  The activations of
// a K-block are shared by every W block of that K-block in the CTA's panel, so they are moved into
// tensor memory once per K-block and reused from there.
//
// One CTA owns 128 token rows x a panel of NP block columns, i.e. NP fp32 accumulators of 128 x 32
// in tensor memory, plus a ring of kSteps activation tiles (128 lanes x 16 columns each) beside them.
// Its prologue turns the BCSR rows of the panel into a schedule in shared memory: kmask[k] = which
// row-blocks of the panel keep K-block k.  All roles walk k = 0 .. K/32 over that schedule
// independently (no per-step messages):
//   warp 4       producer: TMA loads (X tile by coordinate, W blocks gathered by BCSR position) into
//                two rings; every load of a step completes on the step's "full" mbarrier
//   warps 0-3,   converters: shared memory -> registers -> tcgen05.st into the step's slot of the
//   9-12         activation ring (each warp its own 32-lane quadrant; the two sets alternate steps),
//                then arrive on the step's "a_full" mbarrier
//   warps 5-8    MMA issue: each warp owns the accumulators l with l % 4 == its index and one of its
//                threads issues tcgen05.mma with A from tensor memory (two K = 16 slabs per W block);
//                tcgen05.commit arrives on the step's "empty" mbarrier, which frees the X tile, the W
//                blocks and the activation slot once all four have arrived.  One thread sustains about
//                one MMA per 45 cycles, hence four issuers.
//   warps 0-3, 9-12 afterwards: epilogue, tcgen05.ld -> + bias -> fp16 / bf16 -> global
// Every mbarrier wait is bounded; a wait that runs out sets a status word and the CTA winds down.
//
// Replaces sparta_sparse_matmul_dsd.cuh.j2 / openai_sparse_matmul_dsd.cuh.j2 for this layout.
#include <cstdlib>
#include <type_traits>

#include "bsmm.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

using namespace tc;

constexpr int kBlk = 32;            // BCSR block edge (K and N)
constexpr int kTileM = 128;         // token rows per CTA
constexpr int kXBytes = kTileM * kBlk * 2;   // 8 KB: 128 rows x 64 B
constexpr int kWBytes = kBlk * kBlk * 2;     // 2 KB
constexpr int kACols = kBlk / 2;    // tensor-memory columns of one activation tile (two 16-bit values per column)
constexpr int kMaxKb = 1024;        // K-blocks the schedule can hold (K <= 32768)
constexpr int kMmaWarps = 4;        // MMA-issuing warps
constexpr int kConvSets = 2;        // converter warp sets (four warps each) that alternate steps
constexpr int kProdWarps = 4;       // TMA-issuing warps: one thread sustains only about one bulk tensor load per 200 cycles
constexpr int kProd0 = 4;           // first producer warp
constexpr int kMma0 = kProd0 + kProdWarps;  // first MMA-issuing warp
constexpr int kThreads = 32 * (4 + kProdWarps + kMmaWarps + 4 * (kConvSets - 1));  // 512

struct DsdTsParams {
  const int32_t* row_ptr;
  const int32_t* idx;
  const void* bias;
  void* C;
  int M, N, Kb, Nb;
  long long val_stride_blocks;
  int32_t* status;
  int dbg;
};

// NP = 12: 384 accumulator columns + 8 activation slots (128 columns) = all 512 columns, one CTA per SM.
// NP = 6:  192 + 4 slots (64) = 256 columns, two CTAs per SM.
template <int NP>
struct TsLayout {
  static constexpr int kSteps = NP > 6 ? 8 : 4;         // steps (X tiles, activation slots) in flight
  static constexpr int kWSlots = NP > 6 ? 40 : 20;      // W blocks in flight
  static constexpr uint32_t kAccCols = NP * kBlk;
  static constexpr uint32_t kTmemCols = NP > 6 ? 512 : 256;
  static constexpr int kXRing = kSteps * kXBytes;
  static constexpr int kWRing = kWSlots * kWBytes;
  static constexpr int kMaskBytes = kMaxKb * 4;
  static constexpr int kBiasBytes = NP * kBlk * 4;
  static constexpr int kCtlBytes = 512;
  static constexpr int kTotal = kXRing + kWRing + kMaskBytes + kBiasBytes + kCtlBytes + 1024 /* align */;
  static_assert(kAccCols + kSteps * kACols <= kTmemCols, "tensor memory budget");
};

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

}  // namespace
__device__ long long g_trace[1024];
namespace {
#define TRACE(role, i) do { if (blockIdx.x == 3 && blockIdx.y == 5 && lane == 0 && (i) < 128) g_trace[(role) * 128 + (i)] = clock64(); } while (0)

template <int NP, int FMT>
__global__ void __launch_bounds__(kThreads, NP > 6 ? 1 : 2)
bsmm_dsd_ts_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   DsdTsParams p) {
  using T = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
  using L = TsLayout<NP>;
  constexpr int kSteps = L::kSteps, kWSlots = L::kWSlots;
  constexpr int kIssuers = kMmaWarps;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x_ring = smem;
  uint8_t* w_ring = smem + L::kXRing;
  uint32_t* kmask = reinterpret_cast<uint32_t*>(smem + L::kXRing + L::kWRing);
  float* s_bias = reinterpret_cast<float*>(smem + L::kXRing + L::kWRing + L::kMaskBytes);
  uint8_t* ctl = smem + L::kXRing + L::kWRing + L::kMaskBytes + L::kBiasBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctl);   // [kSteps] loads of a step have landed
  uint64_t* afull_bar = full_bar + kSteps;                 // [kSteps] the step's activations are in tensor memory
  uint64_t* empty_bar = afull_bar + kSteps;                // [kSteps] MMAs of a step have read their operands
  uint64_t* accum_bar = empty_bar + kSteps;                // [1]      all MMAs of the tile are done
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_bar + 1);
  int* s_range = reinterpret_cast<int*>(tmem_holder + 1);  // [2] BCSR entries of the panel
  int* s_row_start = s_range + 2;                          // [NP]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int panel = blockIdx.x, m0 = blockIdx.y * kTileM, batch = blockIdx.z;
  const int nb0 = panel * NP;
  const int nb_end = min(nb0 + NP, p.Nb);
  const bool is_conv = warp < 4 || warp >= kMma0 + kIssuers;
  const int conv_set = warp < 4 ? 0 : 1;
  const int quad = warp & 3;  // tensor-memory lane quadrant this warp may access

  // ------------------------------ prologue ------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSteps; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&afull_bar[s], 4);
      mbar_init(&empty_bar[s], kIssuers);
    }
    mbar_init(accum_bar, kIssuers);
    fence_mbar_init();
    s_range[0] = p.row_ptr[nb0];
    s_range[1] = p.row_ptr[nb_end];
  }
  if (warp == kProd0 && lane == 0) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
  }
  if (warp == kMma0) tmem_alloc<L::kTmemCols>(tmem_holder);
  if (threadIdx.x >= 64 && threadIdx.x < 64 + NP) {
    const int l = threadIdx.x - 64;
    s_row_start[l] = nb0 + l < p.Nb ? p.row_ptr[nb0 + l] : 0;
  }
  for (int k = threadIdx.x; k < p.Kb; k += kThreads) kmask[k] = 0;
  {
    const T* bias = p.bias ? static_cast<const T*>(p.bias) + (long long)batch * p.N : nullptr;
    for (int j = threadIdx.x; j < NP * kBlk; j += kThreads) {
      const int n = nb0 * kBlk + j;
      s_bias[j] = (bias && n < p.N) ? to_float(bias[n]) : 0.f;
    }
  }
  __syncthreads();
  // the rows of a panel are consecutive in the BCSR array: entry = (row-block << 16) | K-block
  for (int e = s_range[0] + threadIdx.x; e < s_range[1]; e += kThreads) {
    const int v = __ldg(p.idx + e);
    atomicOr(&kmask[v & 0xffff], 1u << ((v >> 16) - nb0));
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) TRACE(5, 0);
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t a_tmem = tmem_base + L::kAccCols;  // activation ring
  uint32_t written = 0;  // which accumulators receive any product

  if (warp >= kProd0 && warp < kMma0) {
    // ------------------------------ producers ------------------------------
    // Every producer warp runs the same bookkeeping over all steps and issues the loads of every
    // kProdWarps-th step.  Within a warp all lanes keep the ring state; lane l also owns the cursor
    // into BCSR row nb0 + l.
    const int prod = warp - kProd0;
    long long wrow = 0;  // row of this lane's next W block in the [blocks * 32, 32] view of the values
    if (lane < NP) wrow = ((long long)batch * p.val_stride_blocks + s_row_start[lane]) * kBlk;
    int slot = 0, tail = 0, inflight = 0, w_used = 0, w_head = 0;
    uint32_t tail_phase = 0;
    uint64_t cnts = 0;  // W blocks held by each in-flight step, 5 bits per ring slot
    bool ok = true;
    int tstep = 0;
    uint32_t m_next = p.Kb > 0 ? kmask[0] : 0;
    for (int k = 0; k < p.Kb; ++k) {
      const uint32_t m = m_next;
      m_next = (k + 1 < p.Kb) ? kmask[k + 1] : 0;
      if (!m) continue;
      const int need = __popc(m);
      if (prod == 0) TRACE(6, tstep);
      while (inflight == kSteps || w_used + need > kWSlots) {  // free the oldest step
        if (!mbar_wait(&empty_bar[tail], tail_phase)) { ok = false; break; }
        w_used -= (int)((cnts >> (5 * tail)) & 31u);
        --inflight;
        if (++tail == kSteps) { tail = 0; tail_phase ^= 1; }
      }
      if (!ok) break;
      if (prod == 0) TRACE(7, tstep);
      const bool mine = (tstep % kProdWarps) == prod;
      if (mine && lane == 0) {
        mbar_arrive_expect_tx(&full_bar[slot], kXBytes + need * kWBytes);
        tma_load_2d(x_ring + slot * kXBytes, &tm_x, k * kBlk, batch * p.M + m0, &full_bar[slot]);
      }
      __syncwarp();  // the expected byte count is registered before any lane's load can complete
      if ((m >> lane) & 1u) {
        int ws = w_head + __popc(m & ((1u << lane) - 1u));  // rank among the kept row-blocks
        if (ws >= kWSlots) ws -= kWSlots;
        if (mine) tma_load_2d(w_ring + ws * kWBytes, &tm_w, 0, (int)wrow, &full_bar[slot]);
        wrow += kBlk;
      }
      cnts = (cnts & ~(31ull << (5 * slot))) | ((uint64_t)need << (5 * slot));
      w_head += need;
      if (w_head >= kWSlots) w_head -= kWSlots;
      w_used += need;
      ++inflight;
      if (prod == 0) TRACE(0, tstep);
      ++tstep;
      if (++slot == kSteps) slot = 0;
    }
    if (!ok && lane == 0) atomicExch(&p.status[0], 1);
  } else if (warp >= kMma0 && warp < kMma0 + kIssuers) {
    // ------------------------------ MMA issue ------------------------------
    // Operand addresses derive from loop counters only, so they stay warp-uniform; one lane issues.
    constexpr uint32_t idesc = make_idesc_f16(kTileM, kBlk, FMT, 0, 0);
    const uint32_t w_base = smem_u32(w_ring);
    const uint64_t desc_hi = make_smem_desc(0, 16, 512, SW_64B);
    const bool leader = lane == 0;
    uint32_t mine = 0;  // accumulators issued by this warp
    for (int l = warp - kMma0; l < NP; l += kIssuers) mine |= 1u << l;
    int slot = 0, tstep = 0;
    uint32_t phase = 0, ws = 0;  // ws: next W slot, advances exactly like the producer's ring head
    bool ok = true;
    uint32_t m_next = p.Kb > 0 ? kmask[0] : 0;
    for (int k = 0; k < p.Kb; ++k) {
      const uint32_t mask = m_next;
      m_next = (k + 1 < p.Kb) ? kmask[k + 1] : 0;
      if (!mask) continue;
      // every issuer waits for the step's loads, also one without a block in it: that keeps it within
      // one ring turn of the others, so its commits never land in an earlier phase of empty_bar
      uint32_t m = mask & mine;
      if (!mbar_wait(&full_bar[slot], phase) || (m && !mbar_wait(&afull_bar[slot], phase))) { ok = false; break; }
      tc_fence_after_sync();
      if (warp == kMma0) TRACE(1, tstep);
      const uint32_t a_addr = a_tmem + slot * kACols;
      while (m) {
        const int l = __ffs(m) - 1;
        m &= m - 1;
        uint32_t w = ws + __popc(mask & ((1u << l) - 1u));  // rank of block l among the step's blocks
        if (w >= kWSlots) w -= kWSlots;
        const uint32_t b_lo = (w_base + w * kWBytes) >> 4;
        const uint32_t acc = (written >> l) & 1u;
        if (leader && !(p.dbg & 2)) {
          umma_ts(tmem_base + l * kBlk, a_addr, desc_hi | b_lo, idesc, acc);
          umma_ts(tmem_base + l * kBlk, a_addr + kACols / 2, desc_hi | (b_lo + 2), idesc, 1u);
        }
      }
      ws += __popc(mask);
      if (ws >= kWSlots) ws -= kWSlots;
      if (leader) umma_commit(&empty_bar[slot]);  // frees the step's X tile, W blocks and activation slot
      if (warp == kMma0) TRACE(2, tstep);
      ++tstep;
      written |= mask;
      if (++slot == kSteps) { slot = 0; phase ^= 1; }
    }
    if (!ok && lane == 0) atomicExch(&p.status[1], 1);
    if (leader) umma_commit(accum_bar);
  } else if (is_conv) {
    // ------------------------------ converters ------------------------------
    // The X tile was written by TMA with the 64-byte swizzle: the 16-byte chunk c of row r sits at
    // chunk position c ^ ((r >> 1) & 3), which also makes the row-per-thread reads conflict-free.
    const int row = quad * 32 + lane;
    const uint32_t sw = (row >> 1) & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    int slot = 0, step = 0;
    uint32_t phase = 0;
    bool ok = true;
    uint32_t m_next = p.Kb > 0 ? kmask[0] : 0;
    for (int k = 0; k < p.Kb; ++k) {
      const uint32_t mask = m_next;
      m_next = (k + 1 < p.Kb) ? kmask[k + 1] : 0;
      if (!mask) continue;
      written |= mask;
      if ((step & (kConvSets - 1)) == conv_set) {
        if (!mbar_wait(&full_bar[slot], phase)) { ok = false; break; }
        if (quad == 0) TRACE(3, step);
        const uint8_t* xrow = x_ring + slot * kXBytes + row * 64;
        uint32_t r[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 v = (p.dbg & 4) ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(xrow + ((c ^ sw) << 4));
          r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
        }
        if (!(p.dbg & 1)) {
        tmem_st_x16(a_tmem + slot * kACols + lane_addr, r);
        tmem_st_wait();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&afull_bar[slot]);
        if (quad == 0) TRACE(4, step);
      }
      ++step;
      if (++slot == kSteps) { slot = 0; phase ^= 1; }
    }
    if (!ok && lane == 0) atomicExch(&p.status[3], 1);

    // ------------------------------ epilogue ------------------------------
    // the two warps of a lane quadrant take alternate accumulators
    if (!mbar_wait(accum_bar, 0)) {
      if (lane == 0) atomicExch(&p.status[2], 1);
    } else {
      tc_fence_after_sync();
      T* crow = static_cast<T*>(p.C) + ((long long)batch * p.M + m0 + row) * p.N;
      for (int l = conv_set; l < nb_end - nb0; l += kConvSets) {
        uint32_t r[32];
        if ((written >> l) & 1u) {
          tmem_ld_x32(tmem_base + lane_addr + l * kBlk, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 bv = *reinterpret_cast<const float2*>(&s_bias[l * kBlk + 2 * j]);
          const float v0 = __uint_as_float(r[2 * j]) + bv.x, v1 = __uint_as_float(r[2 * j + 1]) + bv.y;
          if constexpr (FMT == 0) {
            __half2 h = __floats2half2_rn(v0, v1);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            packed[j] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        uint4* dst = reinterpret_cast<uint4*>(crow + (nb0 + l) * kBlk);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
      }
    }
  }
  if (warp == 0) TRACE(5, 1);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMma0) {
    tc_fence_after_sync();
    tmem_dealloc<L::kTmemCols>(tmem_base);
  }
}

template <int NP, int FMT>
int launch_dsd_ts(const BsmmParams& p, cudaStream_t st) {
  using L = TsLayout<NP>;
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
  DsdTsParams q;
  q.row_ptr = p.ptr;
  q.idx = static_cast<const int32_t*>(p.idx);
  q.bias = p.bias;
  q.C = p.C;
  q.M = p.M; q.N = p.N; q.Kb = p.K / kBlk; q.Nb = p.N / kBlk;
  q.val_stride_blocks = p.val_stride_blocks;
  q.status = device_status_ptr();
  { const char* e = getenv("SPARTA_DBG"); q.dbg = e ? atoi(e) : 0; }
  if (!q.status) return SPARTA_ERR_DRIVER;
  auto kern = bsmm_dsd_ts_kernel<NP, FMT>;
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

}  // namespace

}  // namespace sparta
extern "C" int sparta_debug_trace(long long* out) { return (int)cudaMemcpyFromSymbol(out, sparta::g_trace, sizeof(long long) * 1024); }
namespace sparta {
bool dsd_ts_supported(const BsmmParams& p) {
  if (p.mode != MODE_DSD || !p.trans_b || p.trans_a || !p.compressed || p.idx_is_64) return false;
  if (p.dtype != SPARTA_F16 && p.dtype != SPARTA_BF16) return false;
  if (p.BM != kTileM || p.BK != kBlk || p.BN != kBlk) return false;
  if (p.M % kTileM || p.K % kBlk || p.N % kBlk) return false;
  if (p.K / kBlk > kMaxKb || p.n_index_sets != 1 || p.val_stride_blocks <= 0) return false;
  if ((long long)p.batch * p.val_stride_blocks * kBlk > 0x7fffffffll) return false;
  if ((long long)p.batch * p.M > 0x7fffffffll || p.batch > 65535 || p.M / kTileM > 65535) return false;
  if (!aligned(p.A, 16) || !aligned(p.B, 16) || !aligned(p.C, 16)) return false;
  return true;
}

int dsd_ts_launch(const BsmmParams& p, cudaStream_t st) {
  const int fmt = p.dtype == SPARTA_F16 ? 0 : 1;
  const char* e = getenv("SPARTA_DSD_NP");
  const int np = (e && e[0] == '6') ? 6 : 12;
  if (np == 6) return fmt == 0 ? launch_dsd_ts<6, 0>(p, st) : launch_dsd_ts<6, 1>(p, st);
  return fmt == 0 ? launch_dsd_ts<12, 0>(p, st) : launch_dsd_ts<12, 1>(p, st);
}

}  // namespace sparta
