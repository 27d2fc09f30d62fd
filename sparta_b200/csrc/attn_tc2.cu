// Fused block-sparse attention forward, two Q tiles per CTA (fp16 / bf16, head dim 64 or 128, 64 x 64 mask
// blocks, Nt a multiple of 256):  O = softmax_mask(Q K^T * scale) V  over the kept blocks only.
//
// Same mathematics and data path as attn_tc.cu (scores in tensor memory, online softmax in registers, P back
// to tensor memory, P.V with A from tensor memory); what differs is the schedule.  With one 128-row Q tile per
// CTA a step is the chain  QK^T -> softmax -> P.V  and the tensor pipe idles while the softmax warps work
// (measured: 27 % of the tensor peak, the step time being the softmax warps' instruction stream).  Here a CTA
// owns 256 query rows as two tiles with their own score / output accumulators and their own eight softmax
// warps, sharing the K / V tiles: while one tile's softmax runs, the other tile's MMAs are issued, sixteen
// softmax warps keep the schedulers busier than eight, and every K / V tile is loaded once for 256 rows.
//
// Tensor memory per tile: scores 128 columns, output D columns; the probabilities of a step overwrite the
// score columns their own thread has already consumed (thread with K block b of the pair: scores in columns
// 64 b .. 64 b + 63, probabilities as 16-bit pairs in columns 64 b .. 64 b + 31), so no third region is needed
// and no thread overwrites what another still has to read.  Q.K^T of the next step is issued by the same
// thread right after the P.V of this one, which orders the two in the tensor pipe; "scores complete" therefore
// also means that the previous P.V is done, and a rescale of the output accumulator never races with an MMA.
//
// Steps walk the merged, sorted list of the K blocks kept by any of the CTA's four block rows, two blocks at
// a time; a tile skips a step in which none of its two block rows keeps either block (its barriers count
// only the steps it takes part in).
//   warps 0-7   softmax + epilogue of tile 0 (two threads per row: one per K block of the pair)
//   warps 8-15  the same for tile 1
//   warp 16     TMA producer (Q tiles once, then K / V pairs through two-stage rings)
//   warp 17     issues all MMAs: Q.K^T (M128 N128, D/16 per tile and step) and P.V (M128 N=D, A from tensor
//               memory, V MN-major in shared memory); a tile's next Q.K^T goes out right behind its P.V
// All mbarrier waits are bounded (status words of sparta_last_status).
#include <cstring>
#include <type_traits>

#include "bsmm.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

using namespace tc;

constexpr int kBlk = 64;       // mask block edge
constexpr int kTileM = 128;    // Q rows per tile
constexpr int kTiles = 2;      // tiles per CTA
constexpr int kPair = 128;     // keys per step (two blocks)
constexpr int kSmWarps = 8;    // softmax warps per tile
constexpr int kWarpLoad = kTiles * kSmWarps, kWarpQK = kWarpLoad + 1;  // kWarpQK issues every MMA
constexpr int kThreads = 32 * (kWarpLoad + 4);  // one idle warp rounds the CTA up to whole warp groups
constexpr int kMaxKb = 1024;   // K blocks per row (Ns <= 65536)
constexpr float kRescaleThreshold = 8.f;
constexpr int kStages = 2;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#ifdef SPARTA_ATTN_TRACE
__device__ unsigned long long g_attn_trace[8][32];
#define TR_DECL unsigned long long* tr = (blockIdx.x % 1000 == 7 && blockIdx.x / 1000 < 8) ? g_attn_trace[blockIdx.x / 1000] : nullptr
#define TR_T0(name) const long long name = clock64()
#define TR_ADD(slot, name) do { if (tr && lane == 0) atomicAdd(&tr[slot], (unsigned long long)(clock64() - name)); } while (0)
#define TR_ADD_IF(cond, slot, name) do { if ((cond) && tr && lane == 0) atomicAdd(&tr[slot], (unsigned long long)(clock64() - name)); } while (0)
#define TR_SET(slot, value) do { if (tr && lane == 0) atomicAdd(&tr[slot], (unsigned long long)(value)); } while (0)
#else
#define TR_DECL
#define TR_T0(name)
#define TR_ADD(slot, name)
#define TR_ADD_IF(cond, slot, name)
#define TR_SET(slot, value)
#endif

struct Attn2Params {
  const int32_t* row_ptr;
  const int32_t* idx;
  const uint8_t* mask;  // [Nt, Ns] element mask or null
  void* O;
  float* lse;
  int Nt, Ns, heads;
  int grouped;          // launch order, see the kernel
  float scale_log2;     // scale * log2(e)
  int32_t* status;
  int n_copies;         // further destinations of O (the peers' gathered outputs), see GatherMaps
};

// Tensor maps of the further destinations of O, each laid out like O itself ([heads * Nt, D]): with the heads
// sharded over GPUs, a rank's output is also stored into its slice of every peer's gathered output, over
// NVLink, from the kernel that computes it.  The tile is staged in the (by then idle) shared memory of its
// Q tile in the 128-byte swizzle and leaves as bulk tensor stores, so that the link carries full lines.
struct GatherMaps {
  CUtensorMap m[SPARTA_ATTN_MAX_COPIES];
};

template <int D>
struct Cfg2 {
  static constexpr int kChunks = D / 64;             // 64-element (128-byte) chunks of the head dim
  static constexpr int kQBytes = kTileM * D * 2;     // one tile
  static constexpr int kKVBytes = kPair * D * 2;     // one stage: two blocks
  static constexpr uint32_t kTileCols = kPair + D;   // tensor-memory columns of a tile: scores, then output
  static constexpr uint32_t kTmemCols = 512;
  static_assert(kTiles * kTileCols <= kTmemCols, "tensor memory budget");
  static constexpr int kListBytes = kMaxKb * 2 + kMaxKb;  // ulist (uint16) + kmask (uint8)
  static constexpr int kSmem = kTiles * kQBytes + 2 * kStages * kKVBytes + kListBytes + 512 + 1024;
};

template <int D, int FMT>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_tc2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ GatherMaps gm, Attn2Params p) {
  using T = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
  using C = Cfg2<D>;
  constexpr int kChunks = C::kChunks;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                                  // [kTiles][128 x D]
  uint8_t* k_s = q_s + kTiles * C::kQBytes;             // [kStages][128 keys x D]
  uint8_t* v_s = k_s + kStages * C::kKVBytes;
  uint16_t* ulist = reinterpret_cast<uint16_t*>(v_s + kStages * C::kKVBytes);  // (K block << 4) | presence bits of the four block rows
  uint8_t* kmask = reinterpret_cast<uint8_t*>(ulist + kMaxKb);
  uint8_t* ctl = kmask + kMaxKb;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctl);
  uint64_t* k_full = q_full + 1;             // [kStages]
  uint64_t* k_empty = k_full + kStages;      // [kStages]
  uint64_t* v_full = k_empty + kStages;      // [kStages]
  uint64_t* v_empty = v_full + kStages;      // [kStages]
  uint64_t* s_full = v_empty + kStages;      // [kTiles] the tile's scores of a step are complete
  uint64_t* p_full = s_full + kTiles;        // [kTiles] its probabilities are in tensor memory
  uint64_t* pv_done = p_full + kTiles;       // [kTiles] its P.V of a step is complete
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + kTiles);
  int* s_count = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_range = s_count + 1;                // [2]

  __shared__ float s_xchg[kTiles][2][2][kTileM];  // [tile][step parity][K block of the pair][row]: row maxima of the two threads of a row
  __shared__ float s_lsum[kTiles][2][kTileM];     // their partial row sums, at the end
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TR_DECL;
  TR_T0(t_cta);
  // Launch order.  grouped: first the first tile of every head (with a global-token row it is the heaviest by
  // far, and long jobs should start first), then the remaining tiles head by head: the tiles of a head share its
  // K and V (4 MB at S 8192, D 128), which then stay in L2 -- head-major order for all tiles kept 148 heads' K / V
  // live at once and sent every K / V tile to HBM again (28 -> 24.5 ms on 2048 heads).  Otherwise (all K / V fit
  // in L2 anyway): head-major, every head's heavy tile first, which balances best.
  const int tiles_per_head = p.Nt / (kTiles * kTileM);
  int head, cta_tile;
  if (!p.grouped) {
    cta_tile = blockIdx.x / p.heads;
    head = blockIdx.x - cta_tile * p.heads;
  } else if (static_cast<int>(blockIdx.x) < p.heads) {
    head = blockIdx.x; cta_tile = 0;
  } else {
    const int i = blockIdx.x - p.heads;
    head = i / (tiles_per_head - 1);
    cta_tile = 1 + (i - head * (tiles_per_head - 1));
  }
  const int br0 = cta_tile * 2 * kTiles;     // first of the CTA's four block rows
  const int ncb = p.Ns / kBlk;

  // ------------------------------ prologue ------------------------------
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < kTiles; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], kSmWarps);
      mbar_init(&pv_done[t], 1);
    }
    fence_mbar_init();
    s_range[0] = p.row_ptr[br0];
    s_range[1] = p.row_ptr[br0 + 2 * kTiles];
  }
  if (warp == kWarpLoad && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == kWarpQK) tmem_alloc<C::kTmemCols>(tmem_holder);
  for (int k = threadIdx.x; k < ncb; k += kThreads) kmask[k] = 0;
  __syncthreads();
  // the four block rows are consecutive in the BCSR array: entry = (block row << 16) | K block
  for (int e = s_range[0] + threadIdx.x; e < s_range[1]; e += kThreads) {
    const int v = __ldg(p.idx + e);
    const int kb = v & 0xffff, r = (v >> 16) - br0;
    if (kb < ncb && r >= 0 && r < 2 * kTiles)  // index arrays come from the caller: never index shared memory with them unchecked
      atomicOr(reinterpret_cast<unsigned int*>(kmask + (kb & ~3)), (1u << r) << (8 * (kb & 3)));
  }
  __syncthreads();
  if (warp == 0) {  // ordered compaction of the merged list
    int n = 0;
    for (int base = 0; base < ncb; base += 32) {
      const int k = base + lane;
      const int m = k < ncb ? kmask[k] : 0;
      const unsigned bal = __ballot_sync(0xffffffffu, m != 0);
      if (m) ulist[n + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>((k << 4) | m);
      n += __popc(bal);
    }
    if (lane == 0) *s_count = n;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const int count = *s_count;
  const int npairs = (count + 1) / 2;
  const long long q_row0 = (long long)head * p.Nt + (long long)cta_tile * (kTiles * kTileM);
  const long long kv_row0 = (long long)head * p.Ns;

  // presence bits of a step (both blocks of the pair): which tiles take part
  auto step_bits = [&](int j) -> uint32_t {
    uint32_t b = ulist[2 * j] & 0xfu;
    if (2 * j + 1 < count) b |= ulist[2 * j + 1] & 0xfu;
    return b;
  };

  bool failed = false;  // a bounded wait of this thread gave up
  if (warp == kWarpLoad) {
    // ------------------------------ producer ------------------------------
    if (lane == 0 && count > 0) {
      mbar_arrive_expect_tx(q_full, kTiles * C::kQBytes);
      for (int t = 0; t < kTiles; ++t)
        for (int c = 0; c < kChunks; ++c)
          tma_load_2d(q_s + t * C::kQBytes + c * (kTileM * 128), &tm_q, c * 64, (int)(q_row0 + t * kTileM), q_full);
      bool ok = true;
      for (int j = 0; j < npairs && ok; ++j) {
        const int nblk = min(2, count - 2 * j);
        const int st = j % kStages;
        const uint32_t par = ((j / kStages) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[st], nblk * kBlk * D * 2);
        for (int b = 0; b < nblk; ++b) {
          const int kb = ulist[2 * j + b] >> 4;
          for (int c = 0; c < kChunks; ++c)
            tma_load_2d(k_s + st * C::kKVBytes + c * (kPair * 128) + b * (kBlk * 128), &tm_k, c * 64,
                        (int)(kv_row0 + (long long)kb * kBlk), &k_full[st]);
        }
        if (!mbar_wait(&v_empty[st], par)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[st], nblk * kBlk * D * 2);
        for (int b = 0; b < nblk; ++b) {
          const int kb = ulist[2 * j + b] >> 4;
          for (int c = 0; c < kChunks; ++c)
            tma_load_2d(v_s + st * C::kKVBytes + c * (kPair * 128) + b * (kBlk * 128), &tm_v, c * 64,
                        (int)(kv_row0 + (long long)kb * kBlk), &v_full[st]);
        }
      }
      failed |= !ok;
      if (!ok) atomicExch(&p.status[0], 1);
    }
  } else if (warp == kWarpQK) {
    // ------------------------------ MMA issue: S_t = Q_t K^T and O_t += P_t V ------------------------------
    // One thread issues both contractions.  MMAs of one thread execute in issue order, so Q.K^T of a tile's
    // next step can be issued right behind the P.V of its current step: it will not overwrite the score
    // columns (which hold P) before that P.V has read them, and no barrier round trip separates the two.
    // The chain between two softmax phases of a tile is then: probabilities complete -> this warp wakes ->
    // 16 MMAs -> scores complete -> the softmax warps wake.  (With one issuing warp per contraction the chain
    // had a third hand-off in the middle; a trace showed the softmax warps waiting 1 700-2 000 cycles per step
    // for 1 024 cycles of MMAs.)
    // P: A operand in tensor memory, lane = row, two 16-bit probabilities per column; the thread holding K
    // block b of the pair left its 64 probabilities in columns 64 b .. 64 b + 31 of the tile's score region.
    // V: MN-major (head dim contiguous), 8 keys per 1024-byte group, 64-element chunks of the head dim
    // kPair * 128 bytes apart.
    // Issuing must not cost more than the 64 cycles an M128 N128 K16 MMA takes to execute, or the single issuing
    // thread becomes the bound (measured with descriptors assembled per instruction in a rolled loop: ~140 cycles
    // per MMA, the whole kernel waiting on this warp).  So the loops below are fully unrolled with compile-time
    // offsets, the per-stage / per-tile descriptor bases live in registers, and a descriptor is one 32-bit add
    // away from its base (only the 14-bit address field in the low word changes).
    const uint64_t desc_hi = make_smem_desc(0, 16, 1024, SW_128B);
    const uint64_t v_desc_hi = make_smem_desc(0, kPair * 128, 1024, SW_128B);
    const uint32_t hi_qk = static_cast<uint32_t>(desc_hi >> 32), hi_v = static_cast<uint32_t>(v_desc_hi >> 32);
    const uint32_t lo_flags = static_cast<uint32_t>(desc_hi) & 0xffff0000u;    // leading-offset field (same for V: LBO differs)
    const uint32_t lo_flags_v = static_cast<uint32_t>(v_desc_hi) & 0xffff0000u;
    // (scalars selected with ?: rather than arrays indexed at run time, which would live in local memory)
    static_assert(kTiles == 2 && kStages == 2, "the selections below are written out for two tiles and two stages");
    const uint32_t q_base0 = lo_flags | (smem_u32(q_s) >> 4), q_base1 = lo_flags | ((smem_u32(q_s) + C::kQBytes) >> 4);
    const uint32_t k_base0 = lo_flags | (smem_u32(k_s) >> 4), k_base1 = lo_flags | ((smem_u32(k_s) + C::kKVBytes) >> 4);
    const uint32_t v_base0 = lo_flags_v | (smem_u32(v_s) >> 4), v_base1 = lo_flags_v | ((smem_u32(v_s) + C::kKVBytes) >> 4);
    const uint32_t t_base0 = tmem_base, t_base1 = tmem_base + C::kTileCols;
    constexpr uint32_t idesc_pv = make_idesc_f16(kTileM, D, FMT, 0, 1);
    constexpr uint32_t idesc_qk2 = make_idesc_f16(kTileM, 2 * kBlk, FMT, 0, 0), idesc_qk1 = make_idesc_f16(kTileM, kBlk, FMT, 0, 0);
    bool ok = count == 0 || mbar_wait(q_full, 0);
    int taken[kTiles] = {0, 0};  // P.V steps issued per tile
    // last step each tile takes part in: only there does its epilogue need "P.V complete"
    int last_step[kTiles] = {-1, -1};
    for (int j = 0; j < npairs; ++j) {
      const uint32_t b = step_bits(j);
      if (b & 3u) last_step[0] = j;
      if (b & 12u) last_step[1] = j;
    }
    // scores of a step for tile t from K stage st (both indexes select registers), then "scores complete"
    auto issue_qk = [&](int t, int st, int nblk) {
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t qb = t ? q_base1 : q_base0, kb = st ? k_base1 : k_base0, d = t ? t_base1 : t_base0;
        const uint32_t idesc = nblk == 2 ? idesc_qk2 : idesc_qk1;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * (kTileM * 128) + (kk % 4) * 32) >> 4;  // kTileM == kPair
          umma_ss_lohi(d, qb + off, hi_qk, kb + off, hi_qk, idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      }
      __syncwarp();
    };
    auto issue_pv = [&](int t, int st, int nblk, bool first, bool last) {
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t vb = st ? v_base1 : v_base0, tb = t ? t_base1 : t_base0;
#pragma unroll
        for (int kk = 0; kk < 2 * (kBlk / 16); ++kk) {
          if (kk < nblk * (kBlk / 16)) {  // the second block of the pair may be missing at the end of the list
            const uint32_t a_col = (kk / 4) * kBlk + (kk % 4) * 8;
            umma_ts_lohi(tb + kPair, tb + a_col, vb + ((kk * 16 * 128) >> 4), hi_v, idesc_pv, (!first || kk > 0) ? 1u : 0u);
          }
        }
        if (last) umma_commit(&pv_done[t]);  // read by the tile's epilogue only
      }
      __syncwarp();
    };
    uint32_t bits_next = npairs > 0 ? step_bits(0) : 0u;
    if (ok && npairs > 0) {
      TR_T0(t_kf);
      ok = mbar_wait(&k_full[0], 0);
      TR_ADD(1, t_kf);
      if (ok) {
        const int nblk0 = min(2, count);
        if (bits_next & 3u) issue_qk(0, 0, nblk0);
        if (bits_next & 12u) issue_qk(1, 0, nblk0);
        if (lane == 0) umma_commit(&k_empty[0]);
        __syncwarp();
      }
    }
    for (int j = 0; j < npairs && ok; ++j) {
      const int nblk = min(2, count - 2 * j);
      const int st = j % kStages, st_next = (j + 1) % kStages;
      const bool more = j + 1 < npairs;
      const uint32_t bits = bits_next;
      bits_next = more ? step_bits(j + 1) : 0u;
      const int nblk_next = min(2, count - 2 * (j + 1));
      TR_T0(t_vf);
      if (!mbar_wait(&v_full[st], (j / kStages) & 1)) { ok = false; break; }
      TR_ADD(3, t_vf);
      bool k_ready = false;
#pragma unroll
      for (int t = 0; t < kTiles; ++t) {
        if (!ok) break;
        if ((bits >> (2 * t)) & 3u) {
          TR_T0(t_pf);
          if (!mbar_wait(&p_full[t], taken[t] & 1)) { ok = false; break; }
          TR_ADD(4, t_pf);
          issue_pv(t, st, nblk, taken[t] == 0, j == last_step[t]);
          ++taken[t];
        }
        if ((bits_next >> (2 * t)) & 3u) {
          if (!k_ready) {
            TR_T0(t_kf);
            if (!mbar_wait(&k_full[st_next], ((j + 1) / kStages) & 1)) { ok = false; break; }
            TR_ADD(1, t_kf);
            k_ready = true;
          }
          issue_qk(t, st_next, nblk_next);
        }
      }
      if (!ok) break;
      if (lane == 0) {
        umma_commit(&v_empty[st]);
        if (more) umma_commit(&k_empty[st_next]);
      }
      __syncwarp();
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[1], 1);
  } else if (warp < kWarpLoad) {
    // ------------------------------ softmax + epilogue ------------------------------
    // Two threads per row: warp w and warp w + 4 of a tile share a tensor-memory lane quadrant; the first takes
    // the first K block of a pair (score columns 0-63), the second the other one.  They exchange their row
    // maxima through shared memory once per step, keep partial row sums, and split the columns of O when it
    // is rescaled or written out.  Every thread of a tile passes the same named barriers whatever happens:
    // after a wait has given up it only keeps the barrier count.
    const int tile = warp / kSmWarps, wt = warp % kSmWarps;
    const int quad = wt & 3, colhalf = wt >> 2;
    const int row = quad * 32 + lane;          // row of the tile == TMEM lane
    const int half = row >> 6;                 // which of the tile's two block rows
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tile_base = tmem_base + lane_base + tile * C::kTileCols;
    const uint32_t o_base = tile_base + kPair;
    const long long grow = (long long)cta_tile * (kTiles * kTileM) + tile * kTileM + row;  // row inside the head
    const int bar_id = 1 + tile;
    constexpr int kOChunks = D / 64;           // 32-column chunks of O per thread
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    int taken = 0;
    for (int j = 0; j < npairs; ++j) {
      const int nblk = min(2, count - 2 * j);
      const uint32_t bits = step_bits(j);
      // neither block row of this tile keeps a block of the pair: nothing to do for this tile (uniform per tile)
      const bool active = (bits >> (2 * tile)) & 3u;
      const int e = colhalf < nblk ? ulist[2 * j + colhalf] : 0;
      const bool mine = (e >> (2 * tile + half)) & 1;  // this thread's block is kept in its block row (warp-uniform)
      const int kb = e >> 4;
      const uint32_t s_addr = tile_base + colhalf * kBlk;
      uint32_t r[32];
      auto mask_scores = [&](uint32_t* v, int h) {  // 32 scores starting at key 32 h of the block
        const uint4* mrow = reinterpret_cast<const uint4*>(p.mask + grow * p.Ns + (long long)kb * kBlk + h * 32);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint4 m4 = __ldg(mrow + q);
          const uint32_t mw[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (!((mw[i >> 2] >> (8 * (i & 3))) & 0xffu)) v[16 * q + i] = 0xff800000u;  // -inf
        }
      };
      bool run = false;  // this thread exponentiates in this step
      if (active) {
        // ---- pass 1: row maximum over the kept, unmasked scores of this thread's block ----
        float mx = -INFINITY;
        TR_T0(t_sf);
        if (ok) {
          if (!mbar_wait_warp(&s_full[tile], taken & 1)) {
            ok = false;
          } else {
            TR_ADD_IF(warp == 0, 5, t_sf);
            TR_ADD_IF(warp == 8, 10, t_sf);
            tc_fence_after_sync();
            if (mine) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                tmem_ld_x32(s_addr + h * 32, r);
                tmem_ld_wait();
                if (p.mask) mask_scores(r, h);
                float m4[4] = {mx, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[i]));
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
              }
            }
          }
        }
        TR_ADD_IF(warp == 0, 6, t_sf);  // wait + pass 1
        TR_T0(t_x);
        s_xchg[tile][taken & 1][colhalf][row] = mx;
        named_barrier_sync(bar_id, kSmWarps * 32);
        TR_ADD_IF(warp == 0, 7, t_x);
        if (ok) {
          run = true;
          mx = fmaxf(mx, s_xchg[tile][taken & 1][colhalf ^ 1][row]);
          const float m_new = mx * p.scale_log2;  // scale > 0
          // ---- lazy rescale of the running state.  The scores of this step exist, so the P.V of the tile's
          // previous step is complete (Q.K^T waited for it): the output accumulator is quiet ----
          float alpha = 1.f;
          if (m_new > m_run + kRescaleThreshold || (m_run == -INFINITY && m_new > -INFINITY)) {
            alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
            m_run = m_new;
            l_run *= alpha;
          }
          if (taken > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {  // the partner warp sees the same alphas and takes the other columns
#pragma unroll
            for (int c = colhalf * kOChunks; c < (colhalf + 1) * kOChunks; ++c) {
              uint32_t o[32];
              tmem_ld_x32(o_base + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_x32(o_base + c * 32, o);
            }
          }
        }
      }
      // ---- pass 2: P = exp2(S * scale * log2e - m) as 16-bit pairs, over the score columns just consumed ----
      // (making the two tiles take turns here, so that one exponentiates while the other's MMAs run, was
      // measured: no gain -- the MMA-issuing warp is busy 85 % of the time either way)
      TR_T0(t_p2);
      if (run) {
        if (colhalf < nblk) {  // this thread's block of the pair (warp-uniform)
          // every score of this row masked so far: subtracting +inf makes every probability zero
          const float neg_m = m_run > -INFINITY ? -m_run : -INFINITY;
          float sum = 0.f, sum1 = 0.f;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t packed[16];
            if (mine) {
              tmem_ld_x32(s_addr + h * 32, r);
              tmem_ld_wait();
              if (p.mask) mask_scores(r, h);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float p0 = ex2_approx(fmaf(__uint_as_float(r[2 * i]), p.scale_log2, neg_m));
                const float p1 = ex2_approx(fmaf(__uint_as_float(r[2 * i + 1]), p.scale_log2, neg_m));
                // the row sum takes the fp32 probabilities (their rounding to 16 bits for P.V is unbiased); two
                // alternating partial sums keep the additions from forming one dependent chain
                if (i & 1) sum1 += p0 + p1; else sum += p0 + p1;
                if constexpr (FMT == 0) {
                  const __half2 hv = __floats2half2_rn(p0, p1);
                  packed[i] = *reinterpret_cast<const uint32_t*>(&hv);
                } else {
                  const __nv_bfloat162 hv = __floats2bfloat162_rn(p0, p1);
                  packed[i] = *reinterpret_cast<const uint32_t*>(&hv);
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) packed[i] = 0;
            }
            // scores 32 h .. 32 h + 31 of this thread are consumed: their probabilities take columns 16 h .. of its region
            tmem_st_x16(s_addr + h * 16, packed);
          }
          l_run += sum + sum1;
        }
        tmem_st_wait();  // P and a rescaled O are in tensor memory
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[tile]);
      }
      TR_ADD_IF(warp == 0, 9, t_p2);
      if (active) ++taken;
    }
    TR_ADD_IF(warp == 0, 11, t_cta);
    if (warp == 0) { TR_SET(12, npairs); TR_SET(13, taken); }
    // ---- epilogue: O / l -> global ----
    if (ok && taken > 0 && !mbar_wait_warp(&pv_done[tile], 0)) ok = false;  // committed once, after the tile's last P.V
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[3], 1);
    tc_fence_after_sync();
    // the staging tile below reuses the Q tile's shared memory: its load must have landed (it has, unless this
    // tile took part in no step), and "P.V complete" above covers the last MMA that read it
    if (p.n_copies > 0 && count > 0 && !mbar_wait_warp(q_full, 0)) {
      ok = false;
      failed = true;
      if (lane == 0) atomicExch(&p.status[3], 1);
    }
    s_lsum[tile][colhalf][row] = l_run;  // the row sum is the two threads' partial sums
    named_barrier_sync(bar_id, kSmWarps * 32);
    l_run += s_lsum[tile][colhalf ^ 1][row];
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* orow = static_cast<T*>(p.O) + (q_row0 + tile * kTileM + row) * D;
#pragma unroll
    for (int c = colhalf * kOChunks; c < (colhalf + 1) * kOChunks; ++c) {
      uint32_t o[32];
      if (taken > 0 && ok) {
        tmem_ld_x32(o_base + c * 32, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0;
      }
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float v0 = __uint_as_float(o[2 * i]) * inv, v1 = __uint_as_float(o[2 * i + 1]) * inv;
        if constexpr (FMT == 0) {
          const __half2 hv = __floats2half2_rn(v0, v1);
          packed[i] = *reinterpret_cast<const uint32_t*>(&hv);
        } else {
          const __nv_bfloat162 hv = __floats2bfloat162_rn(v0, v1);
          packed[i] = *reinterpret_cast<const uint32_t*>(&hv);
        }
      }
      uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      if (p.n_copies > 0) {
        // the same 64 bytes into the staging tile: 64-column chunk c / 2, row `row`, 16-byte pieces
        // (c & 1) * 4 .. + 3 at piece position ^ (row & 7)
        uint8_t* srow = q_s + tile * C::kQBytes + (c >> 1) * (kTileM * 128) + row * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(srow + (((((c & 1) << 2) | q) ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
    }
    if (p.n_copies > 0) {  // uniform over the CTA
      fence_proxy_async_smem();  // the staging tile was written through the generic proxy, TMA reads through the async one
      named_barrier_sync(bar_id, kSmWarps * 32);
      if (wt == 0 && lane == 0) {
        for (int g = 0; g < p.n_copies; ++g)
          for (int ch = 0; ch < kChunks; ++ch)
            tma_store_2d(&gm.m[g], q_s + tile * C::kQBytes + ch * (kTileM * 128), ch * 64, (int)(q_row0 + tile * kTileM));
        tma_store_commit_and_wait_all();  // the peers' copies are complete when the kernel ends
      }
    }
    if (p.lse && colhalf == 0) {
      // natural-log sum of exponentials of the scaled scores (-inf for a fully masked row)
      p.lse[(long long)head * p.Nt + grow] = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc_fence_before_sync();
  sync_and_drain(failed);
  TR_ADD_IF(warp == 0, 0, t_cta);
  if (warp == kWarpQK) {
    tc_fence_after_sync();
    tmem_dealloc<C::kTmemCols>(tmem_base);
  }
}

template <int D, int FMT>
int launch_attn2(const void* Q, const void* K, const void* V, const Attn2Params& p, void* const* copies, int dtype,
                 cudaStream_t st) {
  using C = Cfg2<D>;
  CUtensorMap tm_q, tm_k, tm_v;
  GatherMaps gm;
  std::memset(&gm, 0, sizeof(gm));
  for (int g = 0; g < p.n_copies; ++g) {
    const uint64_t dims[2] = {(uint64_t)D, (uint64_t)p.heads * p.Nt};
    const uint64_t pitch[1] = {(uint64_t)D * 2};
    const uint32_t box[2] = {64, kTileM};
    int rc = make_tensor_map(&gm.m[g], copies[g], dtype, 2, dims, pitch, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  const uint64_t strides[1] = {(uint64_t)D * 2};
  {
    const uint64_t dims[2] = {(uint64_t)D, (uint64_t)p.heads * p.Nt};
    const uint32_t box[2] = {64, kTileM};
    int rc = make_tensor_map(&tm_q, Q, dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)D, (uint64_t)p.heads * p.Ns};
    const uint32_t box[2] = {64, kBlk};
    int rc = make_tensor_map(&tm_k, K, dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
    rc = make_tensor_map(&tm_v, V, dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  auto kern = attn_fwd_tc2_kernel<D, FMT>;
  static SmemAttrOnce attr;
  if (cudaError_t e = attr.ensure(kern, C::kSmem); e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((unsigned)((long long)p.heads * (p.Nt / (kTiles * kTileM))));
  kern<<<grid, kThreads, C::kSmem, st>>>(tm_q, tm_k, tm_v, gm, p);
  return launch_status();
}

}  // namespace

// K and V of all heads against the L2 (126 MB on B200): beyond about three quarters of it, tiles are launched
// grouped by head
bool kv_exceeds_l2(int heads, int Ns, int D) { return 4.0 * heads * Ns * D > 96.0 * 1024 * 1024; }

// The two-tile schedule applies when the query length is a multiple of 256 rows; attn_tc.cu takes the rest.
bool attn_tc2_supported(int Nt) { return Nt % (kTiles * kTileM) == 0; }

int attn_tc2_launch(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                    const int32_t* bcsr_idx, const uint8_t* mask, float scale_log2, int heads, int Nt, int Ns,
                    int D, int dtype, float* lse, int32_t* status, void* const* copies, int n_copies, cudaStream_t st) {
  if (n_copies < 0 || n_copies > SPARTA_ATTN_MAX_COPIES || (n_copies > 0 && !copies)) return SPARTA_ERR_BAD_ARG;
  for (int g = 0; g < n_copies; ++g)
    if (!copies[g] || !aligned(copies[g], 16)) return SPARTA_ERR_ALIGN;
  Attn2Params p;
  p.n_copies = n_copies;
  p.row_ptr = row_ptr; p.idx = bcsr_idx; p.mask = mask; p.O = O; p.lse = lse;
  p.Nt = Nt; p.Ns = Ns; p.heads = heads;
  p.grouped = kv_exceeds_l2(heads, Ns, D);
  p.scale_log2 = scale_log2;
  p.status = status;
  const int fmt = dtype == SPARTA_F16 ? 0 : 1;
  if (D == 64) return fmt == 0 ? launch_attn2<64, 0>(Q, K, V, p, copies, dtype, st) : launch_attn2<64, 1>(Q, K, V, p, copies, dtype, st);
  return fmt == 0 ? launch_attn2<128, 0>(Q, K, V, p, copies, dtype, st) : launch_attn2<128, 1>(Q, K, V, p, copies, dtype, st);
}

}  // namespace sparta

#ifdef SPARTA_ATTN_TRACE
// Instrumented builds only: copies (and clears) the per-role wait counters of the launches so far.
extern "C" int sparta_debug_attn_trace(unsigned long long* h_out) {
  cudaError_t e = cudaMemcpyFromSymbol(h_out, sparta::g_attn_trace, sizeof(unsigned long long) * 8 * 32);
  if (e != cudaSuccess) return static_cast<int>(e);
  static unsigned long long zeros[8 * 32] = {};
  e = cudaMemcpyToSymbol(sparta::g_attn_trace, zeros, sizeof(zeros));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
#endif
