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
// One CTA owns 128 token rows x a panel of NP = 8, 10 or 12 block columns, i.e. NP fp32 accumulators
// of 128 x 32 in tensor memory, plus a ring of kASlots = 4, 3 or 2 activation tiles (128 lanes x 64
// columns each) in the remaining columns.  A "step" is an aligned group of kG = 4 K-blocks (128 values
// of K) of which at least one is kept by a row-block of the panel; its activations arrive as two TMA
// boxes of 128-byte rows (the widest a swizzled box can fetch; a bulk tensor load costs the TMA unit
// about 1.3-1.9 cycles per box row however wide the row is, so 64-byte rows would cost twice as much
// per K-block).  What a step costs is mostly not its work: with loads, conversion and MMAs all
// switched off the kernel still takes three quarters of its time, because every role pays 100-150
// cycles for each mbarrier wait (also one that succeeds at once), 50-80 for a commit and 150-200 for a
// hand-off to the next warp, per step.  Hence steps of four K-blocks rather than two (22 % faster at
// 75 % sparsity, 5 % at 95 %; 10 % slower at 50 %), although only two to four of the larger activation
// tiles fit in tensor memory.  A step is in flight for 3-4 thousand cycles (load issue, load latency,
// conversion, MMA issue, four hand-offs) while its MMAs take a few hundred, so each resource is held
// only as long as it is needed: an X tile's shared-memory slot (four, or three beside 48 W slots) until the
// converters have read it, a W block's ring slot (40 or 48 blocks) and the activation slot until the step's
// MMAs are done; the "full" barriers form a ring of kSSlots = 12 steps.  The prologue turns the BCSR
// rows of the panel into a complete schedule in shared memory -- per step its K-group, the W blocks
// it needs (kmask of its K-blocks), where each of them sits in the value array (wsrc), its position
// in the W ring (cum_w), the latest earlier step whose W blocks still occupy that ring space
// (wait_for) and, per accumulator, the ring slots of its blocks (iss_tab) -- so the roles below run
// without per-step messages and with almost no bookkeeping of their own; a single warp executes
// dependent instructions at only one per ~5 cycles, which made run-time bookkeeping the bottleneck
// of earlier versions.  (With kG = 2 the same source builds the variant with 64-value steps, five X
// slots, four to six activation slots and issuers that release steps in pairs; K up to 32768 instead
// of 16384.)
//   warp 20      X producer: one TMA load per step into the X ring, as soon as the converters have
//                freed the slot; completes on the step's "full" mbarrier
//   warps 21-23  W producers: warp j issues the loads of steps j, j + 3, ... (blocks gathered by BCSR
//                position, one per lane in a single instruction; they complete on the same "full"
//                mbarrier) once the ring space is free.  Issuing one bulk tensor load costs the issuing
//                warp 50-140 cycles, hence three warps.
//   warps 0-3,   converters: shared memory -> registers -> tcgen05.st into the step's slot of the
//   16-19        activation ring (each warp its own 32-lane quadrant; the two sets alternate steps),
//                then arrive on the step's "a_full" mbarrier and on the X slot's "x_free" mbarrier
//   warps 4-15   MMA issue: warp 4 + l owns accumulator l, and one of its threads issues tcgen05.mma
//                with A from tensor memory (two K = 16 slabs per W block); MMAs into one accumulator
//                must come from one thread to stay ordered.  Every issuer commits to the "empty"
//                mbarrier of every step (also of steps in which it has no block), which frees the W
//                blocks and the activation slot once all have arrived and makes releases monotonic.
//                What to issue comes from iss_tab; the next step's barrier is probed ahead.
//   warps 0-3, 16-19 afterwards: epilogue, tcgen05.ld -> + bias -> fp16 / bf16 -> shared memory -> one TMA
//                store per tile of 64 output columns, issued as soon as the tile's four warps are done
// Every mbarrier wait is bounded; a wait that runs out sets a status word and the CTA winds down.
//
// Layouts.  The same kernel serves every product that has this shape -- a dense operand with the reduction
// dimension contiguous, times a block-sparse operand indexed along the output dimension:
//   dsd, B stored [N, K] (BCSR by row-block n)      the SparseLinear forward;
//   dsd, B stored [K, N] (BCSC by column-block n)   its input gradient dX = dY W: the 32 x 32 block then has the
//                                                   output dimension contiguous and enters the MMA as an
//                                                   MN-major B operand; with both index forms built, the
//                                                   64-bit BCSC entries carry the value position (BCSR order);
//   sdd with B stored [N, K]                        C^T = B A^T: the dense B plays the activations, the sparse
//                                                   A (BCSR [M, K] or BCSC [K, M]) the weight, and the
//                                                   epilogue stores the accumulators transposed.
// Replaces sparta_sparse_matmul_{dsd,sdd}.cuh.j2 / openai_sparse_matmul_{dsd,sdd}.cuh.j2 for these layouts.
#include <type_traits>

#include "bsmm.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

using namespace tc;

constexpr int kBlk = 32;            // BCSR block edge (K and N)
constexpr int kTileM = 128;         // token rows per CTA
constexpr int kG = 4;               // K-blocks per step (2 or 4, see above)
constexpr int kSubK = 2 * kBlk;     // K values of one X sub-tile: 128-byte rows, the widest swizzled TMA box
constexpr int kSubTiles = kG / 2;   // X sub-tiles per step
constexpr int kSubBytes = kTileM * kSubK * 2;  // 16 KB: 128 rows x 128 B
constexpr int kStepK = kG * kBlk;   // K values per step
constexpr int kXBytes = kSubTiles * kSubBytes;
constexpr int kWBytes = kBlk * kBlk * 2;      // 2 KB
constexpr int kACols = kStepK / 2;  // tensor-memory columns of one activation tile (two 16-bit values per column)
constexpr int kNPMax = 12;          // block columns per CTA: 8, 10 or 12, chosen per launch (template parameter NP)
constexpr int kMaxKb = kG == 2 ? 512 : 256;   // K-blocks the schedule can hold (K <= 16384 or 8192): shared-memory budget
constexpr int kMaxSteps = kMaxKb / kG;
// X tiles in shared memory; a slot is free again once its tile is in tensor memory.  A load takes well over a
// thousand cycles from issue to landing, a step should take a few hundred, and a slot is tied up for the whole
// flight: the number of X slots bounds the step rate (three slots: a step per ~630 cycles at best).  Panels of up
// to ten block columns need only 40 W slots, which leaves room for a fourth X slot (DEEP_X).  Measured on 4096^3:
// the fourth X slot wins 3 % at 90 / 95 % sparsity, where a step holds few W blocks, and loses 8 % at 75 %, where
// the W ring is the scarcer resource; the launcher picks by the density of the mask.
constexpr int x_slots(int np, bool deep_x) { return kG == 2 ? 5 : ((np >= 12 || !deep_x) ? 3 : 4); }
constexpr int kXSlotsMax = kG == 2 ? 5 : 4;
constexpr int kSSlots = 12;         // steps in flight between the first load and the last MMA: size of the "full" barrier ring
constexpr int kPair = kG == 2 ? 2 : 1;  // steps the issuers release together (pairs 2p, 2p + 1 when steps are small)
constexpr int kPSlots = kSSlots / kPair;  // ring of the issuers' "empty" barriers
// steps whose activations sit in tensor memory: the tiles that fit beside the NP accumulators (at most 6)
constexpr int kASlotsMax = 6;
constexpr int a_slots(int np) {
  const int fit = (512 - np * kBlk) / (kG * kBlk / 2);
  return fit < kASlotsMax ? fit : kASlotsMax;
}
constexpr int w_slots(int np, bool deep_x) { return (np >= 12 || !deep_x) ? 48 : 40; }  // W blocks in flight: at least the blocks of a pair of steps, see the W producers
constexpr int kMmaWarps = 12;       // warps reserved for MMA issue (a multiple of 4); the first NP are used, one per accumulator
constexpr int kConvSets = 2;        // converter warp sets (four warps each) that alternate steps
constexpr int kProdWarps = 4;       // TMA-issuing warps: one for the X tiles, the others for the W blocks
constexpr int kWProd = kProdWarps - 1;
constexpr int kMma0 = 4;            // first MMA-issuing warp
constexpr int kConv1 = kMma0 + kMmaWarps;    // first warp of the second converter set (a multiple of 4)
constexpr int kProd0 = kConv1 + 4;  // first producer warp
constexpr int kThreads = 32 * (kProd0 + kProdWarps);
static_assert(kWProd <= kSSlots, "a producer may run at most one ring turn ahead of the release it waits for");
static_assert(kSSlots % 2 == 0 && kSSlots >= kXSlotsMax + kASlotsMax,
              "the X producer's arrival for step s must find the phase of step s - kSSlots complete, see there");
static_assert(kConv1 % 4 == 0, "converter warps must map onto their tensor-memory lane quadrant");
static_assert(kNPMax <= 12 && kNPMax <= kMmaWarps, "a step record packs 12-bit block masks; one issuer warp per accumulator");
static_assert(w_slots(12, false) >= kPair * kG * 12 && w_slots(10, true) >= kPair * kG * 10 && w_slots(12, false) < 64,
              "the W blocks of a pair of steps must fit the ring; a ring position packs into 6 bits");

struct DsdTcParams {
  const int32_t* row_ptr;  // pointer array along the output dimension (row_ptr of [N, K], col_ptr of [K, N])
  const void* idx;         // packed entries (output block << 16) | reduction block; 64-bit with the value position on top
  int idx64;               // entries are 64-bit (both index forms built): values sit at entry >> 32
  int b_mn;                // the sparse blocks have the output dimension contiguous (stored [K, N]): MN-major B operand
  int out_t;               // store the accumulators transposed: C is [N, M] in this kernel's terms (sdd through B A^T)
  const void* bias;
  void* C;
  int M, N, Kb, Nb;
  long long val_stride_blocks;
  int32_t* status;
};

constexpr uint32_t kTmemCols = 512;

// shared-memory carve-up (byte offsets from a 1 KB aligned base), per panel width
template <int NP, bool DEEP_X>
struct Lay {
  static constexpr int kXSlots = x_slots(NP, DEEP_X), kWSlots = w_slots(NP, DEEP_X);
  static constexpr int kOffX = 0;                                  // X ring   [kXSlots][128 rows x 128 B]
  static constexpr int kOffW = kOffX + kXSlots * kXBytes;           // W ring   [kWSlots][2 KB]
  static constexpr int kOffMask = kOffW + kWSlots * kWBytes;       // kmask    [Kb]        u32: row-blocks keeping K-block k
  static constexpr int kOffSrc = kOffMask + kMaxKb * 4;            // wsrc     [Kb][NP]    u32: position of the block in the value array
  static constexpr int kOffStep = kOffSrc + kMaxKb * NP * 4;       // step_kp  [steps]     u16: K-pair index
  static constexpr int kOffCum = kOffStep + kMaxSteps * 2;         // cum_w    [steps + 1] u16: W blocks of all earlier steps
  static constexpr int kOffWait = kOffCum + (kMaxSteps + 8) * 2;   // wait_for [steps]     s16
  static constexpr int kOffRec = (kOffWait + kMaxSteps * 2 + 7) / 8 * 8;  // rec [steps] u64: 12-bit block mask per K-block | ring pos << 48
  static constexpr int kOffIss = kOffRec + kMaxSteps * 8;          // iss_tab  [steps][NP][kG] u8: W ring slot of the block, 0xff = none
  static constexpr int kOffBias = (kOffIss + kMaxSteps * NP * kG + 7) / 8 * 8;  // bias  [NP * 32]   f32
  static constexpr int kOffCtl = kOffBias + kNPMax * kBlk * 4;     // mbarriers and scalars
  static constexpr int kSmemTotal = kOffCtl + 512 + 1024 /* alignment slack */;
  static_assert(kOffRec % 8 == 0 && kOffBias % 8 == 0 && kOffCtl % 8 == 0, "alignment of the shared-memory tables");
  static_assert(kSmemTotal <= 227 * 1024, "shared memory budget");
  static_assert(kXSlots * kXBytes + kWSlots * kWBytes >= (kNPMax / 2) * kSubBytes,
                "the epilogue stages the output tile in the X ring and the W ring behind it");
};

template <int FMT, int NP, bool DEEP_X>
__global__ void __launch_bounds__(kThreads, 1)
bsmm_dsd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_c, DsdTcParams p) {
  using T = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
  static_assert(NP % 2 == 0 && NP <= kNPMax, "panel width");
  constexpr int kASlots = a_slots(NP);
  constexpr uint32_t kAccCols = NP * kBlk;
  static_assert(kASlots >= 2 && kAccCols + kASlots * kACols <= kTmemCols, "tensor memory budget");
  constexpr int kIssuers = NP;  // issuer warps in use
  constexpr uint32_t kLow = (1u << NP) - 1u;
  using L = Lay<NP, DEEP_X>;
  constexpr int kXSlots = L::kXSlots, kWSlots = L::kWSlots;
  constexpr int kOffX = L::kOffX, kOffW = L::kOffW, kOffMask = L::kOffMask, kOffSrc = L::kOffSrc, kOffStep = L::kOffStep,
                kOffCum = L::kOffCum, kOffWait = L::kOffWait, kOffRec = L::kOffRec, kOffIss = L::kOffIss,
                kOffBias = L::kOffBias, kOffCtl = L::kOffCtl;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x_ring = smem + kOffX;
  uint8_t* w_ring = smem + kOffW;
  uint32_t* kmask = reinterpret_cast<uint32_t*>(smem + kOffMask);
  uint32_t* wsrc = reinterpret_cast<uint32_t*>(smem + kOffSrc);
  uint16_t* step_kp = reinterpret_cast<uint16_t*>(smem + kOffStep);
  uint16_t* cum_w = reinterpret_cast<uint16_t*>(smem + kOffCum);
  int16_t* wait_for = reinterpret_cast<int16_t*>(smem + kOffWait);
  uint64_t* rec = reinterpret_cast<uint64_t*>(smem + kOffRec);
  uint8_t* iss_tab = smem + kOffIss;
  float* s_bias = reinterpret_cast<float*>(smem + kOffBias);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kOffCtl);  // [kSSlots] loads of a step have landed
  uint64_t* empty_bar = full_bar + kSSlots;                // [kPSlots] MMAs of a pair of steps have read their operands
  uint64_t* afull_bar = empty_bar + kPSlots;               // [kASlots] the step's activations are in tensor memory
  uint64_t* xfree_bar = afull_bar + kASlots;               // [kXSlots] the X tile has been read out of its slot
  uint64_t* accum_bar = xfree_bar + kXSlots;               // [1]       all MMAs of the tile are done
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_bar + 1);
  int* s_range = reinterpret_cast<int*>(tmem_holder + 1);  // [2] BCSR entries of the panel
  int* s_nsteps = s_range + 2;
  uint32_t* s_written = reinterpret_cast<uint32_t*>(s_nsteps + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int panel = blockIdx.x, m0 = blockIdx.y * kTileM, batch = blockIdx.z;
  const int nb0 = panel * NP;
  const int nb_end = min(nb0 + NP, p.Nb);
  const bool is_conv = warp < 4 || (warp >= kConv1 && warp < kProd0);
  const int conv_set = warp < 4 ? 0 : 1;
  const int quad = warp & 3;  // tensor-memory lane quadrant this warp may access
  const int n_pairs = (p.Kb + kG - 1) / kG;  // K-groups (steps before the empty ones are dropped)

  // ------------------------------ prologue: barriers, tensor memory, schedule ------------------------------
  // the rows of a panel are consecutive in the BCSR array; every thread reads the panel's range and its
  // first entry now, so that the two dependent trips to memory overlap the set-up below
  const int e0 = __ldg(p.row_ptr + nb0), e1 = __ldg(p.row_ptr + nb_end);
  auto load_entry = [&](int e, uint32_t& pos) -> int {  // packed (output block << 16) | reduction block, and where its values sit
    if (p.idx64) {
      const long long w = __ldg(static_cast<const long long*>(p.idx) + e);
      pos = static_cast<uint32_t>(w >> 32);
      return static_cast<int>(w & 0xffffffffll);
    }
    pos = static_cast<uint32_t>(e);
    return __ldg(static_cast<const int32_t*>(p.idx) + e);
  };
  uint32_t pos_first = 0;
  const int v_first = e0 + static_cast<int>(threadIdx.x) < e1 ? load_entry(e0 + threadIdx.x, pos_first) : 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSSlots; ++s) mbar_init(&full_bar[s], 2);  // the X producer and the step's W producer
    for (int s = 0; s < kPSlots; ++s) mbar_init(&empty_bar[s], kIssuers);
    for (int s = 0; s < kASlots; ++s) mbar_init(&afull_bar[s], 4);
    for (int s = 0; s < kXSlots; ++s) mbar_init(&xfree_bar[s], 4);
    mbar_init(accum_bar, kIssuers);
    fence_mbar_init();
  }
  if (warp == kProd0 && lane == 0) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_c);
  }
  if (warp == kMma0) tmem_alloc<kTmemCols>(tmem_holder);
  for (int k = threadIdx.x; k < kG * n_pairs; k += kThreads) kmask[k] = 0;  // includes the pad blocks of the last group
  {
    // (with the transposed store the bias runs along this kernel's rows and is added in the epilogue)
    const T* bias = p.bias && !p.out_t ? static_cast<const T*>(p.bias) + (long long)batch * p.N : nullptr;
    for (int j = threadIdx.x; j < NP * kBlk; j += kThreads) {
      const int n = nb0 * kBlk + j;
      s_bias[j] = (bias && n < p.N) ? to_float(bias[n]) : 0.f;
    }
  }
  __syncthreads();
  // entry = (row-block << 16) | K-block
  for (int e = e0 + threadIdx.x; e < e1; e += kThreads) {
    uint32_t pos = pos_first;
    const int v = e == e0 + static_cast<int>(threadIdx.x) ? v_first : load_entry(e, pos);
    const int k = v & 0xffff, l = (v >> 16) - nb0;
    if (k < p.Kb && l >= 0 && l < NP) {  // index arrays come from the caller: never index shared memory with them unchecked
      atomicOr(&kmask[k], 1u << l);
      wsrc[k * NP + l] = pos;
    }
  }
  __syncthreads();
  if (warp == 0) {
    // compact the kept K-pairs into steps and prefix-sum their W block counts
    int base = 0, wbase = 0;
    uint32_t wr = 0;
    for (int c = 0; c < n_pairs; c += 32) {
      const int kp = c + lane;
      uint32_t m = 0u;  // which row-blocks keep any of the group's K-blocks; w: how many blocks in all
      int w = 0;
      if (kp < n_pairs) {
#pragma unroll
        for (int j = 0; j < kG; ++j) {
          m |= kmask[kG * kp + j];
          w += __popc(kmask[kG * kp + j]);
        }
      }
      wr |= m;
      const unsigned bal = __ballot_sync(0xffffffffu, m != 0u);
      const int ord = base + __popc(bal & ((1u << lane) - 1u));
      int incl = w;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
      }
      if (m) {
        step_kp[ord] = static_cast<uint16_t>(kp);
        cum_w[ord] = static_cast<uint16_t>(wbase + incl - w);
      }
      base += __popc(bal);
      wbase += __shfl_sync(0xffffffffu, incl, 31);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wr |= __shfl_xor_sync(0xffffffffu, wr, o);
    if (lane == 0) {
      cum_w[base] = static_cast<uint16_t>(wbase);
      *s_nsteps = base;
      *s_written = wr;
    }
  }
  __syncthreads();
  const int n_steps = *s_nsteps;
  // the W blocks of step s may be fetched once step wait_for[s], the latest one whose W blocks still
  // occupy the ring positions s needs, has been released
  for (int s = threadIdx.x; s < n_steps; s += kThreads) {
    const int target = static_cast<int>(cum_w[s + 1]) - kWSlots;
    int f = -1;
    if (target > 0) {
      int lo = 0, hi = s;  // cum_w[s] >= target because a step holds at most kG NP <= kWSlots blocks
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int>(cum_w[mid]) >= target) hi = mid; else lo = mid + 1;
      }
      f = lo - 1;
    }
    wait_for[s] = static_cast<int16_t>(f);
    const int kp = step_kp[s];
    uint64_t rr = static_cast<uint64_t>(cum_w[s] % kWSlots) << 48;
#pragma unroll
    for (int j = 0; j < kG; ++j) rr |= static_cast<uint64_t>(kmask[kG * kp + j]) << (NP * j);
    rec[s] = rr;
  }
  // the issuers' view of a step: for every accumulator and K-block of the step, the W ring slot that
  // holds its block (blocks take consecutive slots in K-block, then accumulator order), 0xff for none
  for (int i = threadIdx.x; i < n_steps * NP; i += kThreads) {
    const int s = i / NP, l = i - s * NP;
    const int kp = step_kp[s];
    int pos = static_cast<int>(cum_w[s] % kWSlots);
#pragma unroll
    for (int j = 0; j < kG; ++j) {
      const uint32_t mk = kmask[kG * kp + j];
      uint8_t b = 0xff;
      if ((mk >> l) & 1u) {
        int q = pos + __popc(mk & ((1u << l) - 1u));  // below 2 kWSlots: a step holds at most kWSlots blocks
        if (q >= kWSlots) q -= kWSlots;
        b = static_cast<uint8_t>(q);
      }
      iss_tab[i * kG + j] = b;
      pos += __popc(mk);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t a_tmem = tmem_base + kAccCols;  // activation ring

  bool failed = false;  // a bounded wait of this thread gave up
  if (warp == kProd0) {
    // ------------------------------ X producer ------------------------------
    // One warp, all steps in order: the slot is free once the converters have read the tile that was
    // in it (step s - kXSlots).  The converter of that step had waited for the release of step
    // s - kXSlots - kASlots, so the issuers -- and before them the converters -- are through every step
    // up to there, step s - kSSlots included: the previous phase of this step's "full" barrier is
    // complete when the arrival for step s is made.
    bool ok = true;
    for (int s = 0; s < n_steps; ++s) {
      const int xslot = s % kXSlots, sslot = s % kSSlots;
      if (s >= kXSlots && !mbar_wait_warp(&xfree_bar[xslot], ((s - kXSlots) / kXSlots) & 1)) { ok = false; break; }
      if (lane == 0) {
        const int kp = step_kp[s];
        mbar_arrive_expect_tx(&full_bar[sslot], kXBytes);
#pragma unroll
        for (int t = 0; t < kSubTiles; ++t)
          tma_load_2d(x_ring + xslot * kXBytes + t * kSubBytes, &tm_x, kp * kStepK + t * kSubK, batch * p.M + m0,
                      &full_bar[sslot]);
      }
      __syncwarp();
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[0], 1);
  } else if (warp > kProd0) {
    // ------------------------------ W producers ------------------------------
    // One instruction per pair of K-blocks; lanes 0 .. NP-1 fetch the blocks of the pair's first
    // K-block, lanes 16 .. 16+NP-1 those of the second
    const long long wrow0 = (long long)batch * p.val_stride_blocks * kBlk;  // row in the [blocks * 32, 32] view
    const int half = lane >> 4, l = lane & 15;
    bool ok = true;
    for (int s = warp - kProd0 - 1; s < n_steps; s += kWProd) {
      const int kp = step_kp[s];
      const uint64_t r = rec[s];
      const int c0 = static_cast<int>(r >> 48) & 0x3f, wf = wait_for[s];
      uint32_t pack[kSubTiles];  // per pair of K-blocks: one bit per lane that has a block to fetch
      uint32_t src[kSubTiles];
      int n_blocks = 0;
#pragma unroll
      for (int t = 0; t < kSubTiles; ++t) {
        pack[t] = (static_cast<uint32_t>(r >> (2 * t * NP)) & kLow) | ((static_cast<uint32_t>(r >> ((2 * t + 1) * NP)) & kLow) << 16);
        src[t] = ((pack[t] >> lane) & 1u) ? wsrc[(kG * kp + 2 * t + half) * NP + l] : 0u;
        n_blocks += __popc(pack[t]);
      }
      // An mbarrier wait names a phase by its parity only, so a waiter must know that the barrier is
      // at most one phase away from the one it names.  Releases are monotonic and this warp's previous
      // step (s - kWProd) confirmed the release of step s - kWProd - kSSlots, at or after the predecessor
      // of step s - kSSlots on that barrier: waiting for s - kSSlots is safe.  After it, everything up to
      // s - kSSlots is known to be released, which covers the predecessor of any later step wf, and the
      // previous phase of this step's "full" barrier is complete.
      // Steps are released in pairs: step t with pair t / 2, on barrier (t / 2) % kPSlots.  wait_for[s]
      // always lies in an earlier pair than s, because the blocks of one pair fit the ring.
      const int sslot = s % kSSlots, pr = s / kPair;
      if (s >= kSSlots && !mbar_wait_warp(&empty_bar[pr % kPSlots], (pr / kPSlots - 1) & 1)) { ok = false; break; }
      if (wf >= 0 && wf > s - kSSlots && !mbar_wait_warp(&empty_bar[(wf / kPair) % kPSlots], ((wf / kPair) / kPSlots) & 1)) { ok = false; break; }
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[sslot], n_blocks * kWBytes);
      __syncwarp();  // the expected byte count is registered before any lane's load can complete
      int before = c0;  // ring position of the pair's first block
#pragma unroll
      for (int t = 0; t < kSubTiles; ++t) {
        if ((pack[t] >> lane) & 1u) {
          int ws = before + __popc(pack[t] & ((1u << lane) - 1u));  // rank among the step's blocks
          if (ws >= kWSlots) ws -= kWSlots;
          tma_load_2d(w_ring + ws * kWBytes, &tm_w, 0, (int)(wrow0 + (long long)src[t] * kBlk), &full_bar[sslot]);
        }
        before += __popc(pack[t]);
      }
      __syncwarp();
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[0], 1);
  } else if (warp >= kMma0 && warp < kMma0 + kIssuers) {  // (warps up to kConv1 are spare when NP < 12)
    // ------------------------------ MMA issue ------------------------------
    // Operand addresses derive from the schedule only, so they stay warp-uniform; one lane issues.
    // K-major B (block stored [n][k]): K = 16 slabs 32 bytes apart inside the 64-byte rows.  MN-major B (block stored
    // [k][n]): 16 rows of 64 bytes per slab, 1 KB apart; eight-row groups 512 bytes apart either way.
    const uint32_t idesc = make_idesc_f16(kTileM, kBlk, FMT, 0, p.b_mn ? 1 : 0);
    const uint32_t slab = p.b_mn ? (16u * kBlk * 2u) >> 4 : 2u;
    const uint32_t w_base16 = smem_u32(w_ring) >> 4;
    const uint64_t desc_hi = p.b_mn ? make_smem_desc(0, kWBytes, 512, SW_64B) : make_smem_desc(0, 16, 512, SW_64B);
    const bool leader = lane == 0;
    const int l = warp - kMma0;                        // the accumulator issued by this warp
    const uint32_t d_tmem = tmem_base + l * kBlk;
    using Word = typename std::conditional<kG == 2, uint16_t, uint32_t>::type;  // kG bytes of the table
    constexpr uint32_t kNone = kG == 2 ? 0xffffu : 0xffffffffu;
    const Word* tab = reinterpret_cast<const Word*>(iss_tab) + l;
    uint32_t pslot = 0, aslot = 0, aphase = 0, accumulate = 0;
    bool ok = true;
    // the MMAs of one step of this accumulator: v holds, per K-block of the step, the W ring slot or 0xff
    auto issue = [&](uint32_t v, uint32_t as) {
#pragma unroll
      for (int j = 0; j < kG; ++j) {
        const uint32_t b = (v >> (8 * j)) & 0xffu;
        if (b != 0xffu) {
          const uint32_t a_addr = a_tmem + as * kACols + j * (kBlk / 2);
          const uint32_t b_lo = w_base16 + b * (kWBytes >> 4);
          umma_ts(d_tmem, a_addr, desc_hi | b_lo, idesc, accumulate);
          umma_ts(d_tmem, a_addr + kBlk / 4, desc_hi | (b_lo + slab), idesc, 1u);
          accumulate = 1u;
        }
      }
    };
    // Steps are taken two at a time.  Every issuer waits for the activations of every step and commits
    // to the "empty" barrier of every pair, also when it has no block in it.  The waits keep it within
    // one ring turn of the converters, so a phase parity is never mistaken for an older one; the commit
    // makes the release of steps monotonic (a released pair implies that every issuer's MMAs of all
    // earlier steps are done), which is what the producers' wait_for table assumes.  A step's "full"
    // phase completed before its converters ran, so the W blocks are in place too.  What to issue
    // comes from the table the prologue built: decoding the step's masks here, on one warp, took
    // longer than the MMAs.  The wait, the commit and the loop cost a warp 200-300 cycles, several
    // times the MMAs of a step: hence pairs, and the probes of the next pair's barriers issued ahead
    // (the issuers usually run a few steps behind the converters, so the probes mostly succeed).
    bool ready0 = false, ready1 = false;
    for (int s = 0; s < n_steps; s += kPair) {
      const bool two = kPair == 2 && s + 1 < n_steps;
      const uint32_t v0 = tab[s * NP], v1 = two ? static_cast<uint32_t>(tab[(s + 1) * NP]) : kNone;
      const uint32_t as0 = aslot, ph0 = aphase;
      if (++aslot == kASlots) { aslot = 0; aphase ^= 1u; }
      const uint32_t as1 = aslot, ph1 = aphase;
      if (kPair == 2 && ++aslot == kASlots) { aslot = 0; aphase ^= 1u; }
      if (!ready0 && !mbar_wait(&afull_bar[as0], ph0)) { ok = false; break; }
      if (v0 != kNone) {
        tc_fence_after_sync();
        if (leader) issue(v0, as0);
      }
      if (two) {
        if (!ready1 && !mbar_wait(&afull_bar[as1], ph1)) { ok = false; break; }
        if (v1 != kNone) {
          tc_fence_after_sync();
          if (leader) issue(v1, as1);
        }
      }
      const uint32_t as3 = aslot + 1 == kASlots ? 0u : aslot + 1, ph3 = aslot + 1 == kASlots ? aphase ^ 1u : aphase;
      ready0 = s + kPair < n_steps && mbar_test_wait(&afull_bar[aslot], aphase);
      ready1 = kPair == 2 && s + 3 < n_steps && mbar_test_wait(&afull_bar[as3], ph3);
      if (leader) umma_commit(&empty_bar[pslot]);  // frees the pair's W blocks and activation slots
      if (++pslot == kPSlots) pslot = 0;
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[1], 1);
    if (leader) umma_commit(accum_bar);
  } else if (is_conv) {
    // ------------------------------ converters ------------------------------
    // The X tile was written by TMA with the 128-byte swizzle: the 16-byte chunk c of row r sits at
    // chunk position c ^ (r & 7), which also makes the row-per-thread reads conflict-free.
    const int row = quad * 32 + lane;
    const uint32_t sw = row & 7;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    for (int s = conv_set; s < n_steps; s += kConvSets) {
      const int slot = s % kXSlots, aslot = s % kASlots;
      // the loads of the step have landed: take the first half of the tile into registers at once, so that
      // only the stores to tensor memory follow the wait for the activation slot
      if (!mbar_wait_warp(&full_bar[s % kSSlots], (s / kSSlots) & 1)) { ok = false; break; }
      uint32_t r[32];
      {
        const uint8_t* xrow = x_ring + slot * kXBytes + row * (kSubK * 2);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(xrow + ((c ^ sw) << 4));
          r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
        }
      }
      // the activation slot is free once the MMAs of step s - kASlots are done (this warp confirmed the
      // release of step s - kConvSets - kASlots on its previous turn, so the parity cannot alias)
      if (s >= kASlots && !mbar_wait_warp(&empty_bar[((s - kASlots) / kPair) % kPSlots], (((s - kASlots) / kPair) / kPSlots) & 1)) { ok = false; break; }
      tmem_st_x32(a_tmem + aslot * kACols + lane_addr, r);
#pragma unroll
      for (int t = 1; t < kSubTiles; ++t) {
        const uint8_t* xrow = x_ring + slot * kXBytes + t * kSubBytes + row * (kSubK * 2);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(xrow + ((c ^ sw) << 4));
          r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
        }
        tmem_st_x32(a_tmem + aslot * kACols + t * (kSubK / 2) + lane_addr, r);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&afull_bar[aslot]);
        mbar_arrive(&xfree_bar[slot]);  // the tile is in registers / tensor memory: the X slot may be refilled
      }
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[3], 1);

    // ------------------------------ epilogue ------------------------------
    // Accumulators -> + bias -> 16 bit -> the idle X ring as six tiles of 128 rows x 64 columns in
    // the 128-byte swizzle, then one TMA store per tile.  (Storing from registers, a lane per row,
    // would touch 32 different lines with every instruction and took four times longer.)  The two
    // warps of a lane quadrant take alternate pairs of accumulators.
    const uint32_t written = *s_written;
    const bool acc_ok = mbar_wait_warp(accum_bar, 0);
    if (!acc_ok) {
      failed = true;
      if (lane == 0) atomicExch(&p.status[2], 1);
    } else {
      tc_fence_after_sync();
    }
    // A tile (two accumulators, 64 output columns) belongs to one converter set; its four warps fill
    // it, meet at the set's named barrier, and one thread issues the tile's TMA store while the set
    // goes on to its next tile.
    const int n_acc = nb_end - nb0, n_tiles = (n_acc + 1) / 2;
    if (p.out_t) {
      // Transposed store (sdd as B A^T): the thread's row is a column of C, so the 32 lanes of a warp write 64
      // contiguous bytes of one row of C per accumulator column, straight from registers.
      if (acc_ok) {
        T* C = static_cast<T*>(p.C);
        const float bt = p.bias ? to_float(static_cast<const T*>(p.bias)[(long long)batch * p.M + m0 + row]) : 0.f;
        for (int l = conv_set; l < n_acc; l += kConvSets) {
          uint32_t r[32];
          if ((written >> l) & 1u) {
            tmem_ld_x32(tmem_base + lane_addr + l * kBlk, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
          }
          T* out = C + ((long long)batch * p.N + (long long)(nb0 + l) * kBlk) * p.M + m0 + row;
#pragma unroll
          for (int j = 0; j < 32; ++j) out[(long long)j * p.M] = from_float<T>(__uint_as_float(r[j]) + bt);
        }
      }
    } else
    for (int t = conv_set; t < n_tiles; t += kConvSets) {
      if (acc_ok) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int l = 2 * t + h;
          if (l >= n_acc) break;
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
              __half2 hh = __floats2half2_rn(v0, v1);
              packed[j] = *reinterpret_cast<uint32_t*>(&hh);
            } else {
              __nv_bfloat162 hh = __floats2bfloat162_rn(v0, v1);
              packed[j] = *reinterpret_cast<uint32_t*>(&hh);
            }
          }
          // tile t, row `row`, 16-byte chunks h * 4 .. + 3, each at chunk position c ^ (row & 7)
          uint8_t* trow = x_ring + t * kSubBytes + row * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t c = static_cast<uint32_t>(h * 4 + j) ^ sw;
            *reinterpret_cast<uint4*>(trow + (c << 4)) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          }
        }
        fence_proxy_async_smem();  // the tile was written through the generic proxy, TMA reads through the async one
      }
      if (conv_set == 0) named_barrier_sync(2, 4 * 32); else named_barrier_sync(3, 4 * 32);  // the four warps of this set
      if (quad == 0 && lane == 0 && acc_ok)
        tma_store_2d(&tm_c, x_ring + t * kSubBytes, (nb0 + 2 * t) * kBlk, batch * p.M + m0);
    }
    if (quad == 0 && lane == 0 && !p.out_t) tma_store_commit_and_wait();  // shared memory must outlive the stores' reads
  }
  tc_fence_before_sync();
  sync_and_drain(failed);
  if (warp == kMma0) {
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

// The product in this kernel's own terms: C[M, N] (or its transpose) = X[M, K] . W^T, W block-sparse along N.
struct DsdView {
  const void* X;
  const void* W;
  int M, N, K;
  int b_mn, out_t;
};

DsdView dsd_view(const BsmmParams& p) {
  if (p.mode == MODE_DSD) return {p.A, p.B, p.M, p.N, p.K, p.trans_b ? 0 : 1, 0};
  return {p.B, p.A, p.N, p.M, p.K, p.trans_a ? 1 : 0, 1};  // sdd: C^T = B A^T
}

template <int FMT, int NP, bool DEEP_X>
int launch_dsd_tc(const BsmmParams& p, const DsdView& v, cudaStream_t st) {
  CUtensorMap tm_x, tm_w;
  {
    const uint64_t dims[2] = {(uint64_t)v.K, (uint64_t)p.batch * v.M};
    const uint64_t strides[1] = {(uint64_t)v.K * 2};
    const uint32_t box[2] = {kSubK, kTileM};
    int rc = make_tensor_map(&tm_x, v.X, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  {
    const uint64_t dims[2] = {kBlk, (uint64_t)p.batch * p.val_stride_blocks * kBlk};
    const uint64_t strides[1] = {kBlk * 2};
    const uint32_t box[2] = {kBlk, kBlk};
    int rc = make_tensor_map(&tm_w, v.W, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != SPARTA_OK) return rc;
  }
  CUtensorMap tm_c;  // unused by the transposed store, which writes from registers
  {
    const uint64_t dims[2] = {(uint64_t)(v.out_t ? v.M : v.N), (uint64_t)p.batch * (v.out_t ? v.N : v.M)};
    const uint64_t strides[1] = {dims[0] * 2};
    const uint32_t box[2] = {kSubK, kTileM};
    int rc = make_tensor_map(&tm_c, p.C, p.dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  DsdTcParams q;
  q.row_ptr = p.ptr;
  q.idx = p.idx;
  q.idx64 = p.idx_is_64;
  q.b_mn = v.b_mn;
  q.out_t = v.out_t;
  q.bias = p.bias;
  q.C = p.C;
  q.M = v.M; q.N = v.N; q.Kb = v.K / kBlk; q.Nb = v.N / kBlk;
  q.val_stride_blocks = p.val_stride_blocks;
  q.status = device_status_ptr();
  if (!q.status) return SPARTA_ERR_DRIVER;
  auto kern = bsmm_dsd_tc_kernel<FMT, NP, DEEP_X>;
  constexpr int kSmemTotal = Lay<NP, DEEP_X>::kSmemTotal;
  static SmemAttrOnce attr;
  if (cudaError_t e = attr.ensure(kern, kSmemTotal); e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((q.Nb + NP - 1) / NP, v.M / kTileM, p.batch);
  kern<<<grid, kThreads, kSmemTotal, st>>>(tm_x, tm_w, tm_c, q);
  return launch_status();
}

}  // namespace
bool bsmm_tc_available() { return true; }

bool dsd_tc_supported(const BsmmParams& p) {
  // dsd with either weight layout (BCSR [N, K]; BCSC [K, N], 32-bit or with the BCSR value position), and sdd
  // against a dense B stored [N, K]; the dense operand must have the reduction dimension contiguous
  if (p.mode == MODE_DSD) {
    if (p.trans_a || p.BM != kTileM || p.BN != kBlk) return false;
    if (p.trans_b && p.idx_is_64) return false;  // 64-bit entries exist in the BCSC order only
  } else if (p.mode == MODE_SDD) {
    if (!p.trans_b || p.BM != kBlk || p.BN != kTileM) return false;
    if (!p.trans_a && p.idx_is_64) return false;
  } else {
    return false;
  }
  if (!p.compressed || p.BK != kBlk) return false;
  if (p.dtype != SPARTA_F16 && p.dtype != SPARTA_BF16) return false;
  const DsdView v = dsd_view(p);
  if (v.M % kTileM || v.K % kBlk || v.N % kBlk) return false;
  if (v.K / kBlk > kMaxKb || v.N / kBlk > 0xffff || p.n_index_sets != 1 || p.val_stride_blocks <= 0) return false;
  if ((long long)p.batch * p.val_stride_blocks * kBlk > 0x7fffffffll) return false;
  if ((long long)p.batch * v.M > 0x7fffffffll || (long long)p.batch * v.N > 0x7fffffffll) return false;
  if (p.batch > 65535 || v.M / kTileM > 65535) return false;
  if (!aligned(p.A, 16) || !aligned(p.B, 16) || !aligned(p.C, 16)) return false;
  return true;
}

int dsd_tc_launch(const BsmmParams& p, cudaStream_t st) {
  // Panel width: narrower panels leave more tensor memory for activation tiles in flight and give more
  // CTAs, wider ones re-read the activations less.  Cost model: waves of CTAs x (a fixed part per CTA
  // + the panel's share of the blocks), fitted to the 4096^3 measurements (10 columns beat 12 by 4 %, 8
  // lost 17 %).
  const DsdView v = dsd_view(p);
  const long long tiles = (long long)(v.M / kTileM) * p.batch;
  int best = 12;
  long long best_cost = -1;
  for (int np : {12, 10, 8}) {
    const long long ctas = (long long)((v.N / kBlk + np - 1) / np) * tiles;
    const long long cost = ((ctas + kNumSMs - 1) / kNumSMs) * (6 + np);
    if (best_cost < 0 || cost < best_cost) { best = np; best_cost = cost; }
  }
  // sparse masks (few W blocks per step) take the variant with a fourth X slot, see x_slots()
  const double density = (double)p.val_stride_blocks / ((double)(v.N / kBlk) * (double)(v.K / kBlk));
  const bool deep_x = best <= 10 && density <= 0.15;
  const bool h = p.dtype == SPARTA_F16;
  switch (best) {
    case 8:
      if (deep_x) return h ? launch_dsd_tc<0, 8, true>(p, v, st) : launch_dsd_tc<1, 8, true>(p, v, st);
      return h ? launch_dsd_tc<0, 8, false>(p, v, st) : launch_dsd_tc<1, 8, false>(p, v, st);
    case 10:
      if (deep_x) return h ? launch_dsd_tc<0, 10, true>(p, v, st) : launch_dsd_tc<1, 10, true>(p, v, st);
      return h ? launch_dsd_tc<0, 10, false>(p, v, st) : launch_dsd_tc<1, 10, false>(p, v, st);
    default: return h ? launch_dsd_tc<0, 12, false>(p, v, st) : launch_dsd_tc<1, 12, false>(p, v, st);
  }
}

}  // namespace sparta
