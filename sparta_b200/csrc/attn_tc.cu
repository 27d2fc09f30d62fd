// Fused block-sparse attention forward on tcgen05 / TMEM / TMA (fp16 / bf16, head dim 64 or 128,
// 64 x 64 mask blocks):  O = softmax_mask(Q K^T * scale) V  over the kept blocks only.  The score
// matrix lives in tensor memory and registers; it is never written to global memory.
//
// Replaces the three launches of SparseAttention.forward
// (sparta/specializer/operators/sparse_attention.py:76-80): dds(Q, K^T) -> sparse softmax -> sdd(P, V).
//
// One CTA owns a 128-row Q tile = two block rows of the mask.  Its prologue merges the BCSR lists of
// the two rows into a sorted list of K blocks with two presence bits each; K blocks are then taken
// two at a time, so that both contractions run as full-width instructions:
//   S[128, 128] = Q[128, D] . [K_a; K_b]^T           (tcgen05.mma M128 N128, D/16 of them)
//   P = exp2(S * scale * log2e - m)  in registers, masked per row half and per element, -> tensor memory
//   O[128, D] += P[128, 128] . [V_a; V_b]             (tcgen05.mma M128 N=D, A = P from tensor memory,
//                                                      B operand MN-major in shared memory)
// The scores of a step are read from tensor memory once and stay in registers between the row-maximum pass
// and the exponential pass, so the score buffer is released right after the read; P goes back to tensor
// memory with one tcgen05.st per thread (no shared-memory round trip, no proxy fence), which also takes
// the 4 KB A-operand read of every P.V instruction off the shared-memory port (with D = 64 that read made
// the instruction take 48 cycles for 32 cycles of math).
// Warps: 0-7 softmax (two threads per row, one for each K block of the pair; online max / sum with a
// lazy rescale of O: the running max is only raised when it grows by more than 8 in log2 units), 8 TMA
// producer, 9 issues the Q.K^T MMAs, 10 issues the P.V MMAs.  All mbarrier waits are bounded (status words of sparta_last_status).
#include <type_traits>

#include "bsmm.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

using namespace tc;

constexpr int kBlk = 64;       // mask block edge
constexpr int kTileM = 128;    // Q rows per CTA
constexpr int kPair = 128;     // keys per step (two blocks)
constexpr int kSoftmaxWarps = 8;  // two per tensor-memory lane quadrant: one for each K block of a pair
constexpr int kWarpLoad = kSoftmaxWarps, kWarpQK = kSoftmaxWarps + 1, kWarpPV = kSoftmaxWarps + 2;
constexpr int kThreads = 32 * (kSoftmaxWarps + 3);
constexpr int kMaxKb = 1024;   // K blocks per row (Ns <= 65536)
constexpr float kRescaleThreshold = 8.f;

// 2^x by the special-function unit alone.  exp2f() wraps the same instruction in a range fix for
// results below the normal range (a compare, two multiplies); probabilities that small round to zero
// in fp16 / bf16 anyway, and the softmax warps are bound by the number of instructions they issue.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnParams {
  const int32_t* row_ptr;
  const int32_t* idx;
  const uint8_t* mask;  // [Nt, Ns] element mask or null
  void* O;
  float* lse;
  int Nt, Ns, heads;
  int grouped;          // launch order, see the kernel
  float scale_log2;     // scale * log2(e)
  int32_t* status;
};

template <int D>
struct Cfg {
  static constexpr int kSBuf = D == 64 ? 1 : 2;      // score buffers in tensor memory
  static constexpr int kKStages = 2;
  static constexpr int kVStages = 2;
  static constexpr int kChunks = D / 64;             // 64-element (128-byte) chunks of the head dim
  static constexpr int kQBytes = kTileM * D * 2;
  static constexpr int kKVBytes = kPair * D * 2;     // one stage: two blocks
  // tensor memory columns: scores (128 per buffer), the output accumulator (D), the probabilities as 16-bit
  // pairs (64): 256 columns for D = 64 (two CTAs share an SM), 512 for D = 128
  static constexpr uint32_t kTmemCols = D == 64 ? 256 : 512;
  static constexpr uint32_t kOCol = kSBuf * kPair;
  static constexpr uint32_t kPCol = kOCol + D;
  static_assert(kPCol + kPair / 2 <= kTmemCols, "tensor memory budget");
  static constexpr int kListBytes = kMaxKb * 2 + kMaxKb;  // ulist (uint16) + kmask (uint8)
  static constexpr int kSmem = kQBytes + (kKStages + kVStages) * kKVBytes + kListBytes + 512 + 1024;
};

template <int D, int FMT>
__global__ void __launch_bounds__(kThreads, D == 64 ? 2 : 1)  // D = 64: two CTAs per SM, 88 registers
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, AttnParams p) {
  using T = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
  using C = Cfg<D>;
  constexpr int kSBuf = C::kSBuf, kKStages = C::kKStages, kVStages = C::kVStages, kChunks = C::kChunks;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + C::kQBytes;
  uint8_t* v_s = k_s + kKStages * C::kKVBytes;
  uint16_t* ulist = reinterpret_cast<uint16_t*>(v_s + kVStages * C::kKVBytes);  // (K block << 2) | presence bits
  uint8_t* kmask = reinterpret_cast<uint8_t*>(ulist + kMaxKb);
  uint8_t* ctl = kmask + kMaxKb;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctl);
  uint64_t* k_full = q_full + 1;             // [kKStages]
  uint64_t* k_empty = k_full + kKStages;     // [kKStages]
  uint64_t* v_full = k_empty + kKStages;     // [kVStages]
  uint64_t* v_empty = v_full + kVStages;     // [kVStages]
  uint64_t* s_full = v_empty + kVStages;     // [kSBuf]
  uint64_t* s_empty = s_full + kSBuf;        // [kSBuf]
  uint64_t* p_full = s_empty + kSBuf;        // [1]
  uint64_t* pv_done = p_full + 1;            // [1]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 1);
  int* s_count = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_range = s_count + 1;                // [2]

  __shared__ float s_xchg[2][2][kTileM];  // [step parity][K block of the pair][row]: row maxima of the two threads of a row
  __shared__ float s_lsum[2][kTileM];     // their partial row sums, at the end
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Launch order (see attn_tc2.cu): grouped by head when the K / V of all heads exceed L2, else head-major
  const int tiles_per_head = p.Nt / kTileM;
  int head, tile;
  if (!p.grouped) {
    tile = blockIdx.x / p.heads;
    head = blockIdx.x - tile * p.heads;
  } else if (static_cast<int>(blockIdx.x) < p.heads) {
    head = blockIdx.x; tile = 0;
  } else {
    const int i = blockIdx.x - p.heads;
    head = i / (tiles_per_head - 1);
    tile = 1 + (i - head * (tiles_per_head - 1));
  }
  const int br0 = tile * 2;
  const int ncb = p.Ns / kBlk;

  // ------------------------------ prologue ------------------------------
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kKStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < kVStages; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int s = 0; s < kSBuf; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], kSoftmaxWarps); }
    mbar_init(p_full, kSoftmaxWarps);
    mbar_init(pv_done, 1);
    fence_mbar_init();
    s_range[0] = p.row_ptr[br0];
    s_range[1] = p.row_ptr[br0 + 2];
  }
  if (warp == kWarpLoad && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == kWarpQK) tmem_alloc<C::kTmemCols>(tmem_holder);
  for (int k = threadIdx.x; k < ncb; k += kThreads) kmask[k] = 0;
  __syncthreads();
  // the two block rows are consecutive in the BCSR array: entry = (block row << 16) | K block
  for (int e = s_range[0] + threadIdx.x; e < s_range[1]; e += kThreads) {
    const int v = __ldg(p.idx + e);
    const int kb = v & 0xffff, r = (v >> 16) - br0;
    if (kb < ncb && r >= 0 && r < 2)  // index arrays come from the caller: never index shared memory with them unchecked
      atomicOr(reinterpret_cast<unsigned int*>(kmask + (kb & ~3)), (1u << r) << (8 * (kb & 3)));
  }
  __syncthreads();
  if (warp == 0) {  // ordered compaction of the merged list
    int n = 0;
    for (int base = 0; base < ncb; base += 32) {
      const int k = base + lane;
      const int m = k < ncb ? kmask[k] : 0;
      const unsigned bal = __ballot_sync(0xffffffffu, m != 0);
      if (m) ulist[n + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>((k << 2) | m);
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
  const long long q_row0 = (long long)head * p.Nt + (long long)tile * kTileM;
  const long long kv_row0 = (long long)head * p.Ns;

  bool failed = false;  // a bounded wait of this thread gave up
  if (warp == kWarpLoad) {
    // ------------------------------ producer ------------------------------
    if (lane == 0 && count > 0) {
      mbar_arrive_expect_tx(q_full, C::kQBytes);
      for (int c = 0; c < kChunks; ++c)
        tma_load_2d(q_s + c * (kTileM * 128), &tm_q, c * 64, (int)q_row0, q_full);
      bool ok = true;
      for (int j = 0; j < npairs && ok; ++j) {
        const int nblk = min(2, count - 2 * j);
        const int ks = j % kKStages, vs = j % kVStages;
        if (!mbar_wait(&k_empty[ks], ((j / kKStages) & 1) ^ 1)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[ks], nblk * kBlk * D * 2);
        for (int b = 0; b < nblk; ++b) {
          const int kb = ulist[2 * j + b] >> 2;
          for (int c = 0; c < kChunks; ++c)
            tma_load_2d(k_s + ks * C::kKVBytes + c * (kPair * 128) + b * (kBlk * 128), &tm_k, c * 64,
                        (int)(kv_row0 + (long long)kb * kBlk), &k_full[ks]);
        }
        if (!mbar_wait(&v_empty[vs], ((j / kVStages) & 1) ^ 1)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[vs], nblk * kBlk * D * 2);
        for (int b = 0; b < nblk; ++b) {
          const int kb = ulist[2 * j + b] >> 2;
          for (int c = 0; c < kChunks; ++c)
            tma_load_2d(v_s + vs * C::kKVBytes + c * (kPair * 128) + b * (kBlk * 128), &tm_v, c * 64,
                        (int)(kv_row0 + (long long)kb * kBlk), &v_full[vs]);
        }
      }
      failed |= !ok;
      if (!ok) atomicExch(&p.status[0], 1);
    }
  } else if (warp == kWarpQK) {
    // ------------------------------ S = Q K^T ------------------------------
    const uint64_t desc_hi = make_smem_desc(0, 16, 1024, SW_128B);
    const uint32_t q_lo = smem_u32(q_s) >> 4, k_lo = smem_u32(k_s) >> 4;
    bool ok = count == 0 || mbar_wait(q_full, 0);
    for (int j = 0; j < npairs && ok; ++j) {
      const int nblk = min(2, count - 2 * j);
      const int ks = j % kKStages, sb = j % kSBuf;
      if (!mbar_wait(&k_full[ks], (j / kKStages) & 1)) { ok = false; break; }
      if (!mbar_wait(&s_empty[sb], ((j / kSBuf) & 1) ^ 1)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t idesc = make_idesc_f16(kTileM, nblk * kBlk, FMT, 0, 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * (kTileM * 128) + (kk % 4) * 32) >> 4;  // kTileM == kPair
          umma_ss(tmem_base + sb * kPair, desc_hi | (q_lo + off),
                  desc_hi | (k_lo + ((ks * C::kKVBytes) >> 4) + off), idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        umma_commit(&k_empty[ks]);
      }
      __syncwarp();
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[1], 1);
  } else if (warp == kWarpPV) {
    // ------------------------------ O += P V ------------------------------
    // P: A operand in tensor memory, lane = row, two 16-bit probabilities per column, keys in order (eight
    // columns per K = 16 slab); V: MN-major (head dim contiguous), 8 keys per 1024-byte group, 64-element
    // chunks of the head dim kPair * 128 bytes apart.
    const uint64_t v_desc_hi = make_smem_desc(0, kPair * 128, 1024, SW_128B);
    const uint32_t v_lo = smem_u32(v_s) >> 4;
    constexpr uint32_t idesc = make_idesc_f16(kTileM, D, FMT, 0, 1);
    bool ok = true;
    for (int j = 0; j < npairs && ok; ++j) {
      const int nblk = min(2, count - 2 * j);
      const int vs = j % kVStages;
      if (!mbar_wait(&v_full[vs], (j / kVStages) & 1)) { ok = false; break; }
      if (!mbar_wait(p_full, j & 1)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        for (int kk = 0; kk < nblk * (kBlk / 16); ++kk) {
          const uint32_t b_off = (vs * C::kKVBytes + kk * 16 * 128) >> 4;
          umma_ts(tmem_base + C::kOCol, tmem_base + C::kPCol + kk * 8, v_desc_hi | (v_lo + b_off), idesc,
                  (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[vs]);
        umma_commit(pv_done);
      }
      __syncwarp();
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[2], 1);
  } else {
    // ------------------------------ softmax + epilogue (warps 0-7) ------------------------------
    // Two threads per row: warp w and warp w + 4 share a tensor-memory lane quadrant; the first takes
    // the first K block of a pair (score columns 0-63), the second the other one.  They exchange their
    // row maxima through shared memory once per step, keep partial row sums, and split the columns of O
    // when it is rescaled or written out.  A single warp runs this instruction stream at one
    // instruction per several cycles, and it sits in the chain QK^T -> softmax -> P V of every step.
    // Every thread passes the same named barriers whatever happens: after a wait has given up it only
    // keeps the barrier count.
    const int quad = warp & 3, colhalf = warp >> 2;
    const int row = quad * 32 + lane;          // row of the Q tile == TMEM lane
    const int half = row >> 6;                 // which of the two block rows
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const long long grow = (long long)tile * kTileM + row;  // row inside the head
    constexpr int kOChunks = D / 64;           // 32-column chunks of O per thread
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < npairs; ++j) {
      const int nblk = min(2, count - 2 * j);
      const int sb = j % kSBuf;
      const int e = colhalf < nblk ? ulist[2 * j + colhalf] : 0;
      const bool mine = (e >> half) & 1;       // this thread's block is kept in its block row (warp-uniform)
      const int kb = e >> 2;
      const uint32_t s_addr = tmem_base + lane_base + sb * kPair + colhalf * kBlk;
      // ---- the 64 scores of this thread's block: masked elements set to -inf, row maximum.  With D = 128
      // (one CTA per SM, registers to spare) they are read once and stay in registers, and the score buffer
      // is released here; with D = 64 (two CTAs per SM, 80 registers) they are read again for the second pass
      constexpr bool kHold = D == 128;
      uint32_t r[kHold ? 64 : 32];
      float mx = -INFINITY;
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
      if (ok) {
        if (!mbar_wait_warp(&s_full[sb], (j / kSBuf) & 1)) {
          ok = false;
        } else {
          tc_fence_after_sync();
          if (mine) {
            if constexpr (kHold) {
              tmem_ld_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
              tmem_ld_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
              tmem_ld_wait();
              if (p.mask) { mask_scores(&r[0], 0); mask_scores(&r[32], 1); }
              {  // four independent chains: one chain of 64 dependent maxima would cost ~300 cycles of latency
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[i]));
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
              }
            } else {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                tmem_ld_x32(s_addr + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                tmem_ld_wait();
                if (p.mask) mask_scores(&r[0], h);
                {
                  float m4[4] = {mx, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                  for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[i]));
                  mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                }
              }
            }
          }
          if constexpr (kHold) {  // the scores are in registers: the buffer may take the next S
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[sb]);
          }
        }
      }
      s_xchg[j & 1][colhalf][row] = mx;
      named_barrier_sync(1, kSoftmaxWarps * 32);
      if (!ok) continue;
      mx = fmaxf(mx, s_xchg[j & 1][colhalf ^ 1][row]);
      const float m_new = mx * p.scale_log2;  // scale > 0
      // ---- lazy rescale of the running state ----
      float alpha = 1.f;
      if (m_new > m_run + kRescaleThreshold || (m_run == -INFINITY && m_new > -INFINITY)) {
        alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
        m_run = m_new;
        l_run *= alpha;
      }
      // previous P V must be finished before P is overwritten or O is rescaled
      if (j > 0 && !mbar_wait_warp(pv_done, (j - 1) & 1)) { ok = false; continue; }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {  // the partner warp sees the same alphas and takes the other columns
        tc_fence_after_sync();
#pragma unroll
        for (int c = colhalf * kOChunks; c < (colhalf + 1) * kOChunks; ++c) {
          uint32_t o[32];
          tmem_ld_x32(tmem_base + lane_base + C::kOCol + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(tmem_base + lane_base + C::kOCol + c * 32, o);
        }
      }
      // ---- P = exp2(S * scale * log2e - m) as 16-bit pairs -> tensor memory (this thread's 32 columns) ----
      if (colhalf < nblk) {  // this thread's block of the pair (warp-uniform)
        // every score of this row masked so far: subtracting +inf makes every probability zero
        const float neg_m = m_run > -INFINITY ? -m_run : -INFINITY;
        float sum = 0.f, sum1 = 0.f;
        auto exp_pack = [&](const uint32_t* v, uint32_t* out) {  // 32 scores -> 16 packed pairs (out may be v)
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, neg_m));
            const float p1 = ex2_approx(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, neg_m));
            // the row sum takes the fp32 probabilities: their rounding to 16 bits for P V is unbiased, and
            // converting them back cost two instructions per pair in warps bound by instruction issue
            // (two alternating partial sums keep the additions from forming one dependent chain)
            if (i & 1) sum1 += p0 + p1; else sum += p0 + p1;
            if constexpr (FMT == 0) {
              const __half2 hv = __floats2half2_rn(p0, p1);
              out[i] = *reinterpret_cast<const uint32_t*>(&hv);
            } else {
              const __nv_bfloat162 hv = __floats2bfloat162_rn(p0, p1);
              out[i] = *reinterpret_cast<const uint32_t*>(&hv);
            }
          }
        };
        const uint32_t p_addr = tmem_base + lane_base + C::kPCol + colhalf * (kBlk / 2);
        if constexpr (kHold) {
          if (mine) {
            exp_pack(&r[0], &r[0]);
            exp_pack(&r[32], &r[16]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0;
          }
          tmem_st_x32(p_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t packed[16];
            if (mine) {
              tmem_ld_x32(s_addr + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
              tmem_ld_wait();
              if (p.mask) mask_scores(&r[0], h);
              exp_pack(&r[0], packed);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) packed[i] = 0;
            }
            tmem_st_x16(p_addr + h * 16, packed);
          }
        }
        l_run += sum + sum1;
      }
      tmem_st_wait();  // P and a rescaled O are in tensor memory
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (!kHold) mbar_arrive(&s_empty[sb]);  // S may be overwritten
        mbar_arrive(p_full);
      }
    }
    // ---- epilogue: O / l -> global ----
    if (ok && npairs > 0 && !mbar_wait_warp(pv_done, (npairs - 1) & 1)) ok = false;
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[3], 1);
    tc_fence_after_sync();
    s_lsum[colhalf][row] = l_run;  // the row sum is the two threads' partial sums
    named_barrier_sync(1, kSoftmaxWarps * 32);
    l_run += s_lsum[colhalf ^ 1][row];
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* orow = static_cast<T*>(p.O) + (q_row0 + row) * D;
#pragma unroll
    for (int c = colhalf * kOChunks; c < (colhalf + 1) * kOChunks; ++c) {
      uint32_t r[32];
      if (npairs > 0 && ok) {
        tmem_ld_x32(tmem_base + lane_base + C::kOCol + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0;
      }
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float v0 = __uint_as_float(r[2 * i]) * inv, v1 = __uint_as_float(r[2 * i + 1]) * inv;
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
    }
    if (p.lse && colhalf == 0) {
      // natural-log sum of exponentials of the scaled scores (-inf for a fully masked row)
      p.lse[(long long)head * p.Nt + grow] = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc_fence_before_sync();
  sync_and_drain(failed);
  if (warp == kWarpQK) {
    tc_fence_after_sync();
    tmem_dealloc<C::kTmemCols>(tmem_base);
  }
}

template <int D, int FMT>
int launch_attn(const void* Q, const void* K, const void* V, const AttnParams& p, int dtype, cudaStream_t st) {
  using C = Cfg<D>;
  CUtensorMap tm_q, tm_k, tm_v;
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
  auto kern = attn_fwd_tc_kernel<D, FMT>;
  static SmemAttrOnce attr;
  if (cudaError_t e = attr.ensure(kern, C::kSmem); e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((unsigned)((long long)p.heads * (p.Nt / kTileM)));
  kern<<<grid, kThreads, C::kSmem, st>>>(tm_q, tm_k, tm_v, p);
  return launch_status();
}

}  // namespace

bool attn_tc_available() { return true; }

}  // namespace sparta

using namespace sparta;

extern "C" size_t sparta_attn_fwd_workspace_bytes(int, int, int, int, int) { return 0; }

namespace {
int attn_fwd_entry(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                   const int32_t* bcsr_idx, const uint8_t* mask, float scale, int heads, int Nt, int Ns, int D,
                   int BLK, int dtype, float* lse, int32_t* status, void* const* copies, int n_copies, void* stream);
}

extern "C" int sparta_attn_fwd(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                               const int32_t* bcsr_idx, const int32_t* nnz, const uint8_t* mask, float scale,
                               int heads, int Nt, int Ns, int D, int BLK, int dtype, float* lse,
                               int32_t* status, void* workspace, size_t workspace_bytes, void* stream) {
  (void)nnz; (void)workspace; (void)workspace_bytes;
  return attn_fwd_entry(Q, K, V, O, row_ptr, bcsr_idx, mask, scale, heads, Nt, Ns, D, BLK, dtype, lse, status, nullptr, 0,
                        stream);
}

extern "C" int sparta_attn_fwd_gather(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                                      const int32_t* bcsr_idx, const int32_t* nnz, const uint8_t* mask, float scale,
                                      int heads, int Nt, int Ns, int D, int BLK, int dtype, float* lse,
                                      int32_t* status, void* const* copies, int n_copies, void* stream) {
  (void)nnz;
  if (n_copies < 0 || n_copies > SPARTA_ATTN_MAX_COPIES || (n_copies > 0 && !copies)) return SPARTA_ERR_BAD_ARG;
  return attn_fwd_entry(Q, K, V, O, row_ptr, bcsr_idx, mask, scale, heads, Nt, Ns, D, BLK, dtype, lse, status, copies,
                        n_copies, stream);
}

namespace {
int attn_fwd_entry(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                   const int32_t* bcsr_idx, const uint8_t* mask, float scale, int heads, int Nt, int Ns, int D,
                   int BLK, int dtype, float* lse, int32_t* status, void* const* copies, int n_copies, void* stream) {
  if (!Q || !K || !V || !O || !row_ptr || !bcsr_idx || heads <= 0 || Nt <= 0 || Ns <= 0) return SPARTA_ERR_BAD_ARG;
  if (dtype != SPARTA_F16 && dtype != SPARTA_BF16) return SPARTA_ERR_UNSUPPORTED;
  if (BLK != kBlk || (D != 64 && D != 128)) return SPARTA_ERR_UNSUPPORTED;
  if (Nt % kTileM || Ns % kBlk) return SPARTA_ERR_SHAPE;
  if (Ns / kBlk > kMaxKb || Nt / kTileM > 65535 || !(scale > 0.f)) return SPARTA_ERR_UNSUPPORTED;
  if ((long long)heads * Nt > 0x7fffffffll || (long long)heads * Ns > 0x7fffffffll) return SPARTA_ERR_SHAPE;
  if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16) || !aligned(O, 16)) return SPARTA_ERR_ALIGN;
  if (mask && (!aligned(mask, 16) || Ns % 16)) return SPARTA_ERR_ALIGN;
  AttnParams p;
  p.row_ptr = row_ptr; p.idx = bcsr_idx; p.mask = mask; p.O = O; p.lse = lse;
  p.Nt = Nt; p.Ns = Ns; p.heads = heads;
  p.grouped = kv_exceeds_l2(heads, Ns, D);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status ? status : tc::device_status_ptr();
  if (!p.status) return SPARTA_ERR_DRIVER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // D = 128: two Q tiles per CTA sharing the K / V tiles (attn_tc2.cu), when the query length allows it.  D = 64
  // stays with one tile per CTA and two CTAs per SM, which measured 25 % faster than the two-tile form there.
  if (D == 128 && attn_tc2_supported(Nt))
    return attn_tc2_launch(Q, K, V, O, row_ptr, bcsr_idx, mask, p.scale_log2, heads, Nt, Ns, D, dtype, lse, p.status,
                           copies, n_copies, st);
  if (n_copies > 0) return SPARTA_ERR_UNSUPPORTED;  // the one-tile kernels store O only
#ifndef SPARTA_ATTN64_TWO_BLOCKS
  if (D == 64)
    return attn_tc64_launch(Q, K, V, O, row_ptr, bcsr_idx, mask, p.scale_log2, heads, Nt, Ns, dtype, lse, p.status, st);
#endif
  const int fmt = dtype == SPARTA_F16 ? 0 : 1;
  if (D == 64) return fmt == 0 ? launch_attn<64, 0>(Q, K, V, p, dtype, st) : launch_attn<64, 1>(Q, K, V, p, dtype, st);
  return fmt == 0 ? launch_attn<128, 0>(Q, K, V, p, dtype, st) : launch_attn<128, 1>(Q, K, V, p, dtype, st);
}
}  // namespace
