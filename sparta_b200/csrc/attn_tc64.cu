// Fused block-sparse attention forward for head dim 64 (fp16 / bf16, 64 x 64 mask blocks), one K block per step
// and four CTAs per SM.
//
// The step of a fused attention tile is a chain -- S = Q K^T, softmax of S, O += P V, next S -- whose links cannot
// overlap inside one tile, so the units stay busy only as far as several tiles are in flight on an SM.  The
// two-block form (attn_tc.cu) needs 256 tensor-memory columns per tile, which is two tiles per SM; for D = 64 its
// tensor pipe was a quarter busy.  Here a step is ONE K block: 64 score columns (the probabilities, as 16-bit
// pairs, go back into the first 32 of them) beside the 64 columns of O make 128 columns per CTA, a row's 64 scores
// are one thread's work (no exchange of row maxima between threads, no partial sums), shared memory holds Q and
// two stages of one K and one V block (52 KB), and four CTAs share an SM.
//   warps 0-3  softmax + epilogue: thread = row of the Q tile = tensor-memory lane
//   warp 4     TMA producer (Q once, then K and V block by block)
//   warp 5     one thread issues every MMA: P V of step j, then Q K^T of step j + 1.  MMAs of one thread execute
//              in issue order, so the next scores cannot overwrite the probabilities before P V has read them, and
//              "scores complete" also means that O is quiet (the softmax warps may rescale it).
// Replaces the three launches of SparseAttention.forward (sparta/specializer/operators/sparse_attention.py:76-80).
#include <type_traits>

#include "bsmm.cuh"
#include "tc_common.cuh"

namespace sparta {
namespace {

using namespace tc;

constexpr int kBlk = 64;       // mask block edge = keys per step
constexpr int kTileM = 128;    // Q rows per CTA (two block rows)
constexpr int kD = 64;         // head dim
constexpr int kSmWarps = 4;
constexpr int kWarpLoad = kSmWarps, kWarpMma = kSmWarps + 1;
constexpr int kThreads = 32 * (kSmWarps + 2);
constexpr int kStages = 2;
constexpr int kCtasPerSM = 4;   // 80 registers: the scores are read again for the second pass
constexpr bool kHold = false;   // (three CTAs per SM with the 64 scores held in 112 registers measured 0.272 ms against 0.194 ms)
constexpr int kMaxKb = 1024;   // K blocks per row (Ns <= 65536)
constexpr float kRescaleThreshold = 8.f;
constexpr int kQBytes = kTileM * kD * 2;   // 16 KB
constexpr int kKVBytes = kBlk * kD * 2;    // 8 KB per block
constexpr uint32_t kTmemCols = 128;        // scores / probabilities 0..63, O 64..127
constexpr uint32_t kOCol = 64;
constexpr int kSmem = kQBytes + 2 * kStages * kKVBytes + kMaxKb * 3 + 512 + 1024;

struct Attn64Params {
  const int32_t* row_ptr;
  const int32_t* idx;
  const uint8_t* mask;  // [Nt, Ns] element mask or null
  void* O;
  float* lse;
  int Nt, Ns, heads;
  int grouped;          // launch order: tiles of a head together when K / V of all heads exceed L2
  float scale_log2;     // scale * log2(e)
  int32_t* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int FMT>
__global__ void __launch_bounds__(kThreads, kCtasPerSM)
attn_fwd_tc64_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, Attn64Params p) {
  using T = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + kQBytes;
  uint8_t* v_s = k_s + kStages * kKVBytes;
  uint16_t* ulist = reinterpret_cast<uint16_t*>(v_s + kStages * kKVBytes);  // (K block << 2) | presence bits of the two block rows
  uint8_t* kmask = reinterpret_cast<uint8_t*>(ulist + kMaxKb);
  uint8_t* ctl = kmask + kMaxKb;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctl);
  uint64_t* k_full = q_full + 1;          // [kStages]
  uint64_t* k_empty = k_full + kStages;   // [kStages]
  uint64_t* v_full = k_empty + kStages;   // [kStages]
  uint64_t* v_empty = v_full + kStages;   // [kStages]
  uint64_t* s_full = v_empty + kStages;   // scores of a step complete (and every earlier MMA)
  uint64_t* p_full = s_full + 1;          // probabilities of a step in tensor memory
  uint64_t* pv_done = p_full + 1;         // last P V complete
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 1);
  int* s_count = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_range = s_count + 1;             // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, kSmWarps);
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
  if (warp == kWarpMma) tmem_alloc<kTmemCols>(tmem_holder);
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
  const int count = *s_count;  // steps
  const long long q_row0 = (long long)head * p.Nt + (long long)tile * kTileM;
  const long long kv_row0 = (long long)head * p.Ns;

  bool failed = false;  // a bounded wait of this thread gave up
  if (warp == kWarpLoad) {
    // ------------------------------ producer ------------------------------
    if (lane == 0 && count > 0) {
      mbar_arrive_expect_tx(q_full, kQBytes);
      tma_load_2d(q_s, &tm_q, 0, (int)q_row0, q_full);
      bool ok = true;
      for (int j = 0; j < count && ok; ++j) {
        const int st = j % kStages;
        const uint32_t par = ((j / kStages) & 1) ^ 1;
        const int kb = ulist[j] >> 2;
        if (!mbar_wait(&k_empty[st], par)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[st], kKVBytes);
        tma_load_2d(k_s + st * kKVBytes, &tm_k, 0, (int)(kv_row0 + (long long)kb * kBlk), &k_full[st]);
        if (!mbar_wait(&v_empty[st], par)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[st], kKVBytes);
        tma_load_2d(v_s + st * kKVBytes, &tm_v, 0, (int)(kv_row0 + (long long)kb * kBlk), &v_full[st]);
      }
      failed |= !ok;
      if (!ok) atomicExch(&p.status[0], 1);
    }
  } else if (warp == kWarpMma) {
    // ------------------------------ MMA issue ------------------------------
    // Q, K: K-major, 128-byte rows, 128-byte swizzle.  P: A operand in tensor memory, lane = row, two 16-bit
    // probabilities per column, eight columns per K = 16 slab.  V: MN-major (head dim contiguous), eight keys per
    // 1024-byte group.
    const uint64_t desc_hi = make_smem_desc(0, 16, 1024, SW_128B);
    const uint64_t v_desc_hi = make_smem_desc(0, kBlk * 128, 1024, SW_128B);
    const uint32_t q_lo = smem_u32(q_s) >> 4, k_lo = smem_u32(k_s) >> 4, v_lo = smem_u32(v_s) >> 4;
    constexpr uint32_t idesc_qk = make_idesc_f16(kTileM, kBlk, FMT, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc_f16(kTileM, kD, FMT, 0, 1);
    auto issue_qk = [&](int st) {
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          umma_ss(tmem_base, desc_hi | (q_lo + 2 * kk), desc_hi | (k_lo + ((st * kKVBytes) >> 4) + 2 * kk), idesc_qk,
                  kk > 0 ? 1u : 0u);
        umma_commit(s_full);
        umma_commit(&k_empty[st]);
      }
      __syncwarp();
    };
    bool ok = count == 0 || (mbar_wait(q_full, 0) && mbar_wait(&k_full[0], 0));
    if (ok && count > 0) issue_qk(0);
    for (int j = 0; j < count && ok; ++j) {
      const int st = j % kStages;
      if (!mbar_wait(&v_full[st], (j / kStages) & 1)) { ok = false; break; }
      if (!mbar_wait(p_full, j & 1)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < kBlk / 16; ++kk)
          umma_ts(tmem_base + kOCol, tmem_base + kk * 8, v_desc_hi | (v_lo + ((st * kKVBytes + kk * 16 * 128) >> 4)),
                  idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&v_empty[st]);
        if (j + 1 == count) umma_commit(pv_done);
      }
      __syncwarp();
      if (j + 1 < count) {
        const int sn = (j + 1) % kStages;
        if (!mbar_wait(&k_full[sn], ((j + 1) / kStages) & 1)) { ok = false; break; }
        issue_qk(sn);
      }
    }
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[1], 1);
  } else {
    // ------------------------------ softmax + epilogue ------------------------------
    const int row = warp * 32 + lane;           // row of the Q tile == tensor-memory lane
    const int half = row >> 6;                  // which of the two block rows (warp-uniform)
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base;
    const long long grow = (long long)tile * kTileM + row;  // row inside the head
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < count; ++j) {
      const int e = ulist[j];
      const bool mine = (e >> half) & 1;        // the block is kept in this thread's block row (warp-uniform)
      const int kb = e >> 2;
      uint32_t r[kHold ? 64 : 32];
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
      if (ok && !mbar_wait_warp(s_full, j & 1)) ok = false;
      if (!ok) continue;
      tc_fence_after_sync();
      // ---- pass 1: row maximum over the block's 64 scores (read once when they fit the registers) ----
      float mx = -INFINITY;
      if (mine) {
        if constexpr (kHold) {
          tmem_ld_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_ld_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_ld_wait();
          if (p.mask) { mask_scores(&r[0], 0); mask_scores(&r[32], 1); }
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < 64; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[i]));
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            tmem_ld_x32(s_addr + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            tmem_ld_wait();
            if (p.mask) mask_scores(r, h);
            float m4[4] = {mx, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(r[i]));
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
          }
        }
      }
      const float m_new = mx * p.scale_log2;  // scale > 0
      // ---- lazy rescale of the running state (O is quiet: "scores complete" covers the previous P V) ----
      float alpha = 1.f;
      if (m_new > m_run + kRescaleThreshold || (m_run == -INFINITY && m_new > -INFINITY)) {
        alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
        m_run = m_new;
        l_run *= alpha;
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld_x32(s_addr + kOCol + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(s_addr + kOCol + c * 32, o);
        }
      }
      // ---- pass 2: P = exp2(S * scale * log2e - m) as 16-bit pairs into columns 0..31 (over scores already read) ----
      const float neg_m = m_run > -INFINITY ? -m_run : -INFINITY;  // all masked so far: every probability zero
      float sum = 0.f, sum1 = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t packed[16];
        if (mine) {
          if constexpr (!kHold) {
            tmem_ld_x32(s_addr + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            tmem_ld_wait();
            if (p.mask) mask_scores(r, h);
          }
          const uint32_t* v = kHold ? &r[32 * h] : &r[0];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, neg_m));
            const float p1 = ex2_approx(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, neg_m));
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
        // h = 0 writes columns 0..15 (scores 0..31 are consumed); h = 1 writes 16..31 after reading 32..63
        tmem_st_x16(s_addr + h * 16, packed);
      }
      l_run += sum + sum1;
      tmem_st_wait();  // P and a rescaled O are in tensor memory
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> global ----
    if (ok && count > 0 && !mbar_wait_warp(pv_done, 0)) ok = false;
    failed |= !ok;
    if (!ok && lane == 0) atomicExch(&p.status[3], 1);
    tc_fence_after_sync();
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* orow = static_cast<T*>(p.O) + (q_row0 + row) * kD;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
      if (count > 0 && ok) {
        tmem_ld_x32(s_addr + kOCol + c * 32, r);
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
    if (p.lse) p.lse[(long long)head * p.Nt + grow] = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
  }
  tc_fence_before_sync();
  sync_and_drain(failed);
  if (warp == kWarpMma) {
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

template <int FMT>
int launch_attn64(const void* Q, const void* K, const void* V, const Attn64Params& p, int dtype, cudaStream_t st) {
  CUtensorMap tm_q, tm_k, tm_v;
  const uint64_t strides[1] = {(uint64_t)kD * 2};
  {
    const uint64_t dims[2] = {(uint64_t)kD, (uint64_t)p.heads * p.Nt};
    const uint32_t box[2] = {64, kTileM};
    int rc = make_tensor_map(&tm_q, Q, dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)kD, (uint64_t)p.heads * p.Ns};
    const uint32_t box[2] = {64, kBlk};
    int rc = make_tensor_map(&tm_k, K, dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
    rc = make_tensor_map(&tm_v, V, dtype, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SPARTA_OK) return rc;
  }
  auto kern = attn_fwd_tc64_kernel<FMT>;
  static SmemAttrOnce attr;
  if (cudaError_t e = attr.ensure(kern, kSmem); e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((unsigned)((long long)p.heads * (p.Nt / kTileM)));
  kern<<<grid, kThreads, kSmem, st>>>(tm_q, tm_k, tm_v, p);
  return launch_status();
}

}  // namespace

int attn_tc64_launch(const void* Q, const void* K, const void* V, void* O, const int32_t* row_ptr,
                     const int32_t* bcsr_idx, const uint8_t* mask, float scale_log2, int heads, int Nt, int Ns,
                     int dtype, float* lse, int32_t* status, cudaStream_t st) {
  Attn64Params p;
  p.row_ptr = row_ptr; p.idx = bcsr_idx; p.mask = mask; p.O = O; p.lse = lse;
  p.Nt = Nt; p.Ns = Ns; p.heads = heads;
  p.grouped = kv_exceeds_l2(heads, Ns, kD);
  p.scale_log2 = scale_log2;
  p.status = status;
  return dtype == SPARTA_F16 ? launch_attn64<0>(Q, K, V, p, dtype, st) : launch_attn64<1>(Q, K, V, p, dtype, st);
}

}  // namespace sparta
