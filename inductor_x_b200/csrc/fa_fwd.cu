// Fused attention forward for sm_100a: softmax(Q K^T * scale [+ causal mask]) V with
// tcgen05 tensor-core MMAs, accumulators in tensor memory and operands brought in by TMA.
// It takes the place of the vendor kernel behind torch.ops.npu_graph.npu_fa
// (inductor_x/npu_fusion_attention_graph.py:20-35).
//
// One CTA owns two 128-row query tiles (A, B) of one (batch, head) and walks the
// key/value tiles (128 keys each) that they can see.  Eleven warps, four roles:
//   warp 0     TMA producer: Q once, then K_j / V_j into two-stage rings
//   warp 1     MMA issuer: S_t(j) = Q_t K_j^T into tile t's TMEM buffer, then
//              O_t += P_t(j) V_j with P read straight from TMEM (it overwrites S as 16-bit
//              values).  The two tiles alternate, so the tensor core works on one tile
//              while the other tile's softmax runs.
//   warps 2-5  softmax of tile A, warps 6-9 softmax of tile B: thread <-> query row.
//   warp 10    forwarder: waits for the K/V tiles of a step and adds its arrival to the
//              tiles' P barriers, so that the issuer makes one wait per tile and step
//              Pass 1 reads the S row for its maximum; pass 2 re-reads it 32 columns at
//              a time, exponentiates and writes P back.  The O accumulator is rescaled
//              only when the maximum has grown by more than 2^8 since the last rescale
//              (the final division by the running sum makes a stale reference exact).
// Hand-offs are mbarriers; every wait is bounded and a wait that gives up raises a flag in
// `status` and lets the CTA drain and exit.
//
// TMEM columns: [0,128) S/P of A, [128,256) S/P of B, [256,384) O of A, [384,512) O of B.
#include <atomic>
#include "host.h"
#include "fa_maps.h"
#include "ixb/tcgen05.cuh"

namespace {

using namespace ixb;

constexpr int BM = 128;          // rows of one query tile
constexpr int NQ = 2;            // query tiles per CTA
constexpr int BN = 128;          // keys per tile
constexpr int HD = 128;          // head dimension
constexpr int kStages = 2;  // (the issuer picks stage descriptors with two-way selects)
constexpr int kTileBytes = BN * HD * 2;     // one operand tile, 16-bit elements
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column TMA box of the tile
constexpr int kThreads = 64 + NQ * 128 + 32;  // producer, issuer, softmax warps, forwarder
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;  // + 128 * tile
constexpr float kRescaleThreshold = 8.f;    // log2 units
constexpr size_t kSmemBytes = (size_t)kTileBytes * (NQ + 2 * kStages) + 1024;

struct FaParams {
  void* o;
  float* lse;            // [B, H, Sq] natural-log sum of exponentials, may be null
  int* status;           // device word set to 1 if a wait gave up, may be null
  long long o_stride_b, o_stride_h, o_stride_s;  // elements
  int B, H, Sq, Sk;
  float scale_log2;      // softmax scale * log2(e), > 0
  int causal;
  int head_group;  // heads whose CTAs are dispatched together (see the CTA order in the kernel)
};

__device__ __forceinline__ uint32_t pack_pair(float lo, float hi, bool is_bf16) {
  if (is_bf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <bool IS_BF16>
__global__ void __launch_bounds__(kThreads, 1)
    fa_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const FaParams p) {
  extern __shared__ unsigned char smem_raw[];
  // operand tiles want 1024-byte alignment for the 128-byte swizzle
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_smem = smem;
  unsigned char* k_smem = smem + kTileBytes * NQ;
  unsigned char* v_smem = smem + kTileBytes * (NQ + kStages);

  __shared__ __align__(8) uint64_t q_full, k_full[kStages], k_empty[kStages], v_full[kStages],
      v_empty[kStages], s_full[NQ], p_full[NQ], pv_done[NQ];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // CTA order.  Heads are taken in groups of p.head_group (their K and V stay in L2 while the
  // group runs); inside a group the query blocks go from the last one to the first, all heads
  // of the group at each: under a causal mask the late blocks see the most keys, so the CTAs
  // still running when the grid drains are the short ones.
  const int n_q_blocks = (p.Sq + BM * NQ - 1) / (BM * NQ);
  const int n_bh = p.B * p.H;
  const int kHeadGroup = p.head_group;
  const int per_group = n_q_blocks * kHeadGroup;
  const int group = (int)blockIdx.x / per_group;
  const int in_group = (int)blockIdx.x - group * per_group;
  const int left = n_bh - group * kHeadGroup;
  const int g_heads = left < kHeadGroup ? left : kHeadGroup;
  const int q_block = n_q_blocks - 1 - in_group / g_heads;
  const int bh = group * kHeadGroup + in_group % g_heads;
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = q_block * BM * NQ;
  const int diag = p.Sk - p.Sq;  // key j is visible to query row i when j <= i + diag
  // number of key tiles each query tile walks (0 for a tile past the end of the sequence)
  int n_kv_t[NQ];
  int n_kv = 0;
#pragma unroll
  for (int t = 0; t < NQ; ++t) {
    const int qt0 = q0 + t * BM;
    int kv_end = p.Sk;
    if (p.causal) {
      const int lim = qt0 + BM + diag;
      kv_end = lim < p.Sk ? lim : p.Sk;
    }
    n_kv_t[t] = qt0 < p.Sq ? (kv_end + BN - 1) / BN : 0;
    n_kv = n_kv_t[t] > n_kv ? n_kv_t[t] : n_kv;
  }

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < NQ; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128 + 1);  // the rows of the tile and the forwarder
      mbar_init(&pv_done[t], 1);
    }
    failed = 0;
    mbar_init_fence();
  }
  if (warp == 1) tc::tmem_alloc(&tmem_base_slot, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_arrive_expect_tx(&q_full, kTileBytes * NQ);
#pragma unroll
      for (int t = 0; t < NQ; ++t) {
        // rows past the end of the tensor are zero-filled by the copy engine
        tc::tma_load_4d(q_smem + t * kTileBytes, &map_q, &q_full, 0, q0 + t * BM, h, b);
        tc::tma_load_4d(q_smem + t * kTileBytes + kHalfBytes, &map_q, &q_full, 64, q0 + t * BM, h, b);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % kStages, n = j / kStages;
        if (n > 0) ok = mbar_wait(&k_empty[s], (n - 1) & 1, &failed);
        if (!ok) break;
        unsigned char* kd = k_smem + (size_t)s * kTileBytes;
        mbar_arrive_expect_tx(&k_full[s], kTileBytes);
        tc::tma_load_4d(kd, &map_k, &k_full[s], 0, j * BN, h, b);
        tc::tma_load_4d(kd + kHalfBytes, &map_k, &k_full[s], 64, j * BN, h, b);
        if (n > 0) ok = mbar_wait(&v_empty[s], (n - 1) & 1, &failed);
        if (!ok) break;
        unsigned char* vd = v_smem + (size_t)s * kTileBytes;
        mbar_arrive_expect_tx(&v_full[s], kTileBytes);
        tc::tma_load_4d(vd, &map_v, &v_full[s], 0, j * BN, h, b);
        tc::tma_load_4d(vd + kHalfBytes, &map_v, &v_full[s], 64, j * BN, h, b);
      }
      if (!ok) failed = 1;
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::instr_desc(BM, BN, IS_BF16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_pv = tc::instr_desc(BM, HD, IS_BF16 ? 1 : 0, 0, 1);
      // S_t = Q_t K_j^T: both operands K-major, 8 steps of 16 along the head dimension;
      // a step moves 32 bytes inside the 128-byte swizzled row, 4 steps per 64-column box
      // Descriptors of the tile bases are formed once; a k-step only adds its byte offset
      // (in 16-byte units) to the address field, which cannot carry out of it.
      uint64_t q_desc[NQ], k_desc[kStages], v_desc[kStages];
#pragma unroll
      for (int t = 0; t < NQ; ++t) q_desc[t] = tc::smem_desc(smem_u32(q_smem + (size_t)t * kTileBytes), 16, 1024);
#pragma unroll
      for (int s = 0; s < kStages; ++s) {
        k_desc[s] = tc::smem_desc(smem_u32(k_smem + (size_t)s * kTileBytes), 16, 1024);
        v_desc[s] = tc::smem_desc(smem_u32(v_smem + (size_t)s * kTileBytes), kHalfBytes, 1024);
      }
      // (descriptors are picked with selects: an array indexed by the run-time stage would
      // live in local memory, and every load of it would sit on this thread's critical path)
      auto issue_qk = [&](int t, int stage) {
        const uint32_t d = tmem_base + kColS + t * 128;
        const uint64_t qd = t ? q_desc[1] : q_desc[0];
        const uint64_t kd = stage ? k_desc[1] : k_desc[0];
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
          tc::mma_ss(d, qd + off, kd + off, idesc_qk, ks > 0);
        }
      };
      // O_t += P_t V_j: A = P from TMEM (two 16-bit values per column, 8 columns per step),
      // B = V_j in MN-major form: 64 head-dim values (128 bytes) are contiguous, 8 keys
      // make one 1024-byte swizzle atom (stride-dimension offset), the second 64-column
      // box sits kHalfBytes further (leading-dimension offset); a step of 16 keys is two
      // atoms = 2048 bytes
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t a = tmem_base + kColS + t * 128;
        const uint32_t d = tmem_base + kColO + t * 128;
        const uint64_t vd = stage ? v_desc[1] : v_desc[0];
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          tc::mma_ts(d, a + ks * 8, vd + (uint32_t)(ks * 2048 >> 4), idesc_pv,
                     (accumulate || ks > 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(&q_full, 0, &failed);
      if (ok && n_kv > 0) ok = mbar_wait(&k_full[0], 0, &failed);
      if (ok && n_kv > 0) {
        tc::fence_after_sync();
#pragma unroll
        for (int t = 0; t < NQ; ++t) {
          if (n_kv_t[t] > 0) {
            issue_qk(t, 0);
            tc::mma_commit(&s_full[t]);
          }
        }
        tc::mma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1, n = j >> 1;
        const int s1 = (j + 1) & 1, n1 = (j + 1) >> 1;
#pragma unroll
        for (int t = 0; t < NQ; ++t) {
          // every wait of this tile's step comes first, so that its sixteen MMAs go to the
          // tensor core back to back and its queue does not drain in between
          const bool do_pv = j < n_kv_t[t], do_qk = j + 1 < n_kv_t[t];
          // one wait per tile and step: the forwarder warp has added its arrival to p_full
          // only after V_j and K_(j+1) landed, so this thread - for which every wait costs
          // about 240 cycles beside the busy softmax warps of the other tile - does not wait
          // for the operand rings itself
          if (do_pv) ok = ok && mbar_wait(&p_full[t], j & 1, &failed);
          if (!ok) break;
          tc::fence_after_sync();
          if (do_pv) {
            issue_pv(t, s, j > 0);
            // only the last product of the tile needs a signal of its own: every earlier one
            // is covered by the commit behind the scores that follow it (a commit tracks all
            // MMAs issued before it)
            if (!do_qk) tc::mma_commit(&pv_done[t]);
          }
          if (do_qk) {
            // P_t(j) has been consumed by the MMAs just issued (the tensor core runs
            // them in order), so tile t's buffer can take S_t(j+1)
            issue_qk(t, s1);
            tc::mma_commit(&s_full[t]);
          }
        }
        if (!ok) break;
        tc::mma_commit(&v_empty[s]);
        if (j + 1 < n_kv) tc::mma_commit(&k_empty[s1]);
      }
      if (!ok) failed = 1;
    }
    __syncwarp();
  } else if (warp == 2 + NQ * 4) {
    // ------------------------------------------------------------------ forwarder
    // Waits for the operand tiles of a step on behalf of the MMA issuer and adds one arrival
    // to p_full of every tile that has work in the step.
    if (lane == 0) {
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1, n = j >> 1;
        const int s1 = (j + 1) & 1, n1 = (j + 1) >> 1;
        ok = mbar_wait(&v_full[s], n & 1, &failed);
        if (ok && j + 1 < n_kv) ok = mbar_wait(&k_full[s1], n1 & 1, &failed);
        if (!ok) break;
#pragma unroll
        for (int t = 0; t < NQ; ++t)
          if (j < n_kv_t[t]) tc::mbar_arrive(&p_full[t]);
        // not ahead of the rows: the arrival for step j + 1 must not fall into phase j
#pragma unroll
        for (int t = 0; t < NQ; ++t)
          if (j < n_kv_t[t]) ok = ok && mbar_wait(&p_full[t], j & 1, &failed);
      }
      if (!ok) failed = 1;
    }
    __syncwarp();
  } else {
    // ----------------------------------------------------------- softmax + epilogue
    const int t = (warp - 2) >> 2;           // query tile of this warp group
    const int quad = warp & 3;               // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;        // row inside the query tile
    const int qt0 = q0 + t * BM;
    const int qi = qt0 + row;
    const int my_n_kv = n_kv_t[t];
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + kColS + t * 128;
    const uint32_t o_addr = lane_addr + kColO + t * 128;
    float m_used = -INFINITY;  // reference maximum (scaled, log2 domain)
    float l = 0.f;             // running sum of exp2(s - m_used)
    bool ok = true;

    for (int j = 0; j < my_n_kv; ++j) {
      if (!__all_sync(kFull, mbar_wait(&s_full[t], j & 1, &failed))) {
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const int col0 = j * BN;
      const bool edge = (col0 + BN > p.Sk) || (p.causal && (col0 + BN - 1 > qt0 + diag));
      // last visible key of this row, relative to the tile
      int lim = BN - 1;
      if (edge) {
        int last = p.Sk - 1;
        if (p.causal && qi + diag < last) last = qi + diag;
        lim = last - col0;
      }
      // ---- pass 1: row maximum of the raw scores, two 64-column round trips
      // (four independent chains: one chain of 64 dependent max3 would cost its latency 64 times)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t raw[64];
        tc::tmem_ld32(s_addr + hh * 64, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
        tc::tmem_ld32(s_addr + hh * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
        tc::tmem_wait_ld();
        if (edge) {
#pragma unroll
          for (int e = 0; e < 64; ++e)
            mx4[e & 3] = fmaxf(mx4[e & 3], (hh * 64 + e <= lim) ? __uint_as_float(raw[e]) : -INFINITY);
        } else {
#pragma unroll
          for (int e = 0; e < 64; e += 2)
            mx4[(e >> 1) & 3] = max3(mx4[(e >> 1) & 3], __uint_as_float(raw[e]), __uint_as_float(raw[e + 1]));
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= p.scale_log2;  // scale > 0: scaling commutes with the maximum
      // lazy rescale: move the reference maximum only when it would grow by > 2^8
      const bool grow = mx > m_used + kRescaleThreshold;  // also true for the first tile
      if (__any_sync(kFull, grow)) {
        const float m_new = grow ? mx : m_used;
        const float f = !grow ? 1.f : ((m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new));
        l *= f;
        if (j > 0) {
          // O may only be touched once O += P(j-1) V(j-1) has completed: it has - S(j),
          // which this warp has waited for, was committed behind it
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tc::tmem_ld32(o_addr + c * 32, o);
            tc::tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tc::tmem_st32(o_addr + c * 32, o);
          }
          tc::tmem_wait_st();
        }
        m_used = m_new;
      }
      // ---- pass 2: P = exp2(s * scale - m_used); the next 32 columns are requested
      // before the current 32 are processed so the TMEM latency overlaps the arithmetic
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(-mref, -mref);
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};  // two chains of packed adds
      uint32_t buf[2][32];
      tc::tmem_ld32(s_addr, buf[0]);
      tc::tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        const uint32_t(&raw)[32] = buf[c & 1];
        // P columns [16c, 16c+16) hold S columns that are already in registers, and the
        // prefetch below reads S columns [32c+32, 32c+64): no overlap with the store
        if (c + 1 < BN / 32) tc::tmem_ld32(s_addr + (c + 1) * 32, buf[(c + 1) & 1]);
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const int col = c * 32 + e;
          const float2 a =
              fma2(make_float2(__uint_as_float(raw[e]), __uint_as_float(raw[e + 1])), sc2, nm2);
          float2 pe = make_float2(fast_exp2(a.x), fast_exp2(a.y));
          if (edge) {
            if (col > lim) pe.x = 0.f;
            if (col + 1 > lim) pe.y = 0.f;
          }
          sum2[(e >> 1) & 1] = add2(sum2[(e >> 1) & 1], pe);
          pk[e / 2] = pack_pair(pe.x, pe.y, IS_BF16);
        }
        tc::tmem_wait_ld();
        tc::tmem_st16(s_addr + c * 16, pk);
      }
      l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      tc::tmem_wait_st();
      tc::fence_before_sync();
      tc::mbar_arrive(&p_full[t]);
    }

    if (ok && my_n_kv > 0) ok = mbar_wait(&pv_done[t], 0, &failed);  // the tile's last product
    ok = __all_sync(kFull, ok);
    if (ok) {
      tc::fence_after_sync();
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      const bool live = qi < p.Sq;
      unsigned char* orow = reinterpret_cast<unsigned char*>(p.o) +
                            2 * ((long long)b * p.o_stride_b + (long long)h * p.o_stride_h +
                                 (long long)qi * p.o_stride_s);
      if (my_n_kv > 0) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tc::tmem_ld32(o_addr + c * 32, o);
          tc::tmem_wait_ld();
          if (live) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 w;
              w.x = pack_pair(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv, IS_BF16);
              w.y = pack_pair(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv, IS_BF16);
              w.z = pack_pair(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv, IS_BF16);
              w.w = pack_pair(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv, IS_BF16);
              *reinterpret_cast<uint4*>(orow + (c * 32 + e) * 2) = w;
            }
          }
        }
        if (live && p.lse != nullptr) {
          const float lse = (l > 0.f) ? (m_used + log2f(l)) * 0.69314718055994530942f : -INFINITY;
          p.lse[((long long)b * p.H + h) * p.Sq + qi] = lse;
        }
      }
    } else {
      failed = 1;
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && failed && p.status != nullptr) atomicExch(p.status, 1);
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

extern "C" int ixb_fa_fwd(int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                          int32_t B, int32_t H, int32_t Sq, int32_t Sk, int32_t D,
                          const int64_t* q_strides, const int64_t* k_strides,
                          const int64_t* v_strides, const int64_t* o_strides, float scale,
                          int causal, int32_t* status, ixb_stream stream) {
  if (B < 0 || H < 0 || Sq < 0 || Sk < 0) return IXB_ERR_ARG;
  if (B == 0 || H == 0 || Sq == 0) return IXB_OK;
  if (!q || !k || !v || !o || !q_strides || !k_strides || !v_strides || !o_strides) return IXB_ERR_ARG;
  if (dtype != IXB_BF16 && dtype != IXB_F16) return IXB_ERR_DTYPE;
  if (D != HD) return IXB_ERR_SHAPE;
  if (Sk <= 0) return IXB_ERR_SHAPE;
  if (causal && Sk < Sq) return IXB_ERR_SHAPE;  // some rows would see no key at all
  if ((long long)B * H > 65535) return IXB_ERR_SHAPE;
  const void* ptrs[4] = {q, k, v, o};
  const int64_t* strs[4] = {q_strides, k_strides, v_strides, o_strides};
  for (int t = 0; t < 4; ++t) {
    if (!ixb_host::aligned16(ptrs[t])) return IXB_ERR_ALIGN;
    for (int i = 0; i < 3; ++i)
      if (strs[t][i] <= 0 || (strs[t][i] * 2) % 16 != 0) return IXB_ERR_ALIGN;
  }
  const int is_bf16 = dtype == IXB_BF16;
  CUtensorMap mq, mk, mv;
  if (int st = ixb_host::make_fa_map(&mq, q, is_bf16, B, H, Sq, q_strides[0], q_strides[1], q_strides[2])) return st;
  if (int st = ixb_host::make_fa_map(&mk, k, is_bf16, B, H, Sk, k_strides[0], k_strides[1], k_strides[2])) return st;
  if (int st = ixb_host::make_fa_map(&mv, v, is_bf16, B, H, Sk, v_strides[0], v_strides[1], v_strides[2])) return st;
  FaParams p;
  p.o = o;
  p.lse = lse;
  p.status = status;
  p.o_stride_b = o_strides[0];
  p.o_stride_h = o_strides[1];
  p.o_stride_s = o_strides[2];
  p.B = B;
  p.H = H;
  p.Sq = Sq;
  p.Sk = Sk;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  // Without a mask every query block of a head reads all of its K and V, so the heads go one
  // after the other (group of 1: blockIdx order = head-major, as a 2-D grid would give).
  // Under a causal mask 8 heads run together (measured at 4096 keys: 1, 8, 16 heads within 1 %
  // of each other, 64 and more slower - their K and V no longer stay in L2).
  static const int group_env = [] { const char* v = getenv("IXB_FA_HEAD_GROUP"); return v != nullptr ? atoi(v) : 0; }();
  p.head_group = group_env > 0 ? group_env : (causal ? 8 : 1);
  if (!(scale > 0.f)) return IXB_ERR_ARG;  // the row maximum is taken before scaling
  const dim3 grid((unsigned)(((Sq + BM * NQ - 1) / (BM * NQ)) * (long long)B * H));
  auto kern = is_bf16 ? fa_fwd_kernel<true> : fa_fwd_kernel<false>;
  // the shared-memory opt-in is a property of (kernel, device): set once per device
  static std::atomic<bool> configured[2][64];
  int devid = 0;
  cudaGetDevice(&devid);
  std::atomic<bool>& done = configured[is_bf16][devid & 63];
  if (!done.load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return ixb_host::cuda_status(e);
    done.store(true, std::memory_order_release);
  }
  kern<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(mq, mk, mv, p);
  return ixb_host::cuda_status(cudaGetLastError());
}
