// Fused attention backward for sm_100a: gradients of softmax(Q K^T * scale [+ causal mask]) V
// with tcgen05 tensor-core MMAs, accumulators in tensor memory and operands brought in by
// TMA.  It takes the place of the vendor kernel behind torch.ops.npu_graph.npu_fa_backward
// (inductor_x/npu_fusion_attention_graph.py:38-42).
//
// With P = exp(S * scale - lse), dP = dO V^T, delta = rowsum(dO * O) and
// dS = P * (dP - delta):   dV = P^T dO,   dK = scale * dS^T Q,   dQ = scale * dS K.
// Three launches, no atomics, no scratch besides `delta`:
//   fa_bwd_delta_kernel  delta[b, h, i] (one warp per row)
//   fa_bwd_dkv_kernel    one CTA owns a 128-key tile and walks the query tiles that see it;
//                        it forms S^T = K Q^T and dP^T = V dO^T (thread <-> key, columns <->
//                        queries), so that P^T and dS^T - written back over S^T and dP^T as
//                        16-bit values - are the TMEM operands of dV += P^T dO and
//                        dK += dS^T Q, which stay in TMEM until the tile is finished
//   fa_bwd_dq_kernel     one CTA owns a 128-row query tile and walks its key tiles;
//                        S = Q K^T, dP = dO V^T (thread <-> query), dS over dP, dQ += dS K
// The probabilities are recomputed in both kernels (7 products instead of 5) - that is what
// keeps each output with a single owner.
//
// Warp 0 is the TMA producer, warp 1 the MMA issuer, the other 4 * NG warps do the
// element-wise work in NG groups of four warps that split the 128 columns of a tile between
// them (a warp may only touch the 32 TMEM lanes of its quadrant; no row reduction is needed
// here - lse and delta come in precomputed - so the split costs nothing).  Every wait is
// bounded; a wait that gives up raises a flag in `status` and lets the CTA drain and exit.
//
// Measured on B200 (4096 keys, causal): per 128 x 128 tile pair the tensor core needs about
// 2050 cycles for the four products (one 128x128x16 MMA per 64 cycles, SS or TS form, one or
// two issuing threads alike) and the element-wise warps about 2300 (the exponentials alone
// fill the ex2 unit for 1024); with one tile in flight the two add up (4330 cycles per tile
// pair).  A variant with 64-query sub-tiles, double-buffered score columns and a four-stage
// ring overlapped them but ran 30 % slower: an SS-form MMA with N = 64 takes 48 cycles, not 32
// (both operands come from shared memory at 128 bytes per cycle), and the hand-offs double.
#include <atomic>
#include "fa_maps.h"
#include "ixb/tcgen05.cuh"

namespace {

using namespace ixb;

constexpr int BM = 128;  // query rows per tile
constexpr int BN = 128;  // keys per tile
constexpr int HD = 128;  // head dimension
constexpr int kStages = 2;  // (the issuers pick stage descriptors with two-way selects: no local-memory arrays)
constexpr int kTileBytes = 128 * HD * 2;
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int NG = 2;             // groups of element-wise warps; each takes 128 / NG columns of a tile
constexpr int GC = 128 / NG;      // columns per group
constexpr int kWorkers = 128 * NG;
constexpr int kThreads = 64 + kWorkers;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColDP = 128, kColAcc0 = 256, kColAcc1 = 384;
constexpr size_t kSmemBytes = (size_t)kTileBytes * 6 + 1024;

struct Out {
  void* ptr;
  long long sb, sh, ss;  // strides in elements
};
struct BwdParams {
  const float* lse;    // [B, H, Sq] natural-log sum of exponentials of the forward
  const float* delta;  // [B, H, Sq] rowsum(dO * O)
  Out dq, dk, dv;
  int* status;
  int B, H, Sq, Sk;
  float scale, scale_log2;
  int causal;
  int head_group;
};

__device__ __forceinline__ uint32_t pack_pair(float lo, float hi, bool is_bf16) {
  if (is_bf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_pair(uint32_t w, bool is_bf16) {
  if (is_bf16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// One arrival per warp: every lane has fenced its tensor-memory accesses, the warp
// synchronises, lane 0 arrives (the barrier counts warps, not threads).
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) tc::mbar_arrive(bar);
}

// ------------------------------------------------------------------------------ delta
template <bool IS_BF16>
__global__ void __launch_bounds__(256)
    fa_bwd_delta_kernel(const unsigned char* o, const unsigned char* dout, float* delta, int H, int Sq,
                        long long rows, long long o_sb, long long o_sh, long long o_ss, long long d_sb,
                        long long d_sh, long long d_ss) {
  // half a warp per row: 16 lanes x 16 bytes = the 128 16-bit values of a row
  const int lane = threadIdx.x & 31, sub = lane & 15;
  const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  float s = 0.f;
  if (row < rows) {
    const long long bh = row / Sq;
    const long long i = row - bh * Sq;
    const long long b = bh / H, h = bh - b * H;
    const uint4 a = ldg_stream(reinterpret_cast<const uint4*>(o + 2 * (b * o_sb + h * o_sh + i * o_ss) + sub * 16));
    const uint4 g = ldg_stream(reinterpret_cast<const uint4*>(dout + 2 * (b * d_sb + h * d_sh + i * d_ss) + sub * 16));
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = unpack_pair(aw[e], IS_BF16), y = unpack_pair(gw[e], IS_BF16);
      s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
    }
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(kFull, s, off);
  if (sub == 0 && row < rows) delta[row] = s;
}

// --------------------------------------------------------------------- shared pieces
// CTA order: heads in groups of `head_group` (their operands stay in L2 while the group
// runs); inside a group tile `slot` of every head before tile `slot + 1` of any.
__device__ __forceinline__ void cta_order(int n_tiles, int n_bh, int head_group, int* slot, int* bh) {
  const int per_group = n_tiles * head_group;
  const int group = (int)blockIdx.x / per_group;
  const int in_group = (int)blockIdx.x - group * per_group;
  const int left = n_bh - group * head_group;
  const int g_heads = left < head_group ? left : head_group;
  *slot = in_group / g_heads;
  *bh = group * head_group + in_group % g_heads;
}

__device__ __forceinline__ void load_tile(unsigned char* dst, const CUtensorMap* map, uint64_t* bar, int row0,
                                          int h, int b) {
  tc::tma_load_4d(dst, map, bar, 0, row0, h, b);
  tc::tma_load_4d(dst + kHalfBytes, map, bar, 64, row0, h, b);
}

// D = A B^T, both operands K-major tiles of 128 x 128 (8 steps of 16 along the head dimension)
__device__ __forceinline__ void issue_ss(uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
    tc::mma_ss(d, a_desc + off, b_desc + off, idesc, ks > 0);
  }
}
// D (+)= A B with A in TMEM as 16-bit pairs (group g wrote its GC values of the reduced index
// as GC / 2 columns starting at column a + GC * g) and B a tile in MN-major form (16 rows =
// 2048 bytes a step)
__device__ __forceinline__ void issue_ts(uint32_t d, uint32_t a, uint64_t b_desc_mn, uint32_t idesc,
                                         bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < 128 / 16; ++ks) {
    constexpr int kStepsPerGroup = GC / 16;
    const uint32_t col = a + (ks / kStepsPerGroup) * GC + (ks % kStepsPerGroup) * 8;
    tc::mma_ts(d, col, b_desc_mn + (uint32_t)(ks * 2048 >> 4), idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// GC accumulator columns of this thread's row -> 16-bit values in global memory
template <bool IS_BF16>
__device__ __forceinline__ void store_cols(uint32_t taddr, unsigned char* dst, float mult, bool live) {
#pragma unroll
  for (int c = 0; c < GC / 32; ++c) {
    uint32_t acc[32];
    tc::tmem_ld32(taddr + c * 32, acc);
    tc::tmem_wait_ld();
    if (live) {
#pragma unroll
      for (int e = 0; e < 32; e += 8) {
        uint4 w;
        w.x = pack_pair(__uint_as_float(acc[e]) * mult, __uint_as_float(acc[e + 1]) * mult, IS_BF16);
        w.y = pack_pair(__uint_as_float(acc[e + 2]) * mult, __uint_as_float(acc[e + 3]) * mult, IS_BF16);
        w.z = pack_pair(__uint_as_float(acc[e + 4]) * mult, __uint_as_float(acc[e + 5]) * mult, IS_BF16);
        w.w = pack_pair(__uint_as_float(acc[e + 6]) * mult, __uint_as_float(acc[e + 7]) * mult, IS_BF16);
        *reinterpret_cast<uint4*>(dst + (c * 32 + e) * 2) = w;
      }
    }
  }
}

// ------------------------------------------------------------------------------ dK, dV
// TMEM columns: [0,128) S^T then P^T, [128,256) dP^T then dS^T, [256,384) dV, [384,512) dK.
template <bool IS_BF16>
__global__ void __launch_bounds__(kThreads, 1)
    fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                      const BwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* k_smem = smem;
  unsigned char* v_smem = smem + kTileBytes;
  unsigned char* q_smem = smem + 2 * kTileBytes;   // kStages tiles
  unsigned char* do_smem = smem + 4 * kTileBytes;  // kStages tiles

  __shared__ __align__(8) uint64_t kv_full, qdo_full[kStages], qdo_empty[kStages], s_full, dp_full, p_full,
      ds_full, acc_done;
  __shared__ __align__(16) float lse_s[kStages][BM], delta_s[kStages][BM];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int n_kv_tiles = (p.Sk + BN - 1) / BN;
  const int n_q_tiles = (p.Sq + BM - 1) / BM;
  int kv_tile, bh;
  cta_order(n_kv_tiles, p.B * p.H, p.head_group, &kv_tile, &bh);  // early key tiles see the most queries
  const int b = bh / p.H, h = bh % p.H;
  const int kt0 = kv_tile * BN;
  const int diag = p.Sk - p.Sq;  // key j is visible to query i when j <= i + diag
  int i0 = 0;
  if (p.causal) {
    const int first = kt0 - diag;  // first query that sees the first key of the tile
    i0 = first > 0 ? first / BM : 0;
  }
  const int n_it = n_q_tiles > i0 ? n_q_tiles - i0 : 0;

  if (threadIdx.x == 0) {
    mbar_init(&kv_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&dp_full, 1);
    mbar_init(&p_full, kWorkers / 32);
    mbar_init(&ds_full, kWorkers / 32);
    mbar_init(&acc_done, 1);
    failed = 0;
    mbar_init_fence();
  }
  if (warp == 1) tc::tmem_alloc(&tmem_base_slot, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0 && n_it > 0) {
      mbar_arrive_expect_tx(&kv_full, 2 * kTileBytes);
      load_tile(k_smem, &map_k, &kv_full, kt0, h, b);
      load_tile(v_smem, &map_v, &kv_full, kt0, h, b);
    }
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it % kStages, n = it / kStages;
      const int qt0 = (i0 + it) * BM;
      if (n > 0) {
        int mine = 1;
        if (lane == 0) mine = mbar_wait(&qdo_empty[s], (n - 1) & 1, &failed) ? 1 : 0;
        ok = __shfl_sync(kFull, mine, 0) != 0;
        if (!ok) break;
      }
      // per-query statistics of the tile: lse in log2 units (+inf past the end: P = 0), delta
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = lane * 4 + e;
        const int qi = qt0 + r;
        const bool live = qi < p.Sq;
        const long long at = (long long)bh * p.Sq + qi;
        lse_s[s][r] = live ? p.lse[at] * kLog2e : INFINITY;
        delta_s[s][r] = live ? p.delta[at] : 0.f;
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_expect_tx(&qdo_full[s], 2 * kTileBytes);
        load_tile(q_smem + (size_t)s * kTileBytes, &map_q, &qdo_full[s], qt0, h, b);
        load_tile(do_smem + (size_t)s * kTileBytes, &map_do, &qdo_full[s], qt0, h, b);
      }
    }
    if (!ok && lane == 0) failed = 1;
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_kk = tc::instr_desc(128, 128, IS_BF16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_mn = tc::instr_desc(128, 128, IS_BF16 ? 1 : 0, 0, 1);
      const uint64_t k_desc = tc::smem_desc(smem_u32(k_smem), 16, 1024);
      const uint64_t v_desc = tc::smem_desc(smem_u32(v_smem), 16, 1024);
      uint64_t q_desc[kStages], do_desc[kStages], q_desc_mn[kStages], do_desc_mn[kStages];
#pragma unroll
      for (int s = 0; s < kStages; ++s) {
        const uint32_t qa = smem_u32(q_smem + (size_t)s * kTileBytes);
        const uint32_t da = smem_u32(do_smem + (size_t)s * kTileBytes);
        q_desc[s] = tc::smem_desc(qa, 16, 1024);
        do_desc[s] = tc::smem_desc(da, 16, 1024);
        q_desc_mn[s] = tc::smem_desc(qa, kHalfBytes, 1024);
        do_desc_mn[s] = tc::smem_desc(da, kHalfBytes, 1024);
      }
      const uint32_t t_s = tmem_base + kColS, t_dp = tmem_base + kColDP;
      const uint32_t t_dv = tmem_base + kColAcc0, t_dk = tmem_base + kColAcc1;
      bool ok = mbar_wait(&kv_full, 0, &failed);
      ok = ok && mbar_wait(&qdo_full[0], 0, &failed);
      if (ok) {
        tc::fence_after_sync();
        issue_ss(t_s, k_desc, q_desc[0], idesc_kk);  // S^T = K Q^T
        tc::mma_commit(&s_full);
        issue_ss(t_dp, v_desc, do_desc[0], idesc_kk);  // dP^T = V dO^T
        tc::mma_commit(&dp_full);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1, s1 = (it + 1) & 1;
        const bool next = it + 1 < n_it;
        ok = mbar_wait(&p_full, it & 1, &failed);
        if (!ok) break;
        tc::fence_after_sync();
        issue_ts(t_dv, t_s, (s ? do_desc_mn[1] : do_desc_mn[0]), idesc_mn, it > 0);  // dV += P^T dO
        if (next) {
          ok = mbar_wait(&qdo_full[s1], ((it + 1) >> 1) & 1, &failed);
          if (!ok) break;
          tc::fence_after_sync();
          // the tensor core runs its MMAs in order: P^T has been consumed when this one starts
          issue_ss(t_s, k_desc, (s1 ? q_desc[1] : q_desc[0]), idesc_kk);
          tc::mma_commit(&s_full);
        }
        ok = mbar_wait(&ds_full, it & 1, &failed);
        if (!ok) break;
        tc::fence_after_sync();
        issue_ts(t_dk, t_dp, (s ? q_desc_mn[1] : q_desc_mn[0]), idesc_mn, it > 0);  // dK += dS^T Q
        tc::mma_commit(&qdo_empty[s]);
        if (next) {
          issue_ss(t_dp, v_desc, (s1 ? do_desc[1] : do_desc[0]), idesc_kk);
          tc::mma_commit(&dp_full);
        }
      }
      if (ok) tc::mma_commit(&acc_done);
      if (!ok) failed = 1;
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ element-wise work
    const int g = (warp - 2) >> 2;  // group: query columns [GC g, GC g + GC) of a tile
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // key inside the tile
    const int kj = kt0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + kColS + GC * g;
    const uint32_t dp_addr = lane_addr + kColDP + GC * g;
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    bool ok = true;

    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const int qt0 = (i0 + it) * BM;
      bool w = mbar_wait(&qdo_full[s], (it >> 1) & 1, &failed);
      w = w && mbar_wait(&s_full, it & 1, &failed);
      if (!__all_sync(kFull, w)) {
        ok = false;
        break;
      }
      tc::fence_after_sync();
      // query column e of this group is visible to key kj when qt0 + GC g + e >= kj - diag
      const bool edge = p.causal && (kt0 + BN - 1 > qt0 + diag);
      const int lo = edge ? kj - diag - (qt0 + GC * g) : 0;
      const float* lse_row = &lse_s[s][GC * g];
      float pr[GC];
#pragma unroll
      for (int c = 0; c < GC / 32; ++c) {
        uint32_t raw[32];
        tc::tmem_ld32(s_addr + c * 32, raw);
        tc::tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse_row + c * 32 + e);
          const float2 a0 = fma2(make_float2(__uint_as_float(raw[e]), __uint_as_float(raw[e + 1])), sc2,
                                 make_float2(-l4.x, -l4.y));
          const float2 a1 = fma2(make_float2(__uint_as_float(raw[e + 2]), __uint_as_float(raw[e + 3])), sc2,
                                 make_float2(-l4.z, -l4.w));
          float* o = &pr[c * 32 + e];
          o[0] = fast_exp2(a0.x);
          o[1] = fast_exp2(a0.y);
          o[2] = fast_exp2(a1.x);
          o[3] = fast_exp2(a1.y);
          if (edge) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (c * 32 + e + u < lo) o[u] = 0.f;
          }
        }
      }
      // all of this group's S columns are in registers: P^T goes over their first half
#pragma unroll
      for (int c = 0; c < GC / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = pack_pair(pr[c * 32 + 2 * e], pr[c * 32 + 2 * e + 1], IS_BF16);
        tc::tmem_st16(s_addr + c * 16, pk);
      }
      tc::tmem_wait_st();
      tc::fence_before_sync();
      warp_arrive(&p_full, lane);

      if (!__all_sync(kFull, mbar_wait(&dp_full, it & 1, &failed))) {
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const float* delta_row = &delta_s[s][GC * g];
#pragma unroll
      for (int c = 0; c < GC / 32; ++c) {
        uint32_t d[32];
        tc::tmem_ld32(dp_addr + c * 32, d);
        tc::tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(delta_row + c * 32 + e);
          const float x0 = pr[c * 32 + e] * (__uint_as_float(d[e]) - d4.x);
          const float x1 = pr[c * 32 + e + 1] * (__uint_as_float(d[e + 1]) - d4.y);
          const float x2 = pr[c * 32 + e + 2] * (__uint_as_float(d[e + 2]) - d4.z);
          const float x3 = pr[c * 32 + e + 3] * (__uint_as_float(d[e + 3]) - d4.w);
          pk[e / 2] = pack_pair(x0, x1, IS_BF16);
          pk[e / 2 + 1] = pack_pair(x2, x3, IS_BF16);
        }
        // columns [16c, 16c+16) of this group: their dP values are already in registers
        tc::tmem_st16(dp_addr + c * 16, pk);
      }
      tc::tmem_wait_st();
      tc::fence_before_sync();
      warp_arrive(&ds_full, lane);
    }

    if (ok && n_it > 0) ok = mbar_wait(&acc_done, 0, &failed);
    ok = __all_sync(kFull, ok);
    if (ok) {
      tc::fence_after_sync();
      const bool live = kj < p.Sk;
      unsigned char* dv_row = reinterpret_cast<unsigned char*>(p.dv.ptr) +
                              2 * ((long long)b * p.dv.sb + (long long)h * p.dv.sh + (long long)kj * p.dv.ss) +
                              2 * GC * g;
      unsigned char* dk_row = reinterpret_cast<unsigned char*>(p.dk.ptr) +
                              2 * ((long long)b * p.dk.sb + (long long)h * p.dk.sh + (long long)kj * p.dk.ss) +
                              2 * GC * g;
      if (n_it > 0) {
        store_cols<IS_BF16>(lane_addr + kColAcc0 + GC * g, dv_row, 1.f, live);
        store_cols<IS_BF16>(lane_addr + kColAcc1 + GC * g, dk_row, p.scale, live);
      } else if (live) {
        // no query sees this key tile: the gradients are zero
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int e = 0; e < GC / 8; ++e) {
          reinterpret_cast<uint4*>(dv_row)[e] = z;
          reinterpret_cast<uint4*>(dk_row)[e] = z;
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

// ------------------------------------------------------------------------------ dQ
// TMEM columns: [0,128) S, [128,256) dP then dS (group g's GC values as GC / 2 columns at
// 128 + GC g), [256,384) dQ.
template <bool IS_BF16>
__global__ void __launch_bounds__(kThreads, 1)
    fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                     const BwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_smem = smem;
  unsigned char* do_smem = smem + kTileBytes;
  unsigned char* k_smem = smem + 2 * kTileBytes;  // kStages tiles
  unsigned char* v_smem = smem + 4 * kTileBytes;  // kStages tiles

  __shared__ __align__(8) uint64_t qdo_full, k_full[kStages], k_empty[kStages], v_full[kStages],
      v_empty[kStages], s_full, dp_full, s_read, ds_full, acc_done;
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int n_q_tiles = (p.Sq + BM - 1) / BM;
  int slot, bh;
  cta_order(n_q_tiles, p.B * p.H, p.head_group, &slot, &bh);
  const int q_tile = n_q_tiles - 1 - slot;  // late query tiles see the most keys: first
  const int b = bh / p.H, h = bh % p.H;
  const int qt0 = q_tile * BM;
  const int diag = p.Sk - p.Sq;
  int kv_end = p.Sk;
  if (p.causal) {
    const int lim = qt0 + BM + diag;
    kv_end = lim < p.Sk ? lim : p.Sk;
  }
  const int n_kv = (kv_end + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&qdo_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&dp_full, 1);
    mbar_init(&s_read, kWorkers / 32);
    mbar_init(&ds_full, kWorkers / 32);
    mbar_init(&acc_done, 1);
    failed = 0;
    mbar_init_fence();
  }
  if (warp == 1) tc::tmem_alloc(&tmem_base_slot, kTmemCols);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      mbar_arrive_expect_tx(&qdo_full, 2 * kTileBytes);
      load_tile(q_smem, &map_q, &qdo_full, qt0, h, b);
      load_tile(do_smem, &map_do, &qdo_full, qt0, h, b);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % kStages, n = j / kStages;
        if (n > 0) ok = mbar_wait(&k_empty[s], (n - 1) & 1, &failed);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[s], kTileBytes);
        load_tile(k_smem + (size_t)s * kTileBytes, &map_k, &k_full[s], j * BN, h, b);
        if (n > 0) ok = mbar_wait(&v_empty[s], (n - 1) & 1, &failed);
        if (!ok) break;
        mbar_arrive_expect_tx(&v_full[s], kTileBytes);
        load_tile(v_smem + (size_t)s * kTileBytes, &map_v, &v_full[s], j * BN, h, b);
      }
      if (!ok) failed = 1;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_kk = tc::instr_desc(128, 128, IS_BF16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_mn = tc::instr_desc(128, 128, IS_BF16 ? 1 : 0, 0, 1);
      const uint64_t q_desc = tc::smem_desc(smem_u32(q_smem), 16, 1024);
      const uint64_t do_desc = tc::smem_desc(smem_u32(do_smem), 16, 1024);
      uint64_t k_desc[kStages], v_desc[kStages], k_desc_mn[kStages];
#pragma unroll
      for (int s = 0; s < kStages; ++s) {
        const uint32_t ka = smem_u32(k_smem + (size_t)s * kTileBytes);
        k_desc[s] = tc::smem_desc(ka, 16, 1024);
        k_desc_mn[s] = tc::smem_desc(ka, kHalfBytes, 1024);
        v_desc[s] = tc::smem_desc(smem_u32(v_smem + (size_t)s * kTileBytes), 16, 1024);
      }
      const uint32_t t_s = tmem_base + kColS, t_dp = tmem_base + kColDP, t_dq = tmem_base + kColAcc0;
      bool ok = mbar_wait(&qdo_full, 0, &failed);
      ok = ok && mbar_wait(&k_full[0], 0, &failed);
      ok = ok && mbar_wait(&v_full[0], 0, &failed);
      if (ok) {
        tc::fence_after_sync();
        issue_ss(t_s, q_desc, k_desc[0], idesc_kk);  // S = Q K^T
        tc::mma_commit(&s_full);
        issue_ss(t_dp, do_desc, v_desc[0], idesc_kk);  // dP = dO V^T
        tc::mma_commit(&dp_full);
        tc::mma_commit(&v_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1, s1 = (j + 1) & 1, n1 = (j + 1) >> 1;
        const bool next = j + 1 < n_kv;
        if (next) {
          // S(j) is in registers of the element-wise warps: its columns can take S(j+1)
          ok = mbar_wait(&s_read, j & 1, &failed);
          ok = ok && mbar_wait(&k_full[s1], n1 & 1, &failed);
          if (!ok) break;
          tc::fence_after_sync();
          issue_ss(t_s, q_desc, (s1 ? k_desc[1] : k_desc[0]), idesc_kk);
          tc::mma_commit(&s_full);
        }
        ok = mbar_wait(&ds_full, j & 1, &failed);
        if (!ok) break;
        tc::fence_after_sync();
        issue_ts(t_dq, t_dp, (s ? k_desc_mn[1] : k_desc_mn[0]), idesc_mn, j > 0);  // dQ += dS K
        tc::mma_commit(&k_empty[s]);
        if (next) {
          ok = mbar_wait(&v_full[s1], n1 & 1, &failed);
          if (!ok) break;
          tc::fence_after_sync();
          issue_ss(t_dp, do_desc, (s1 ? v_desc[1] : v_desc[0]), idesc_kk);  // after dQ(j): dS(j) has been consumed
          tc::mma_commit(&dp_full);
          tc::mma_commit(&v_empty[s1]);
        }
      }
      if (ok) tc::mma_commit(&acc_done);
      if (!ok) failed = 1;
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ element-wise work
    const int g = (warp - 2) >> 2;  // group: key columns [GC g, GC g + GC) of a tile
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int qi = qt0 + row;
    const bool live = qi < p.Sq;
    const long long stat_at = (long long)bh * p.Sq + qi;
    const float lse2 = live ? p.lse[stat_at] * kLog2e : INFINITY;
    const float dl = live ? p.delta[stat_at] : 0.f;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + kColS + GC * g;
    const uint32_t dp_addr = lane_addr + kColDP + GC * g;
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    const float2 nl2 = make_float2(-lse2, -lse2);
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      if (!__all_sync(kFull, mbar_wait(&s_full, j & 1, &failed))) {
        ok = false;
        break;
      }
      tc::fence_after_sync();
      uint32_t raw[GC];
#pragma unroll
      for (int c = 0; c < GC / 32; ++c) tc::tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[c * 32]));
      tc::tmem_wait_ld();
      tc::fence_before_sync();
      warp_arrive(&s_read, lane);
      const int col0 = j * BN + GC * g;
      const bool edge = (j * BN + BN > p.Sk) || (p.causal && (j * BN + BN - 1 > qt0 + diag));
      int lim = GC - 1;  // last visible key of this row, relative to this group's columns
      if (edge) {
        int last = p.Sk - 1;
        if (p.causal && qi + diag < last) last = qi + diag;
        lim = last - col0;
      }
      float pr[GC];
#pragma unroll
      for (int e = 0; e < GC; e += 2) {
        const float2 a = fma2(make_float2(__uint_as_float(raw[e]), __uint_as_float(raw[e + 1])), sc2, nl2);
        pr[e] = fast_exp2(a.x);
        pr[e + 1] = fast_exp2(a.y);
        if (edge) {
          if (e > lim) pr[e] = 0.f;
          if (e + 1 > lim) pr[e + 1] = 0.f;
        }
      }
      if (!__all_sync(kFull, mbar_wait(&dp_full, j & 1, &failed))) {
        ok = false;
        break;
      }
      tc::fence_after_sync();
#pragma unroll
      for (int c = 0; c < GC / 32; ++c) {
        uint32_t d[32];
        tc::tmem_ld32(dp_addr + c * 32, d);
        tc::tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float x0 = pr[c * 32 + e] * (__uint_as_float(d[e]) - dl);
          const float x1 = pr[c * 32 + e + 1] * (__uint_as_float(d[e + 1]) - dl);
          pk[e / 2] = pack_pair(x0, x1, IS_BF16);
        }
        tc::tmem_st16(dp_addr + c * 16, pk);
      }
      tc::tmem_wait_st();
      tc::fence_before_sync();
      warp_arrive(&ds_full, lane);
    }

    if (ok) ok = mbar_wait(&acc_done, 0, &failed);
    ok = __all_sync(kFull, ok);
    if (ok) {
      tc::fence_after_sync();
      unsigned char* dq_row = reinterpret_cast<unsigned char*>(p.dq.ptr) +
                              2 * ((long long)b * p.dq.sb + (long long)h * p.dq.sh + (long long)qi * p.dq.ss) +
                              2 * GC * g;
      store_cols<IS_BF16>(lane_addr + kColAcc0 + GC * g, dq_row, p.scale, live);
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

template <class K>
int opt_in_smem(K kern, std::atomic<bool>& done) {
  if (!done.load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return ixb_host::cuda_status(e);
    done.store(true, std::memory_order_release);
  }
  return IXB_OK;
}

}  // namespace

extern "C" int ixb_fa_bwd(int dtype, const void* q, const void* k, const void* v, const void* o,
                          const void* dout, const float* lse, void* dq, void* dk, void* dv, float* delta,
                          int32_t B, int32_t H, int32_t Sq, int32_t Sk, int32_t D, const int64_t* q_strides,
                          const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                          const int64_t* do_strides, const int64_t* dq_strides, const int64_t* dk_strides,
                          const int64_t* dv_strides, float scale, int causal, int32_t* status,
                          ixb_stream stream) {
  if (B < 0 || H < 0 || Sq < 0 || Sk < 0) return IXB_ERR_ARG;
  if (B == 0 || H == 0 || Sq == 0 || Sk == 0) return IXB_OK;
  if (!q || !k || !v || !o || !dout || !lse || !dq || !dk || !dv || !delta) return IXB_ERR_ARG;
  if (dtype != IXB_BF16 && dtype != IXB_F16) return IXB_ERR_DTYPE;
  if (D != HD) return IXB_ERR_SHAPE;
  if (causal && Sk < Sq) return IXB_ERR_SHAPE;
  if (!(scale > 0.f)) return IXB_ERR_ARG;
  const void* ptrs[8] = {q, k, v, o, dout, dq, dk, dv};
  const int64_t* strs[8] = {q_strides, k_strides, v_strides, o_strides, do_strides, dq_strides, dk_strides,
                            dv_strides};
  for (int t = 0; t < 8; ++t) {
    if (strs[t] == nullptr) return IXB_ERR_ARG;
    if (!ixb_host::aligned16(ptrs[t])) return IXB_ERR_ALIGN;
    for (int i = 0; i < 3; ++i)
      if (strs[t][i] <= 0 || (strs[t][i] * 2) % 16 != 0) return IXB_ERR_ALIGN;
  }
  const long long n_q_tiles = (Sq + BM - 1) / BM, n_kv_tiles = (Sk + BN - 1) / BN;
  const long long n_bh = (long long)B * H;
  if (n_q_tiles * n_bh > 0x7fffffffLL || n_kv_tiles * n_bh > 0x7fffffffLL) return IXB_ERR_SHAPE;
  const int is_bf16 = dtype == IXB_BF16;
  CUtensorMap mq, mk, mv, mdo;
  if (int st = ixb_host::make_fa_map(&mq, q, is_bf16, B, H, Sq, q_strides[0], q_strides[1], q_strides[2])) return st;
  if (int st = ixb_host::make_fa_map(&mk, k, is_bf16, B, H, Sk, k_strides[0], k_strides[1], k_strides[2])) return st;
  if (int st = ixb_host::make_fa_map(&mv, v, is_bf16, B, H, Sk, v_strides[0], v_strides[1], v_strides[2])) return st;
  if (int st = ixb_host::make_fa_map(&mdo, dout, is_bf16, B, H, Sq, do_strides[0], do_strides[1], do_strides[2]))
    return st;
  BwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq = Out{dq, dq_strides[0], dq_strides[1], dq_strides[2]};
  p.dk = Out{dk, dk_strides[0], dk_strides[1], dk_strides[2]};
  p.dv = Out{dv, dv_strides[0], dv_strides[1], dv_strides[2]};
  p.status = status;
  p.B = B;
  p.H = H;
  p.Sq = Sq;
  p.Sk = Sk;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.causal = causal ? 1 : 0;
  static const int group_env = [] { const char* e = getenv("IXB_FA_HEAD_GROUP"); return e != nullptr ? atoi(e) : 0; }();
  p.head_group = group_env > 0 ? group_env : (causal ? 8 : 1);

  auto kern_delta = is_bf16 ? fa_bwd_delta_kernel<true> : fa_bwd_delta_kernel<false>;
  auto kern_dkv = is_bf16 ? fa_bwd_dkv_kernel<true> : fa_bwd_dkv_kernel<false>;
  auto kern_dq = is_bf16 ? fa_bwd_dq_kernel<true> : fa_bwd_dq_kernel<false>;
  static std::atomic<bool> configured[2][2][64];
  int devid = 0;
  cudaGetDevice(&devid);
  if (int st = opt_in_smem(kern_dkv, configured[0][is_bf16][devid & 63])) return st;
  if (int st = opt_in_smem(kern_dq, configured[1][is_bf16][devid & 63])) return st;

  cudaStream_t cs = (cudaStream_t)stream;
  const long long rows = n_bh * Sq;
  kern_delta<<<(unsigned)((rows + 15) / 16), 256, 0, cs>>>(
      static_cast<const unsigned char*>(o), static_cast<const unsigned char*>(dout), delta, H, Sq, rows,
      o_strides[0], o_strides[1], o_strides[2], do_strides[0], do_strides[1], do_strides[2]);
  kern_dkv<<<(unsigned)(n_kv_tiles * n_bh), kThreads, kSmemBytes, cs>>>(mq, mk, mv, mdo, p);
  kern_dq<<<(unsigned)(n_q_tiles * n_bh), kThreads, kSmemBytes, cs>>>(mq, mk, mv, mdo, p);
  return ixb_host::cuda_status(cudaGetLastError());
}
