// Fused attention forward for sm_100a: softmax(Q K^T * scale [+ causal mask]) V with
// tcgen05 tensor-core MMAs, accumulators in tensor memory and operands brought in by TMA.
// It takes the place of the vendor kernel behind torch.ops.npu_graph.npu_fa
// (inductor_x/npu_fusion_attention_graph.py:20-35).
//
// One CTA owns a 128-row query tile of one (batch, head) and walks the key/value tiles
// (128 keys each) that the tile can see.  Six warps, three roles:
//   warp 0     TMA producer: Q once, then K_j / V_j into two-stage rings
//   warp 1     MMA issuer: S_j = Q K_j^T into one of two TMEM buffers, then O += P_j V_j
//              with P_j read straight from TMEM (it overwrites S_j as 16-bit values)
//   warps 2-5  softmax: thread <-> query row.  Reads its S row from TMEM, applies scale
//              and mask, keeps a running maximum and sum, writes P_j back to TMEM, and
//              rescales the O accumulator only when the maximum has grown by more than
//              2^8 since the last rescale (the final division by the sum makes any stale
//              reference maximum exact).
// Hand-offs are mbarriers; every wait is bounded and a wait that gives up raises a flag in
// `status` and lets the CTA drain and exit.
//
// TMEM columns: [0,128) S/P buffer 0, [128,256) S/P buffer 1, [256,384) O.
#include "host.h"
#include "ixb/tcgen05.cuh"

namespace {

using namespace ixb;

constexpr int BM = 128;          // query rows per CTA
constexpr int BN = 128;          // keys per tile
constexpr int HD = 128;          // head dimension
constexpr int kStages = 2;
constexpr int kTileBytes = BN * HD * 2;   // one operand tile, 16-bit elements
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column TMA box of the tile
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256;
constexpr float kRescaleThreshold = 8.f;  // log2 units
constexpr size_t kSmemBytes = (size_t)kTileBytes * (1 + 2 * kStages) + 1024;

struct FaParams {
  void* o;
  float* lse;            // [B, H, Sq] natural-log sum of exponentials, may be null
  int* status;           // device word set to 1 if a wait gave up, may be null
  long long o_stride_b, o_stride_h, o_stride_s;  // elements
  int B, H, Sq, Sk;
  float scale_log2;      // softmax scale * log2(e)
  int causal;
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
  unsigned char* k_smem = smem + kTileBytes;
  unsigned char* v_smem = smem + kTileBytes * (1 + kStages);

  __shared__ __align__(8) uint64_t q_full, k_full[kStages], k_empty[kStages], v_full[kStages],
      v_empty[kStages], s_full[2], p_full[2], pv_done[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // heavy (late) query tiles first: they see the most keys under a causal mask
  const int n_q_tiles = (p.Sq + BM - 1) / BM;
  const int q_tile = n_q_tiles - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = q_tile * BM;
  const int diag = p.Sk - p.Sq;  // key index allowed for query row i: j <= i + diag
  int kv_end = p.Sk;
  if (p.causal) {
    const int lim = q0 + BM + diag;
    kv_end = lim < p.Sk ? lim : p.Sk;
  }
  const int n_kv = (kv_end + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&pv_done[s], 1);
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
      mbar_arrive_expect_tx(&q_full, kTileBytes);
      tc::tma_load_4d(q_smem, &map_q, &q_full, 0, q0, h, b);
      tc::tma_load_4d(q_smem + kHalfBytes, &map_q, &q_full, 64, q0, h, b);
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
      const uint32_t q_addr = smem_u32(q_smem);
      // S_j = Q K_j^T: both operands K-major, 8 steps of 16 along the head dimension;
      // a step moves 32 bytes inside the 128-byte swizzled row, 4 steps per 64-column box
      auto issue_qk = [&](int buf, int stage) {
        const uint32_t k_addr = smem_u32(k_smem + (size_t)stage * kTileBytes);
        const uint32_t d = tmem_base + (buf ? kColS1 : kColS0);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
          tc::mma_ss(d, tc::smem_desc(q_addr + off, 16, 1024), tc::smem_desc(k_addr + off, 16, 1024),
                     idesc_qk, ks > 0);
        }
      };
      // O += P_j V_j: A = P from TMEM (two 16-bit values per column, 8 columns per step),
      // B = V_j in MN-major form: 64 head-dim values (128 bytes) are contiguous, 8 keys
      // make one 1024-byte swizzle atom (stride-dimension offset), the second 64-column
      // box sits kHalfBytes further (leading-dimension offset); a step of 16 keys is two
      // atoms = 2048 bytes
      auto issue_pv = [&](int buf, int stage, bool accumulate) {
        const uint32_t v_addr = smem_u32(v_smem + (size_t)stage * kTileBytes);
        const uint32_t a = tmem_base + (buf ? kColS1 : kColS0);
        const uint32_t d = tmem_base + kColO;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          tc::mma_ts(d, a + ks * 8, tc::smem_desc(v_addr + ks * 2048, kHalfBytes, 1024), idesc_pv,
                     (accumulate || ks > 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(&q_full, 0, &failed);
      if (ok && n_kv > 0) ok = mbar_wait(&k_full[0], 0, &failed);
      if (ok && n_kv > 0) {
        tc::fence_after_sync();
        issue_qk(0, 0);
        tc::mma_commit(&s_full[0]);
        tc::mma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int s1 = (j + 1) & 1, n1 = (j + 1) >> 1;
          ok = mbar_wait(&k_full[s1], n1 & 1, &failed);
          // buffer s1 still holds P_{j-1} until O += P_{j-1} V_{j-1} has finished
          if (ok && j >= 1) ok = mbar_wait(&pv_done[s1], ((j - 1) >> 1) & 1, &failed);
          if (!ok) break;
          tc::fence_after_sync();
          issue_qk(s1, s1);
          tc::mma_commit(&s_full[s1]);
          tc::mma_commit(&k_empty[s1]);
        }
        const int s = j & 1, n = j >> 1;
        ok = mbar_wait(&p_full[s], n & 1, &failed);
        if (ok) ok = mbar_wait(&v_full[s], n & 1, &failed);
        if (!ok) break;
        tc::fence_after_sync();
        issue_pv(s, s, j > 0);
        tc::mma_commit(&pv_done[s]);
        tc::mma_commit(&v_empty[s]);
      }
      if (!ok) failed = 1;
    }
    __syncwarp();
  } else {
    // ----------------------------------------------------------- softmax + epilogue
    const int quad = warp & 3;               // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;        // row of the query tile
    const int qi = q0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    float m_used = -INFINITY;  // reference maximum (scaled, log2 domain)
    float l = 0.f;             // running sum of exp2(s - m_used)
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1, n = j >> 1;
      if (!__all_sync(kFull, mbar_wait(&s_full[s], n & 1, &failed))) {
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const uint32_t s_addr = lane_addr + (s ? kColS1 : kColS0);
      float v[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c)
        tc::tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
      tc::tmem_wait_ld();

      const int col0 = j * BN;
      const bool edge = (col0 + BN > p.Sk) || (p.causal && (col0 + BN - 1 > q0 + diag));
      float mx = -INFINITY;
      if (edge) {
        const int lim = p.causal ? (qi + diag < p.Sk - 1 ? qi + diag : p.Sk - 1) : p.Sk - 1;
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          v[c] = (col0 + c <= lim) ? v[c] * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, v[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          v[c] *= p.scale_log2;
          mx = fmaxf(mx, v[c]);
        }
      }
      // lazy rescale: move the reference maximum only when it would grow by > 2^8
      const bool grow = mx > m_used + kRescaleThreshold;  // also true for the first tile
      if (__any_sync(kFull, grow)) {
        const float m_new = grow ? mx : m_used;
        const float factor = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        l *= grow ? factor : 1.f;
        if (j > 0) {
          // O may only be touched once O += P_{j-1} V_{j-1} has completed
          if (!__all_sync(kFull, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, &failed))) {
            ok = false;
            break;
          }
          tc::fence_after_sync();
          const float f = grow ? factor : 1.f;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tc::tmem_ld32(lane_addr + kColO + c * 32, o);
            tc::tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tc::tmem_st32(lane_addr + kColO + c * 32, o);
          }
          tc::tmem_wait_st();
        }
        m_used = m_new;
      }
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
      float sum = 0.f;
      uint32_t pk[BN / 2];
#pragma unroll
      for (int c = 0; c < BN; c += 2) {
        const float p0 = fast_exp2(v[c] - mref);
        const float p1 = fast_exp2(v[c + 1] - mref);
        sum += p0 + p1;
        pk[c / 2] = pack_pair(p0, p1, IS_BF16);
      }
      l += sum;
      // P_j overwrites the first 64 columns of the S buffer it came from
#pragma unroll
      for (int c = 0; c < BN / 64; ++c)
        tc::tmem_st32(s_addr + c * 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[c * 32]));
      tc::tmem_wait_st();
      tc::fence_before_sync();
      tc::mbar_arrive(&p_full[s]);
    }

    if (ok && n_kv > 0) {
      const int jl = n_kv - 1;
      ok = mbar_wait(&pv_done[jl & 1], (jl >> 1) & 1, &failed);
    }
    ok = __all_sync(kFull, ok);
    if (ok) {
      tc::fence_after_sync();
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      const bool live = qi < p.Sq;
      unsigned char* orow = reinterpret_cast<unsigned char*>(p.o) +
                            2 * ((long long)b * p.o_stride_b + (long long)h * p.o_stride_h +
                                 (long long)qi * p.o_stride_s);
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        if (n_kv > 0) {
          tc::tmem_ld32(lane_addr + kColO + c * 32, o);
          tc::tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0;
        }
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

// cuTensorMapEncodeTiled, fetched through the runtime so the library does not link libcuda
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [B, H, S, 128] view with arbitrary (16-byte multiple) strides: dims (d, s, h, b),
// box = 64 x 128 x 1 x 1 elements with the 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int is_bf16, int B, int H, int S, long long sb,
             long long sh, long long ss) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return IXB_ERR_CUDA;
  const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)BN, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IXB_OK : IXB_ERR_ARG;
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
  if (int st = make_map(&mq, q, is_bf16, B, H, Sq, q_strides[0], q_strides[1], q_strides[2])) return st;
  if (int st = make_map(&mk, k, is_bf16, B, H, Sk, k_strides[0], k_strides[1], k_strides[2])) return st;
  if (int st = make_map(&mv, v, is_bf16, B, H, Sk, v_strides[0], v_strides[1], v_strides[2])) return st;
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
  const dim3 grid((Sq + BM - 1) / BM, B * H);
  auto kern = is_bf16 ? fa_fwd_kernel<true> : fa_fwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return ixb_host::cuda_status(e);
  kern<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(mq, mk, mv, p);
  return ixb_host::cuda_status(cudaGetLastError());
}
