// Context-parallel attention merge kernels: fold the partial result of one ring step into
// the running result.  They stand where the reference keeps hand-written Triton kernels
//   tl_fn_forward_update     (test/npu_indexing/written/attn_cp_triton_kernel_3d.py:15-82)
//   tl_fn_forward_update_la  (test/npu_indexing/written/attn_cp_triton_kernel_3d_la.py:11-55)
// and the eager gradient accumulation of its ring backward
//   backward_update          (test/npu_indexing/written/test_attn_cp.py:267-287).
// All three are streaming kernels: every byte is read once and written once, 128 bits per
// thread per access, persistent grids.
#pragma once
#include "common.cuh"

namespace ixb {

// ---- (max, sum) form ------------------------------------------------------------------
// attn tensors are [S, B, H] (H = N * D, stride-1), statistics are [B, N, S, 8] fp32 with
// the 8 entries of a row holding the same value (the layout of the vendor attention op);
// `*_nstride` is the element stride of their N axis, so a slice along S of a longer buffer
// can be passed as it is.  Per (s, b, n):
//   m = max(pm, cm); ps = psum * exp(pm - m); cs = csum * exp(cm - m); l = ps + cs
//   out = prev * (ps / l) + cur * (cs / l)          (fp32 math, stored in T)
// The statistics are updated entry by entry, the attention scale uses entry 0
// (attn_cp_test.py:24-33).
// A CTA walks tiles of kCpRows consecutive s for one b.  Per tile, one thread per (head, s)
// first merges that pair's statistics (all eight entries, written out; the kCpRows entries
// of a head are adjacent in memory, so a head's statistics move as whole 128-byte lines)
// and leaves the two attention weights in shared memory; then the whole CTA streams the
// tile's rows, 128 bits per access, looking its weights up by head.  The weight buffers
// alternate between tiles, so one barrier per tile is enough.
constexpr int kCpRows = 4;

template <typename T>
__global__ void __launch_bounds__(256)
    cp_forward_update_kernel(const T* __restrict__ prev_attn, const float* __restrict__ prev_max,
                             const float* __restrict__ prev_sum, const T* __restrict__ cur_attn,
                             const float* __restrict__ cur_max, const float* __restrict__ cur_sum,
                             T* __restrict__ out_attn, float* __restrict__ out_max,
                             float* __restrict__ out_sum, int S, int B, int N, int D,
                             long long prev_nstride, long long cur_nstride, long long out_nstride,
                             int head_shift) {
  extern __shared__ float2 cp_weights[];   // [2][kCpRows][N]
  constexpr int kVec = Elem<T>::kVec;
  const int H = N * D;
  const int vec_per_row = H / kVec;
  const int vph = D / kVec;              // vectors of one head; head_shift = log2(vph) or -1
  const long long tiles = (long long)B * ((S + kCpRows - 1) / kCpRows);
  int parity = 0;
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x, parity ^= 1) {
    const int b = (int)(tile % B);
    const int s0 = (int)(tile / B) * kCpRows;
    float2* w = cp_weights + parity * kCpRows * N;
    for (int idx = threadIdx.x; idx < N * kCpRows; idx += blockDim.x) {
      const int n = idx / kCpRows, sl = idx - n * kCpRows;
      const int s = s0 + sl;
      if (s >= S) continue;
      const long long bn = (long long)b * N + n;
      const long long po = bn * prev_nstride + (long long)s * 8;
      const long long co = bn * cur_nstride + (long long)s * 8;
      const long long oo = bn * out_nstride + (long long)s * 8;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const float4 pm4 = *reinterpret_cast<const float4*>(prev_max + po + q * 4);
        const float4 cm4 = *reinterpret_cast<const float4*>(cur_max + co + q * 4);
        const float4 ps4 = *reinterpret_cast<const float4*>(prev_sum + po + q * 4);
        const float4 cs4 = *reinterpret_cast<const float4*>(cur_sum + co + q * 4);
        float4 m4, l4;
        m4.x = fmaxf(pm4.x, cm4.x);
        m4.y = fmaxf(pm4.y, cm4.y);
        m4.z = fmaxf(pm4.z, cm4.z);
        m4.w = fmaxf(pm4.w, cm4.w);
        const float psx = ps4.x * expf(pm4.x - m4.x), csx = cs4.x * expf(cm4.x - m4.x);
        l4.x = psx + csx;
        l4.y = ps4.y * expf(pm4.y - m4.y) + cs4.y * expf(cm4.y - m4.y);
        l4.z = ps4.z * expf(pm4.z - m4.z) + cs4.z * expf(cm4.z - m4.z);
        l4.w = ps4.w * expf(pm4.w - m4.w) + cs4.w * expf(cm4.w - m4.w);
        *reinterpret_cast<float4*>(out_max + oo + q * 4) = m4;
        *reinterpret_cast<float4*>(out_sum + oo + q * 4) = l4;
        if (q == 0) w[sl * N + n] = make_float2(psx / l4.x, csx / l4.x);   // entry 0 scales the output
      }
    }
    __syncthreads();
#pragma unroll
    for (int sl = 0; sl < kCpRows; ++sl) {
      const int s = s0 + sl;
      if (s >= S) break;
      const long long row = (long long)s * B + b;
      const T* pa = prev_attn + row * H;
      const T* ca = cur_attn + row * H;
      T* oa = out_attn + row * H;
      const float2* wr = w + sl * N;
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        const uint4 praw = ldg_stream(pa + (long long)v * kVec);
        const uint4 craw = ldg_stream(ca + (long long)v * kVec);
        const float2 ww = wr[head_shift >= 0 ? (v >> head_shift) : (v / vph)];
        float a[kVec], c[kVec];
        unpack<T>(praw, a);
        unpack<T>(craw, c);
#pragma unroll
        for (int i = 0; i < kVec; ++i) a[i] = a[i] * ww.x + c[i] * ww.y;
        stg_stream(oa + (long long)v * kVec, pack<T>(a));
      }
    }
  }
}

// ---- log-sum-exp form, in place ---------------------------------------------------------
// attn tensors are [B, N, S, D] fp32 (D stride-1, `*_attn_nstride` = element stride of N),
// lse tensors [B, N, S] fp32.  Per (b, n, s):
//   lse = log(exp(p) + exp(c)); prev_attn = exp(p - lse) * prev_attn + exp(c - lse) * cur_attn
//   prev_lse = lse
// The sum of exponentials is taken relative to max(p, c), which is the same value without
// the overflow of the literal form.
__global__ void __launch_bounds__(256)
    cp_forward_update_lse_kernel(float* __restrict__ prev_attn, float* __restrict__ prev_lse,
                                 const float* __restrict__ cur_attn, const float* __restrict__ cur_lse,
                                 int BN, int S, int D, long long prev_attn_nstride,
                                 long long prev_lse_nstride, long long cur_attn_nstride,
                                 long long cur_lse_nstride) {
  // one warp per (b, n, s) row: every lane reads the row's old lse before lane 0 replaces it
  const int vec_per_row = D / 4;
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)BN * S;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const long long bn = r / S;
    const int s = (int)(r - bn * S);
    float* lse_slot = prev_lse + bn * prev_lse_nstride + s;
    const float p = *lse_slot;
    const float c = cur_lse[bn * cur_lse_nstride + s];
    __syncwarp();
    const float m = fmaxf(p, c);
    const float lse = (m == -INFINITY) ? -INFINITY : m + logf(expf(p - m) + expf(c - m));
    const float wp = (lse == -INFINITY) ? 0.f : expf(p - lse);
    const float wc = (lse == -INFINITY) ? 0.f : expf(c - lse);
    float* pa = prev_attn + bn * prev_attn_nstride + (long long)s * D;
    const float* ca = cur_attn + bn * cur_attn_nstride + (long long)s * D;
    for (int v = lane; v < vec_per_row; v += 32) {
      float4 a = *reinterpret_cast<const float4*>(pa + v * 4);
      const uint4 craw = ldg_stream(ca + v * 4);
      a.x = wp * a.x + wc * __uint_as_float(craw.x);
      a.y = wp * a.y + wc * __uint_as_float(craw.y);
      a.z = wp * a.z + wc * __uint_as_float(craw.z);
      a.w = wp * a.w + wc * __uint_as_float(craw.w);
      *reinterpret_cast<float4*>(pa + v * 4) = a;
    }
    if (lane == 0) *lse_slot = lse;
  }
}

// ---- gradient accumulation: acc += cur, fp32 add, rounded to T (torch's add_ on 16-bit) ---
template <typename T>
__global__ void __launch_bounds__(256)
    accumulate_kernel(T* __restrict__ acc, const T* __restrict__ cur, long long nvec) {
  constexpr int kVec = Elem<T>::kVec;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < nvec; g += stride) {
    float a[kVec], c[kVec];
    unpack<T>(*reinterpret_cast<const uint4*>(acc + g * kVec), a);
    unpack<T>(ldg_stream(cur + g * kVec), c);
#pragma unroll
    for (int i = 0; i < kVec; ++i) a[i] += c[i];
    *reinterpret_cast<uint4*>(acc + g * kVec) = pack<T>(a);
  }
}

}  // namespace ixb
