// Persistent row template: the whole reduced axis of one row lives in the registers of
// a "team" of threads, so a chain of reductions with pointwise stages between them
// (softmax -> layer-norm, RMSNorm, fused pointwise + row-sum ...) costs one read and at
// most one write of HBM.  It replaces the reference's persistent and looped inner
// reductions (inductor_x/codegen/triton.py:1163-1253), which re-read the row per pass.
//
// Work split: a team of TEAM threads owns one row at a time; thread t holds the 128-bit
// vectors t, t+TEAM, ... (VPT of them), so every load instruction of a warp covers 512
// contiguous bytes.  CTAs are persistent: a grid sized to the resident capacity of the
// 148 SMs strides over the rows, and the raw vectors of the next row are requested
// before the current row is processed so HBM latency overlaps the arithmetic.
//
// A Body supplies the math:
//   using in_t            element type of the row-shaped inputs
//   struct Params         plain-old-data kernel argument
//   kRowInputs            number of row-shaped inputs prefetched by the template
//   row_ptr(p, k)         base pointer of row input k
//   init(p, ctx)          once per thread (cache per-column constants)
//   row(p, ctx, r, raw)   process row r given its raw vectors raw[k][i]
#pragma once
#include <type_traits>

#include "common.cuh"

namespace ixb {

template <typename T, int TEAM, int TEAMS, int VPT, bool ALIGNED> struct RowCtx {
  static constexpr int kVec = Elem<T>::kVec;
  static constexpr bool kAligned = ALIGNED;
  static constexpr int kTeam = TEAM;
  static constexpr int kVpt = VPT;
  static constexpr int kWarpsPerTeam = TEAM / 32;

  int lane;   // thread index inside the team
  int team;   // team index inside the CTA
  int cols;   // row length in elements
  int phase;  // ping-pong slot of the exchange buffer
  float* red; // shared exchange buffer of this team: [2 phases][kWarpsPerTeam][4 floats]

  // first column of the i-th vector held by this thread
  __device__ __forceinline__ int vec_col(int i) const { return (lane + i * TEAM) * kVec; }
  __device__ __forceinline__ bool valid(int i) const { return vec_col(i) < cols; }
  // element j of vector i lies inside the row.  With ALIGNED rows (length a multiple of
  // the vector width, 16-byte aligned base) validity is per vector and hoists out of the
  // element loops; otherwise it is per element and access falls back to scalar.
  __device__ __forceinline__ bool ok(int i, int j) const {
    return ALIGNED ? valid(i) : (vec_col(i) + j < cols);
  }
  // Load / store vector i of a row-shaped operand whose row starts at `base`.
  template <bool STREAM = true> __device__ __forceinline__ uint4 load(const T* base, int i) const {
    if constexpr (ALIGNED) {
      if (!valid(i)) return make_uint4(0, 0, 0, 0);
      return STREAM ? ldg_stream(base + vec_col(i)) : ldg_keep(base + vec_col(i));
    } else {
      union {
        uint4 u;
        T e[kVec];
      } v;
      v.u = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int j = 0; j < kVec; ++j)
        if (vec_col(i) + j < cols) v.e[j] = base[vec_col(i) + j];
      return v.u;
    }
  }
  __device__ __forceinline__ void store(T* base, int i, const float* vals) const {
    if constexpr (ALIGNED) {
      if (valid(i)) stg_stream(base + vec_col(i), pack<T>(vals));
    } else {
#pragma unroll
      for (int j = 0; j < kVec; ++j)
        if (vec_col(i) + j < cols) base[vec_col(i) + j] = Elem<T>::from_f(vals[j]);
    }
  }

  // Reduce one value per thread over the whole team; every thread gets the result.
  template <class Op> __device__ __forceinline__ float reduce(float v) {
    v = warp_reduce<Op>(v);
    if constexpr (TEAM > 32) {
      float* slot = red + phase * kWarpsPerTeam * 4;
      if ((lane & 31) == 0) slot[lane >> 5] = v;
      team_barrier(team + 1, TEAM);
      v = slot[0];
#pragma unroll
      for (int w = 1; w < kWarpsPerTeam; ++w) v = Op::combine(v, slot[w]);
      phase ^= 1;
    }
    return v;
  }
  // Two sums at once (one barrier instead of two).
  __device__ __forceinline__ float2 reduce_sum2(float a, float b) {
    a = warp_reduce<SumOp>(a);
    b = warp_reduce<SumOp>(b);
    if constexpr (TEAM > 32) {
      float2* slot = reinterpret_cast<float2*>(red + phase * kWarpsPerTeam * 4);
      if ((lane & 31) == 0) slot[lane >> 5] = make_float2(a, b);
      team_barrier(team + 1, TEAM);
      float2 r = slot[0];
#pragma unroll
      for (int w = 1; w < kWarpsPerTeam; ++w) {
        r.x += slot[w].x;
        r.y += slot[w].y;
      }
      phase ^= 1;
      return r;
    }
    return make_float2(a, b);
  }
  template <bool IS_MAX> __device__ __forceinline__ ArgPair reduce_arg(ArgPair p) {
    p = warp_reduce_arg<IS_MAX>(p);
    if constexpr (TEAM > 32) {
      // reuse the float exchange buffer: value and index halves in three floats' space
      float* slot = red + phase * kWarpsPerTeam * 4;
      if ((lane & 31) == 0) {
        slot[(lane >> 5) * 4] = p.v;
        *reinterpret_cast<long long*>(slot + (lane >> 5) * 4 + 2) = p.i;
      }
      team_barrier(team + 1, TEAM);
      ArgPair r{slot[0], *reinterpret_cast<long long*>(slot + 2)};
#pragma unroll
      for (int w = 1; w < kWarpsPerTeam; ++w) {
        ArgPair q{slot[w * 4], *reinterpret_cast<long long*>(slot + w * 4 + 2)};
        r = ArgOp<IS_MAX>::combine(r, q);
      }
      phase ^= 1;
      return r;
    }
    return p;
  }
};

template <class Body, int TEAM, int TEAMS, int VPT, bool ALIGNED>
__global__ void __launch_bounds__(TEAM* TEAMS)
    row_kernel(const typename Body::Params p, const long long rows, const int cols) {
  using T = typename Body::in_t;
  using Ctx = RowCtx<T, TEAM, TEAMS, VPT, ALIGNED>;
  constexpr int NIN = Body::kRowInputs;
  // [team][phase][warp] with 4 floats per warp so arg-reductions fit as well
  __shared__ __align__(16) float exchange[TEAMS * 2 * (TEAM / 32) * 4];

  Ctx c;
  c.lane = threadIdx.x % TEAM;
  c.team = threadIdx.x / TEAM;
  c.cols = cols;
  c.phase = 0;
  c.red = exchange + c.team * 2 * (TEAM / 32) * 4;

  typename Body::template Impl<VPT> body;
  body.init(p, c);

  const long long stride = (long long)gridDim.x * TEAMS;
  long long r = (long long)blockIdx.x * TEAMS + c.team;

  uint4 nxt[NIN][VPT];
  auto fetch = [&](long long row) {
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
      const T* base = Body::row_ptr(p, k) + row * (long long)cols;
#pragma unroll
      for (int i = 0; i < VPT; ++i) nxt[k][i] = c.load(base, i);
    }
  };
  if (r < rows) fetch(r);
  while (r < rows) {
    uint4 cur[NIN][VPT];
#pragma unroll
    for (int k = 0; k < NIN; ++k)
#pragma unroll
      for (int i = 0; i < VPT; ++i) cur[k][i] = nxt[k][i];
    const long long rn = r + stride;
    if (rn < rows) fetch(rn);
    body.row(p, c, r, cur);
    r = rn;
  }
}

// Host launcher: persistent grid = min(row groups, SMs x resident CTAs).
template <class Body, int TEAM, int TEAMS, int VPT, bool ALIGNED>
cudaError_t launch_row(const typename Body::Params& p, long long rows, int cols, int sm_count,
                       int grid_override, cudaStream_t stream) {
  auto kern = row_kernel<Body, TEAM, TEAMS, VPT, ALIGNED>;
  static int resident = 0;  // CTAs per SM; identical on every B200 of a box
  if (resident == 0) {
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, TEAM * TEAMS, 0);
    if (e != cudaSuccess) return e;
    resident = n > 0 ? n : 1;
  }
  const long long groups = (rows + TEAMS - 1) / TEAMS;
  long long grid = (long long)sm_count * resident;
  if (grid_override > 0) grid = grid_override;
  if (grid > groups) grid = groups;
  if (grid < 1) return cudaSuccess;
  kern<<<(unsigned)grid, TEAM * TEAMS, 0, stream>>>(p, rows, cols);
  return cudaGetLastError();
}

}  // namespace ixb
