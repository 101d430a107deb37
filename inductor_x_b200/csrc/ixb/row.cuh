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
//   smem_bytes(cols, vpt) CTA-shared scratch the body wants (0 for most)
//   init(p, ctx, smem)    once per thread (cache per-column constants); ends with a
//                         CTA-wide barrier if it filled the scratch
//   row(p, ctx, r, raw)   process row r given its raw vectors raw[k][i]
#pragma once
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"

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
      if constexpr (kWarpsPerTeam % 4 == 0) {
        // the partials of four warps per 128-bit shared load
        const float4 q0 = *reinterpret_cast<const float4*>(slot);
        v = Op::combine(Op::combine(q0.x, q0.y), Op::combine(q0.z, q0.w));
#pragma unroll
        for (int w = 4; w < kWarpsPerTeam; w += 4) {
          const float4 q = *reinterpret_cast<const float4*>(slot + w);
          v = Op::combine(v, Op::combine(Op::combine(q.x, q.y), Op::combine(q.z, q.w)));
        }
      } else {
        v = slot[0];
#pragma unroll
        for (int w = 1; w < kWarpsPerTeam; ++w) v = Op::combine(v, slot[w]);
      }
      phase ^= 1;
    }
    return v;
  }
  // Online-softmax reduction: one exchange for a maximum, NS sums that were accumulated
  // relative to each thread's own maximum, and NP ordinary sums (NS + NP <= 3).
  // In: m = this thread's maximum; scaled[n] = sum of terms exp2((x - m) * k);
  // plain[n] = any partial sum.  Out: m = team maximum, scaled[n] = team totals relative
  // to it, plain[n] = team totals.  Returns this thread's factor
  // exp2((m_thread - m_team) * k), by which its own terms must be scaled.
  template <int NS, int NP>
  __device__ __forceinline__ float reduce_rescaled(float& m, float (&scaled)[NS],
                                                   float (&plain)[NP > 0 ? NP : 1], float k) {
    static_assert(NS + NP <= 3, "exchange slot holds a maximum and three sums");
    const float mt = m;
    const float mw = warp_max_fast(mt);
    float r = (mt == -INFINITY) ? 0.f : fast_exp2((mt - mw) * k);
    float v[3] = {0.f, 0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NS; ++n) v[n] = warp_reduce<SumOp>(scaled[n] * r);
#pragma unroll
    for (int n = 0; n < NP; ++n) v[NS + n] = warp_reduce<SumOp>(plain[n]);
    if constexpr (TEAM > 32) {
      float* slot = red + phase * kWarpsPerTeam * 4;
      if ((lane & 31) == 0)
        *reinterpret_cast<float4*>(slot + (lane >> 5) * 4) = make_float4(mw, v[0], v[1], v[2]);
      team_barrier(team + 1, TEAM);
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarpsPerTeam; ++w) mm = fmaxf(mm, slot[w * 4]);
      v[0] = v[1] = v[2] = 0.f;
#pragma unroll
      for (int w = 0; w < kWarpsPerTeam; ++w) {
        const float4 part = *reinterpret_cast<const float4*>(slot + w * 4);
        const float f = (part.x == -INFINITY) ? 0.f : fast_exp2((part.x - mm) * k);
        const float pv[3] = {part.y, part.z, part.w};
#pragma unroll
        for (int n = 0; n < NS; ++n) v[n] = fmaf(pv[n], f, v[n]);
#pragma unroll
        for (int n = 0; n < NP; ++n) v[NS + n] += pv[NS + n];
      }
      r *= (mw == -INFINITY) ? 0.f : fast_exp2((mw - mm) * k);
      m = mm;
      phase ^= 1;
    } else {
      m = mw;
    }
#pragma unroll
    for (int n = 0; n < NS; ++n) scaled[n] = v[n];
#pragma unroll
    for (int n = 0; n < NP; ++n) plain[n] = v[NS + n];
    return r;
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

template <class Body, int TEAM, int TEAMS, int VPT, bool ALIGNED, int MIN_CTAS = 1>
__global__ void __launch_bounds__(TEAM* TEAMS, MIN_CTAS)
    row_kernel(const typename Body::Params p, const long long rows, const int cols) {
  using T = typename Body::in_t;
  using Ctx = RowCtx<T, TEAM, TEAMS, VPT, ALIGNED>;
  constexpr int NIN = Body::kRowInputs;
  // [team][phase][warp] with 4 floats per warp so arg-reductions fit as well
  __shared__ __align__(16) float exchange[TEAMS * 2 * (TEAM / 32) * 4];
  extern __shared__ __align__(128) unsigned char body_smem[];  // Body::smem_bytes(cols, VPT)

  Ctx c;
  c.lane = threadIdx.x % TEAM;
  c.team = threadIdx.x / TEAM;
  c.cols = cols;
  c.phase = 0;
  c.red = exchange + c.team * 2 * (TEAM / 32) * 4;

  // Programmatic dependent launch: the next launch of the stream may place its CTAs as ours
  // retire (its launch latency then overlaps our tail), and we touch no global memory
  // until the launch before us has completed and flushed.  Both are no-ops for a launch
  // without the attribute.
  pdl_launch_dependents();
  pdl_wait();

  typename Body::template Impl<VPT> body;
  body.init(p, c, body_smem);

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

// Staged variant: rows arrive in a shared-memory ring filled by bulk asynchronous copies
// (one TMA instruction per row, issued by lane 0 of the team) STAGES-1 rows ahead, so the
// bytes in flight per SM no longer depend on how many registers a thread can spare for
// prefetch.  Needs ALIGNED rows: 16-byte aligned base and a row pitch that is a multiple
// of 16 bytes.  Ring layout: [team][stage][input][row bytes].
template <class Body, int TEAM, int TEAMS, int VPT, int STAGES, int MIN_CTAS>
__global__ void __launch_bounds__(TEAM* TEAMS, MIN_CTAS)
    row_staged_kernel(const typename Body::Params p, const long long rows, const int cols) {
  using T = typename Body::in_t;
  using Ctx = RowCtx<T, TEAM, TEAMS, VPT, true>;
  constexpr int NIN = Body::kRowInputs;
  extern __shared__ __align__(128) unsigned char ring_raw[];
  __shared__ __align__(16) float exchange[TEAMS * 2 * (TEAM / 32) * 4];
  __shared__ __align__(8) uint64_t full[TEAMS][STAGES];

  Ctx c;
  c.lane = threadIdx.x % TEAM;
  c.team = threadIdx.x / TEAM;
  c.cols = cols;
  c.phase = 0;
  c.red = exchange + c.team * 2 * (TEAM / 32) * 4;

  const uint32_t row_bytes = (uint32_t)cols * sizeof(T);
  // body scratch first (rounded up to 128 bytes), then the rings
  const size_t body_bytes = (Body::smem_bytes(cols, VPT) + 127) & ~(size_t)127;
  unsigned char* ring = ring_raw + body_bytes + (size_t)c.team * STAGES * NIN * row_bytes;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int t = 0; t < TEAMS; ++t)
#pragma unroll
      for (int s = 0; s < STAGES; ++s) mbar_init(&full[t][s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  typename Body::template Impl<VPT> body;
  body.init(p, c, ring_raw);

  const long long stride = (long long)gridDim.x * TEAMS;
  const long long r0 = (long long)blockIdx.x * TEAMS + c.team;

  auto issue = [&](long long row, int slot) {
    mbar_arrive_expect_tx(&full[c.team][slot], row_bytes * NIN);
#pragma unroll
    for (int k = 0; k < NIN; ++k)
      bulk_g2s(ring + ((size_t)slot * NIN + k) * row_bytes,
               Body::row_ptr(p, k) + row * (long long)cols, row_bytes, &full[c.team][slot]);
  };
  if (c.lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      const long long row = r0 + (long long)s * stride;
      if (row < rows) issue(row, s);
    }
  }

  int slot = 0;
  uint32_t parity = 0;
  bool ok = true;
  for (long long r = r0; r < rows; r += stride) {
    if (!mbar_wait(&full[c.team][slot], parity)) {
      ok = false;
      break;
    }
    uint4 cur[NIN][VPT];
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
      const unsigned char* src = ring + ((size_t)slot * NIN + k) * row_bytes;
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        cur[k][i] = c.valid(i) ? *reinterpret_cast<const uint4*>(src + (size_t)c.vec_col(i) * sizeof(T))
                               : make_uint4(0, 0, 0, 0);
    }
    // every thread of the team has taken its vectors: the slot can be refilled
    if constexpr (TEAM > 32) team_barrier(c.team + 1, TEAM); else __syncwarp();
    if (c.lane == 0) {
      const long long nr = r + (long long)STAGES * stride;
      if (nr < rows) issue(nr, slot);
    }
    body.row(p, c, r, cur);
    if (++slot == STAGES) {
      slot = 0;
      parity ^= 1;
    }
  }
  if (!ok) {
    // a wait gave up: drain what this team still has in flight (bounded) before the CTA's
    // shared memory is released, then leave
    for (int s = 0; s < STAGES; ++s) mbar_wait(&full[c.team][s], parity);
  }
}

// Per-device launch state of one kernel instantiation: the dynamic shared-memory opt-in and
// the occupancy are properties of (kernel, device), and several host threads may launch at
// once, so the cache is indexed by the current device and guarded by a mutex.
struct RowLaunchState {
  std::mutex mu;
  size_t configured[64] = {};   // largest dynamic shared-memory size opted in, per device
  size_t sized_for[64] = {};    // shared-memory size the cached occupancy was computed for
  int resident[64] = {};        // CTAs per SM (0 = not computed yet)
};
template <class K>
inline cudaError_t row_launch_capacity(RowLaunchState& st, K kern, int threads, size_t smem, int* resident) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const int d = dev & 63;
  std::lock_guard<std::mutex> lock(st.mu);
  if (smem > st.configured[d]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    st.configured[d] = smem;
    st.resident[d] = 0;
  }
  if (st.resident[d] == 0 || st.sized_for[d] != smem) {
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem);
    if (e != cudaSuccess) return e;
    if (n < 1) return cudaErrorInvalidConfiguration;
    st.resident[d] = n;
    st.sized_for[d] = smem;
  }
  *resident = st.resident[d];
  return cudaSuccess;
}

template <class Body, int TEAM, int TEAMS, int VPT, int STAGES, int MIN_CTAS>
cudaError_t launch_row_staged(const typename Body::Params& p, long long rows, int cols,
                              int sm_count, int grid_override, cudaStream_t stream) {
  auto kern = row_staged_kernel<Body, TEAM, TEAMS, VPT, STAGES, MIN_CTAS>;
  const size_t smem = ((Body::smem_bytes(cols, VPT) + 127) & ~(size_t)127) +
                      (size_t)TEAMS * STAGES * Body::kRowInputs * cols * sizeof(typename Body::in_t);
  static RowLaunchState state;
  int resident = 0;
  if (cudaError_t e = row_launch_capacity(state, kern, TEAM * TEAMS, smem, &resident)) return e;
  const long long groups = (rows + TEAMS - 1) / TEAMS;
  long long grid = (long long)sm_count * resident;
  if (grid_override > 0) grid = grid_override;
  if (grid > groups) grid = groups;
  if (grid < 1) return cudaSuccess;
  kern<<<(unsigned)grid, TEAM * TEAMS, smem, stream>>>(p, rows, cols);
  return cudaGetLastError();
}

// Host launcher: persistent grid = min(row groups, SMs x resident CTAs).
template <class Body, int TEAM, int TEAMS, int VPT, bool ALIGNED, int MIN_CTAS = 1>
cudaError_t launch_row(const typename Body::Params& p, long long rows, int cols, int sm_count,
                       int grid_override, cudaStream_t stream) {
  auto kern = row_kernel<Body, TEAM, TEAMS, VPT, ALIGNED, MIN_CTAS>;
  const size_t smem = Body::smem_bytes(cols, VPT);
  static RowLaunchState state;
  int resident = 0;
  if (cudaError_t e = row_launch_capacity(state, kern, TEAM * TEAMS, smem, &resident)) return e;
  const long long groups = (rows + TEAMS - 1) / TEAMS;
  long long grid = (long long)sm_count * resident;
  if (grid_override > 0) grid = grid_override;
  if (grid > groups) grid = groups;
  if (grid < 1) return cudaSuccess;
  return launch_pdl(kern, (unsigned)grid, TEAM * TEAMS, smem, stream, p, rows, cols);
}

}  // namespace ixb
