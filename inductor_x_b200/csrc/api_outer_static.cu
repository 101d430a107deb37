// ixb_outer_reduce_static: the split outer reduction for callers that cannot hand the
// library a scratch buffer.  The fp32 partials live in a fixed array inside the library
// image instead; the entry point allocates nothing.
#include <atomic>
#include <mutex>

#include "host.h"
#include "ixb/outer.cuh"

namespace {

// Partials of the split: [rsplit][outer * inner] floats.  4 MiB per GPU that loads the
// library, held until the process exits.
constexpr size_t kStaticScratchFloats = IXB_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// `g_static_scratch` names a host-side handle here, not device memory: the device
// address has to be asked for, once per device, while that device is current.
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices];
std::atomic<int> g_scratch_ready[kMaxDevices];
std::mutex g_scratch_mutex;

int scratch_for_current_device(float** out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return ixb_host::cuda_status(e);
  if (device < 0 || device >= kMaxDevices) return IXB_ERR_ARG;
  if (!g_scratch_ready[device].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ready[device].load(std::memory_order_relaxed)) {
      float* p = nullptr;
      e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
      if (e != cudaSuccess) return ixb_host::cuda_status(e);
      if (p == nullptr) return IXB_ERR_CUDA;
      g_scratch_addr[device] = p;
      g_scratch_ready[device].store(1, std::memory_order_release);
    }
  }
  *out = g_scratch_addr[device];
  return IXB_OK;
}

template <typename T, class Op, int VC>
cudaError_t launch_partial(const T* x, float* scratch, int64_t outer, int64_t R, int64_t inner,
                           int chunks, int rsplit, cudaStream_t s) {
  const long long grid = outer * chunks * rsplit;
  ixb::outer_reduce_kernel<T, float, Op, 256, VC, 8>
      <<<(unsigned)grid, 256, 0, s>>>(x, scratch, R, inner, chunks, rsplit, outer * inner, 1.f);
  return cudaGetLastError();
}

template <typename T, class Op>
int run_op(const void* x, void* out, int64_t outer, int64_t R, int64_t inner, int rsplit,
           float post, float* scratch, cudaStream_t s) {
  constexpr int kVec = ixb::Elem<T>::kVec;
  const int64_t nv = inner / kVec;
  int vc = 1;
  while (vc < 32 && vc < nv) vc <<= 1;
  const int chunks = (int)((nv + vc - 1) / vc);
  if (outer * chunks * rsplit > 0x7fffffffLL) return IXB_ERR_SHAPE;
  const T* xt = (const T*)x;
  cudaError_t e;
  switch (vc) {
    case 1: e = launch_partial<T, Op, 1>(xt, scratch, outer, R, inner, chunks, rsplit, s); break;
    case 2: e = launch_partial<T, Op, 2>(xt, scratch, outer, R, inner, chunks, rsplit, s); break;
    case 4: e = launch_partial<T, Op, 4>(xt, scratch, outer, R, inner, chunks, rsplit, s); break;
    case 8: e = launch_partial<T, Op, 8>(xt, scratch, outer, R, inner, chunks, rsplit, s); break;
    case 16: e = launch_partial<T, Op, 16>(xt, scratch, outer, R, inner, chunks, rsplit, s); break;
    default: e = launch_partial<T, Op, 32>(xt, scratch, outer, R, inner, chunks, rsplit, s); break;
  }
  if (e != cudaSuccess) return ixb_host::cuda_status(e);
  const int64_t out_numel = outer * inner;
  ixb::outer_reduce_finalize_kernel<T, Op><<<(unsigned)((out_numel + 255) / 256), 256, 0, s>>>(
      scratch, (T*)out, out_numel, rsplit, post);
  return ixb_host::cuda_status(cudaGetLastError());
}

template <typename T>
int run_t(int kind, const void* x, void* out, int64_t outer, int64_t R, int64_t inner, int rsplit,
          float* scratch, cudaStream_t s) {
  switch (kind) {
    case IXB_SUM: return run_op<T, ixb::SumOp>(x, out, outer, R, inner, rsplit, 1.f, scratch, s);
    case IXB_MEAN: return run_op<T, ixb::SumOp>(x, out, outer, R, inner, rsplit, 1.f / (float)R, scratch, s);
    case IXB_AMAX: return run_op<T, ixb::MaxOp>(x, out, outer, R, inner, rsplit, 1.f, scratch, s);
    case IXB_AMIN: return run_op<T, ixb::MinOp>(x, out, outer, R, inner, rsplit, 1.f, scratch, s);
    default: return IXB_ERR_UNSUPPORTED;
  }
}

}  // namespace

extern "C" int ixb_outer_reduce_static(int dtype, int kind, const void* x, void* out,
                                       int64_t outer, int64_t R, int64_t inner, int rsplit,
                                       ixb_stream stream) {
  if (outer < 0 || R <= 0 || inner < 0 || rsplit < 1) return IXB_ERR_ARG;
  if (outer == 0 || inner == 0) return IXB_OK;
  if (x == nullptr || out == nullptr) return IXB_ERR_ARG;
  if (dtype != IXB_F32 && dtype != IXB_F16 && dtype != IXB_BF16) return IXB_ERR_DTYPE;
  const int es = ixb_host::elem_size(dtype);
  if (inner % (16 / es) != 0 || !ixb_host::aligned16(x)) return IXB_ERR_ALIGN;
  if (rsplit > R) rsplit = (int)R;
  // the partials must fit the fixed array: refuse anything larger, never spill over.  Each
  // factor is checked against what is left of the capacity, so the product cannot wrap.
  const unsigned long long cap = kStaticScratchFloats;
  if ((unsigned long long)outer > cap || (unsigned long long)inner > cap / (unsigned long long)outer ||
      (unsigned long long)rsplit > cap / ((unsigned long long)outer * (unsigned long long)inner))
    return IXB_ERR_SCRATCH;
  float* scratch = nullptr;
  if (int st = scratch_for_current_device(&scratch)) return st;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case IXB_F32: return run_t<float>(kind, x, out, outer, R, inner, rsplit, scratch, s);
    case IXB_F16: return run_t<ixb::f16>(kind, x, out, outer, R, inner, rsplit, scratch, s);
    default: return run_t<ixb::bf16>(kind, x, out, outer, R, inner, rsplit, scratch, s);
  }
}
