// Library-level entry points of the C ABI: version, error strings, device facts and the
// launch-config chooser.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "host.h"

namespace ixb_host {

static thread_local char g_last_error[256] = "";

int cuda_status(cudaError_t e) {
  if (e == cudaSuccess) return IXB_OK;
  std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", cudaGetErrorName(e),
                cudaGetErrorString(e));
  return IXB_ERR_CUDA;
}

static constexpr int kMaxDevices = 64;
static ixb_devinfo g_dev[kMaxDevices];
static std::atomic<int> g_dev_ready[kMaxDevices];
static std::mutex g_dev_mutex;

static int fill_device(int device, ixb_devinfo* out) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return cuda_status(e);
  std::memset(out, 0, sizeof(*out));
  out->sm_count = prop.multiProcessorCount;
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->max_threads_per_sm = prop.maxThreadsPerMultiProcessor;
  out->l2_bytes = prop.l2CacheSize;
  out->smem_per_block_optin = (int64_t)prop.sharedMemPerBlockOptin;
  out->global_mem_bytes = (int64_t)prop.totalGlobalMem;
  out->vector_bytes = 16;
  return IXB_OK;
}

static const ixb_devinfo* device_entry(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  if (!g_dev_ready[device].load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    if (!g_dev_ready[device].load(std::memory_order_relaxed)) {
      if (fill_device(device, &g_dev[device]) != IXB_OK) return nullptr;
      g_dev_ready[device].store(1, std::memory_order_release);
    }
  }
  return &g_dev[device];
}

const ixb_devinfo* current_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
  return device_entry(device);
}

bool choose_row(int64_t cols, int elsize, int max_vpt, ixb_cfg* cfg) {
  const int vec = 16 / elsize;
  const int64_t nvec = (cols + vec - 1) / vec;
  // instantiated (team, vpt) pairs in order of preference for a given row length
  static const int pairs[][2] = {{32, 1},  {32, 2},  {32, 4},  {64, 4},   {128, 2},  {128, 4},
                                 {256, 2}, {256, 4}, {512, 2}, {512, 4}, {1024, 4}, {1024, 8}};
  // Prefer the pair with the least padding; among equals, two vectors per thread for
  // teams of 128+ (more warps to hide the exchange barrier), else the smaller team.
  int best = -1;
  int64_t best_cap = 0;
  for (int i = 0; i < (int)(sizeof(pairs) / sizeof(pairs[0])); ++i) {
    if (pairs[i][1] > max_vpt) continue;
    const int64_t cap = (int64_t)pairs[i][0] * pairs[i][1];
    if (cap < nvec) continue;
    if (best < 0 || cap < best_cap) {
      best = i;
      best_cap = cap;
    }
  }
  if (best < 0) return false;
  cfg->team = pairs[best][0];
  cfg->vpt = pairs[best][1];
  return true;
}

}  // namespace ixb_host

extern "C" {

int ixb_abi_version(void) { return IXB_ABI_VERSION; }

const char* ixb_strerror(int status) {
  switch (status) {
    case IXB_OK: return "ok";
    case IXB_ERR_ARG: return "invalid argument";
    case IXB_ERR_DTYPE: return "dtype not supported by this entry point";
    case IXB_ERR_ALIGN: return "pointer or pitch is not 16-byte aligned";
    case IXB_ERR_SHAPE: return "extent outside the supported range";
    case IXB_ERR_UNSUPPORTED: return "no kernel instantiated for this configuration";
    case IXB_ERR_SCRATCH: return "scratch buffer missing or too small";
    case IXB_ERR_CUDA: return "CUDA runtime error (see ixb_last_cuda_error)";
    case IXB_ERR_INDEX: return "index out of range";
    default: return "unknown status";
  }
}

const char* ixb_last_cuda_error(void) { return ixb_host::g_last_error; }

int ixb_device_info(int device, ixb_devinfo* out) {
  if (out == nullptr) return IXB_ERR_ARG;
  if (device < 0) {
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return ixb_host::cuda_status(e);
  }
  const ixb_devinfo* d = ixb_host::device_entry(device);
  if (d == nullptr) return IXB_ERR_CUDA;
  *out = *d;
  return IXB_OK;
}

int ixb_choose_config(const ixb_problem* pb, const ixb_devinfo* dev, ixb_cfg* out) {
  if (pb == nullptr || out == nullptr) return IXB_ERR_ARG;
  const int es = ixb_host::elem_size(pb->dtype);
  if (es == 0) return IXB_ERR_DTYPE;
  const int sms = (dev != nullptr && dev->sm_count > 0) ? dev->sm_count : 148;
  std::memset(out, 0, sizeof(*out));
  switch (pb->family) {
    case IXB_FAM_ROW: {
      if (pb->reduce <= 0) return IXB_ERR_SHAPE;
      // two row inputs double the prefetch registers: cap vectors per thread at 4
      const int max_vpt = pb->row_inputs > 1 ? 4 : 8;
      if (!ixb_host::choose_row(pb->reduce, es, max_vpt, out)) return IXB_ERR_SHAPE;
      out->threads = out->team >= 256 ? out->team : 256;
      return IXB_OK;
    }
    case IXB_FAM_OUTER: {
      if (pb->reduce <= 0 || pb->inner <= 0 || pb->outer <= 0) return IXB_ERR_SHAPE;
      const int vec = 16 / es;
      const int64_t nv = (pb->inner + vec - 1) / vec;
      int vc = 1;
      while (vc < 32 && vc < nv) vc <<= 1;
      const int64_t chunks = (nv + vc - 1) / vc;
      const int64_t ctas = pb->outer * chunks;
      // Split the reduced axis only when the kept extent alone cannot occupy the SMs
      // twice over and every segment still gets at least 256 rows; the reference's
      // trigger is a reduced length above 32768 (inductor_x/codegen/split_tiling.py:160).
      int rsplit = 1;
      const int64_t want = 4LL * sms;
      if (ctas < 2LL * sms && pb->reduce >= 512) {
        int64_t s = (want + ctas - 1) / ctas;
        const int64_t max_s = pb->reduce / 256;
        if (s > max_s) s = max_s;
        if (s > 64) s = 64;
        if (s < 1) s = 1;
        rsplit = (int)s;
      }
      out->rsplit = rsplit;
      out->threads = 256;
      out->vpt = vc;  // inner vectors per CTA row
      out->unroll = 8;
      out->grid = (int)(ctas * rsplit);
      return IXB_OK;
    }
    case IXB_FAM_SHORT_ROW:
      out->threads = 256;
      out->unroll = 4;
      return IXB_OK;
    case IXB_FAM_GATHER: {
      out->threads = 256;
      out->unroll = 4;
      const int64_t vecs = pb->outer * ((pb->inner + 15) / 16);
      int64_t grid = (vecs + 256LL * 4 - 1) / (256LL * 4);
      const int64_t cap = 16LL * sms;
      if (grid > cap) grid = cap;
      if (grid < 1) grid = 1;
      out->grid = (int)grid;
      return IXB_OK;
    }
    case IXB_FAM_POINTWISE:
      out->threads = 256;
      out->unroll = 4;
      return IXB_OK;
    default:
      return IXB_ERR_ARG;
  }
}

}  // extern "C"
