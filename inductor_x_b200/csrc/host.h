// Host-side helpers shared by the C-ABI translation units: status plumbing, the
// per-device attribute cache and the launch-config chooser.
#pragma once
#include <cuda_runtime.h>

#include "../../include/ixb.h"

namespace ixb_host {

// Records a CUDA error for ixb_last_cuda_error() and maps it to a status code.
int cuda_status(cudaError_t e);

// Cached attributes of the current device (filled on first use, then read-only).
const ixb_devinfo* current_device();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int elem_size(int dtype) {
  switch (dtype) {
    case IXB_F32: return 4;
    case IXB_F16: return 2;
    case IXB_BF16: return 2;
    case IXB_I64: return 8;
    case IXB_I32: return 4;
    case IXB_U8: return 1;
    default: return 0;
  }
}

// Row-family chooser: smallest team that covers the row with at most `max_vpt` vectors
// per thread.  Returns false if the row does not fit the persistent form.
bool choose_row(int64_t cols, int elsize, int max_vpt, ixb_cfg* cfg);

}  // namespace ixb_host

// Dispatch over the instantiated (TEAM, VPT) pairs of the row template.  TEAMS is
// derived: CTAs are 256 threads unless a single team is larger.
#define IXB_ROW_TEAMS(TEAM_) ((TEAM_) >= 256 ? 1 : 256 / (TEAM_))
// Register budget: CTAs of 256 threads are compiled for two resident CTAs per SM (at
// most 128 registers per thread), which measured fastest for the fused bodies; larger
// CTAs take what they need.
#define IXB_ROW_MIN_CTAS(TEAM_) ((TEAM_) <= 256 ? 2 : 1)
#define IXB_ROW_CASE(BODY, TEAM_, VPT_, AL_)                                                    \
  if (cfg.team == (TEAM_) && cfg.vpt == (VPT_))                                                 \
    return ixb_host::cuda_status(                                                               \
        ixb::launch_row<BODY, TEAM_, IXB_ROW_TEAMS(TEAM_), VPT_, AL_, IXB_ROW_MIN_CTAS(TEAM_)>( \
            p, rows, (int)cols, dev->sm_count, cfg.grid, (cudaStream_t)stream));
#define IXB_ROW_DISPATCH(BODY, AL_) \
  IXB_ROW_CASE(BODY, 32, 1, AL_)    \
  IXB_ROW_CASE(BODY, 32, 2, AL_)    \
  IXB_ROW_CASE(BODY, 32, 4, AL_)    \
  IXB_ROW_CASE(BODY, 64, 4, AL_)    \
  IXB_ROW_CASE(BODY, 128, 2, AL_)   \
  IXB_ROW_CASE(BODY, 128, 4, AL_)   \
  IXB_ROW_CASE(BODY, 256, 2, AL_)   \
  IXB_ROW_CASE(BODY, 256, 4, AL_)   \
  IXB_ROW_CASE(BODY, 512, 2, AL_)   \
  IXB_ROW_CASE(BODY, 512, 4, AL_)   \
  IXB_ROW_CASE(BODY, 1024, 4, AL_)  \
  IXB_ROW_CASE(BODY, 1024, 8, AL_)
