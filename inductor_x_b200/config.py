"""Backend configuration and B200 device parameters.

Counterpart of ``inductor_x/config.py:6-28`` (flags, core counts, the 32-byte alignment
unit) and ``inductor_x/codegen/triton_utils.py:6-27`` (bytes per element).  Unlike the
reference this module does not mutate ``torch._inductor.config`` at import.
"""
import os

import torch

# -- flags -------------------------------------------------------------------------------
#: register the backend for device "cuda" when the package is imported
register_on_import = os.environ.get("IXB_REGISTER", "1") != "0"
#: print ms / GB / GB/s for every generated kernel launch (the reference's
#: NPUDebugAutotuner, inductor_x/npu_triton_heuristics.py:268-299)
profile_bandwidth = os.environ.get("IXB_PROFILE_BANDWIDTH", "0") == "1"
#: keep Inductor's own two-kernel split of long reductions everywhere (the reference forces
#: num_splits == 1, inductor_x/codegen/ir.py:13-24).  Off: a reduction with at least
#: ``min_kept_for_single_kernel`` outputs stays one kernel and is split over a thread-block
#: cluster on chip instead.
allow_multilayer_reduction = os.environ.get("IXB_MULTILAYER_REDUCTION", "0") == "1"
min_kept_for_single_kernel = 32
#: one exchange for LayerNorm-style (mean, m2) statistics by merging partial statistics.
#: Off by default: on the bf16 softmax->LayerNorm chain at 16384 x 4096 the merged form
#: measured slower (106 us -> 151 us) - the divisions of the merge cost more than the
#: barrier they save - and the reference's variance is the two-pass form anyway.
merged_welford = os.environ.get("IXB_MERGED_WELFORD", "0") == "1"
#: softmax's (max, sum of exp) from one exchange: every thread sums relative to its own
#: maximum, keeps its exponentials for the normalisation that follows, and later row sums
#: that are linear in them (a mean after the softmax) ride in the same exchange.
merged_online_softmax = os.environ.get("IXB_MERGED_ONLINE_SOFTMAX", "1") == "1"
#: measure the launch shapes of large generated row kernels on their first call and keep the
#: fastest (decision cached on disk beside the compiled modules); kernels that stream less
#: than ``autotune_min_bytes`` keep the static choice
autotune = os.environ.get("IXB_AUTOTUNE", "1") == "1"
autotune_min_bytes = int(os.environ.get("IXB_AUTOTUNE_MIN_BYTES", str(32 << 20)))
autotune_max_candidates = int(os.environ.get("IXB_AUTOTUNE_MAX_CANDIDATES", "5"))
autotune_launches = 20
#: a candidate launch shape whose kernel spills more than this many bytes is not measured
autotune_spill_bytes = 32
autotune_verbose = os.environ.get("IXB_AUTOTUNE_VERBOSE", "0") == "1"
compile_threads = int(os.environ.get("IXB_COMPILE_THREADS", str(min(8, os.cpu_count() or 1))))
#: in dry-run mode, also build every candidate launch shape (used by the build step that
#: prepares modules on a machine without a GPU)
prebuild_candidates = os.environ.get("IXB_PREBUILD_CANDIDATES", "0") == "1"
#: generate kernels that check every data-dependent index against the extent it addresses;
#: an out-of-range index is reported by the launcher as an IndexError (and replaced by 0 on
#: the device, so nothing faults).  Off by default, as in eager mode.
debug_bounds = os.environ.get("IXB_DEBUG_BOUNDS", "0") == "1"
#: float64 buffers: the templates compute every floating value in fp32, so a graph that
#: reads or writes float64 is refused unless this is set (then it is computed in fp32)
fp64_as_fp32 = os.environ.get("IXB_FP64_AS_FP32", "0") == "1"
#: float32 attention operands: the tensor-core kernel takes 16-bit operands, so a float32
#: graph is matched (and narrowed to float16) only with this set
attention_fp32_as_fp16 = os.environ.get("IXB_ATTENTION_FP32_AS_FP16", "0") == "1"
#: compile generated kernels but never launch them (host-logic tests without a GPU)
dry_run = os.environ.get("IXB_DRY_RUN", "0") == "1"
#: where generated functor modules are cached
#: (inside the package by default, so that modules built ahead of time travel with it)
cache_dir = os.environ.get("IXB_CACHE_DIR") or os.path.join(
    os.path.dirname(os.path.abspath(__file__)), "_jit_cache")

# -- device parameters (B200) -------------------------------------------------------------
num_sms = 148
l2_bytes = 126 * 1024 * 1024
#: bytes of one coalesced per-thread access (the reference's npu_block is 32)
vector_bytes = 16
#: longest reduced row, in 128-bit vectors, that the persistent row template holds on chip
max_row_vectors = 1024 * 32

BYTES_PER_ELEMENT = {
    torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.float64: 8, torch.int64: 8,
    torch.int32: 4, torch.int16: 2, torch.int8: 1, torch.uint8: 1, torch.bool: 1,
}


def byte_per_numel(dtype: torch.dtype) -> int:
    return BYTES_PER_ELEMENT[dtype]


def get_aligned_numel(dtype: torch.dtype) -> int:
    """Elements per 128-bit vector (the reference returns elements per 32-byte block)."""
    return vector_bytes // byte_per_numel(dtype)
