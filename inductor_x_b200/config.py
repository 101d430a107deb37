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
#: keep Inductor's own multi-layer split of long reductions (the reference forces
#: num_splits == 1, inductor_x/codegen/ir.py:13-24)
allow_multilayer_reduction = True
#: one exchange for LayerNorm-style (mean, m2) statistics by merging partial statistics,
#: and one for softmax's (max, sum of exp), instead of one exchange per plain reduction.
#: Off by default: on the bf16 softmax->LayerNorm chain at 16384 x 4096 the merged forms
#: measured slower (106 us -> 151 us and 115 us) - the extra shuffles and divisions of the
#: merge cost more than the barrier they save.
merged_welford = os.environ.get("IXB_MERGED_WELFORD", "0") == "1"
merged_online_softmax = os.environ.get("IXB_MERGED_ONLINE_SOFTMAX", "0") == "1"
#: compile generated kernels but never launch them (host-logic tests without a GPU)
dry_run = os.environ.get("IXB_DRY_RUN", "0") == "1"
#: where generated functor modules are cached
cache_dir = os.environ.get("IXB_CACHE_DIR") or os.path.join(
    os.environ.get("TORCHINDUCTOR_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache"),
    "inductor_x_b200")

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
