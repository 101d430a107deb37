"""inductor_x_b200 - a B200 (sm_100a) TorchInductor backend.

Drop-in for the registration surface of BD-Seed-HHW/inductor-x (imported there as
``inductor_npu``): importing the package registers the backend for CUDA devices, the way
``inductor_x/__init__.py:16-58`` does for ``"npu"``.  Underneath, kernels come from
hand-written CUDA templates in ``libixb.so`` instead of generated Triton.
"""
from . import runtime  # noqa: F401
from . import ops  # noqa: F401
from .runtime import raw_stream as get_current_raw_stream  # noqa: F401

__all__ = ["ops", "runtime", "get_current_raw_stream"]
