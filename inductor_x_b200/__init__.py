"""inductor_x_b200 - a B200 (sm_100a) TorchInductor backend.

Drop-in for the registration surface of BD-Seed-HHW/inductor-x (imported there as
``inductor_npu``).  Importing the package does for ``"cuda"`` what
``inductor_x/__init__.py:16-63`` does for ``"npu"``:

* registers the scheduling and wrapper classes (``_inductor_register_backend_for_device``),
* registers device-op overrides so that generated wrappers import
  ``get_current_raw_stream`` from this package (``NewNPUDeviceOpOverrides``),
* registers the Dynamo device interface (``NewNpuInterface``),
* applies the lowering policy and decomposition edits, and
* registers the fused-attention FX pattern.

After that ``torch.compile(fn)`` on CUDA tensors emits no Triton: every fused group becomes
an instantiation of a hand-written CUDA template, compiled once and called through the C ABI.
Set ``IXB_REGISTER=0`` to import the kernels (``inductor_x_b200.ops``) without touching
Inductor.
"""
import torch

from . import config  # noqa: F401
from . import runtime  # noqa: F401
from . import ops  # noqa: F401


def get_current_raw_stream(device=None) -> int:
    """Raw handle of the current CUDA stream (``inductor_x/__init__.py:26-27``)."""
    return torch.cuda.current_stream(device).cuda_stream


_registered = False


def _inductor_register_backend_for_device():
    from torch._inductor.codegen.common import register_backend_for_device

    from .codegen import B200Scheduling, B200WrapperCodeGen
    from .fusion_attention_graph import B200AttentionPass

    register_backend_for_device("cuda", B200Scheduling, B200WrapperCodeGen,
                                device_custom_pass=B200AttentionPass())


def _inductor_register_device_op_overrides():
    from torch._inductor.codegen.common import register_device_op_overrides
    from torch._inductor.codegen.cuda.device_op_overrides import CUDADeviceOpOverrides

    class B200DeviceOpOverrides(CUDADeviceOpOverrides):
        def import_get_raw_stream_as(self, name):
            return f"from inductor_x_b200 import get_current_raw_stream as {name}"

    register_device_op_overrides("cuda", B200DeviceOpOverrides())


def _register_device_interface():
    from torch._dynamo.device_interface import CudaInterface, register_interface_for_device

    class B200Interface(CudaInterface):
        @staticmethod
        def is_available() -> bool:
            return torch.cuda.is_available() and torch.cuda.device_count() > 0

        @staticmethod
        def is_triton_capable(device=None) -> bool:
            # generated kernels come from CUDA templates; Triton is never asked to compile
            return True

        @staticmethod
        def raise_if_triton_unavailable(device=None) -> None:
            return None

    register_interface_for_device("cuda", B200Interface)


def _enable_online_softmax_pattern():
    """Inductor rewrites softmax's max and sum into one ``online_softmax_reduce`` only when its
    own Triton backend is selected for the device; the row template has that reduction too
    (one exchange per row instead of two), so the check is widened to this backend."""
    import torch._inductor.fx_passes.post_grad as post_grad
    from torch._inductor import config as inductor_config

    def extra_check(match):
        device_type = match.kwargs["x"].meta["val"].device.type
        return inductor_config.online_softmax and (device_type == "cuda" or config.dry_run)

    post_grad.prepare_softmax_extra_check = extra_check


def _route_random_ops_to_aten():
    """Random numbers come from ATen's generators (``fallback_random``): ``rand`` / ``randn`` /
    ``randint`` / ``bernoulli`` / ``native_dropout`` stay extern kernels that draw from the same
    Philox stream as eager mode, so a compiled dropout is bit-identical to the eager one under the
    same seed.  Inductor's own seed-and-offset generator exists only inside its Triton kernels (the
    reference inherits it unchanged); the pointwise work around the random tensor is still fused
    by the templates."""
    from torch._inductor import config as inductor_config

    inductor_config.fallback_random = True


def _specialize_python_floats():
    """Python ``float`` arguments of a compiled function are baked into the graph as constants
    (Dynamo's ``specialize_float``; a new value recompiles).  Left symbolic, such a float enters
    the graph as a 0-dim float64 host tensor - with ``dynamic=True`` that happens to the softmax
    scale or the rotary scaling factor of library models - and generated kernels take device
    pointers and integer scalars only, and no float64."""
    import torch._dynamo.config as dynamo_config

    dynamo_config.specialize_float = True


def register():
    """Perform the registrations (idempotent).  Called at import unless IXB_REGISTER=0."""
    global _registered
    if _registered:
        return
    from .decomposition import _register_b200_inductor_decompositions
    from .lowering import _register_b200_inductor_fallbacks

    _inductor_register_backend_for_device()
    _inductor_register_device_op_overrides()
    _register_device_interface()
    _enable_online_softmax_pattern()
    _route_random_ops_to_aten()
    _specialize_python_floats()
    from .codegen.ir import install_num_splits

    install_num_splits()
    _register_b200_inductor_fallbacks()
    _register_b200_inductor_decompositions()
    from . import fusion_attention_graph

    fusion_attention_graph.register_fx_pass()
    _registered = True


if config.register_on_import:
    register()

__all__ = ["ops", "runtime", "config", "get_current_raw_stream", "register"]
