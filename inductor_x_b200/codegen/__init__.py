"""Code generation of the B200 backend: index analysis, launch chooser, template
instantiator, scheduling, wrapper and the compile-once loader.

The reference's ``inductor_x/codegen/__init__.py:23-38`` applies class-level monkey patches
to stock Inductor (``Reduction.num_splits``, ``LoopBody.__call__``,
``TritonScheduling.group_fn/select_index_dtype/select_tiling``, ``TritonKernel.is_compatible``,
``SizeVarAllocator.simplify``).  Here the same decisions are overrides on the backend's own
subclasses, so importing this package changes nothing for other backends.
"""
from .scheduling import B200Scheduling  # noqa: F401
from .kernel import B200Kernel, UnsupportedByTemplates  # noqa: F401
from .wrapper import B200WrapperCodeGen  # noqa: F401
