"""Wrapper codegen of the B200 backend.

The reference subclasses the Python wrapper to change the import header, to emit one numel
expression per axis and to never free buffers or assert input sizes
(``inductor_x/codegen/wrapper.py:3-47``).  None of those workarounds is wanted here: stock
``PythonWrapperCodegen`` is used unchanged (buffers are freed, inputs are asserted) and the
only addition - importing the kernel loader - is made by ``B200Scheduling``.
"""
from torch._inductor.codegen.wrapper import PythonWrapperCodegen


class B200WrapperCodeGen(PythonWrapperCodegen):
    pass
