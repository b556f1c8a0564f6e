"""tornadovm_b200 -- host side of the ``b200/linalg`` library-task module.

Python mirror of the Java module ``tornado-b200`` (factories, provider and
native binding) over the C ABI of ``libtornado_b200.so``; see include/tornado_b200.h.
"""
from .native import B200Native, TornadoB200Error  # noqa: F401
