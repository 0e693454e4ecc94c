"""wein-b200: sm_100a kernels for wein's MTP draft -> verify -> accept path.

The product is the C-ABI shared library ``libwein_b200.so`` (declared in
``include/wein_b200.h``).  This package is the Python-side harness around it:
``inferulm_b200.lib`` loads the library and fails loudly when it is missing,
``inferulm_b200.ops`` mirrors the reference's Op traits one to one, and
``inferulm_b200.engine`` drives the speculative step.
"""
from .lib import load, LibraryMissing  # noqa: F401
