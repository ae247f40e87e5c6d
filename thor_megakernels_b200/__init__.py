"""B200-native decode megakernel behind the thor-megakernels Python surface.

Sub-modules mirror the reference package layout: ``instructions``, ``scheduler``,
``demos.latency.{instructions,scheduler,mk}``, ``dispatch``, ``mk``,
``generators``, ``llama``.  ``runtime`` is the ctypes handle over the C-ABI
library ``libb200mk.so`` built from ``csrc/``.
"""

__version__ = "0.1.0"
