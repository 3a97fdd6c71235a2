"""Top-level module name of the reference project (``import block_linear``), bound to the implementation in
the ``blockwise_int8_linear_b200`` package: both names are the same module object, so assigning a knob through
either one is seen by the other."""
import sys

from blockwise_int8_linear_b200 import block_linear as _impl

sys.modules[__name__] = _impl
