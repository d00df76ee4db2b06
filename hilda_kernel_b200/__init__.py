"""hilda_kernel_b200: the token-parallel operator path of hilda-kernel on hand-written sm_100a
CUDA kernels, behind the reference's Python API (``hilda_*`` functions, autograd Functions and
nn.Modules). ``from hilda_kernel_b200 import hilda_rms_norm`` or, as with the reference,
``from hilda_kernel_b200.kernels.rms_norm import hilda_rms_norm``."""
from .kernels import *  # noqa: F401,F403
from .kernels import __all__ as _kernel_names

__all__ = list(_kernel_names)
__version__ = "0.1.0"
