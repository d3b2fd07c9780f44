"""B200-native constant folding for the NPU compiler's Const dialect: the ContentAttr
transformation chain and weight compression as sm_100a CUDA kernels behind a C ABI
(include/b200const.h).  `const` mirrors the reference's host API; `_cabi` is the raw binding."""
from . import _cabi  # noqa: F401
from . import const  # noqa: F401

__all__ = ["_cabi", "const"]
