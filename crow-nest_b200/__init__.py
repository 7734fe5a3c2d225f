"""crownest_b200: sm_100a kernels for the quantized GEMV / MoE decode path, behind a C ABI.

The directory name carries a hyphen, so the importable name is ``crownest_b200`` (the shim
package beside it points here).
"""
from ._lib import CN_BF16, CN_F32, CN_MAX_M, CrownestError, build, device_status, lib  # noqa: F401
