"""mixlab_b200 - B200 (sm_100a) kernels for mixlab's gated-delta and Mamba-3 scans.

The product is ``libmixlab_b200.so`` (C ABI in ``include/mixlab_b200.h``).  This
package is a thin ctypes binding plus a torch-tensor front end used by the
tests and the benchmark; torch only provides device memory and streams.
"""
from ._lib import lib, load_library, MxbError, GdnDesc, Mamba3Desc, MXB_F32, MXB_BF16  # noqa: F401
from . import ops  # noqa: F401
