"""fusedmm_b200 -- B200-native FusedMM (the ``fusedMM_csr`` operation of HipGraph/FusedMM) as hand-written
sm_100a CUDA kernels behind a C ABI, plus the Python mirror of that ABI.

The compute lives in ``fusedmm_b200/lib/libfusedmm_b200.so`` (sources in ``fusedmm_b200/csrc``, interface in
``include/fusedmm_b200.h``).  Importing this package does not load it; :func:`fusedmm_b200.api.lib` does and
raises if it has not been built -- there is no fallback implementation.
"""
from . import messages  # noqa: F401
from .api import fusedMM_csr, lib, call_info, set_sop, set_option, get_option, FusedMMError  # noqa: F401
