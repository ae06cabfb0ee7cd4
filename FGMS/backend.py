"""Drop-in module: ``from FGMS.backend import fgms_fwd_cuda, fgms_fusion_fwd_cuda, fgms_bwd_cuda``
works unchanged for callers of hkeee21/FGMS (``cpu-check.py:2``, ``cpu-check-back.py:2``,
``spconv-test.py:2``) and resolves to the B200-native implementation."""
from fgms_b200.backend import fgms_bwd_cuda, fgms_fusion_fwd_cuda, fgms_fwd_cuda  # noqa: F401
