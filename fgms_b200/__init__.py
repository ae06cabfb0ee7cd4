"""fgms_b200 — B200-native backend for the FGMS fused gather-GEMM-scatter sparse convolution.

``fgms_b200.backend`` (also importable as ``FGMS.backend``) holds the three operator entry
points; ``fgms_b200.maps`` / ``fgms_b200.clouds`` build kernel maps and synthetic inputs on the
host.  Importing ``fgms_b200.backend`` needs the compiled ``libfgms_b200.so``
(``python -m fgms_b200.build``); nothing falls back to the CPU.
"""
__version__ = "0.1"
