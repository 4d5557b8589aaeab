"""B200-native quantised Linear (FP8 e4m3 / NVFP4) behind EmbodiInfer's operator-registry API.

The compute path is hand-written sm_100a CUDA in ``csrc/`` reached through the C ABI declared in
``include/embodiinfer_b200.h``; this package is the PyTorch host side: registries, weight bundles
and plan objects with the reference's names, argument meaning and error behaviour.
"""

__version__ = "0.1.0"
