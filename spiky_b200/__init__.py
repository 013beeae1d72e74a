"""spiky_b200 - B200-native (sm_100a) implementation of the LUT-layer hot path.

Public surface (drop-in for the reference's ``spiky.lut``): :mod:`spiky_b200.lut_layer` and
:mod:`spiky_b200.lut_transformer`.  The compute path is the C-ABI CUDA library
``libspiky_b200.so`` (include/spiky_b200.h); there is no CPU or PyTorch fallback.
"""
__version__ = "0.1.0"
