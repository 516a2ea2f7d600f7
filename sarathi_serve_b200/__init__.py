"""B200-native (sm_100a) implementation of Sarathi-Serve's tensor-parallel
decoder-layer hot path, behind the reference's layer-module and ops API.

Sub-modules are imported lazily by their users; importing the package does not
load the CUDA library (``sarathi_serve_b200._native.lib()`` does, loudly)."""

__version__ = "0.1.0"
