"""CUDA sources (sm_100a), their build script and the ctypes bindings."""
