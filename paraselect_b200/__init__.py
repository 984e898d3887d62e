"""B200 (sm_100a) IVF-PQ search path behind ParaSelect's view API: CUDA kernels + C ABI (csrc/, libpsb.so)
and the ctypes binding (api.py)."""
