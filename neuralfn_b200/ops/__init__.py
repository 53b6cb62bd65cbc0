"""Kernel front-ends. CUDA paths call the hand-written sm_100a library through
ctypes; each op also carries a plain PyTorch fp32 reference used by the tests
and by CPU execution."""
