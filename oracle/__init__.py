"""CPU oracle for the verify-step hot path: TEST INFRASTRUCTURE ONLY.

`oracle.binding` loads `libsz_oracle.so` (built by `make -C oracle`) through ctypes.  Only tests/, the smoke check
and the CPU-baseline leg of bench.py may import this package; the CUDA library never does.
"""
