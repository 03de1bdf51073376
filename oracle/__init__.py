"""TEST INFRASTRUCTURE - NOT PRODUCT CODE.

CPU checkers for the CUDA hot path: `exb_oracle` (our plain-C restatement) and `ref_lib`
(ctypes driver for the unmodified reference library when oracle/_ref has been built).
Only tests, the smoke check and the benchmark's CPU-baseline leg import this package.
"""
