"""spork_b200: hand-written sm_100a (B200) GEMM and attention kernels behind the
launch interface of the akeley98/spork testbed.

The product is ``libspork_b200.so`` (a C-ABI library, ``include/spork_b200.h``).
This package is the Python face of it: ``spork_b200.api`` binds the C ABI with
ctypes and accepts torch tensors (torch is used for device memory and streams
only).  There is no CPU fallback: every call raises if the library is missing
or the device is not a B200-class GPU.
"""
from .api import (  # noqa: F401
    DATA_IDENTITY,
    DATA_NORMAL,
    DATA_NORMAL_BM,
    DATA_RANDOM,
    DATA_TILED_NUMBERS,
    DATA_UNIFORM_PM1,
    SEED_A,
    SEED_B,
    SporkError,
    attn_fwd,
    choice,
    compare_f32,
    gemm_baseline,
    init_test_data,
    last_clock_mhz,
    lib,
    library_path,
    matmul_sm100,
    matmul_sm100_batched,
    matmul_sm100_htod,
    matmul_sm100_supports,
    matmul_sm100_tf32,
    status,
    ring_model,
    tmap_cache_stats,
    stream_k_counters,
    trace,
    tune,
    tuning,
    version,
)
