"""ctypes binding of the CPU oracle (``libspork_oracle.so``).

Test infrastructure only: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libspork_oracle.so")

DATA_RANDOM = 0
DATA_IDENTITY = 1
DATA_TILED_NUMBERS = 2
DATA_UNIFORM_PM1 = 3
DATA_NORMAL = 4
DATA_NORMAL_BM = 5  # Box-Muller unit normal: statistically, not bitwise, the device's fixture

# The reference's two hash constants (gemm/gemm_test.cu:73,86) double as the
# seeds of the A and B operands of the uniform fixtures.
SEED_A = 20010106
SEED_B = 19980724


def build(force: bool = False) -> str:
    """Compile the oracle with the system gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "spork_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libspork_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        u16p = ctypes.POINTER(ctypes.c_uint16)
        f32p = ctypes.POINTER(ctypes.c_float)
        f64p = ctypes.POINTER(ctypes.c_double)
        L.spork_oracle_pcg3d.restype = ctypes.c_uint64
        L.spork_oracle_pcg3d.argtypes = [ctypes.c_uint32] * 3
        L.spork_oracle_half_to_float.restype = ctypes.c_float
        L.spork_oracle_half_to_float.argtypes = [ctypes.c_uint16]
        L.spork_oracle_float_to_half.restype = ctypes.c_uint16
        L.spork_oracle_float_to_half.argtypes = [ctypes.c_float]
        L.spork_oracle_fill_f16.restype = None
        L.spork_oracle_fill_f16.argtypes = [u16p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_uint32,
                                            ctypes.c_int]
        L.spork_oracle_gemm_f16f32.restype = ctypes.c_int
        L.spork_oracle_gemm_f16f32.argtypes = [ctypes.c_uint32] * 3 + [u16p, u16p, f32p]
        L.spork_oracle_gemm_f16f64.restype = ctypes.c_int
        L.spork_oracle_gemm_f16f64.argtypes = [ctypes.c_uint32] * 3 + [u16p, u16p, f64p]
        L.spork_oracle_gemm_f32.restype = ctypes.c_int
        L.spork_oracle_gemm_f32.argtypes = [ctypes.c_uint32] * 3 + [f32p, f32p, f32p, ctypes.c_int]
        L.spork_oracle_gemm_f16f32_rows.restype = ctypes.c_int
        L.spork_oracle_gemm_f16f32_rows.argtypes = [ctypes.c_uint32] * 3 + [u16p, u16p, ctypes.c_uint32,
                                                                             ctypes.c_uint32, f32p]
        L.spork_oracle_normalised_error.restype = ctypes.c_double
        L.spork_oracle_normalised_error.argtypes = [ctypes.c_uint64, f32p, f32p, ctypes.c_double, ctypes.c_double,
                                                    ctypes.c_uint32]
        L.spork_oracle_ratio_compare.restype = ctypes.c_uint64
        L.spork_oracle_ratio_compare.argtypes = [f32p, f32p, ctypes.c_uint32, ctypes.c_uint32]
        L.spork_oracle_attn_f16.restype = ctypes.c_int
        L.spork_oracle_attn_f16.argtypes = [ctypes.c_int] * 3 + [u16p, u16p, u16p, u16p, f32p, ctypes.c_float]
        L.spork_oracle_attn_bf16.restype = ctypes.c_int
        L.spork_oracle_attn_bf16.argtypes = [ctypes.c_int] * 3 + [u16p, u16p, u16p, u16p, f32p, ctypes.c_float]
        L.spork_oracle_float_to_bf16.restype = ctypes.c_uint16
        L.spork_oracle_float_to_bf16.argtypes = [ctypes.c_float]
        L.spork_oracle_bf16_to_float.restype = ctypes.c_float
        L.spork_oracle_bf16_to_float.argtypes = [ctypes.c_uint16]
        L.spork_oracle_attn_ex.restype = ctypes.c_int
        L.spork_oracle_attn_ex.argtypes = [ctypes.c_int] * 3 + [u16p, u16p, u16p, u16p, f32p, ctypes.c_float,
                                                                  ctypes.c_int, ctypes.c_int]
        L.spork_oracle_num_threads.restype = ctypes.c_int
        L.spork_oracle_set_threads.argtypes = [ctypes.c_int]
        L.spork_oracle_set_threads.restype = None
        _lib = L
    return _lib


def _u16(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))


def _f32(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _as_bits(a: np.ndarray) -> np.ndarray:
    """fp16 array (or its uint16 bit pattern) -> contiguous uint16 bits."""
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16
    return np.ascontiguousarray(a)


def num_threads() -> int:
    return int(lib().spork_oracle_num_threads())


def use_all_cores() -> int:
    """Use every core this process may run on, whatever OMP_NUM_THREADS says; returns the thread count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().spork_oracle_set_threads(n)
    return num_threads()


def pcg3d(x: int, y: int, z: int) -> int:
    return int(lib().spork_oracle_pcg3d(x & 0xFFFFFFFF, y & 0xFFFFFFFF, z & 0xFFFFFFFF))


def fill_f16(rows: int, cols: int, code: int, seed: int = 0, transpose_rule: bool = False) -> np.ndarray:
    """rows x cols fp16 fixture matrix (see ``fixture_value`` in spork_oracle.c)."""
    out = np.empty((rows, cols), dtype=np.uint16)
    if rows and cols:
        lib().spork_oracle_fill_f16(_u16(out), rows, cols, code, seed & 0xFFFFFFFF, int(transpose_rule))
    return out.view(np.float16)


def gemm_f16f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """C = A . B^T with A (M, K) and B (N, K) fp16, fp32 accumulation, k ascending."""
    A = _as_bits(a)
    B = _as_bits(b)
    M, K = A.shape
    N, K2 = B.shape
    assert K == K2
    C = np.zeros((M, N), dtype=np.float32)
    if M and N:
        rc = lib().spork_oracle_gemm_f16f32(M, N, K, _u16(A), _u16(B), _f32(C))
        if rc:
            raise MemoryError("oracle gemm allocation failed")
    return C


def gemm_f32(a: np.ndarray, b: np.ndarray, tf32_mode: int = 0) -> np.ndarray:
    """fp32 operands (the reference's type): C = A . B^T, fp32 accumulation, k ascending.
    tf32_mode 0 = plain fp32, 1 = operands truncated to tf32, 2 = operands rounded to tf32."""
    A = np.ascontiguousarray(a, dtype=np.float32)
    B = np.ascontiguousarray(b, dtype=np.float32)
    M, K = A.shape
    N, K2 = B.shape
    assert K == K2
    C = np.zeros((M, N), dtype=np.float32)
    if M and N:
        lib().spork_oracle_gemm_f32(M, N, K, _f32(A), _f32(B), _f32(C), tf32_mode)
    return C


def gemm_f16f64(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    A = _as_bits(a)
    B = _as_bits(b)
    M, K = A.shape
    N, _ = B.shape
    C = np.zeros((M, N), dtype=np.float64)
    if M and N:
        lib().spork_oracle_gemm_f16f64(M, N, K, _u16(A), _u16(B), C.ctypes.data_as(ctypes.POINTER(ctypes.c_double)))
    return C


def gemm_f16f32_rows(a: np.ndarray, b: np.ndarray, m0: int, rows: int) -> np.ndarray:
    A = _as_bits(a)
    B = _as_bits(b)
    M, K = A.shape
    N, _ = B.shape
    C = np.zeros((rows, N), dtype=np.float32)
    rc = lib().spork_oracle_gemm_f16f32_rows(M, N, K, _u16(A), _u16(B), m0, rows, _f32(C))
    if rc:
        raise ValueError(f"oracle gemm rows failed: {rc}")
    return C


def normalised_error(c: np.ndarray, ref: np.ndarray, max_abs_a: float, max_abs_b: float, K: int) -> float:
    """max|c - ref| / (max|A| max|B| K 2^-10); the headline tolerance is <= 1."""
    c = np.ascontiguousarray(c, dtype=np.float32)
    ref = np.ascontiguousarray(ref, dtype=np.float32)
    assert c.shape == ref.shape
    return float(lib().spork_oracle_normalised_error(c.size, _f32(c), _f32(ref), max_abs_a, max_abs_b, K))


def ratio_compare(a: np.ndarray, b: np.ndarray):
    """The reference's comparator; returns None if all pass, else (row, col) of the first failure."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    rows, cols = a.shape
    packed = int(lib().spork_oracle_ratio_compare(_f32(a), _f32(b), rows, cols))
    if packed == 0xFFFFFFFFFFFFFFFF:
        return None
    return packed >> 32, packed & 0xFFFFFFFF


def attn_f16(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float | None = None):
    """softmax(Q K^T scale) V per head; q, k, v are (BH, S, D) fp16.  Returns (o_fp16, o_fp32)."""
    Q = _as_bits(q)
    Kb = _as_bits(k)
    V = _as_bits(v)
    BH, S, D = Q.shape
    if scale is None:
        scale = 1.0 / float(np.sqrt(D))
    o16 = np.zeros((BH, S, D), dtype=np.uint16)
    o32 = np.zeros((BH, S, D), dtype=np.float32)
    rc = lib().spork_oracle_attn_f16(BH, S, D, _u16(Q), _u16(Kb), _u16(V), _u16(o16), _f32(o32), scale)
    if rc:
        raise RuntimeError(f"oracle attention failed: {rc}")
    return o16.view(np.float16), o32


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 bit patterns -> fp32 values."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def attn_bf16(q_bits: np.ndarray, k_bits: np.ndarray, v_bits: np.ndarray, scale: float | None = None):
    """Attention on bfloat16 inputs given as uint16 bit patterns (BH, S, D); returns (o_bf16_bits, o_fp32)."""
    Q, Kb, V = (np.ascontiguousarray(x, dtype=np.uint16) for x in (q_bits, k_bits, v_bits))
    BH, S, D = Q.shape
    if scale is None:
        scale = 1.0 / float(np.sqrt(D))
    o16 = np.zeros((BH, S, D), dtype=np.uint16)
    o32 = np.zeros((BH, S, D), dtype=np.float32)
    rc = lib().spork_oracle_attn_bf16(BH, S, D, _u16(Q), _u16(Kb), _u16(V), _u16(o16), _f32(o32), scale)
    if rc:
        raise RuntimeError(f"oracle attention failed: {rc}")
    return o16, o32


def attn_causal_f16(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float | None = None):
    """Causal attention (query i sees keys j <= i) on fp16 inputs; returns (o_fp16, o_fp32)."""
    Q, Kb, V = _as_bits(q), _as_bits(k), _as_bits(v)
    BH, S, D = Q.shape
    if scale is None:
        scale = 1.0 / float(np.sqrt(D))
    o16 = np.zeros((BH, S, D), dtype=np.uint16)
    o32 = np.zeros((BH, S, D), dtype=np.float32)
    rc = lib().spork_oracle_attn_ex(BH, S, D, _u16(Q), _u16(Kb), _u16(V), _u16(o16), _f32(o32), scale, 0, 1)
    if rc:
        raise RuntimeError(f"oracle attention failed: {rc}")
    return o16.view(np.float16), o32
