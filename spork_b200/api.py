"""ctypes binding of ``libspork_b200.so`` for torch tensors.

Function names follow the reference's launch functions (``matmul_sm90`` /
``matmul_sm80_supports`` / ``matmul_baseline`` in gemm/gemm_sm90.h:14,
gemm/gemm_sm80.h:5-6, gemm/gemm_baseline.h:5); argument meaning is that of the
harness's hot call ``GPU_Tensors{M,N,K,d_a,d_bCol,d_c,0,1,0}``
(gemm/gemm_test.cu:365): ``a`` is (M, K), ``b`` is (N, K), both fp16 and
contiguous; ``c`` is (M, N) fp32.
"""
from __future__ import annotations

import ctypes
import os
import struct

_HERE = os.path.dirname(os.path.abspath(__file__))
# SPORK_B200_LIBRARY selects another build of the library (the range-checked debug build
# libspork_b200_checked.so of `python -m spork_b200.build --checked`).
_LIB_PATH = os.environ.get("SPORK_B200_LIBRARY") or os.path.join(_HERE, "libspork_b200.so")

# Fixture codes of init_test_data: 0..2 are the reference's TestDataCode (gemm/gemm_test.h:6-11).
DATA_RANDOM, DATA_IDENTITY, DATA_TILED_NUMBERS, DATA_UNIFORM_PM1, DATA_NORMAL, DATA_NORMAL_BM = range(6)
# The reference's two hash constants (gemm/gemm_test.cu:73,86) seed the A and B operands.
SEED_A = 20010106
SEED_B = 19980724

ERR_BASE = 10000
_ERR_NAMES = {
    10001: "bad argument (null or misaligned pointer, unknown variant)",
    10002: "unsupported shape (K must be a multiple of 8)",
    10003: "current device is not an sm_100 (B200-class) GPU",
    10004: "driver call failed (tensor map encode)",
    10005: "a bounded device-side wait ran out",
    10006: "size beyond the fixed capacity of this entry point",
    10007: "a range check of the debug build failed on the device",
}


class SporkError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        detail = _ERR_NAMES.get(code, f"cudaError_t {code}" if code < ERR_BASE else "unknown")
        super().__init__(f"{what} failed with code {code}: {detail}")


def library_path() -> str:
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    """Load the C-ABI library; raises (never falls back) if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise FileNotFoundError(
                f"{_LIB_PATH} is missing: build it with `python -m spork_b200.build` (needs nvcc); "
                "there is no CPU fallback")
        L = ctypes.CDLL(_LIB_PATH)
        u32, i32, vp = ctypes.c_uint32, ctypes.c_int, ctypes.c_void_p
        L.spork_gemm_sm100_supports.argtypes = [u32, u32, u32]
        L.spork_gemm_sm100_supports.restype = i32
        L.spork_gemm_sm100_f16f32.argtypes = [u32, u32, u32, vp, vp, vp, i32, vp]
        L.spork_gemm_sm100_f16f32.restype = i32
        L.spork_gemm_sm100_tf32f32.argtypes = [u32, u32, u32, vp, vp, vp, i32, i32, vp]
        L.spork_gemm_sm100_tf32f32.restype = i32
        L.spork_gemm_sm100_f16f32_ex.argtypes = [u32, u32, u32, vp, vp, vp, i32, i32, i32, i32, vp]
        L.spork_gemm_sm100_f16f32_ex.restype = i32
        L.spork_gemm_sm100_f16f32_batched.argtypes = [u32, u32, u32, u32, vp, vp, vp, i32, i32, vp]
        L.spork_gemm_sm100_f16f32_batched.restype = i32
        L.spork_gemm_sm100_f16f32_static.argtypes = [u32, u32, u32, vp, vp, vp, i32, vp]
        L.spork_gemm_sm100_f16f32_static.restype = i32
        L.spork_selftest_bounded_wait.argtypes = [u32, vp]
        L.spork_selftest_bounded_wait.restype = i32
        L.spork_selftest_range_check.argtypes = [i32, vp]
        L.spork_selftest_range_check.restype = i32
        L.spork_gemm_sm100_last_clock_mhz.argtypes = [vp, ctypes.POINTER(ctypes.c_double)]
        L.spork_gemm_sm100_last_clock_mhz.restype = i32
        L.spork_gemm_sm100_tune.argtypes = [i32, i32, i32, i32]
        L.spork_gemm_sm100_tune.restype = i32
        L.spork_gemm_sm100_ring_model.argtypes = [u32, u32, u32, i32, i32, i32, i32, i32, i32, i32, u32, u32, i32,
                                                  ctypes.POINTER(ctypes.c_uint64)]
        L.spork_gemm_sm100_ring_model.restype = i32
        L.spork_gemm_sm100_choice.argtypes = [u32, u32, u32, i32, i32, i32, i32, ctypes.POINTER(i32)]
        L.spork_gemm_sm100_choice.restype = i32
        L.spork_gemm_sm100_tmap_cache_stats.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
        L.spork_gemm_sm100_tmap_cache_stats.restype = i32
        L.spork_gemm_sm100_stream_k_counters.argtypes = [ctypes.POINTER(u32), vp]
        L.spork_gemm_sm100_stream_k_counters.restype = i32
        L.spork_gemm_sm100_trace.argtypes = [vp, u32]
        L.spork_gemm_sm100_trace.restype = i32
        L.spork_gemm_sm100_tuning.argtypes = [ctypes.POINTER(i32), i32]
        L.spork_gemm_sm100_tuning.restype = i32
        L.spork_gemm_sm100_status.argtypes = [vp, ctypes.POINTER(u32)]
        L.spork_gemm_sm100_status.restype = i32
        L.spork_gemm_sm100_htod_f16f32.argtypes = [u32, u32, u32, vp, vp, vp]
        L.spork_gemm_sm100_htod_f16f32.restype = i32
        L.spork_init_test_data_f16.argtypes = [vp, u32, u32, i32, u32, i32, vp]
        L.spork_init_test_data_f16.restype = i32
        L.spork_init_test_data_f16_at.argtypes = [vp, u32, u32, i32, u32, i32, u32, u32, vp]
        L.spork_init_test_data_f16_at.restype = i32
        L.spork_gemm_baseline_f16f32.argtypes = [u32, u32, u32, vp, vp, vp, vp]
        L.spork_gemm_baseline_f16f32.restype = i32
        L.spork_compare_f32.argtypes = [vp, vp, u32, u32, vp, vp]
        L.spork_compare_f32.restype = i32
        if hasattr(L, "spork_attn_sm100_fwd_f16"):
            L.spork_attn_sm100_supports.argtypes = [i32, i32, i32]
            L.spork_attn_sm100_supports.restype = i32
            L.spork_attn_sm100_fwd_f16.argtypes = [i32, i32, i32, vp, vp, vp, vp, ctypes.c_float, vp]
            L.spork_attn_sm100_fwd_f16.restype = i32
            L.spork_attn_sm100_fwd_bf16.argtypes = [i32, i32, i32, vp, vp, vp, vp, ctypes.c_float, vp]
            L.spork_attn_sm100_fwd_bf16.restype = i32
            L.spork_attn_sm100_fwd_ex.argtypes = [i32, i32, i32, vp, vp, vp, vp, ctypes.c_float, i32, i32, vp]
            L.spork_attn_sm100_fwd_ex.restype = i32
            L.htod_f32_attn_sm100_fwd.argtypes = [i32, i32, vp, vp, vp, vp]
            L.htod_f32_attn_sm100_fwd.restype = None
        L.spork_b200_version.restype = ctypes.c_char_p
        _lib = L
    return _lib


def version() -> str:
    return lib().spork_b200_version().decode()


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise SporkError(rc, what)


def _stream_ptr(stream) -> int:
    import torch

    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def _dev_ptr(t, dtype, what: str) -> int:
    import torch

    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{what} must be a CUDA tensor")
    if t.dtype != dtype:
        raise TypeError(f"{what} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    return int(t.data_ptr())


class _OnDevice:
    """``with _OnDevice(t.device)``: the launch runs with that GPU current.  Nothing is switched (and nothing
    is paid) when it already is, the usual case."""

    __slots__ = ("_ctx",)

    def __init__(self, device):
        import torch

        index = device if isinstance(device, int) else torch.device(device).index
        current = torch.cuda.current_device()
        self._ctx = None if index is None or index == current else torch.cuda.device(index)

    def __enter__(self):
        if self._ctx is not None:
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            return self._ctx.__exit__(*exc)
        return False


def _same_device(first, *others) -> None:
    """All operands of a launch must live on one GPU: the kernel runs on the first one's device and would
    otherwise read or write addresses that mean nothing there."""
    for t in others:
        if t.device != first.device:
            raise ValueError(f"tensors are on different devices: {first.device} and {t.device}")


def matmul_sm100_supports(M: int, N: int, K: int) -> bool:
    return bool(lib().spork_gemm_sm100_supports(M, N, K))


def matmul_sm100(a, b, c=None, *, variant: int = 0, block_n: int | None = None, cta_group: int | None = None,
                 split_k: int = 1, max_ctas: int = 0, stream=None):
    """c[M,N] (fp32) = a[M,K] (fp16) @ b[N,K]^T (fp16); asynchronous on ``stream``.

    ``variant`` 0/64/128/256 picks the output-tile width like the reference's
    n64/n128/n256 kernels.  ``block_n``/``cta_group``/``split_k``/``max_ctas``
    select the explicit-tunables entry point instead; ``split_k=0`` alone leaves
    tile and K mode (whole tiles, split-K or stream-K) to the library.
    """
    import torch

    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if c is None:
        c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    if tuple(c.shape) != (M, N):
        raise ValueError(f"c must be {(M, N)}, got {tuple(c.shape)}")
    _same_device(a, b, c)
    pa = _dev_ptr(a, torch.float16, "a")
    pb = _dev_ptr(b, torch.float16, "b")
    pc = _dev_ptr(c, torch.float32, "c")
    with _OnDevice(a.device):
        sp = _stream_ptr(stream)
        if block_n is None and cta_group is None and split_k == 1 and max_ctas == 0:
            rc = lib().spork_gemm_sm100_f16f32(M, N, K, pa, pb, pc, variant, sp)
        else:
            bn = block_n if block_n is not None else (variant or (64 if N <= 64 else 128 if N <= 128 else 256))
            cg = cta_group or 2
            if block_n is None and cta_group is None and variant == 0 and split_k == 0:
                cg = 0  # fully automatic: the library picks the tile and the K mode
            rc = lib().spork_gemm_sm100_f16f32_ex(M, N, K, pa, pb, pc, bn, cg, split_k, max_ctas, sp)
    _check(rc, "spork_gemm_sm100_f16f32")
    return c


def matmul_sm100_batched(a, b, c=None, *, variant: int = 0, split_k: int = 1, stream=None):
    """c[L,M,N] (fp32) = a[L,M,K] (fp16) @ b[L,N,K]^T (fp16), one launch for the whole batch.

    The batch dimension of the reference's generated entry points (xgemm_Sm90.py:45-48).
    """
    import torch

    L, M, K = a.shape
    L2, N, K2 = b.shape
    if K != K2 or L != L2:
        raise ValueError(f"shapes do not match: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if c is None:
        c = torch.empty((L, M, N), dtype=torch.float32, device=a.device)
    if tuple(c.shape) != (L, M, N):
        raise ValueError(f"c must be {(L, M, N)}, got {tuple(c.shape)}")
    _same_device(a, b, c)
    pa = _dev_ptr(a, torch.float16, "a")
    pb = _dev_ptr(b, torch.float16, "b")
    pc = _dev_ptr(c, torch.float32, "c")
    with _OnDevice(a.device):
        rc = lib().spork_gemm_sm100_f16f32_batched(L, M, N, K, pa, pb, pc, variant, split_k, _stream_ptr(stream))
    _check(rc, "spork_gemm_sm100_f16f32_batched")
    return c


def matmul_sm100_tf32(a, b, c=None, *, variant: int = 0, split_k: int = 1, stream=None):
    """c[M,N] = a[M,K] @ b[N,K]^T with fp32 operands read as tf32 (the reference's own operand type)."""
    import torch

    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    if c is None:
        c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    if tuple(c.shape) != (M, N):
        raise ValueError(f"c must be {(M, N)}, got {tuple(c.shape)}")
    _same_device(a, b, c)
    pa, pb, pc = (_dev_ptr(t, torch.float32, n) for t, n in ((a, "a"), (b, "b"), (c, "c")))
    with _OnDevice(a.device):
        rc = lib().spork_gemm_sm100_tf32f32(M, N, K, pa, pb, pc, variant, split_k, _stream_ptr(stream))
    _check(rc, "spork_gemm_sm100_tf32f32")
    return c


def last_clock_mhz(stream=None) -> float:
    """SM clock the most recent GEMM or attention launch on the current device ran at (measured inside the kernel)."""
    mhz = ctypes.c_double(0.0)
    _check(lib().spork_gemm_sm100_last_clock_mhz(_stream_ptr(stream), ctypes.byref(mhz)), "last_clock_mhz")
    return float(mhz.value)


def tune(stages: int = 0, group_m: int = 0, l2_hints: int = 0, backoff_ns: int = 0, *, experiment: int = 0,
         k_atoms: int = 0, wide: int = 0, wide_skew: int = 0, wide_group_m: int = 0,
         no_early_launch: bool = False, keep_wide_tiles: bool = False) -> None:
    """Process-wide tuning knobs of later GEMM launches (see spork_gemm_sm100_tune in the header).

    ``l2_hints`` may carry the packed upper bits itself (the C form); the keyword arguments are OR-ed in."""
    packed = l2_hints | ((experiment & 15) << 4) | ((k_atoms & 3) << 8) | ((wide & 3) << 10) | \
        ((wide_skew & 15) << 12) | ((wide_group_m & 255) << 16) | (int(bool(no_early_launch)) << 24) | \
        (int(bool(keep_wide_tiles)) << 25)
    _check(lib().spork_gemm_sm100_tune(stages, group_m, packed, backoff_ns), "spork_gemm_sm100_tune")


def ring_model(M: int, N: int, K: int, *, block_n: int = 256, cta_group: int = 2, split_k: int = 1, max_ctas: int = 0,
               sm_count: int = 148, stages: int | None = None, skew: int = 4, seed: int = 0, group: int = 0,
               inject: int = 0):
    """Run the host-side model of the kernels' barrier protocol for one CTA group of a launch plan
    (spork_gemm_sm100_ring_model); returns (code, stats) with code 0 = every invariant held."""
    if stages is None:
        stages = 4 if block_n == 512 else 6
    stats = (ctypes.c_uint64 * 4)()
    rc = lib().spork_gemm_sm100_ring_model(M, N, K, block_n, cta_group, split_k, max_ctas, sm_count, stages, skew, seed,
                                           group, inject, stats)
    return rc, {"items": int(stats[0]), "mma_ops": int(stats[1]), "steps": int(stats[2]), "groups": int(stats[3])}


def choice(M: int, N: int, K: int, *, variant: int = 0, split_k: int = 1, sm_count: int = 148, tf32: bool = False) -> dict:
    """What a launch of this shape resolves to (tile width, CTAs per tile, column blocks per stage, K split),
    computed without a GPU (spork_gemm_sm100_choice)."""
    out = (ctypes.c_int * 4)()
    _check(lib().spork_gemm_sm100_choice(M, N, K, variant, split_k, sm_count, int(tf32), out), "spork_gemm_sm100_choice")
    return {"block_n": int(out[0]), "cta_group": int(out[1]), "k_atoms": int(out[2]), "split_k": int(out[3])}


def tmap_cache_stats() -> tuple[int, int]:
    """(hits, misses) of the per-thread cache of encoded TMA descriptors, summed over the process."""
    h, m = ctypes.c_uint64(0), ctypes.c_uint64(0)
    _check(lib().spork_gemm_sm100_tmap_cache_stats(ctypes.byref(h), ctypes.byref(m)), "spork_gemm_sm100_tmap_cache_stats")
    return int(h.value), int(m.value)


def stream_k_counters(stream=None) -> list[tuple[int, int]]:
    """The 16 counter pairs stream-K launches meet at, after ``stream`` has drained: all zero unless a launch
    gave up half way (see spork_gemm_sm100_stream_k_counters)."""
    out = (ctypes.c_uint32 * 32)()
    _check(lib().spork_gemm_sm100_stream_k_counters(out, _stream_ptr(stream)), "spork_gemm_sm100_stream_k_counters")
    return [(int(out[2 * i]), int(out[2 * i + 1])) for i in range(16)]


def trace(buffer=None) -> None:
    """Switch the tile hand-over trace of the 256 x 512 kernel on (``buffer``: an int64 CUDA tensor of
    8 * items elements that outlives the traced launches) or off (None).  See spork_gemm_sm100_trace."""
    import torch

    if buffer is None:
        _check(lib().spork_gemm_sm100_trace(None, 0), "spork_gemm_sm100_trace")
        return
    if not buffer.is_cuda or buffer.dtype != torch.int64 or not buffer.is_contiguous() or buffer.numel() < 8:
        raise TypeError("the trace buffer must be a contiguous int64 CUDA tensor of at least 8 elements")
    _check(lib().spork_gemm_sm100_trace(int(buffer.data_ptr()), buffer.numel() // 8), "spork_gemm_sm100_trace")


def tuning() -> dict:
    """The knobs as the next launch will see them (``l2_hints`` is the effective hint mask)."""
    out = (ctypes.c_int * 10)()
    _check(lib().spork_gemm_sm100_tuning(out, 10), "spork_gemm_sm100_tuning")
    keys = ("stages", "group_m", "l2_hints", "backoff_ns", "experiment", "k_atoms", "wide", "wide_skew", "wide_group_m",
            "no_early_launch")
    return dict(zip(keys, (int(v) for v in out)))


def status(stream=None, device=None) -> None:
    """Synchronise ``stream`` and raise SporkError if a kernel reported a device-side timeout."""
    import torch

    with _OnDevice(device if device is not None else torch.cuda.current_device()):
        detail = ctypes.c_uint32(0)
        rc = lib().spork_gemm_sm100_status(_stream_ptr(stream), ctypes.byref(detail))
    if rc != 0:
        raise SporkError(rc, f"device status (detail 0x{detail.value:08x})")


def matmul_sm100_htod(a_host, b_host, c_host=None):
    """Host-buffer GEMM: fp16 CPU tensors in, fp32 CPU tensor out (copies inside the call)."""
    import torch

    M, K = a_host.shape
    N, _ = b_host.shape
    if c_host is None:
        c_host = torch.empty((M, N), dtype=torch.float32)
    for t, dt in ((a_host, torch.float16), (b_host, torch.float16), (c_host, torch.float32)):
        if t.is_cuda or t.dtype != dt or not t.is_contiguous():
            raise TypeError("host tensors must be contiguous CPU tensors (fp16, fp16, fp32)")
    rc = lib().spork_gemm_sm100_htod_f16f32(M, N, K, a_host.data_ptr(), b_host.data_ptr(), c_host.data_ptr())
    _check(rc, "spork_gemm_sm100_htod_f16f32")
    return c_host


def init_test_data(t, code: int, seed: int = 0, transpose_rule: bool = False, stream=None, row0: int = 0,
                   col0: int = 0):
    """Fill the 2-D fp16 CUDA tensor ``t`` with fixture ``code`` (gemm/gemm_test.cu:55-96 plus codes 3, 4).

    ``row0``/``col0`` place ``t`` inside a larger logical matrix (a rank's slab of a sharded operand)."""
    import torch

    rows, cols = t.shape
    with _OnDevice(t.device):
        rc = lib().spork_init_test_data_f16_at(_dev_ptr(t, torch.float16, "t"), rows, cols, code, seed & 0xFFFFFFFF,
                                               int(transpose_rule), row0, col0, _stream_ptr(stream))
    _check(rc, "spork_init_test_data_f16")
    return t


def gemm_baseline(a, b, c=None, stream=None):
    """The slow CUDA-core comparison GEMM (same operand layout as matmul_sm100)."""
    import torch

    M, K = a.shape
    N, _ = b.shape
    if c is None:
        c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    with _OnDevice(a.device):
        rc = lib().spork_gemm_baseline_f16f32(M, N, K, _dev_ptr(a, torch.float16, "a"), _dev_ptr(b, torch.float16, "b"),
                                              _dev_ptr(c, torch.float32, "c"), _stream_ptr(stream))
    _check(rc, "spork_gemm_baseline_f16f32")
    return c


def compare_f32(x, y, stream=None):
    """On-device comparison; returns (first_failure or None, max_abs_diff) like the reference's comparator."""
    import torch

    rows, cols = x.shape
    out = torch.empty(2, dtype=torch.int64, device=x.device)
    with _OnDevice(x.device):
        rc = lib().spork_compare_f32(_dev_ptr(x, torch.float32, "x"), _dev_ptr(y, torch.float32, "y"), rows, cols,
                                     int(out.data_ptr()), _stream_ptr(stream))
    _check(rc, "spork_compare_f32")
    packed, diff_bits = (int(v) & 0xFFFFFFFFFFFFFFFF for v in out.cpu().tolist())
    first = None if packed == 0xFFFFFFFFFFFFFFFF else (packed >> 32, packed & 0xFFFFFFFF)
    max_diff = struct.unpack("<d", struct.pack("<Q", diff_bits))[0]
    return first, max_diff


def attn_fwd(q, k, v, o=None, scale: float | None = None, stream=None, causal: bool = False):
    """o = softmax(q k^T scale) v per head; q, k, v are (BH, S, D) CUDA tensors, all fp16 or all bfloat16
    (the reference interface's type)."""
    import torch

    if q.dim() != 3:
        raise ValueError(f"q must be (BH, S, D), got {tuple(q.shape)}")
    BH, S, D = q.shape
    if o is None:
        o = torch.empty_like(q)
    # every tensor map and every store is sized from q: a shorter k or v, or a smaller o, would be read or
    # written past its end
    for t, name in ((k, "k"), (v, "v"), (o, "o")):
        if tuple(t.shape) != (BH, S, D):
            raise ValueError(f"{name} must have q's shape {(BH, S, D)}, got {tuple(t.shape)}")
    _same_device(q, k, v, o)
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    dt = q.dtype
    if dt not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q must be float16 or bfloat16, got {dt}")
    with _OnDevice(q.device):
        rc = lib().spork_attn_sm100_fwd_ex(BH, S, D, _dev_ptr(q, dt, "q"), _dev_ptr(k, dt, "k"), _dev_ptr(v, dt, "v"),
                                           _dev_ptr(o, dt, "o"), ctypes.c_float(scale), int(dt == torch.bfloat16),
                                           int(bool(causal)), _stream_ptr(stream))
    _check(rc, "spork_attn_sm100_fwd")
    return o
