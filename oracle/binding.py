"""ctypes bindings of the CPU oracle libraries: TEST INFRASTRUCTURE, not part of the product.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark import this module.
`port()` is the C restatement (oracle/attention_cpu.c); `ref()` is the reference's own CPU
attention compiled from the reference sources (oracle/_ref/), present only where those sources
were available at build time.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "liboracle_attn.so")
REF_PATH = os.path.join(_HERE, "_ref", "libref_attention.so")

_port = None
_ref = None


def port():
    global _port
    if _port is None:
        L = ctypes.CDLL(PORT_PATH)
        vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.oracle_attention_rows.argtypes = [vp, vp, vp, f, i, i, i, i, i, i, f, vp, i, vp]
        L.oracle_attention_rows.restype = i
        L.oracle_attention_forward.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, i]
        L.oracle_attention_forward.restype = i
        L.oracle_abs_error.argtypes = [vp, vp, ctypes.c_size_t, vp, vp, vp]
        L.oracle_abs_error.restype = None
        L.oracle_uses_simd.restype = i
        _port = L
    return _port


def ref_available():
    return os.path.exists(REF_PATH)


def ref():
    global _ref
    if _ref is None:
        L = ctypes.CDLL(REF_PATH)
        vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.ref_attention_forward_cpu.argtypes = [vp, vp, vp, f, i, i, i, i, vp, i, i, vp]
        L.ref_attention_forward_cpu.restype = None
        L.ref_attention_forward_cpu_mt.argtypes = [vp, vp, vp, f, i, i, i, i, vp, i, i, vp, i]
        L.ref_attention_forward_cpu_mt.restype = None
        _ref = L
    return _ref


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype in (np.float16, np.uint16)
    return a.view(np.uint16)


def attention(q, k, v, causal=False, window_left=-1, window_right=-1, scale=None, alibi_slopes=None, nthreads=None):
    """Oracle attention of fp16 arrays [B, H, N, d] -> fp16 array of the same shape."""
    B, H, N, d = q.shape
    q16, k16, v16 = _u16(q), _u16(k), _u16(v)
    out = np.empty((B, H, N, d), dtype=np.uint16)
    if scale is None:
        scale = np.float32(1.0) / np.sqrt(np.float32(d))
    sl = None
    if alibi_slopes is not None:
        sl = np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    nt = nthreads or min(os.cpu_count() or 1, B * H)
    rc = port().oracle_attention_forward(q16.ctypes.data, k16.ctypes.data, v16.ctypes.data, out.ctypes.data, B, H, N, d,
                                         float(scale), int(causal), window_left, window_right,
                                         sl.ctypes.data if sl is not None else None, nt)
    if rc != 0:
        raise MemoryError("oracle_attention_forward failed")
    return out.view(np.float16)


def attention_dropout(q, k, v, dropout_p, seed, causal=False, window_left=-1, window_right=-1, scale=None,
                      alibi_slopes=None, nthreads=None):
    """Oracle attention with dropout on the probabilities (the library's documented keep rule: Philox-4x32-10, keep
    threshold round(256 * (1 - p))). Not pinned by the reference, whose CPU function has no dropout."""
    B, H, N, d = q.shape
    q16, k16, v16 = _u16(q), _u16(k), _u16(v)
    out = np.empty((B, H, N, d), dtype=np.uint16)
    if scale is None:
        scale = np.float32(1.0) / np.sqrt(np.float32(d))
    sl = None if alibi_slopes is None else np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    nt = nthreads or min(os.cpu_count() or 1, B * H)
    keep_thr = min(int(np.rint(np.float32(256.0) * (np.float32(1.0) - np.float32(dropout_p)))), 256)
    fn = port().oracle_attention_forward_dropout
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_float] + [ctypes.c_int] * 3 + [
        ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_uint64]
    rc = fn(q16.ctypes.data, k16.ctypes.data, v16.ctypes.data, out.ctypes.data, B, H, N, d, float(scale), int(causal),
            window_left, window_right, sl.ctypes.data if sl is not None else None, nt, keep_thr, seed)
    if rc != 0:
        raise MemoryError("oracle_attention_forward_dropout failed")
    return out.view(np.float16)


def dropout_keep(seed, bh, row, col, keep_thr):
    fn = port().oracle_dropout_keep
    fn.argtypes = [ctypes.c_uint64, ctypes.c_uint, ctypes.c_int, ctypes.c_int, ctypes.c_uint]
    return bool(fn(seed, bh, row, col, keep_thr))


def attention_rows(q, k, v, rows, causal=False, window_left=-1, window_right=-1, scale=None, slope=None):
    """Oracle attention of selected query rows of ONE head: q, k, v fp16 [N, d] -> fp16 [len(rows), d]."""
    N, d = q.shape
    q16, k16, v16 = _u16(q), _u16(k), _u16(v)
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((len(rows), d), dtype=np.uint16)
    if scale is None:
        scale = np.float32(1.0) / np.sqrt(np.float32(d))
    rc = port().oracle_attention_rows(q16.ctypes.data, k16.ctypes.data, v16.ctypes.data, float(scale), N, d,
                                      int(causal), window_left, window_right, int(slope is not None),
                                      float(slope or 0.0), rows.ctypes.data, len(rows), out.ctypes.data)
    if rc != 0:
        raise MemoryError("oracle_attention_rows failed")
    return out.view(np.float16)


def reference_attention(q, k, v, causal=False, window_size=-1, scale=None, alibi_slopes=None, nthreads=1):
    """The reference's own attention_forward_cpu (symmetric window, `window_size < 0` = none)."""
    B, H, N, d = q.shape
    q16, k16, v16 = _u16(q), _u16(k), _u16(v)
    out = np.zeros((B, H, N, d), dtype=np.uint16)
    if scale is None:
        scale = np.float32(1.0) / np.sqrt(np.float32(d))
    sl = None
    if alibi_slopes is not None:
        sl = np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    slp = sl.ctypes.data if sl is not None else None
    if nthreads <= 1:
        ref().ref_attention_forward_cpu(q16.ctypes.data, k16.ctypes.data, v16.ctypes.data, float(scale), B, H, N, d,
                                        out.ctypes.data, int(causal), window_size, slp)
    else:
        ref().ref_attention_forward_cpu_mt(q16.ctypes.data, k16.ctypes.data, v16.ctypes.data, float(scale), B, H, N,
                                           d, out.ctypes.data, int(causal), window_size, slp, nthreads)
    return out.view(np.float16)


def abs_error(a, b):
    """(max_abs, mean_abs, nan_count) of fp16 arrays compared in fp32."""
    a16, b16 = _u16(a).ravel(), _u16(b).ravel()
    assert a16.size == b16.size
    mx, mean, nans = ctypes.c_double(), ctypes.c_double(), ctypes.c_longlong()
    port().oracle_abs_error(a16.ctypes.data, b16.ctypes.data, a16.size, ctypes.byref(mx), ctypes.byref(mean),
                            ctypes.byref(nans))
    return mx.value, mean.value, nans.value


def log_sum_exp_fp64(q, k, softmax_scale=0.0, causal=False, window_left=-1, window_right=-1, alibi_slopes=None,
                     rows=None):
    """Natural-log sum of exp(scale * q_i.k_j - slope_h * |i - j|) over the keys row i may see, in float64 (numpy).

    The reference has no such output (its L/M arguments are dead, src/flash_forward.h:602-603), so this is
    the mathematical definition evaluated exactly on the same fp16 inputs, with the reference's masks
    (src/main.cu:200-222: ALiBi, causal j <= i, window |i - j| <= w, here two-sided with -1 = unbounded).
    q, k: fp16 [B, H, N, d]; rows: optional 1-D index array. Returns float64 [B, H, len(rows) or N]."""
    B, H, N, d = q.shape
    scale = softmax_scale if softmax_scale > 0 else 1.0 / np.sqrt(d)
    rows = np.arange(N) if rows is None else np.asarray(rows)
    i = rows[:, None].astype(np.int64)
    j = np.arange(N, dtype=np.int64)[None, :]
    wr = 0 if causal else window_right
    visible = np.ones((rows.size, N), dtype=bool)
    if wr >= 0:
        visible &= j <= i + wr
    if window_left >= 0:
        visible &= j >= i - window_left
    out = np.empty((B, H, rows.size))
    for b in range(B):
        for h in range(H):
            s = (q[b, h, rows].astype(np.float64) @ k[b, h].astype(np.float64).T) * scale
            if alibi_slopes is not None:
                s -= float(alibi_slopes[h]) * np.abs(i - j)
            s = np.where(visible, s, -np.inf)
            m = s.max(axis=1, keepdims=True)
            out[b, h] = (m + np.log(np.exp(s - m).sum(axis=1, keepdims=True)))[:, 0]
    return out
