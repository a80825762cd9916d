"""ctypes binding of libflashfwd_b200.so, the B200 (sm_100a) attention-forward library.

The shared library is the product; this module only loads it and mirrors the reference's host
entry point for Python callers (tests, the benchmark). There is no fallback of any kind: if the
library is missing or fails to load, importing `lib()` raises, and every call goes to the CUDA
kernels.

The directory name contains a hyphen, so the package is imported by path (see `load_package`
in `__graft_entry__.py`) under the module name `flash_attn_rtx5060_b200`.

Reference interface mirrored here: run_flash_attention (src/flash_forward.h:593-612 of the
reference) and its call site (src/main.cu:99).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashfwd_b200.so")

FA_OK, FA_INVALID_ARG, FA_UNSUPPORTED, FA_CUDA_ERROR, FA_DEVICE_TIMEOUT = range(5)
STATUS_NAMES = {0: "FA_OK", 1: "FA_INVALID_ARG", 2: "FA_UNSUPPORTED", 3: "FA_CUDA_ERROR", 4: "FA_DEVICE_TIMEOUT"}

# every symbol include/flash_forward_b200.h declares
EXPORTS = (
    "flash_forward",
    "flash_forward_ex",
    "flash_forward_alibi",
    "flash_forward_lse",
    "flash_forward_dropout",
    "flash_forward_dropout_keep_probability",
    "flash_forward_multi_gpu",
    "flash_forward_host",
    "flash_forward_host_workspace_bytes",
    "flash_forward_check",
    "flash_forward_noalloc",
    "flash_forward_noalloc_check",
    "run_flash_attention_c",
    "flash_forward_last_error",
    "flash_forward_flops",
    "flash_forward_kv_range",
    "flash_forward_head_group",
    "flash_forward_shutdown",
)

_lib = None


class FlashForwardError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


def lib():
    """Loads the shared library once. Raises OSError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise OSError(f"{LIB_PATH} not found: build it with `make -C {os.path.join(_HERE, 'csrc')}`")
    L = ctypes.CDLL(LIB_PATH)
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    L.flash_forward.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp]
    L.flash_forward.restype = i
    L.flash_forward_alibi.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, vp]
    L.flash_forward_alibi.restype = i
    L.flash_forward_lse.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, vp]
    L.flash_forward_lse.restype = i
    L.flash_forward_dropout.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, f, ctypes.c_ulonglong, vp]
    L.flash_forward_dropout.restype = i
    L.flash_forward_dropout_keep_probability.argtypes = [f]
    L.flash_forward_dropout_keep_probability.restype = ctypes.c_double
    pp = ctypes.POINTER(vp)
    L.flash_forward_multi_gpu.argtypes = [i, ctypes.POINTER(i), pp, pp, pp, pp, ctypes.POINTER(i), i, i, f, i, i, i, pp, i]
    L.flash_forward_multi_gpu.restype = i
    L.flash_forward_ex.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, i, i, vp]
    L.flash_forward_ex.restype = i
    L.flash_forward_host.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, ctypes.c_size_t, i]
    L.flash_forward_host.restype = i
    L.flash_forward_host_workspace_bytes.argtypes = [i, i, i]
    L.flash_forward_host_workspace_bytes.restype = ctypes.c_size_t
    L.flash_forward_noalloc.argtypes = [vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, i, i]
    L.flash_forward_noalloc.restype = i
    L.flash_forward_noalloc_check.argtypes = [vp, i]
    L.flash_forward_noalloc_check.restype = i
    L.flash_forward_check.argtypes = [vp]
    L.flash_forward_check.restype = i
    L.run_flash_attention_c.argtypes = [i, i, i, i, vp, vp, vp, vp, vp, vp, i, i, i, i, i, vp, f, vp]
    L.run_flash_attention_c.restype = i
    L.flash_forward_last_error.argtypes = []
    L.flash_forward_last_error.restype = ctypes.c_char_p
    L.flash_forward_flops.argtypes = [i, i, i, i, i, i, i]
    L.flash_forward_flops.restype = ctypes.c_double
    ip = ctypes.POINTER(ctypes.c_int)
    L.flash_forward_kv_range.argtypes = [i, i, i, i, i, i, ip, ip, ip]
    L.flash_forward_kv_range.restype = i
    L.flash_forward_head_group.argtypes = [i, i, i, i, i, i, i]
    L.flash_forward_head_group.restype = i
    L.flash_forward_shutdown.argtypes = []
    L.flash_forward_shutdown.restype = i
    _lib = L
    return L


def _raise(code):
    raise FlashForwardError(code, lib().flash_forward_last_error().decode())


def flash_forward(q, k, v, o, batch, heads, seqlen, head_dim, softmax_scale=0.0, is_causal=False, window_left=-1,
                  window_right=-1, stream=None, kernel=0, variant=0, dbg=None):
    """Enqueues the attention forward on raw device pointers (ints). Asynchronous."""
    rc = lib().flash_forward_ex(q, k, v, o, batch, heads, seqlen, head_dim, softmax_scale, int(bool(is_causal)),
                                window_left, window_right, stream, kernel, variant, dbg)
    if rc != FA_OK:
        _raise(rc)


def flash_forward_multi_gpu(devices, q, k, v, o, slab_heads, seqlen, head_dim, softmax_scale=0.0, is_causal=False,
                            window_left=-1, window_right=-1, streams=None, wait=True):
    """One slab of heads per entry of `devices`; q, k, v, o are lists of raw device pointers (ints)."""
    n = len(devices)
    assert len(q) == len(k) == len(v) == len(o) == len(slab_heads) == n
    ints = lambda xs: (ctypes.c_int * n)(*xs)  # noqa: E731
    ptrs = lambda xs: (ctypes.c_void_p * n)(*xs)  # noqa: E731
    rc = lib().flash_forward_multi_gpu(n, ints(devices), ptrs(q), ptrs(k), ptrs(v), ptrs(o), ints(slab_heads), seqlen,
                                       head_dim, softmax_scale, int(bool(is_causal)), window_left, window_right,
                                       None if streams is None else ptrs(streams), int(bool(wait)))
    if rc != FA_OK:
        _raise(rc)


def flash_forward_host(q_host, k_host, v_host, o_host, batch, heads, seqlen, head_dim, workspace, workspace_bytes,
                       chunk_heads, softmax_scale=0.0, is_causal=False, window_left=-1, window_right=-1):
    """Forward on HOST buffers (raw pointers): chunked upload / kernel / download pipeline. Blocking."""
    rc = lib().flash_forward_host(q_host, k_host, v_host, o_host, batch, heads, seqlen, head_dim, softmax_scale,
                                  int(bool(is_causal)), window_left, window_right, workspace, workspace_bytes,
                                  chunk_heads)
    if rc != FA_OK:
        _raise(rc)


def host_workspace_bytes(seqlen, head_dim, chunk_heads):
    return lib().flash_forward_host_workspace_bytes(seqlen, head_dim, chunk_heads)


def check(stream=None):
    """Waits for the stream and raises if a device-side wait gave up."""
    rc = lib().flash_forward_check(stream)
    if rc != FA_OK:
        _raise(rc)


def flops(batch, heads, seqlen, head_dim, is_causal=False, window_left=-1, window_right=-1):
    return lib().flash_forward_flops(batch, heads, seqlen, head_dim, int(bool(is_causal)), window_left, window_right)


def kv_range(seqlen, is_causal, window_left, window_right, row_begin, row_end):
    """(tile_begin, tile_end, masked_tiles) of the kv tiles a block of query rows reads."""
    a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    rc = lib().flash_forward_kv_range(seqlen, int(bool(is_causal)), window_left, window_right, row_begin, row_end,
                                      ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
    if rc != FA_OK:
        _raise(rc)
    return a.value, b.value, c.value


def head_group(batch_heads, seqlen, head_dim, is_causal=False, window_left=-1, window_right=-1, num_sms=148):
    """Heads per scheduling group the default kernel uses for this shape (host logic)."""
    return lib().flash_forward_head_group(batch_heads, seqlen, head_dim, int(bool(is_causal)), window_left, window_right,
                                          num_sms)


def run_flash_attention(B, N, S, d, Q, K, V, O, L=None, M=None, Is_dropout=False, Is_causal=False, Is_local=False,
                        Has_alibi=False, window_size=0, alibi_slopes=None, dropout_prob=0.0, states=None):
    """The reference's entry point, argument for argument (N = heads, S = sequence length there).

    Q, K, V, O are raw device pointers. Blocks until the result is ready and prints `TIME: <ms>`
    as the reference does. Raises FlashForwardError where the reference would exit or abort.
    """
    rc = lib().run_flash_attention_c(B, N, S, d, Q, K, V, O, L, M, int(bool(Is_dropout)), int(bool(Is_causal)),
                                     int(bool(Is_local)), int(bool(Has_alibi)), window_size, alibi_slopes,
                                     dropout_prob, states)
    if rc != FA_OK:
        _raise(rc)


def attention_forward(q, k, v, causal=False, window_left=-1, window_right=-1, softmax_scale=0.0, out=None, kernel=0,
                      variant=0, alibi_slopes=None, return_lse=False, dropout_p=0.0, seed=0):
    """Convenience wrapper for torch CUDA tensors of shape [B, H, N, d], fp16, contiguous.

    torch is used for device memory and the current stream only; the computation is the library's.
    With return_lse the result is (out, lse), lse a float32 [B, H, N] tensor (flash_forward_lse).
    With dropout_p > 0 the call is flash_forward_dropout(dropout_p, seed).
    """
    import torch

    assert q.is_cuda and q.dtype == torch.float16 and q.is_contiguous() and q.dim() == 4
    assert k.shape == q.shape and v.shape == q.shape and k.is_contiguous() and v.is_contiguous()
    B, H, N, d = q.shape
    if out is None:
        out = torch.empty_like(q)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        if alibi_slopes is not None:
            assert alibi_slopes.is_cuda and alibi_slopes.dtype == torch.float32 and alibi_slopes.numel() == H
        if dropout_p > 0.0:
            assert kernel == 0 and variant == 0 and not return_lse
            rc = lib().flash_forward_dropout(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, N, d,
                                             softmax_scale, int(bool(causal)), window_left, window_right,
                                             None if alibi_slopes is None else alibi_slopes.data_ptr(), dropout_p,
                                             seed, stream)
            if rc != FA_OK:
                _raise(rc)
            return out
        if return_lse:
            assert kernel == 0 and variant == 0
            lse = torch.empty((B, H, N), device=q.device, dtype=torch.float32)
            rc = lib().flash_forward_lse(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, H,
                                         N, d, softmax_scale, int(bool(causal)), window_left, window_right,
                                         None if alibi_slopes is None else alibi_slopes.data_ptr(), stream)
            if rc != FA_OK:
                _raise(rc)
            return out, lse
        if alibi_slopes is not None:  # float32 CUDA tensor with one slope per head
            assert alibi_slopes.is_cuda and alibi_slopes.dtype == torch.float32 and alibi_slopes.numel() == H
            rc = lib().flash_forward_alibi(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, N, d,
                                           softmax_scale, int(bool(causal)), window_left, window_right,
                                           alibi_slopes.data_ptr(), stream)
            if rc != FA_OK:
                _raise(rc)
        else:
            flash_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, N, d, softmax_scale, causal,
                          window_left, window_right, stream, kernel, variant)
    return out
