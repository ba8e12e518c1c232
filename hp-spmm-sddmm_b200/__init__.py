"""ctypes binding of libhpspmm.so, the C-ABI library of the B200 FP32 CSR SpMM / SDDMM path.

The product is the shared library and the C++ headers under include/; this module is the
thin Python face used by the tests and the benchmark.  There is no fallback of any kind:
if the library is missing, loading raises.

The directory name contains hyphens, so it is imported by path:

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location(
        "hp_spmm_sddmm_b200", "<repo>/hp-spmm-sddmm_b200/__init__.py")
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
"""
import ctypes
import os
from ctypes import (POINTER, byref, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_uint64, c_void_p)

import numpy as np

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "lib", "libhpspmm.so")

OK = 0
ERR_INVALID = 1
ERR_OOM = 2
ERR_CUDA = 3
ERR_TIMEOUT = 4
ERR_UNSUPPORTED = 5
ERR_BAD_CSR = 6

ALGO_AUTO = 0
ALGO_BALANCED = 1
ALGO_ROW_SPLIT = 2
ALGO_TMA = 3

EXCHANGE_NEEDED_ROWS = 0
EXCHANGE_ALL_ROWS = 1
EXCHANGE_NEEDED_ROWS_NCCL = 2
COMM_ID_BYTES = 128

VALS_ONES = 0
VALS_U01 = 1
VALS_UPM1 = 2


class Opts(ctypes.Structure):
    """Mirror of hpspmm_opts."""
    _fields_ = [("algo", c_int32), ("chunk_nnz", c_int32), ("b_l2_hint", c_int32),
                ("reserved", c_int32)]


class HpspmmError(RuntimeError):
    def __init__(self, status, what, detail=""):
        self.status = status
        super().__init__("%s failed with status %d%s" % (what, status, (": " + detail) if detail else ""))


_P = c_void_p
_I64 = c_int64

# name -> (restype, argtypes); every symbol include/hpspmm.h declares
PROTOTYPES = {
    "hpspmm_status_string": (c_char_p, [c_int]),
    "hpspmm_version": (c_char_p, []),
    "hpspmm_ctx_create": (c_int, [c_int, POINTER(_P)]),
    "hpspmm_ctx_destroy": (c_int, [_P]),
    "hpspmm_last_error": (c_char_p, [_P]),
    "hpspmm_ctx_device": (c_int, [_P]),
    "hpspmm_ctx_sm_count": (c_int, [_P]),
    "hpspmm_ctx_l2_bytes": (_I64, [_P]),
    "hpspmm_ctx_launch_count": (_I64, [_P]),
    "hpspmm_dev_alloc": (c_int, [_P, c_size_t, POINTER(_P)]),
    "hpspmm_dev_free": (c_int, [_P, _P]),
    "hpspmm_host_alloc_pinned": (c_int, [_P, c_size_t, POINTER(_P)]),
    "hpspmm_host_free_pinned": (c_int, [_P, _P]),
    "hpspmm_memcpy_h2d": (c_int, [_P, _P, _P, c_size_t, _P]),
    "hpspmm_memcpy_d2h": (c_int, [_P, _P, _P, c_size_t, _P]),
    "hpspmm_memcpy_d2d": (c_int, [_P, _P, _P, c_size_t, _P]),
    "hpspmm_memset": (c_int, [_P, _P, c_int, c_size_t, _P]),
    "hpspmm_stream_create": (c_int, [_P, POINTER(_P)]),
    "hpspmm_stream_sync": (c_int, [_P, _P]),
    "hpspmm_stream_destroy": (c_int, [_P, _P]),
    "hpspmm_event_create": (c_int, [_P, POINTER(_P)]),
    "hpspmm_event_record": (c_int, [_P, _P, _P]),
    "hpspmm_event_sync": (c_int, [_P, _P]),
    "hpspmm_event_elapsed_ms": (c_int, [_P, _P, _P, POINTER(c_float)]),
    "hpspmm_event_destroy": (c_int, [_P, _P]),
    "hpspmm_fill_f32": (c_int, [_P, _P, _I64, c_float, _P]),
    "hpspmm_fill_uniform_f32": (c_int, [_P, _P, _I64, c_uint64, c_uint64, c_float, c_float, _P]),
    "hpspmm_host_fill_uniform_f32": (c_int, [_P, _I64, c_uint64, c_uint64, c_float, c_float]),
    "hpspmm_spmm_csr_f32": (c_int, [_P, _P, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P,
                                    POINTER(Opts), _P]),
    "hpspmm_plan_create": (c_int, [_P, _I64, _I64, _I64, _P, _P, _I64, POINTER(Opts), _P, POINTER(_P)]),
    "hpspmm_plan_destroy": (c_int, [_P, _P]),
    "hpspmm_plan_info": (c_int, [_P, POINTER(_I64), POINTER(_I64), POINTER(_I64), POINTER(_I64)]),
    "hpspmm_spmm_csr_f32_static_scratch": (c_int, [c_int, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P,
                                                   ctypes.c_char_p, c_size_t]),
    "hpspmm_spmm_csr_f32_host": (c_int, [_P, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P,
                                         POINTER(Opts)]),
    "hpspmm_spmm_csr_f32_host_multi": (c_int, [_P, _I64, _I64, _I64, _P, _P, _P, c_int32, _P, _P, _P,
                                               POINTER(Opts)]),
    "hpspmm_spmm_coo_f32": (c_int, [_P, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, POINTER(Opts), _P]),
    "hpspmm_sddmm_csr_f32": (c_int, [_P, _P, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P,
                                     POINTER(Opts), _P]),
    "hpspmm_csr_transpose": (c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _P]),
    "hpspmm_spmm_kernel_signature": (c_int, [_P, _I64, c_int32, ctypes.c_char_p, c_size_t]),
    "hpspmm_plan_tables": (c_int, [_P, POINTER(_P), POINTER(_P), POINTER(_P)]),
    "hpspmm_plan_row_list": (c_int, [_P, POINTER(_P), POINTER(_P), POINTER(_P)]),
    "hpspmm_layer_create": (c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _I64, _P, POINTER(_P)]),
    "hpspmm_layer_destroy": (c_int, [_P, _P]),
    "hpspmm_layer_info": (c_int, [_P, POINTER(_I64), POINTER(_I64), POINTER(_I64), POINTER(_I64),
                                  POINTER(_I64)]),
    "hpspmm_layer_transposed": (c_int, [_P, POINTER(_P), POINTER(_P), POINTER(_P), POINTER(_P)]),
    "hpspmm_layer_forward": (c_int, [_P, _P, _I64, _P, _P, _P]),
    "hpspmm_layer_backward_features": (c_int, [_P, _P, _I64, _P, _P, _P]),
    "hpspmm_layer_backward_weights": (c_int, [_P, _P, _I64, _P, _P, _P, _P]),
    "hpspmm_layer_update_values": (c_int, [_P, _P, _P, _P]),
    "hpspmm_padded_nnz": (_I64, [_I64, _I64]),
    "hpspmm_csr_to_coo_padded": (c_int, [_P, _I64, _I64, _P, _P, _P, _I64, _P, _P, _P, _P]),
    "hpspmm_csr_to_coo_reordered": (c_int, [_P, _I64, _I64, _P, _P, _P, _P, _I64, _P, _P, _P, _P]),
    "hpspmm_csr_permute": (c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "hpspmm_order_rows_by_degree": (c_int, [_P, _I64, _P, _P, _P]),
    "hpspmm_invert_permutation": (c_int, [_P, _I64, _P, _P, _P]),
    "hpspmm_gather_rows_f32": (c_int, [_P, _I64, _I64, _P, _P, _P, _P]),
    "hpspmm_read_row_order": (c_int, [c_char_p, _I64, _P]),
    "hpspmm_validate_csr": (c_int, [_P, _I64, _I64, _I64, _P, _P, POINTER(_I64), _P]),
    "hpspmm_gen_uniform_degree": (c_int, [_I64, _I64, c_int32, c_int32, c_uint64, c_int32, POINTER(_P)]),
    "hpspmm_gen_erdos_renyi": (c_int, [_I64, _I64, c_double, c_uint64, c_int32, POINTER(_P)]),
    "hpspmm_gen_rmat": (c_int, [c_int32, c_int32, c_double, c_double, c_double, c_uint64, c_int32,
                                POINTER(_P)]),
    "hpspmm_gen_shape": (c_int, [_P, POINTER(_I64), POINTER(_I64), POINTER(_I64)]),
    "hpspmm_gen_export": (c_int, [_P, _P, _P, _P]),
    "hpspmm_gen_free": (c_int, [_P]),
    "hpspmm_read_smtx": (c_int, [c_char_p, POINTER(_P)]),
    "hpspmm_shard_bounds": (c_int, [_I64, _P, c_int32, _P]),
    "hpspmm_shard_bounds_weighted": (c_int, [_I64, _P, c_int32, c_double, _P]),
    "hpspmm_shard_row_ptr": (c_int, [_P, _I64, _I64, _P, POINTER(_I64), POINTER(_I64)]),
    "hpspmm_gflops": (c_double, [_I64, _I64, c_double]),
    "hpspmm_row_length_cv": (c_double, [_I64, _P]),
    "hpspmm_spmm_algorithmic_bytes": (c_double, [_I64, _I64, _I64, _I64]),
    "hpspmm_sddmm_algorithmic_bytes": (c_double, [_I64, _I64, _I64, _I64, _I64]),
    "hpspmm_shard_needed_rows": (c_int, [_I64, _P, _I64, c_int32, _P, _P, _P, _P, POINTER(_I64)]),
    "hpspmm_comm_unique_id": (c_int, [_P]),
    "hpspmm_comm_create": (c_int, [_P, c_int32, c_int32, _P, POINTER(_P)]),
    "hpspmm_comm_destroy": (c_int, [_P]),
    "hpspmm_comm_info": (c_int, [_P, POINTER(c_int32), POINTER(c_int32)]),
    "hpspmm_shard_plan_create": (c_int, [_P, _P, _I64, _I64, _I64, _P, _P, _P, _I64, c_int32, _P, POINTER(_P)]),
    "hpspmm_shard_plan_destroy": (c_int, [_P, _P]),
    "hpspmm_shard_plan_info": (c_int, [_P, POINTER(_I64), POINTER(_I64), POINTER(_I64), POINTER(_I64)]),
    "hpspmm_sharded_exchange_begin": (c_int, [_P, _P, c_int32, _I64, _P, _P]),
    "hpspmm_sharded_product": (c_int, [_P, _P, c_int32, _I64, _P, _P, POINTER(Opts), _P]),
    "hpspmm_spmm_sharded_f32": (c_int, [_P, _P, _I64, _P, _P, _P, POINTER(Opts), _P]),
    "hpspmm_debug_fail_device_alloc": (c_int, [_I64, _I64]),
    "hpspmm_probe_gather_gbs": (c_int, [_P, c_int32, _I64, _I64, c_int32, _I64, c_double, c_int32,
                                        POINTER(c_double), POINTER(c_double)]),
    "hpspmm_ctx_tma_fallbacks": (c_int, [_P, POINTER(_I64)]),
    "hpspmm_probe_tma_gather_gbs": (c_int, [_P, c_int32, _I64, _I64, c_int32, c_int32, POINTER(c_double),
                                            POINTER(c_double), POINTER(c_double), POINTER(_I64)]),
}

_lib = None


def load_library(path=None):
    """Loads libhpspmm.so and attaches the prototypes.  Raises if the library is absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(
            "libhpspmm.so not found at %s: build it with `python hp-spmm-sddmm_b200/build.py` "
            "(there is no CPU or PyTorch fallback)" % p)
    lib = ctypes.CDLL(p)
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means the build is stale
        fn.restype = restype
        fn.argtypes = argtypes
    if path is None:
        _lib = lib
    return lib


def _ptr(a):
    """Address of a numpy array's buffer, or a raw integer address, or NULL."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if isinstance(a, DeviceBuffer):
        return a.ptr
    return int(a)


class DeviceBuffer:
    """A device allocation owned through the C ABI."""

    def __init__(self, ctx, nbytes, dtype=None, shape=None):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        self.dtype = dtype
        self.shape = shape
        out = _P()
        ctx._check(ctx.lib.hpspmm_dev_alloc(ctx.handle, self.nbytes, byref(out)), "hpspmm_dev_alloc")
        self.ptr = out.value or 0

    def free(self):
        if self.ptr:
            self.ctx.lib.hpspmm_dev_free(self.ctx.handle, self.ptr)
            self.ptr = 0

    def to_host(self, stream=None):
        out = np.empty(self.shape, dtype=self.dtype)
        self.ctx.memcpy_d2h(out, self, stream)
        self.ctx.stream_sync(stream)
        return out


class Context:
    """One hpspmm context on one device."""

    def __init__(self, device=0):
        self.lib = load_library()
        h = _P()
        st = self.lib.hpspmm_ctx_create(device, byref(h))
        if st != OK:
            raise HpspmmError(st, "hpspmm_ctx_create", self.lib.hpspmm_status_string(st).decode())
        self.handle = h
        self._buffers = []

    def close(self):
        if self.handle:
            for b in self._buffers:
                b.free()
            self._buffers = []
            self.lib.hpspmm_ctx_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, st, what):
        if st != OK:
            raise HpspmmError(st, what, self.lib.hpspmm_last_error(self.handle).decode())

    # -- memory ---------------------------------------------------------------------
    def alloc(self, shape, dtype):
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = int(np.prod(shape)) if shape else 1
        b = DeviceBuffer(self, max(n, 1) * np.dtype(dtype).itemsize, np.dtype(dtype), shape)
        self._buffers.append(b)
        return b

    def upload(self, arr, stream=None):
        arr = np.ascontiguousarray(arr)
        b = self.alloc(arr.shape, arr.dtype)
        if arr.nbytes:
            self._check(self.lib.hpspmm_memcpy_h2d(self.handle, b.ptr, arr.ctypes.data, arr.nbytes,
                                                   stream), "hpspmm_memcpy_h2d")
            self.stream_sync(stream)
        return b

    def memcpy_d2h(self, host_arr, dev, stream=None):
        if host_arr.nbytes:
            self._check(self.lib.hpspmm_memcpy_d2h(self.handle, host_arr.ctypes.data, _ptr(dev),
                                                   host_arr.nbytes, stream), "hpspmm_memcpy_d2h")

    def stream_sync(self, stream=None):
        self._check(self.lib.hpspmm_stream_sync(self.handle, stream), "hpspmm_stream_sync")

    def fill(self, dev, count, value, stream=None):
        self._check(self.lib.hpspmm_fill_f32(self.handle, _ptr(dev), count, value, stream),
                    "hpspmm_fill_f32")

    def fill_uniform(self, dev, count, seed, stream_id, lo, hi, stream=None):
        self._check(self.lib.hpspmm_fill_uniform_f32(self.handle, _ptr(dev), count, seed, stream_id,
                                                     lo, hi, stream), "hpspmm_fill_uniform_f32")

    # -- events ---------------------------------------------------------------------
    def event(self):
        e = _P()
        self._check(self.lib.hpspmm_event_create(self.handle, byref(e)), "hpspmm_event_create")
        return e

    def record(self, ev, stream=None):
        self._check(self.lib.hpspmm_event_record(self.handle, ev, stream), "hpspmm_event_record")

    def elapsed_ms(self, a, b):
        ms = c_float()
        self._check(self.lib.hpspmm_event_elapsed_ms(self.handle, a, b, byref(ms)),
                    "hpspmm_event_elapsed_ms")
        return ms.value

    # -- the path -------------------------------------------------------------------
    def plan_create(self, M, nnz, row_ptr, max_K, opts=None, stream=None, N=0, col_idx=None):
        """Chunk table for (M, nnz, row_ptr).  With N and col_idx the pieces of heavy rows are also
        ordered by the column band they read (better L2 reuse of B)."""
        p = _P()
        self._check(self.lib.hpspmm_plan_create(self.handle, M, N, nnz, _ptr(row_ptr),
                                                _ptr(col_idx) if col_idx is not None else None, max_K,
                                                byref(opts) if opts else None, stream, byref(p)),
                    "hpspmm_plan_create")
        return p

    def plan_destroy(self, plan):
        self.lib.hpspmm_plan_destroy(self.handle, plan)

    def plan_info(self, plan):
        a, b, c, d = _I64(), _I64(), _I64(), _I64()
        self._check(self.lib.hpspmm_plan_info(plan, byref(a), byref(b), byref(c), byref(d)),
                    "hpspmm_plan_info")
        return {"n_chunks": a.value, "n_split_chunks": b.value, "chunk_nnz": c.value,
                "scratch_bytes": d.value}

    def kernel_signature(self, plan, K, b_l2_hint=0):
        buf = ctypes.create_string_buffer(256)
        self._check(self.lib.hpspmm_spmm_kernel_signature(plan, K, b_l2_hint, buf, 256), "hpspmm_spmm_kernel_signature")
        return buf.value.decode()

    def plan_tables(self, plan):
        """Device addresses of chunk_start, chunk_row, chunk_order."""
        a, b, c = _P(), _P(), _P()
        self._check(self.lib.hpspmm_plan_tables(plan, byref(a), byref(b), byref(c)), "hpspmm_plan_tables")
        return a.value, b.value, c.value

    def plan_row_list(self, plan):
        """Device addresses of nz_id, nz_end, chunk_ri."""
        a, b, c = _P(), _P(), _P()
        self._check(self.lib.hpspmm_plan_row_list(plan, byref(a), byref(b), byref(c)), "hpspmm_plan_row_list")
        return a.value, b.value, c.value

    def spmm_csr(self, M, N, K, nnz, row_ptr, col_idx, vals, B, C, plan=None, opts=None, stream=None):
        self._check(self.lib.hpspmm_spmm_csr_f32(self.handle, plan, M, N, K, nnz, _ptr(row_ptr),
                                                 _ptr(col_idx), _ptr(vals), _ptr(B), _ptr(C),
                                                 byref(opts) if opts else None, stream),
                    "hpspmm_spmm_csr_f32")

    def spmm_csr_host(self, M, N, K, nnz, row_ptr, col_idx, vals, B, C, opts=None):
        self._check(self.lib.hpspmm_spmm_csr_f32_host(self.handle, M, N, K, nnz, _ptr(row_ptr),
                                                      _ptr(col_idx), _ptr(vals), _ptr(B), _ptr(C),
                                                      byref(opts) if opts else None),
                    "hpspmm_spmm_csr_f32_host")

    def spmm_csr_host_multi(self, M, N, nnz, row_ptr, col_idx, vals, Ks, Bs, Cs, opts=None):
        """C_i = A * B_i for host arrays (or raw host addresses) B_i, C_i; A is uploaded once."""
        n = len(Ks)
        ks = (_I64 * n)(*[int(k) for k in Ks])
        bs = (_P * n)(*[_ptr(b) for b in Bs])
        cs = (_P * n)(*[_ptr(c) for c in Cs])
        self._check(self.lib.hpspmm_spmm_csr_f32_host_multi(self.handle, M, N, nnz, _ptr(row_ptr), _ptr(col_idx),
                                                            _ptr(vals), n, ks, bs, cs,
                                                            byref(opts) if opts else None),
                    "hpspmm_spmm_csr_f32_host_multi")

    def spmm_coo(self, M, N, K, nnz_padded, row_idx, col_idx, vals, B, C, opts=None, stream=None):
        self._check(self.lib.hpspmm_spmm_coo_f32(self.handle, M, N, K, nnz_padded, _ptr(row_idx),
                                                 _ptr(col_idx), _ptr(vals), _ptr(B), _ptr(C),
                                                 byref(opts) if opts else None, stream),
                    "hpspmm_spmm_coo_f32")

    def sddmm_csr(self, M, N, K, nnz, row_ptr, col_idx, X, Y, out, plan=None, opts=None, stream=None):
        self._check(self.lib.hpspmm_sddmm_csr_f32(self.handle, plan, M, N, K, nnz, _ptr(row_ptr),
                                                  _ptr(col_idx), _ptr(X), _ptr(Y), _ptr(out),
                                                  byref(opts) if opts else None, stream),
                    "hpspmm_sddmm_csr_f32")

    def csr_transpose(self, M, N, nnz, row_ptr, col_idx, vals, row_ptr_t, col_idx_t, vals_t,
                      perm=None, stream=None):
        self._check(self.lib.hpspmm_csr_transpose(self.handle, M, N, nnz, _ptr(row_ptr), _ptr(col_idx),
                                                  _ptr(vals), _ptr(row_ptr_t), _ptr(col_idx_t),
                                                  _ptr(vals_t), _ptr(perm), stream),
                    "hpspmm_csr_transpose")

    def csr_to_coo_reordered(self, M, nnz, row_ptr, col_idx, vals, row_order, padding, row_out, col_out,
                             val_out, stream=None):
        self._check(self.lib.hpspmm_csr_to_coo_reordered(self.handle, M, nnz, _ptr(row_ptr), _ptr(col_idx),
                                                         _ptr(vals), _ptr(row_order), padding, _ptr(row_out),
                                                         _ptr(col_out), _ptr(val_out), stream),
                    "hpspmm_csr_to_coo_reordered")

    def csr_permute(self, M, N, nnz, row_ptr, col_idx, vals, row_order, col_new_id, row_ptr_out, col_out,
                    val_out, stream=None):
        self._check(self.lib.hpspmm_csr_permute(self.handle, M, N, nnz, _ptr(row_ptr), _ptr(col_idx), _ptr(vals),
                                                _ptr(row_order), _ptr(col_new_id), _ptr(row_ptr_out),
                                                _ptr(col_out), _ptr(val_out), stream), "hpspmm_csr_permute")

    def order_rows_by_degree(self, M, row_ptr, order_out, stream=None):
        self._check(self.lib.hpspmm_order_rows_by_degree(self.handle, M, _ptr(row_ptr), _ptr(order_out), stream),
                    "hpspmm_order_rows_by_degree")

    def invert_permutation(self, M, order, inverse_out, stream=None):
        self._check(self.lib.hpspmm_invert_permutation(self.handle, M, _ptr(order), _ptr(inverse_out), stream),
                    "hpspmm_invert_permutation")

    def gather_rows(self, M, K, src, order, dst, stream=None):
        self._check(self.lib.hpspmm_gather_rows_f32(self.handle, M, K, _ptr(src), _ptr(order), _ptr(dst), stream),
                    "hpspmm_gather_rows_f32")

    def csr_to_coo_padded(self, M, nnz, row_ptr, col_idx, vals, padding, row_out, col_out, val_out,
                          stream=None):
        self._check(self.lib.hpspmm_csr_to_coo_padded(self.handle, M, nnz, _ptr(row_ptr),
                                                      _ptr(col_idx), _ptr(vals), padding,
                                                      _ptr(row_out), _ptr(col_out), _ptr(val_out),
                                                      stream), "hpspmm_csr_to_coo_padded")

    def validate_csr(self, M, N, nnz, row_ptr, col_idx, stream=None):
        """Returns (status, first bad position or -1)."""
        bad = _I64(-1)
        st = self.lib.hpspmm_validate_csr(self.handle, M, N, nnz, _ptr(row_ptr), _ptr(col_idx),
                                          byref(bad), stream)
        return st, bad.value

    def launch_count(self):
        return self.lib.hpspmm_ctx_launch_count(self.handle)

    def probe_gather(self, row_bytes, table_rows, n_gathers, pattern=1, hot_rows=0, hot_share=0.0, repeats=10):
        """GB/s and ms per launch of the bare gather shape (hpspmm_probe_gather_gbs)."""
        gbs, ms = c_double(), c_double()
        self._check(self.lib.hpspmm_probe_gather_gbs(self.handle, row_bytes, table_rows, n_gathers, pattern,
                                                     hot_rows, hot_share, repeats, byref(gbs), byref(ms)),
                    "hpspmm_probe_gather_gbs")
        return gbs.value, ms.value

    def tma_fallbacks(self):
        """Warps of the HPSPMM_ALGO_TMA kernel that gave up waiting for a TMA copy (expected 0); synchronises."""
        n = _I64()
        self._check(self.lib.hpspmm_ctx_tma_fallbacks(self.handle, byref(n)), "hpspmm_ctx_tma_fallbacks")
        return n.value

    def probe_tma_gather(self, row_bytes, table_rows, n_gathers, ctas_per_sm=2, repeats=10):
        """The same random rows fetched by TMA gather4 into shared memory (hpspmm_probe_tma_gather_gbs):
        GB/s, ms per launch, the sum of everything read and the number of gathers per launch."""
        gbs, ms, checksum, done = c_double(), c_double(), c_double(), _I64()
        self._check(self.lib.hpspmm_probe_tma_gather_gbs(self.handle, row_bytes, table_rows, n_gathers, ctas_per_sm,
                                                         repeats, byref(gbs), byref(ms), byref(checksum),
                                                         byref(done)),
                    "hpspmm_probe_tma_gather_gbs")
        return gbs.value, ms.value, checksum.value, done.value


# ---- host side ---------------------------------------------------------------------------

class Layer:
    """One aggregation layer C = A·H with both backward products (hpspmm_layer_* of the C ABI).

    row_ptr, col_idx and vals are device arrays (DeviceBuffer or raw addresses) that the caller
    keeps alive.  All products run on `stream` and only enqueue work."""

    def __init__(self, ctx, M, N, nnz, row_ptr, col_idx, vals, max_K, stream=None):
        self.ctx, self.M, self.N, self.nnz, self.max_K = ctx, M, N, nnz, max_K
        h = _P()
        ctx._check(ctx.lib.hpspmm_layer_create(ctx.handle, M, N, nnz, _ptr(row_ptr), _ptr(col_idx), _ptr(vals),
                                               max_K, stream, byref(h)), "hpspmm_layer_create")
        self.handle = h

    def close(self):
        if self.handle:
            self.ctx.lib.hpspmm_layer_destroy(self.ctx.handle, self.handle)
            self.handle = None

    def info(self):
        v = [_I64() for _ in range(5)]
        self.ctx._check(self.ctx.lib.hpspmm_layer_info(self.handle, *[byref(x) for x in v]), "hpspmm_layer_info")
        return dict(zip(("M", "N", "nnz", "max_K", "owned_bytes"), (x.value for x in v)))

    def transposed(self):
        """Device addresses of the transpose the layer owns: row_ptr_t, col_idx_t, vals_t, perm."""
        v = [_P() for _ in range(4)]
        self.ctx._check(self.ctx.lib.hpspmm_layer_transposed(self.handle, *[byref(x) for x in v]),
                        "hpspmm_layer_transposed")
        return tuple(x.value for x in v)

    def forward(self, K, H, C, stream=None):
        self.ctx._check(self.ctx.lib.hpspmm_layer_forward(self.ctx.handle, self.handle, K, _ptr(H), _ptr(C),
                                                          stream), "hpspmm_layer_forward")

    def backward_features(self, K, dC, dH, stream=None):
        self.ctx._check(self.ctx.lib.hpspmm_layer_backward_features(self.ctx.handle, self.handle, K, _ptr(dC),
                                                                    _ptr(dH), stream),
                        "hpspmm_layer_backward_features")

    def backward_weights(self, K, dC, H, dA, stream=None):
        self.ctx._check(self.ctx.lib.hpspmm_layer_backward_weights(self.ctx.handle, self.handle, K, _ptr(dC),
                                                                   _ptr(H), _ptr(dA), stream),
                        "hpspmm_layer_backward_weights")

    def update_values(self, vals, stream=None):
        self.ctx._check(self.ctx.lib.hpspmm_layer_update_values(self.ctx.handle, self.handle, _ptr(vals), stream),
                        "hpspmm_layer_update_values")


def _export_graph(lib, g):
    M, N, nnz = _I64(), _I64(), _I64()
    lib.hpspmm_gen_shape(g, byref(M), byref(N), byref(nnz))
    row_ptr = np.empty(M.value + 1, dtype=np.int32)
    col_idx = np.empty(nnz.value, dtype=np.int32)
    vals = np.empty(nnz.value, dtype=np.float32)
    lib.hpspmm_gen_export(g, row_ptr.ctypes.data, col_idx.ctypes.data, vals.ctypes.data)
    lib.hpspmm_gen_free(g)
    return {"M": M.value, "N": N.value, "nnz": nnz.value, "row_ptr": row_ptr, "col_idx": col_idx,
            "vals": vals}


def _gen_check(lib, st, what):
    if st != OK:
        raise HpspmmError(st, what, lib.hpspmm_status_string(st).decode())


def gen_uniform_degree(M, N, deg_lo, deg_hi, seed, vals_kind=VALS_UPM1):
    lib = load_library()
    g = _P()
    _gen_check(lib, lib.hpspmm_gen_uniform_degree(M, N, deg_lo, deg_hi, seed, vals_kind, byref(g)),
               "hpspmm_gen_uniform_degree")
    return _export_graph(lib, g)


def gen_erdos_renyi(M, N, mean_degree, seed, vals_kind=VALS_U01):
    lib = load_library()
    g = _P()
    _gen_check(lib, lib.hpspmm_gen_erdos_renyi(M, N, mean_degree, seed, vals_kind, byref(g)),
               "hpspmm_gen_erdos_renyi")
    return _export_graph(lib, g)


def gen_rmat(scale, edge_factor, seed, a=0.57, b=0.19, c=0.19, vals_kind=VALS_U01):
    lib = load_library()
    g = _P()
    _gen_check(lib, lib.hpspmm_gen_rmat(scale, edge_factor, a, b, c, seed, vals_kind, byref(g)),
               "hpspmm_gen_rmat")
    return _export_graph(lib, g)


def read_smtx(path):
    lib = load_library()
    g = _P()
    _gen_check(lib, lib.hpspmm_read_smtx(path.encode(), byref(g)), "hpspmm_read_smtx")
    return _export_graph(lib, g)


def read_row_order(path, M):
    """Reads the reference's row order file (one line of M row ids); raises unless it is a permutation."""
    lib = load_library()
    out = np.empty(M, dtype=np.int32)
    _gen_check(lib, lib.hpspmm_read_row_order(path.encode(), M, out.ctypes.data), "hpspmm_read_row_order")
    return out


def host_fill_uniform(count, seed, stream_id, lo, hi):
    lib = load_library()
    out = np.empty(int(count), dtype=np.float32)
    _gen_check(lib, lib.hpspmm_host_fill_uniform_f32(out.ctypes.data, int(count), seed, stream_id,
                                                     lo, hi), "hpspmm_host_fill_uniform_f32")
    return out


def shard_bounds(row_ptr, G):
    lib = load_library()
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    out = np.empty(G + 1, dtype=np.int64)
    _gen_check(lib, lib.hpspmm_shard_bounds(len(row_ptr) - 1, row_ptr.ctypes.data, G, out.ctypes.data),
               "hpspmm_shard_bounds")
    return out


def shard_bounds_weighted(row_ptr, G, row_weight):
    """Row blocks balanced by entries + row_weight per row (hpspmm_shard_bounds_weighted)."""
    lib = load_library()
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    out = np.empty(G + 1, dtype=np.int64)
    _gen_check(lib, lib.hpspmm_shard_bounds_weighted(len(row_ptr) - 1, row_ptr.ctypes.data, G, float(row_weight),
                                                     out.ctypes.data), "hpspmm_shard_bounds_weighted")
    return out


def shard_csr(row_ptr, col_idx, vals, row_lo, row_hi):
    """Local CSR of rows [row_lo, row_hi): rebased row_ptr, views of col_idx / vals."""
    lib = load_library()
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    local = np.empty(row_hi - row_lo + 1, dtype=np.int32)
    lo, n = _I64(), _I64()
    _gen_check(lib, lib.hpspmm_shard_row_ptr(row_ptr.ctypes.data, row_lo, row_hi, local.ctypes.data,
                                             byref(lo), byref(n)), "hpspmm_shard_row_ptr")
    return local, col_idx[lo.value:lo.value + n.value], vals[lo.value:lo.value + n.value]


def shard_needed_rows(col_idx, N, b_bounds):
    """Rows of B a shard references: (col_compact, need_rows, need_off) of hpspmm_shard_needed_rows."""
    lib = load_library()
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    b_bounds = np.ascontiguousarray(b_bounds, dtype=np.int64)
    world = len(b_bounds) - 1
    nnz = len(col_idx)
    col_compact = np.empty(nnz, dtype=np.int32)
    need = np.empty(max(1, min(int(N), max(nnz, 1))), dtype=np.int32)
    off = np.empty(world + 1, dtype=np.int64)
    n = _I64()
    _gen_check(lib, lib.hpspmm_shard_needed_rows(nnz, col_idx.ctypes.data, N, world, b_bounds.ctypes.data,
                                                 col_compact.ctypes.data, need.ctypes.data, off.ctypes.data,
                                                 byref(n)), "hpspmm_shard_needed_rows")
    return col_compact, need[:n.value].copy(), off


def comm_unique_id():
    """128 bytes that identify a new communicator; create on one rank, carry to the others."""
    lib = load_library()
    buf = (ctypes.c_ubyte * COMM_ID_BYTES)()
    _gen_check(lib, lib.hpspmm_comm_unique_id(buf), "hpspmm_comm_unique_id")
    return bytes(buf)


class ShardedSpmm:
    """One rank's side of the row-sharded product (hpspmm_comm_* / hpspmm_shard_plan_* / hpspmm_sharded_*).

    row_ptr / col_idx are the shard's HOST arrays (global column ids); b_bounds says which rank owns
    which rows of B.  comm_id: bytes from comm_unique_id() of one rank (None when world == 1)."""

    def __init__(self, ctx, world, rank, comm_id, M_local, N, row_ptr, col_idx, b_bounds, max_K,
                 exchange=EXCHANGE_NEEDED_ROWS, stream=None):
        self.ctx, self.world, self.rank = ctx, world, rank
        self.comm, self.plan = _P(), _P()
        idbuf = (ctypes.c_ubyte * COMM_ID_BYTES).from_buffer_copy(comm_id) if comm_id is not None else None
        ctx._check(ctx.lib.hpspmm_comm_create(ctx.handle, world, rank, idbuf, byref(self.comm)), "hpspmm_comm_create")
        self._row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
        self._col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
        self._bounds = np.ascontiguousarray(b_bounds, dtype=np.int64)
        self.M_local, self.N, self.nnz_local = int(M_local), int(N), len(self._col_idx)
        self.rows_own = int(self._bounds[rank + 1] - self._bounds[rank])
        try:
            ctx._check(ctx.lib.hpspmm_shard_plan_create(ctx.handle, self.comm, self.M_local, self.N, self.nnz_local,
                                                        self._row_ptr.ctypes.data, self._col_idx.ctypes.data,
                                                        self._bounds.ctypes.data, max_K, exchange, stream,
                                                        byref(self.plan)), "hpspmm_shard_plan_create")
        except Exception:
            ctx.lib.hpspmm_comm_destroy(self.comm)
            self.comm = _P()
            raise

    def info(self):
        v = [_I64() for _ in range(4)]
        self.ctx._check(self.ctx.lib.hpspmm_shard_plan_info(self.plan, *[byref(x) for x in v]), "hpspmm_shard_plan_info")
        return dict(zip(("rows_local", "rows_received", "rows_sent", "device_bytes"), (x.value for x in v)))

    def begin(self, slot, K, B_own, stream=None):
        self.ctx._check(self.ctx.lib.hpspmm_sharded_exchange_begin(self.ctx.handle, self.plan, slot, K, _ptr(B_own),
                                                                   stream), "hpspmm_sharded_exchange_begin")

    def product(self, slot, K, vals, C_local, opts=None, stream=None):
        self.ctx._check(self.ctx.lib.hpspmm_sharded_product(self.ctx.handle, self.plan, slot, K, _ptr(vals),
                                                            _ptr(C_local), byref(opts) if opts else None, stream),
                        "hpspmm_sharded_product")

    def spmm(self, K, vals, B_own, C_local, opts=None, stream=None):
        self.ctx._check(self.ctx.lib.hpspmm_spmm_sharded_f32(self.ctx.handle, self.plan, K, _ptr(vals), _ptr(B_own),
                                                             _ptr(C_local), byref(opts) if opts else None, stream),
                        "hpspmm_spmm_sharded_f32")

    def close(self):
        if self.plan:
            self.ctx.lib.hpspmm_shard_plan_destroy(self.ctx.handle, self.plan)
            self.plan = _P()
        if self.comm:
            self.ctx.lib.hpspmm_comm_destroy(self.comm)
            self.comm = _P()


def gflops(nnz, K, ms):
    return load_library().hpspmm_gflops(nnz, K, ms)


def spmm_algorithmic_bytes(M, N_ref, K, nnz):
    return load_library().hpspmm_spmm_algorithmic_bytes(M, N_ref, K, nnz)


def sddmm_algorithmic_bytes(M_ref, N_ref, K, M, nnz):
    return load_library().hpspmm_sddmm_algorithmic_bytes(M_ref, N_ref, K, M, nnz)
