"""ctypes binding of libflutter_ml_b200.so (the C ABI declared in include/fml.h).

This is the Python counterpart of the Dart binding the library is designed for
(lib/cuda/cudacaller.dart:6-19 in the reference binds its native stub the same
way: open the shared object, look symbols up, call).  There is no fallback: if
the shared object is missing or no B200 is present, the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libflutter_ml_b200.so")

PREC_TF32, PREC_3XTF32, PREC_FP32 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH, ACT_GELU = 0, 1, 2, 3, 4
ACT_BY_NAME = {None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "sigmoid": ACT_SIGMOID, "tanh": ACT_TANH,
               "gelu": ACT_GELU}

i32, i64, f32 = C.c_int32, C.c_int64, C.c_float
fp = C.c_void_p  # device pointers travel as plain addresses


class FmlError(RuntimeError):
    pass


class Config(C.Structure):
    _fields_ = [("device", i32), ("precision", i32), ("workspace_bytes", i64)]


class GemmDesc(C.Structure):
    _fields_ = [("M", i32), ("N", i32), ("K", i32), ("transA", i32), ("transB", i32),
                ("lda", i64), ("ldb", i64), ("ldc", i64),
                ("A", fp), ("B", fp), ("C", fp), ("bias", fp), ("preact", fp),
                ("act", i32), ("alpha", f32), ("beta", f32), ("batch1", i32), ("batch2", i32),
                ("sA1", i64), ("sA2", i64), ("sB1", i64), ("sB2", i64), ("sC1", i64), ("sC2", i64),
                ("precision", i32), ("dact_saved", fp), ("dact", i32),
                ("rowop", i32), ("rowop_causal", i32), ("rowop_aux", fp)]


class LstmDesc(C.Structure):
    _fields_ = [("T", i32), ("B", i32), ("I", i32), ("H", i32), ("W", fp), ("b", fp), ("x", fp),
                ("gates", fp), ("cells", fp), ("hs", fp), ("xproj", fp)]


class AttentionDesc(C.Structure):
    _fields_ = [("n_seq", i32), ("seq_len", i32), ("heads", i32), ("d_head", i32), ("q", fp), ("k", fp), ("v", fp),
                ("ld_qkv", i64), ("out", fp), ("ld_out", i64), ("lse", fp), ("scale", f32), ("causal", i32)]


class Op(C.Structure):
    """fml_op: one autograd node of a tape handed to fml_tape_run."""
    _fields_ = [("kind", i32), ("rows", i32), ("cols", i32), ("inner", i32), ("inp", fp * 3), ("gin", fp * 3),
                ("out", fp), ("gout", fp), ("aux", fp * 2), ("ids", fp), ("parts", fp), ("gparts", fp),
                ("part_cols", fp), ("n_parts", i32), ("s", f32), ("iparam", i32), ("precision", i32)]


# name -> argument types (restype is int32 unless listed in _RESTYPES)
PROTOTYPES = {
    "fml_init": [C.POINTER(Config), C.POINTER(fp)],
    "fml_shutdown": [fp],
    "fml_last_error": [fp],
    "fml_device_count": [C.POINTER(i32)],
    "fml_device_name": [i32, C.c_char_p, i32],
    "fml_sm_count": [fp, C.POINTER(i32)],
    "fml_set_sm_reserve": [fp, i32],
    "fml_set_stream": [fp, fp],
    "fml_sync": [fp],
    "fml_device_status": [fp, C.POINTER(i32)],
    "fml_selftest_wait_timeout": [fp, i32],
    "fml_selftest_per_device_once": [i32, C.POINTER(i32)],
    "fml_alloc": [fp, i64, C.POINTER(fp)],
    "fml_mem_info": [fp, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)],
    "fml_free": [fp, fp],
    "fml_zero": [fp, fp, i64],
    "fml_fill": [fp, fp, i64, f32],
    "fml_upload_f32": [fp, fp, fp, i64],
    "fml_upload_f64": [fp, fp, fp, i64],
    "fml_upload_i32": [fp, fp, fp, i64],
    "fml_download_f32": [fp, fp, fp, i64],
    "fml_download_f64": [fp, fp, fp, i64],
    "fml_copy": [fp, fp, fp, i64],
    "fml_host_alloc": [fp, i64, C.POINTER(fp)],
    "fml_host_free": [fp, fp],
    "fml_event_sync": [fp, i32],
    "fml_stage_rows": [fp, fp, fp, i32, i64, fp, i64, i64, i32],
    "fml_stage_rows_async": [fp, fp, fp, i32, i64, fp, i64, i64, i32],
    "fml_stage_wait": [fp],
    "fml_event_record": [fp, i32],
    "fml_event_elapsed_ms": [fp, i32, i32, C.POINTER(f32)],
    "fml_lane_h2d": [fp, i32, fp, fp, i64],
    "fml_lane_d2h": [fp, i32, fp, fp, i64],
    "fml_lane_sync": [fp, i32],
    "fml_event_record_on": [fp, i32, i32],
    "fml_wait_event": [fp, i32, i32],
    "fml_graph_begin": [fp],
    "fml_graph_end": [fp, C.POINTER(i32)],
    "fml_graph_launch": [fp, i32],
    "fml_graph_destroy": [fp, i32],
    "fml_timer_start": [fp],
    "fml_timer_stop_ms": [fp, C.POINTER(f32)],
    "fml_gemm": [fp, C.POINTER(GemmDesc)],
    "fml_gemm_last_path": [fp, C.POINTER(i32)],
    "fml_gemm_last_tile": [fp, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)],
    "multiplyMatrices": [fp, fp, fp, i32, i32, i32],
    "benchtest": [],
    "fml_act_fwd": [fp, i32, fp, fp, i64],
    "fml_act_bwd": [fp, i32, fp, fp, fp, i64, i64, i32, fp],
    "fml_add": [fp, fp, fp, fp, i64],
    "fml_axpy": [fp, f32, fp, fp, i64],
    "fml_mul": [fp, fp, fp, fp, i64],
    "fml_add_bias": [fp, fp, fp, fp, i64, i64],
    "fml_col_sum": [fp, fp, fp, i64, i64, i32],
    "fml_transpose": [fp, fp, fp, i64, i64],
    "fml_softmax_rows_fwd": [fp, fp, fp, i64, i32, f32, i32],
    "fml_softmax_rows_bwd": [fp, fp, fp, fp, i64, i32, f32, i32],
    "fml_layernorm_fwd": [fp, fp, fp, fp, fp, fp, fp, fp, i64, i32, f32],
    "fml_layernorm_bwd": [fp, fp, fp, fp, fp, fp, fp, fp, i64, i32, i32],
    "fml_softmax_xent": [fp, fp, fp, fp, fp, i64, i32, f32],
    "fml_softmax_xent_dbias": [fp, fp, fp, fp, fp, i64, i32, f32, fp],
    "fml_softmax_xent_static": [fp, fp, fp, fp, fp, i64, i32, f32],
    "fml_mse": [fp, fp, fp, fp, fp, i64, f32],
    "fml_embedding_fwd": [fp, fp, fp, fp, fp, i64, i32, i32, i32],
    "fml_embedding_bwd": [fp, fp, fp, fp, i64, i32, i32],
    "fml_positional_table": [fp, fp, i32, i32],
    "fml_sgd_step": [fp, fp, fp, i64, C.c_double, C.c_double],
    "fml_adam_step": [fp, fp, fp, fp, fp, i64, C.c_double, C.c_double, C.c_double, C.c_double, i32, C.c_double],
    "fml_adam_step_on": [fp, i32, fp, fp, fp, fp, i64, C.c_double, C.c_double, C.c_double, C.c_double, i32, C.c_double, i32],
    "fml_optimizer_step": [fp, i32, fp, fp, fp, fp, fp, i64, C.c_double, C.c_double, C.c_double, C.c_double, C.c_double, i32],
    "fml_act2_fwd": [fp, i32, f32, fp, fp, i64],
    "fml_act2_bwd": [fp, i32, f32, fp, fp, fp, i64, i32],
    "fml_attention_fwd": [fp, C.POINTER(AttentionDesc)],
    "fml_attention_bwd": [fp, C.POINTER(AttentionDesc), fp, i64, fp, fp, fp, i64, i32, fp],
    "fml_conv2d_fwd": [fp, fp, fp, fp, fp, i32, i32, i32, i32, i32, i32, i32],
    "fml_conv2d_bwd": [fp, fp, fp, fp, fp, fp, fp, i32, i32, i32, i32, i32, i32, i32],
    "fml_checkpoint_save": [fp, C.c_char_p, i64, i32, fp, fp, fp],
    "fml_checkpoint_load": [fp, C.c_char_p, C.POINTER(i64), i32, fp, fp, fp],
    "fml_tape_run": [fp, C.POINTER(Op), i32, i32],
    "fml_tape_kind": [C.c_char_p],
    "fml_lstm_fwd": [fp, C.POINTER(LstmDesc)],
    "fml_lstm_bwd": [fp, C.POINTER(LstmDesc), fp, fp, fp, fp, fp],
    "fml_lstm_cell_fwd": [fp, fp, fp, fp, fp, fp, i64, i64],
    "fml_lstm_cell_bwd": [fp, fp, fp, fp, fp, fp, fp, fp, i32, i64, i64],
    "fml_dp_unique_id": [C.c_char_p],
    "fml_dp_init": [fp, C.c_char_p, i32, i32],
    "fml_dp_set_timeout": [fp, i32],
    "fml_dp_set_max_ctas": [fp, i32],
    "fml_dp_allreduce_sum": [fp, fp, i64],
    "fml_dp_allreduce_sum_on": [fp, i32, fp, i64],
    "fml_dp_shutdown": [fp],
}
_RESTYPES = {"fml_last_error": C.c_char_p, "multiplyMatrices": None}

_lib = None


def load():
    """Open the shared library and attach prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FmlError(f"{LIB_PATH} is missing: build it with `python -m flutter_ml_b200._build` "
                           "(there is no CPU implementation to fall back to)")
        lib = C.CDLL(LIB_PATH)
        for name, args in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, i32)
        _lib = lib
    return _lib


def _addr(x):
    """Device address of a DeviceArray / int / None, or host address of a numpy array."""
    if x is None:
        return None
    if isinstance(x, DeviceArray):
        return x.ptr
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    return int(x)


class DeviceArray:
    """A float32 (or int32) buffer in device memory with a logical shape."""

    __slots__ = ("ctx", "ptr", "shape", "dtype", "_owner", "_base")

    def __init__(self, ctx, ptr, shape, dtype=np.float32, owner=True):
        self.ctx, self.ptr, self.shape, self.dtype, self._owner = ctx, ptr, tuple(shape), dtype, owner

    @property
    def size(self):
        return int(np.prod(self.shape)) if self.shape else 1

    def view(self, offset_elems, shape):
        v = DeviceArray(self.ctx, self.ptr + 4 * int(offset_elems), shape, self.dtype, owner=False)
        v._base = self  # keeps the allocation alive while the view is
        return v

    def reshape(self, *shape):
        return self.view(0, shape)

    def numpy(self, dtype=np.float32):
        return self.ctx.download(self, dtype)

    def free(self):
        if self._owner and self.ptr and self.ctx.h:
            self.ctx.lib.fml_free(self.ctx.h, self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Context:
    """One fml_ctx: a device, a stream, a scratch arena."""

    def __init__(self, device=0, precision=PREC_TF32, workspace_bytes=0):
        self.lib = load()
        self.h = fp()
        cfg = Config(device, precision, workspace_bytes)
        rc = self.lib.fml_init(C.byref(cfg), C.byref(self.h))
        if rc != 0:
            raise FmlError(f"fml_init failed ({rc}): {self.lib.fml_last_error(None).decode()}")
        self.device = device
        self.precision = precision
        self.launches = 0  # kernels of this library launched through this context (host-side count)

    def check(self, rc):
        if rc != 0:
            raise FmlError(f"fml error {rc}: {self.lib.fml_last_error(self.h).decode()}")

    def close(self):
        if self.h:
            self.lib.fml_shutdown(self.h)
            self.h = fp()

    # ---------------------------------------------------------------- memory
    def empty(self, *shape, dtype=np.float32):
        n = int(np.prod(shape)) if shape else 1
        p = fp()
        self.check(self.lib.fml_alloc(self.h, n, C.byref(p)))
        return DeviceArray(self, p.value, shape, dtype)

    def mem_info(self):
        """(free bytes on the device, total bytes, bytes of the context's scratch arena)."""
        v = [i64(0) for _ in range(3)]
        self.check(self.lib.fml_mem_info(self.h, *[C.byref(x) for x in v]))
        return tuple(x.value for x in v)

    def zeros(self, *shape, dtype=np.float32):
        a = self.empty(*shape, dtype=dtype)
        self.check(self.lib.fml_zero(self.h, a.ptr, a.size))
        return a

    def upload(self, host, out=None):
        host = np.asarray(host)
        if host.dtype == np.float64:
            host = np.ascontiguousarray(host)
            out = out or self.empty(*host.shape)
            self.check(self.lib.fml_upload_f64(self.h, out.ptr, host.ctypes.data, host.size))
        elif host.dtype in (np.int32, np.int64):
            host = np.ascontiguousarray(host, dtype=np.int32)
            out = out or self.empty(*host.shape, dtype=np.int32)
            self.check(self.lib.fml_upload_i32(self.h, out.ptr, host.ctypes.data, host.size))
            self.sync()
        else:
            host = np.ascontiguousarray(host, dtype=np.float32)
            out = out or self.empty(*host.shape)
            self.check(self.lib.fml_upload_f32(self.h, out.ptr, host.ctypes.data, host.size))
            self.sync()
        return out

    def download(self, arr, dtype=np.float32):
        if arr.dtype == np.int32:
            host = np.empty(arr.shape, dtype=np.int32)
            self.check(self.lib.fml_download_f32(self.h, host.ctypes.data, arr.ptr, arr.size))
            return host
        host = np.empty(arr.shape, dtype=dtype)
        fn = self.lib.fml_download_f64 if dtype == np.float64 else self.lib.fml_download_f32
        self.check(fn(self.h, host.ctypes.data, arr.ptr, arr.size))
        return host

    def zero(self, arr):
        self.check(self.lib.fml_zero(self.h, arr.ptr, arr.size))

    def copy(self, dst, src):
        self.check(self.lib.fml_copy(self.h, dst.ptr, src.ptr, src.size))

    def sync(self):
        self.check(self.lib.fml_sync(self.h))

    def device_status(self):
        code = i32(0)
        self.check(self.lib.fml_device_status(self.h, C.byref(code)))
        return code.value

    def sm_count(self):
        n = i32(0)
        self.check(self.lib.fml_sm_count(self.h, C.byref(n)))
        return n.value

    def timer_start(self):
        self.check(self.lib.fml_timer_start(self.h))

    def timer_stop_ms(self):
        ms = f32(0)
        self.check(self.lib.fml_timer_stop_ms(self.h, C.byref(ms)))
        return ms.value

    def graph_begin(self):
        self.check(self.lib.fml_graph_begin(self.h))

    def graph_end(self):
        gid = i32(-1)
        self.check(self.lib.fml_graph_end(self.h, C.byref(gid)))
        return gid.value

    def graph_launch(self, gid, launches=0):
        self.check(self.lib.fml_graph_launch(self.h, gid))
        self.launches += launches

    def event_record(self, slot):
        self.check(self.lib.fml_event_record(self.h, slot))

    def event_elapsed_ms(self, a, b):
        ms = f32(0)
        self.check(self.lib.fml_event_elapsed_ms(self.h, a, b, C.byref(ms)))
        return ms.value

    def pinned(self, shape, dtype=np.float32):
        """numpy array over page-locked host memory (kept alive by the returned array's base)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = fp()
        self.check(self.lib.fml_host_alloc(self.h, n, C.byref(p)))
        buf = (C.c_char * n).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dtype).reshape(shape)
        self._pinned = getattr(self, "_pinned", [])
        self._pinned.append(p.value)
        return arr

    def upload_async(self, host, out):
        """Enqueue a host->device copy of a float32/int32 array (pinned for true asynchrony)."""
        fn = self.lib.fml_upload_i32 if host.dtype == np.int32 else self.lib.fml_upload_f32
        self.check(fn(self.h, out.ptr, host.ctypes.data, host.size))

    def download_into(self, arr, host):
        self.check(self.lib.fml_download_f32(self.h, host.ctypes.data, arr.ptr, arr.size))

    # ------------------------------------------------------------------ gemm
    def gemm(self, A, B, C_, M, N, K, transA=False, transB=False, lda=None, ldb=None, ldc=None, bias=None,
             preact=None, act=ACT_NONE, alpha=1.0, beta=0.0, batch=(1, 1), sA=(0, 0), sB=(0, 0), sC=(0, 0),
             precision=-1, dact_saved=None, dact=ACT_NONE, rowop=0, rowop_causal=False, rowop_aux=None):
        d = GemmDesc()
        d.M, d.N, d.K = M, N, K
        d.transA, d.transB = int(transA), int(transB)
        d.lda = lda if lda is not None else (M if transA else K)
        d.ldb = ldb if ldb is not None else (K if transB else N)
        d.ldc = ldc if ldc is not None else N
        d.A, d.B, d.C = _addr(A), _addr(B), _addr(C_)
        d.bias, d.preact = _addr(bias), _addr(preact)
        d.act = ACT_BY_NAME.get(act, act) if not isinstance(act, int) else act
        d.alpha, d.beta = alpha, beta
        d.batch1, d.batch2 = batch
        d.sA1, d.sA2 = sA
        d.sB1, d.sB2 = sB
        d.sC1, d.sC2 = sC
        d.precision = precision
        d.dact_saved = _addr(dact_saved)
        d.dact = ACT_BY_NAME.get(dact, dact) if not isinstance(dact, int) else dact
        d.rowop, d.rowop_causal, d.rowop_aux = int(rowop), int(bool(rowop_causal)), _addr(rowop_aux)
        self.check(self.lib.fml_gemm(self.h, C.byref(d)))
        self.launches += 3 if (precision == PREC_3XTF32 or (precision < 0 and self.precision == PREC_3XTF32)) else 1

    def gemm_last_path(self):
        p = i32(0)
        self.check(self.lib.fml_gemm_last_path(self.h, C.byref(p)))
        return p.value

    def gemm_last_tile(self):
        """(CTAs per tile, tile columns, K splits, K chunks) of the last tensor-core product."""
        v = [i32(0) for _ in range(4)]
        self.check(self.lib.fml_gemm_last_tile(self.h, *[C.byref(x) for x in v]))
        return tuple(x.value for x in v)

    def call(self, name, *args, launches=1):
        """Call any fml_* entry point that takes the context first; DeviceArrays become addresses."""
        self.check(getattr(self.lib, name)(self.h, *[_addr(a) if isinstance(a, (DeviceArray, np.ndarray)) else a for a in args]))
        self.launches += launches
