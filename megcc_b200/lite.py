"""ctypes face of the LITE_* C API (include/megcc_b200_lite.h), shaped like the calls a C
program makes: make_network -> load_model_from_mem -> get_io_tensor -> reset_tensor_memory
-> forward -> wait -> get_tensor_memory."""
import ctypes as C

import numpy as np

from ._lib import LIB_PATH, lib as _ops_lib

LITE_CPU, LITE_CUDA = 0, 1
LITE_IO, LITE_INPUT, LITE_OUTPUT = 0, 1, 2


class LiteOptions(C.Structure):
    _fields_ = [(k, C.c_int) for k in (
        "weight_preprocess", "fuse_preprocess", "fake_next_exec", "var_sanity_check_first_run",
        "const_shape", "force_dynamic_alloc", "force_output_dynamic_alloc",
        "no_profiling_on_shape_change", "jit_level", "comp_node_seq_record_level",
        "graph_opt_level", "async_exec_level", "enable_nchw44", "enable_nchw44_dot",
        "enable_nchw88", "enable_nhwcd4", "enable_nchw4", "enable_nchw32", "enable_nchw64")]


class LiteConfig(C.Structure):
    _fields_ = [("has_compression", C.c_int), ("device_id", C.c_int), ("device_type", C.c_int),
                ("backend", C.c_int), ("bare_model_cryption_name", C.c_char_p),
                ("options", LiteOptions)]


class LiteLayout(C.Structure):
    _fields_ = [("shapes", C.c_size_t * 7), ("ndim", C.c_size_t), ("data_type", C.c_int)]


class LiteIO(C.Structure):
    _fields_ = [("name", C.c_char_p), ("is_host", C.c_int), ("io_type", C.c_int),
                ("config_layout", LiteLayout)]


class LiteNetworkIO(C.Structure):
    _fields_ = [("inputs", C.POINTER(LiteIO)), ("outputs", C.POINTER(LiteIO)),
                ("input_size", C.c_size_t), ("output_size", C.c_size_t)]


_P = C.c_void_p
SIGNATURES = {
    "default_config": (C.POINTER(LiteConfig), []),
    "default_network_io": (C.POINTER(LiteNetworkIO), []),
    "LITE_make_network": (C.c_int, [C.POINTER(_P), LiteConfig, LiteNetworkIO]),
    "LITE_load_model_from_mem": (C.c_int, [_P, _P, C.c_size_t]),
    "LITE_load_model_with_shared_mem": (C.c_int, [_P, _P, C.c_size_t]),
    "LITE_load_model_from_path": (C.c_int, [_P, C.c_char_p]),
    "LITE_get_io_tensor": (C.c_int, [_P, C.c_char_p, C.c_int, C.POINTER(_P)]),
    "LITE_get_tensor_total_size_in_byte": (C.c_int, [_P, C.POINTER(C.c_size_t)]),
    "LITE_forward": (C.c_int, [_P]),
    "LITE_wait": (C.c_int, [_P]),
    "LITE_get_input_name": (C.c_int, [_P, C.c_size_t, C.POINTER(C.c_char_p)]),
    "LITE_get_output_name": (C.c_int, [_P, C.c_size_t, C.POINTER(C.c_char_p)]),
    "LITE_get_all_input_name": (C.c_int, [_P, C.POINTER(C.c_size_t), C.POINTER(C.c_char_p)]),
    "LITE_get_all_output_name": (C.c_int, [_P, C.POINTER(C.c_size_t), C.POINTER(C.c_char_p)]),
    "LITE_share_runtime_memroy": (C.c_int, [_P, _P]),
    "LITE_destroy_network": (C.c_int, [_P]),
    "LITE_get_tensor_memory": (C.c_int, [_P, C.POINTER(_P)]),
    "LITE_set_tensor_layout": (C.c_int, [_P, LiteLayout]),
    "LITE_reset_tensor_memory": (C.c_int, [_P, _P, C.c_size_t]),
    "LITE_get_tensor_layout": (C.c_int, [_P, C.POINTER(LiteLayout)]),
    "LITE_destroy_tensor": (C.c_int, [_P]),
    "LITE_set_log_level": (C.c_int, [C.c_int]),
    "LITE_get_log_level": (C.c_int, [C.POINTER(C.c_int)]),
    "LITE_get_last_error": (C.c_char_p, []),
    "LITE_get_device_id": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "LITE_set_device_id": (C.c_int, [_P, C.c_int]),
    "LITE_get_device_type": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "LITE_get_tensor_device_type": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "mb200_lite_stream": (C.c_int, [_P, C.POINTER(_P)]),
    "mb200_lite_set_profile": (C.c_int, [_P, C.c_int]),
    "mb200_lite_set_option": (C.c_int, [_P, C.c_char_p, C.c_int]),
    "mb200_lite_set_kernel_tables": (C.c_int, [_P, _P, C.c_int, _P, C.c_int]),
    "mb200_lite_profile": (C.c_int, [_P, C.c_char_p, C.c_size_t]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        _ops_lib()  # raises the loud "no fallback" error when the library is missing
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class LiteError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"TinyNNStatus {status}: {msg}")
        self.status = status


def check(status):
    if status != 0:
        raise LiteError(status, lib().LITE_get_last_error().decode())


class Network:
    """One LiteNetwork. ``device_outputs``/``device_inputs`` name the I/O tensors that stay
    in device memory (LiteIO.is_host = 0)."""

    def __init__(self, model_bytes, device_id=0, device_io=(), kernel_tables=None):
        """kernel_tables: (address of kernels[], count, address of init_kernels[], count) of a
        generated kernels.c that was compiled and loaded by the caller, or None."""
        L = lib()
        cfg = L.default_config().contents
        cfg = LiteConfig.from_buffer_copy(cfg)
        cfg.device_id = device_id
        cfg.device_type = LITE_CUDA
        self._io_keep = [LiteIO(n.encode(), 0, 0, LiteLayout()) for n in device_io]
        io = LiteNetworkIO()
        if self._io_keep:
            arr = (LiteIO * len(self._io_keep))(*self._io_keep)
            self._io_arr = arr
            io.outputs = arr
            io.output_size = len(self._io_keep)
        self._net = _P()
        check(L.LITE_make_network(C.byref(self._net), cfg, io))
        if kernel_tables is not None:
            k, nk, i, ni = kernel_tables
            check(L.mb200_lite_set_kernel_tables(self._net, _P(k), nk, _P(i), ni))
        # the runtime borrows the buffer for the life of the network
        self._model = C.create_string_buffer(model_bytes, len(model_bytes))
        try:
            check(L.LITE_load_model_from_mem(self._net, self._model, len(model_bytes)))
        except Exception:
            L.LITE_destroy_network(self._net)
            self._net = None
            raise
        self._tensors = {}
        self._in_keep = {}

    def close(self):
        if getattr(self, "_net", None):
            lib().LITE_destroy_network(self._net)
            self._net = None

    __del__ = close

    def _names(self, fn):
        n = C.c_size_t()
        check(fn(self._net, C.byref(n), None))
        arr = (C.c_char_p * n.value)()
        check(fn(self._net, None, arr))
        return [a.decode() for a in arr]

    def input_names(self):
        return self._names(lib().LITE_get_all_input_name)

    def output_names(self):
        return self._names(lib().LITE_get_all_output_name)

    def tensor(self, name, phase=LITE_IO):
        key = (name, phase)
        if key not in self._tensors:
            t = _P()
            check(lib().LITE_get_io_tensor(self._net, name.encode(), phase, C.byref(t)))
            self._tensors[key] = t
        return self._tensors[key]

    def tensor_bytes(self, name, phase=LITE_IO):
        n = C.c_size_t()
        check(lib().LITE_get_tensor_total_size_in_byte(self.tensor(name, phase), C.byref(n)))
        return n.value

    def _shape(self, name, phase):
        # quantised tensors have no lite data type: for them the call fails with
        # TinyNN_ERROR_OUT_OF_RANGE, as the reference's does (runtime/src/lite/tensor.c:11-40)
        lay = LiteLayout()
        check(lib().LITE_get_tensor_layout(self.tensor(name, phase), C.byref(lay)))
        return tuple(int(lay.shapes[i]) for i in range(lay.ndim))

    def input_shape(self, name):
        return self._shape(name, LITE_INPUT)

    def output_shape(self, name):
        return self._shape(name, LITE_OUTPUT)

    def set_input(self, name, array):
        """Host numpy array: borrowed until the next set_input / close."""
        a = np.ascontiguousarray(array)
        self._in_keep[name] = a
        check(lib().LITE_reset_tensor_memory(self.tensor(name, LITE_INPUT), a.ctypes.data,
                                             a.nbytes))

    def set_input_ptr(self, name, ptr, nbytes):
        """Raw pointer (pinned host or device memory owned by the caller)."""
        check(lib().LITE_reset_tensor_memory(self.tensor(name, LITE_INPUT), _P(ptr), nbytes))

    def select_batch(self, name, shape):
        lay = LiteLayout()
        for i, d in enumerate(shape):
            lay.shapes[i] = d
        lay.ndim = len(shape)
        lay.data_type = 4
        check(lib().LITE_set_tensor_layout(self.tensor(name, LITE_INPUT), lay))

    def stream(self):
        """cudaStream_t (as int) the network issues its work on."""
        p = _P()
        check(lib().mb200_lite_stream(self._net, C.byref(p)))
        return p.value or 0

    def set_option(self, name, value):
        check(lib().mb200_lite_set_option(self._net, name.encode(), int(value)))

    def set_profile(self, enable):
        check(lib().mb200_lite_set_profile(self._net, int(enable)))

    def profile(self):
        """[(opr name, kernel symbol, mean ms, samples)] gathered while profiling was on."""
        buf = C.create_string_buffer(1 << 16)
        check(lib().mb200_lite_profile(self._net, buf, len(buf)))
        rows = []
        for line in buf.value.decode().splitlines():
            name, sym, ms, cnt = line.rsplit(" ", 3)
            rows.append((name, sym, float(ms), int(cnt)))
        return rows

    def forward(self):
        check(lib().LITE_forward(self._net))

    def wait(self):
        check(lib().LITE_wait(self._net))

    def output_ptr(self, name):
        p = _P()
        check(lib().LITE_get_tensor_memory(self.tensor(name, LITE_OUTPUT), C.byref(p)))
        return p.value

    def output(self, name, dtype=np.int8):
        """Host copy of an output as a flat numpy array."""
        n = self.tensor_bytes(name, LITE_OUTPUT)
        p = self.output_ptr(name)
        return np.frombuffer(C.string_at(p, n), dtype=dtype).copy()
