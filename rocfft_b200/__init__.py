"""Python host-side mirror of the rocFFT C API, bound to the in-tree
``librocfft.so`` (hand-written CUDA for sm_100a) through ctypes.

The functions have the names, argument order, argument meaning and status codes
of ``rocfft.h`` (reference: ``library/include/rocfft/rocfft.h``), so a test or an
application written against rocFFT reads the same here.  Device memory comes
from PyTorch tensors (``tensor.data_ptr()``) or any other CUDA allocator; the
library itself never touches PyTorch.

There is no CPU fallback: importing works without a GPU (the symbols can be
inspected), but every compute call needs the CUDA library and a device.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "librocfft.so")

# ---- enums (values match rocfft.h) ------------------------------------------
rocfft_status_success = 0
rocfft_status_failure = 1
rocfft_status_invalid_arg_value = 2
rocfft_status_invalid_dimensions = 3
rocfft_status_invalid_array_type = 4
rocfft_status_invalid_strides = 5
rocfft_status_invalid_distance = 6
rocfft_status_invalid_offset = 7
rocfft_status_invalid_work_buffer = 8

rocfft_transform_type_complex_forward = 0
rocfft_transform_type_complex_inverse = 1
rocfft_transform_type_real_forward = 2
rocfft_transform_type_real_inverse = 3

rocfft_precision_single = 0
rocfft_precision_double = 1
rocfft_precision_half = 2

rocfft_placement_inplace = 0
rocfft_placement_notinplace = 1

rocfft_array_type_complex_interleaved = 0
rocfft_array_type_complex_planar = 1
rocfft_array_type_real = 2
rocfft_array_type_hermitian_interleaved = 3
rocfft_array_type_hermitian_planar = 4
rocfft_array_type_unset = 5

rocfft_comm_none = 0
rocfft_comm_mpi = 1
rocfft_comm_nccl = 2

EXPORTED_SYMBOLS = [
    "rocfft_setup", "rocfft_cleanup", "rocfft_plan_create", "rocfft_execute", "rocfft_plan_destroy",
    "rocfft_plan_description_set_scale_factor", "rocfft_plan_description_set_data_layout",
    "rocfft_field_create", "rocfft_field_destroy", "rocfft_get_version_string",
    "rocfft_plan_description_set_comm", "rocfft_brick_create", "rocfft_brick_destroy",
    "rocfft_field_add_brick", "rocfft_plan_description_add_infield",
    "rocfft_plan_description_add_outfield", "rocfft_plan_get_work_buffer_size", "rocfft_plan_get_print",
    "rocfft_plan_description_create", "rocfft_plan_description_destroy", "rocfft_execution_info_create",
    "rocfft_execution_info_destroy", "rocfft_execution_info_set_work_buffer",
    "rocfft_execution_info_set_stream", "rocfft_execution_info_set_load_callback",
    "rocfft_execution_info_set_store_callback", "rocfft_cache_serialize", "rocfft_cache_buffer_free",
    "rocfft_cache_deserialize",
]

_lib = None


class LibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load librocfft.so; raises loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m rocfft_b200.build` "
                "(there is no CPU fallback)")
        _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def _declare(L):
    sz_p = POINTER(c_size_t)
    L.rocfft_setup.restype = c_int
    L.rocfft_cleanup.restype = c_int
    L.rocfft_plan_create.argtypes = [POINTER(c_void_p), c_int, c_int, c_int, c_size_t, sz_p, c_size_t, c_void_p]
    L.rocfft_execute.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_void_p]
    L.rocfft_plan_destroy.argtypes = [c_void_p]
    L.rocfft_plan_description_set_scale_factor.argtypes = [c_void_p, c_double]
    L.rocfft_plan_description_set_data_layout.argtypes = [c_void_p, c_int, c_int, sz_p, sz_p, c_size_t, sz_p,
                                                          c_size_t, c_size_t, sz_p, c_size_t]
    L.rocfft_field_create.argtypes = [POINTER(c_void_p)]
    L.rocfft_field_destroy.argtypes = [c_void_p]
    L.rocfft_get_version_string.argtypes = [c_char_p, c_size_t]
    L.rocfft_plan_description_set_comm.argtypes = [c_void_p, c_int, c_void_p]
    L.rocfft_brick_create.argtypes = [POINTER(c_void_p), sz_p, sz_p, sz_p, c_size_t, c_int]
    L.rocfft_brick_destroy.argtypes = [c_void_p]
    L.rocfft_field_add_brick.argtypes = [c_void_p, c_void_p]
    L.rocfft_plan_description_add_infield.argtypes = [c_void_p, c_void_p]
    L.rocfft_plan_description_add_outfield.argtypes = [c_void_p, c_void_p]
    L.rocfft_plan_get_work_buffer_size.argtypes = [c_void_p, sz_p]
    L.rocfft_plan_get_print.argtypes = [c_void_p]
    L.rocfft_plan_description_create.argtypes = [POINTER(c_void_p)]
    L.rocfft_plan_description_destroy.argtypes = [c_void_p]
    L.rocfft_execution_info_create.argtypes = [POINTER(c_void_p)]
    L.rocfft_execution_info_destroy.argtypes = [c_void_p]
    L.rocfft_execution_info_set_work_buffer.argtypes = [c_void_p, c_void_p, c_size_t]
    L.rocfft_execution_info_set_stream.argtypes = [c_void_p, c_void_p]
    L.rocfft_execution_info_set_load_callback.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_size_t]
    L.rocfft_execution_info_set_store_callback.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_size_t]
    L.rocfft_cache_serialize.argtypes = [POINTER(c_void_p), sz_p]
    L.rocfft_cache_buffer_free.argtypes = [c_void_p]
    L.rocfft_cache_deserialize.argtypes = [c_void_p, c_size_t]
    for name in EXPORTED_SYMBOLS:
        getattr(L, name).restype = c_int


def _sz_array(values):
    if values is None:
        return None
    values = list(values)
    return (c_size_t * len(values))(*values)


# ---- thin functional mirror of the C API ------------------------------------
def rocfft_setup():
    return lib().rocfft_setup()


def rocfft_cleanup():
    return lib().rocfft_cleanup()


def rocfft_get_version_string(length=64):
    buf = ctypes.create_string_buffer(length)
    st = lib().rocfft_get_version_string(buf, length)
    return st, buf.value.decode()


def rocfft_plan_description_create():
    h = c_void_p()
    st = lib().rocfft_plan_description_create(byref(h))
    return st, h


def rocfft_plan_description_destroy(desc):
    return lib().rocfft_plan_description_destroy(desc)


def rocfft_plan_description_set_scale_factor(desc, scale):
    return lib().rocfft_plan_description_set_scale_factor(desc, float(scale))


def rocfft_plan_description_set_data_layout(desc, in_array_type, out_array_type, in_offsets, out_offsets,
                                            in_strides, in_distance, out_strides, out_distance):
    """Stride sizes are taken from the sequences; pass None for defaults."""
    return lib().rocfft_plan_description_set_data_layout(
        desc, in_array_type, out_array_type, _sz_array(in_offsets), _sz_array(out_offsets),
        len(in_strides) if in_strides is not None else 0, _sz_array(in_strides), in_distance,
        len(out_strides) if out_strides is not None else 0, _sz_array(out_strides), out_distance)


def rocfft_plan_create(placement, transform_type, precision, lengths, number_of_transforms, description=None):
    h = c_void_p()
    lengths = list(lengths)
    st = lib().rocfft_plan_create(byref(h), placement, transform_type, precision, len(lengths),
                                  _sz_array(lengths), number_of_transforms, description)
    return st, h


def rocfft_plan_destroy(plan):
    return lib().rocfft_plan_destroy(plan)


def rocfft_plan_get_work_buffer_size(plan):
    n = c_size_t(0)
    st = lib().rocfft_plan_get_work_buffer_size(plan, byref(n))
    return st, n.value


def rocfft_plan_get_print(plan):
    return lib().rocfft_plan_get_print(plan)


def rocfft_execution_info_create():
    h = c_void_p()
    st = lib().rocfft_execution_info_create(byref(h))
    return st, h


def rocfft_execution_info_destroy(info):
    return lib().rocfft_execution_info_destroy(info)


def rocfft_execution_info_set_work_buffer(info, ptr, size_in_bytes):
    return lib().rocfft_execution_info_set_work_buffer(info, c_void_p(ptr) if ptr else None, size_in_bytes)


def rocfft_execution_info_set_stream(info, stream):
    return lib().rocfft_execution_info_set_stream(info, c_void_p(stream) if stream else None)


def rocfft_execute(plan, in_ptrs, out_ptrs=None, info=None):
    """in_ptrs / out_ptrs: sequences of integer device addresses."""
    ins = (c_void_p * max(len(in_ptrs), 1))(*[c_void_p(p) for p in in_ptrs])
    outs = None
    if out_ptrs is not None:
        outs = (c_void_p * max(len(out_ptrs), 1))(*[c_void_p(p) for p in out_ptrs])
    return lib().rocfft_execute(plan, ins, outs, info)


def rocfft_field_create():
    h = c_void_p()
    st = lib().rocfft_field_create(byref(h))
    return st, h


def rocfft_field_destroy(field):
    return lib().rocfft_field_destroy(field)


def rocfft_brick_create(lower, upper, stride, device):
    h = c_void_p()
    st = lib().rocfft_brick_create(byref(h), _sz_array(lower), _sz_array(upper), _sz_array(stride), len(lower), device)
    return st, h


def rocfft_brick_destroy(brick):
    return lib().rocfft_brick_destroy(brick)


def rocfft_field_add_brick(field, brick):
    return lib().rocfft_field_add_brick(field, brick)


def rocfft_plan_description_add_infield(desc, field):
    return lib().rocfft_plan_description_add_infield(desc, field)


def rocfft_plan_description_add_outfield(desc, field):
    return lib().rocfft_plan_description_add_outfield(desc, field)


def rocfft_plan_description_set_comm(desc, comm_type, handle):
    return lib().rocfft_plan_description_set_comm(desc, comm_type, handle)


# ---- convenience wrapper used by tests and the benchmark ---------------------
class Plan:
    """Owns a plan, its description and an execution info; the call sequence
    is the canonical one of the reference's test harness
    (shared/rocfft_params.h:341-503): description -> layout -> [scale] ->
    plan -> info -> work buffer -> execute."""

    def __init__(self, placement, transform_type, precision, lengths, batch=1, *, in_array_type=None,
                 out_array_type=None, in_offsets=None, out_offsets=None, in_strides=None, in_distance=0,
                 out_strides=None, out_distance=0, scale=None):
        self.desc = None
        self.plan = None
        self.info = None
        self._work = None
        st, self.desc = rocfft_plan_description_create()
        assert st == rocfft_status_success
        if any(v is not None for v in (in_array_type, out_array_type, in_offsets, out_offsets, in_strides,
                                       out_strides)) or in_distance or out_distance:
            st = rocfft_plan_description_set_data_layout(
                self.desc,
                rocfft_array_type_unset if in_array_type is None else in_array_type,
                rocfft_array_type_unset if out_array_type is None else out_array_type,
                in_offsets, out_offsets, in_strides, in_distance, out_strides, out_distance)
            if st != rocfft_status_success:
                raise RuntimeError(f"set_data_layout failed: {st}")
        if scale is not None:
            st = rocfft_plan_description_set_scale_factor(self.desc, scale)
            if st != rocfft_status_success:
                raise RuntimeError(f"set_scale_factor failed: {st}")
        st, self.plan = rocfft_plan_create(placement, transform_type, precision, lengths, batch, self.desc)
        self.status = st
        if st != rocfft_status_success:
            raise RuntimeError(f"rocfft_plan_create failed with status {st}")
        st, self.work_bytes = rocfft_plan_get_work_buffer_size(self.plan)
        assert st == rocfft_status_success
        st, self.info = rocfft_execution_info_create()
        assert st == rocfft_status_success

    def set_work_buffer(self, ptr, nbytes):
        return rocfft_execution_info_set_work_buffer(self.info, ptr, nbytes)

    def set_stream(self, stream):
        return rocfft_execution_info_set_stream(self.info, stream)

    def execute(self, in_ptrs, out_ptrs=None):
        return rocfft_execute(self.plan, in_ptrs, out_ptrs, self.info)

    def describe(self):
        """Plan text: one line per kernel launch (b200fft_plan_describe)."""
        L = lib()
        L.b200fft_plan_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
        buf = ctypes.create_string_buffer(1 << 16)
        st = L.b200fft_plan_describe(self.plan, buf, len(buf))
        if st != rocfft_status_success:
            raise RuntimeError(f"b200fft_plan_describe failed: {st}")
        return buf.value.decode()

    def device_error(self):
        """True if a kernel of this plan ever gave up a bounded wait (blocks until the device is idle)."""
        L = lib()
        L.b200fft_plan_device_error.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        v = ctypes.c_int(0)
        st = L.b200fft_plan_device_error(self.plan, ctypes.byref(v))
        if st != rocfft_status_success:
            raise RuntimeError(f"b200fft_plan_device_error failed: {st}")
        return bool(v.value)

    def destroy(self):
        if self.info:
            rocfft_execution_info_destroy(self.info)
            self.info = None
        if self.plan:
            rocfft_plan_destroy(self.plan)
            self.plan = None
        if self.desc:
            rocfft_plan_description_destroy(self.desc)
            self.desc = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
