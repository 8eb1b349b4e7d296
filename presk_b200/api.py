"""Executor and Host: numpy-facing wrappers over the C ABI."""
import ctypes as C
import os

import numpy as np

from . import abi

_NP_OF = {abi.F64: np.float64, abi.F32: np.float32, abi.BF16: np.uint16, abi.I64: np.int64, abi.F16: np.uint16, abi.E8M15: np.uint8, abi.I8: np.int8, abi.E4M3: np.uint8, abi.U8: np.uint8}


class PreskError(RuntimeError):
    """A call of the library that did not return PSK_OK; `code` is the reference's E-number."""

    def __init__(self, code, message):
        super().__init__(f"E{code}: {message}")
        self.code = code
        self.message = message


def _dtype_of_array(a):
    if a.dtype == np.float64:
        return abi.F64
    if a.dtype == np.float32:
        return abi.F32
    if a.dtype == np.int64:
        return abi.I64
    raise TypeError(f"host values are float32, float64 or int64 arrays, not {a.dtype}")


class Executor:
    """`KernelExec` on one CUDA device. Buffers are raw device pointers (ints)."""

    def __init__(self, device=0):
        self.lib = abi.load()
        self.handle = self.lib.psk_exec_create(device)
        if not self.handle:
            raise PreskError(abi.E10001, self.lib.psk_last_error(None).decode())

    def close(self):
        if getattr(self, "handle", None):
            self.lib.psk_exec_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != abi.OK:
            raise PreskError(rc, self.lib.psk_last_error(self.handle).decode())

    def alloc(self, nbytes):
        p = self.lib.psk_exec_alloc(self.handle, nbytes)
        if not p:
            raise PreskError(abi.E10001, self.lib.psk_last_error(self.handle).decode())
        return p

    def free(self, p):
        self.lib.psk_exec_free(self.handle, p)

    def upload(self, array):
        """A device buffer holding the bytes of `array`."""
        a = np.ascontiguousarray(array)
        p = self.alloc(max(a.nbytes, 1))
        if a.nbytes:
            self._check(self.lib.psk_exec_upload(self.handle, p, a.ctypes.data, a.nbytes))
        return p

    def download(self, p, nbytes):
        out = np.empty(nbytes, dtype=np.uint8)
        if nbytes:
            self._check(self.lib.psk_exec_download(self.handle, out.ctypes.data, p, nbytes))
        return out

    def run(self, launch, table):
        arr = (C.c_void_p * len(table))(*table)
        self._check(self.lib.psk_exec_run(self.handle, C.byref(launch), arr))

    def gemm(self, g, a, b, c):
        self._check(self.lib.psk_exec_gemm(self.handle, C.byref(g), a, b, c))

    def gap(self, a, a_dtype, b, b_dtype, n):
        """(largest |a - b|, largest |a|) of two device buffers of n reals: `presk solve --measure`'s gap on the device."""
        g, m = C.c_double(), C.c_double()
        self._check(self.lib.psk_exec_gap(self.handle, a, a_dtype, b, b_dtype, n, C.byref(g), C.byref(m)))
        return g.value, m.value

    def sync(self):
        self._check(self.lib.psk_exec_sync(self.handle))

    def overflow(self):
        return self.lib.psk_exec_overflow(self.handle)

    def counts(self):
        a, b = C.c_int64(), C.c_int64()
        self.lib.psk_exec_counts(self.handle, C.byref(a), C.byref(b))
        return a.value, b.value

    def memory(self):
        a, b = C.c_size_t(), C.c_size_t()
        self.lib.psk_exec_memory(self.handle, C.byref(a), C.byref(b))
        return a.value, b.value

    def set_profiling(self, on=True):
        self.lib.psk_exec_set_profiling(self.handle, 1 if on else 0)

    def profile(self):
        """[(kernel family, launch name, ms, flops, bytes)] of the launches since the last call."""
        rows = []
        for line in self.lib.psk_exec_profile(self.handle).decode().splitlines():
            k, n, ms, fl, by = line.split("\t")
            rows.append((k, n, float(ms), float(fl), float(by)))
        return rows

    def stream(self):
        return self.lib.psk_exec_stream(self.handle)

    def vtable(self):
        vt = abi.ExecVtable()
        self.lib.psk_exec_as_vtable(self.handle, C.byref(vt))
        return vt


class Comm:
    """The exchange step of a sharded call (`psk_comm_*`): one communicator a rank, over the executor's stream."""

    @staticmethod
    def unique_id():
        lib = abi.load()
        buf = C.create_string_buffer(abi.COMM_ID_BYTES)
        rc = lib.psk_comm_unique_id(buf)
        if rc != abi.OK:
            raise PreskError(rc, lib.psk_comm_error(None).decode())
        return buf.raw

    def __init__(self, executor, nranks, rank, unique_id):
        self.lib = executor.lib
        self.executor = executor
        self.handle = self.lib.psk_comm_create(executor.handle, nranks, rank, C.create_string_buffer(unique_id, abi.COMM_ID_BYTES))
        if not self.handle:
            raise PreskError(abi.E10001, self.lib.psk_comm_error(None).decode())

    def allreduce(self, device_ptr, count, dtype, op):
        rc = self.lib.psk_comm_allreduce(self.handle, device_ptr, count, dtype, op)
        if rc != abi.OK:
            raise PreskError(rc, self.lib.psk_comm_error(self.handle).decode())

    def size(self):
        return self.lib.psk_comm_size(self.handle)

    def close(self):
        if self.handle:
            self.lib.psk_comm_destroy(self.handle)
            self.handle = None


class Host:
    """`Backend`: prepare a model under a realization, give it parameters, call an entry.

    `executor` is an `Executor`, or an `abi.ExecVtable` of another executor
    (tests hand it the CPU oracle's, loaded from oracle/; the product never does).
    """

    def __init__(self, executor, realization="f32", lib=None):
        self.executor = executor
        if isinstance(executor, Executor):
            self.lib = executor.lib
            self._vt = executor.vtable()
        else:
            self.lib = lib if lib is not None else abi.load()
            self._vt = executor
        text = realization if isinstance(realization, str) else __import__("json").dumps(realization, ensure_ascii=False)
        self.handle = self.lib.psk_host_create(C.byref(self._vt), text.encode())
        if not self.handle:
            msg = self.lib.psk_host_error(None).decode()
            m = __import__("re").match(r"\[E(\d+)\] (.*)", msg, __import__("re").S)
            raise PreskError(int(m.group(1)), m.group(2)) if m else PreskError(abi.E7001, msg)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.psk_host_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != abi.OK:
            raise PreskError(rc, self.lib.psk_host_error(self.handle).decode())

    def prepare(self, model, **consts):
        text = " ".join(f"{k}={int(v)}" for k, v in consts.items())
        self._check(self.lib.psk_host_prepare(self.handle, model.encode(), text.encode()))
        return self

    def set_param(self, path, array):
        a = np.ascontiguousarray(array)
        dims = (C.c_int64 * max(a.ndim, 1))(*a.shape)
        self._check(self.lib.psk_host_set_param(self.handle, path.encode(), a.ctypes.data, _dtype_of_array(a), dims, a.ndim))

    def init_param(self, path, seed, std, shape):
        dims = (C.c_int64 * max(len(shape), 1))(*shape)
        self._check(self.lib.psk_host_init_param(self.handle, path.encode(), seed, std, dims, len(shape)))

    @staticmethod
    def _values(inputs, device_ptrs=None):
        vals = (abi.Value * max(len(inputs), 1))()
        keep = []
        for i, x in enumerate(inputs):
            if device_ptrs is not None:
                ptr, dtype, shape = x
                vals[i].data, vals[i].dtype, vals[i].rank = ptr, dtype, len(shape)
                for k, d in enumerate(shape):
                    vals[i].dims[k] = d
            else:
                shape = np.shape(x)  # a rank-0 value stays rank 0 (ascontiguousarray would make it [1])
                a = np.ascontiguousarray(x)
                keep.append(a)
                vals[i].data, vals[i].dtype, vals[i].rank = a.ctypes.data, _dtype_of_array(a), len(shape)
                for k, d in enumerate(shape):
                    vals[i].dims[k] = d
        return vals, keep

    def call(self, entry, inputs, out_shape, out_dtype=np.float32):
        """Backend::call with host arrays; returns the result as a numpy array of `out_shape`."""
        vals, keep = self._values(inputs)
        out = np.empty(out_shape, dtype=out_dtype)
        n = C.c_int64()
        code = {np.dtype(np.float32): abi.F32, np.dtype(np.float64): abi.F64, np.dtype(np.int64): abi.I64}[np.dtype(out_dtype)]
        self._check(self.lib.psk_host_call(self.handle, entry.encode(), vals, len(inputs), out.ctypes.data, code, out.size, C.byref(n)))
        if n.value != out.size:
            raise PreskError(abi.E7001, f"the result has {n.value} elements, not {out.size}")
        return out

    def mean_over_ranks(self, comm, device_scalar, dtype):
        """The mean over all ranks of a per-rank mean left on the executor by `call_device`."""
        out = C.c_double()
        self._check(self.lib.psk_host_mean_over_ranks(self.handle, comm.handle, device_scalar, dtype, C.byref(out)))
        return out.value

    def grads_allreduce(self, comm):
        """The last gradient's leaves averaged over the ranks of `comm` (a data-parallel training step)."""
        self._check(self.lib.psk_host_grads_allreduce(self.handle, comm.handle))

    def envelope_allreduce(self, comm):
        """Merges the calibrated magnitudes over the ranks."""
        self._check(self.lib.psk_host_envelope_allreduce(self.handle, comm.handle))

    def result(self, path, shape, out_dtype=np.float32):
        """A leaf of the last call's result when that is a tree (a gradient), by the parameter's path."""
        out = np.empty(shape, dtype=out_dtype)
        n = C.c_int64()
        code = {np.dtype(np.float32): abi.F32, np.dtype(np.float64): abi.F64}[np.dtype(out_dtype)]
        self._check(self.lib.psk_host_result(self.handle, path.encode(), out.ctypes.data, code, out.size, C.byref(n)))
        if n.value != out.size:
            raise PreskError(abi.E7001, f"the result `{path}` has {n.value} elements, not {out.size}")
        return out

    def set_result(self, path, array):
        """Gives a leaf of a gradient (what `adamw.step` takes as `g`) in place of a computed one."""
        a = np.ascontiguousarray(array, dtype=np.float64)
        dims = (C.c_int64 * max(a.ndim, 1))(*a.shape)
        self._check(self.lib.psk_host_set_result(self.handle, path.encode(), a.ctypes.data, abi.F64, dims, a.ndim))

    def adamw(self, **hyperparameters):
        """`optimizer adamw { … }`: lr, beta1, beta2, eps, weight_decay, schedule, warmup; forgets the moments."""
        self._check(self.lib.psk_host_adamw(self.handle, " ".join(f"{k}={v!r}" if isinstance(v, float) else f"{k}={v}" for k, v in hyperparameters.items()).encode()))
        return self

    def adamw_step(self, t, total):
        """`adamw.step` on the last gradient's leaves; the parameters and moments are replaced."""
        self._check(self.lib.psk_host_adamw_step(self.handle, t, total))

    def adamw_lr(self, t, total):
        out = C.c_double()
        self._check(self.lib.psk_host_adamw_lr(self.handle, t, total, C.byref(out)))
        return out.value

    def call_device(self, entry, inputs):
        """Backend::call with device inputs [(ptr, dtype, shape)]; returns (ptr, dtype, numel), queued."""
        vals, _ = self._values(inputs, device_ptrs=True)
        out, dt, n = C.c_void_p(), C.c_int32(), C.c_int64()
        self._check(self.lib.psk_host_call_device(self.handle, entry.encode(), vals, len(inputs), C.byref(out), C.byref(dt), C.byref(n)))
        return out.value, dt.value, n.value

    def set_calibrating(self, on=True):
        """`presk calibrate`: fold every launch's output into its site's magnitudes from now on."""
        self.lib.psk_host_set_calibrating(self.handle, 1 if on else 0)

    def envelope(self):
        """{site: (max |x|, least non-zero |x|, lo, hi)} of everything seen while calibrating."""
        out = {}
        for line in self.lib.psk_host_envelope(self.handle).decode().splitlines():
            site, mx, mn, lo, hi = line.split("\t")
            out[site] = (float(mx), float(mn), float(lo), float(hi))
        return out

    def launches(self):
        return self.lib.psk_host_launches(self.handle)

    def set_logging(self, on=True):
        self.lib.psk_host_set_logging(self.handle, 1 if on else 0)

    def launch_log(self):
        return self.lib.psk_host_launch_log(self.handle).decode().splitlines()


def describe(kernel_text, order=abi.ORDER_SEQUENTIAL):
    """`psk_describe` on every kernel of a listing in the reference's text form: [(name, psk_launch)].
    The launches keep their names alive (each holds a pointer into its own buffer)."""
    lib = abi.load()
    out = []
    text = kernel_text.encode() if isinstance(kernel_text, str) else kernel_text
    while b"kernel " in text:
        l = abi.Launch()
        name = C.create_string_buffer(256)
        err = C.create_string_buffer(512)
        rest = C.c_char_p()
        rc = lib.psk_describe(text, order, C.byref(l), name, 256, C.byref(rest), err, 512)
        if rc != abi.OK:
            raise PreskError(rc, err.value.decode())
        l._name_keep = name
        out.append((name.value.decode(), l))
        text = rest.value or b""
    return out


class DataFile:
    """A .psk.d file open for reading into device buffers (`psk_data_*`). `leaves`: [(bound, n)] of the sample
    type's leaves in order, bound 0 for reals."""

    def __init__(self, path, sample_type, leaves):
        self.lib = abi.load()
        self.leaves = [(int(b), int(n)) for b, n in leaves]
        arr = (abi.DataLeaf * max(len(self.leaves), 1))()
        for i, (b, n) in enumerate(self.leaves):
            arr[i].bound, arr[i].n = b, n
        h = C.c_void_p()
        err = C.create_string_buffer(1024)
        rc = self.lib.psk_data_open(os.fsencode(path), sample_type.encode(), arr, len(self.leaves), C.byref(h), err, 1024)
        if rc != abi.OK:
            raise PreskError(rc, err.value.decode())
        self.handle = h

    @property
    def count(self):
        return self.lib.psk_data_count(self.handle)

    @property
    def sample_bytes(self):
        return self.lib.psk_data_sample_bytes(self.handle)

    def read(self, ex, first, count, dst, dtypes):
        """Samples first .. first + count - 1 into the device buffers `dst` (one a leaf, count x n elements of dtypes[i])."""
        ptrs = (C.c_void_p * max(len(dst), 1))(*dst)
        dts = (C.c_int32 * max(len(dtypes), 1))(*dtypes)
        rc = self.lib.psk_data_read(self.handle, ex.handle, first, count, ptrs, dts)
        if rc != abi.OK:
            raise PreskError(rc, self.lib.psk_data_error(self.handle).decode())

    def close(self):
        if self.handle:
            self.lib.psk_data_close(self.handle)
            self.handle = None


def launch_desc(op, dtype, dims_outer, dims_inner=(), order=abi.ORDER_SEQUENTIAL, name=b"launch"):
    """An empty `psk_launch` over an iteration space; the caller fills the operands."""
    l = abi.Launch()
    l.name = name
    l.op = op
    l.dtype = dtype
    l.order = order
    l.guarded = 1
    l.n_outer = len(dims_outer)
    l.n_inner = len(dims_inner)
    for i, d in enumerate(list(dims_outer) + list(dims_inner)):
        l.dims[i] = d
    return l
