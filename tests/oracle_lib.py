"""Loads the CPU oracle for the tests and wraps its entry points.

The oracle (oracle/psk_oracle.c) is test infrastructure: nothing under
presk_b200/ imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from presk_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "libpsk_oracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libpresk_ref.so")


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.psk_oracle_run.restype = C.c_int
        lib.psk_oracle_run.argtypes = [C.POINTER(abi.Launch), C.POINTER(C.c_void_p), C.POINTER(C.c_uint32)]
        lib.psk_oracle_vtable.argtypes = [C.POINTER(abi.ExecVtable)]
        lib.psk_oracle_quantize.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
        for name, res, args in [
            ("psk_o_bf16_to_f32", C.c_float, [C.c_uint16]), ("psk_o_f32_to_bf16", C.c_uint16, [C.c_float]),
            ("psk_o_f16_to_f32", C.c_float, [C.c_uint16]), ("psk_o_f32_to_f16", C.c_uint16, [C.c_float]),
            ("psk_o_f64_to_f16", C.c_uint16, [C.c_double]), ("psk_o_f64_to_e8m15", C.c_uint32, [C.c_double]),
            ("psk_o_e8m15_to_f32", C.c_float, [C.c_uint32]), ("psk_o_f32_to_e8m15", C.c_uint32, [C.c_float]),
            ("psk_o_e4m3_to_f32", C.c_float, [C.c_uint8]), ("psk_o_f32_to_e4m3", C.c_uint8, [C.c_float]),
            ("psk_o_overflows", C.c_uint32, [C.c_int, C.c_float]),
        ]:
            getattr(lib, name).restype = res
            getattr(lib, name).argtypes = args

    def run(self, launch, arrays):
        """Runs a launch on host arrays (inputs..., output[, scales...]); returns the overflow flag."""
        table = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
        ovf = C.c_uint32(0)
        rc = self.lib.psk_oracle_run(C.byref(launch), table, C.byref(ovf))
        if rc != 0:
            raise RuntimeError(f"oracle: launch refused ({rc})")
        return ovf.value

    def vtable(self):
        vt = abi.ExecVtable()
        self.lib.psk_oracle_vtable(C.byref(vt))
        return vt

    def convert(self, array, to):
        """`array` (float32/float64) stored as dtype `to`: the bytes, as the host's Buf::of."""
        a = np.ascontiguousarray(array)
        frm = abi.F64 if a.dtype == np.float64 else abi.F32
        out = np.zeros(a.size * abi.DTYPE_BYTES[to], dtype=np.uint8)
        l = abi.Launch()
        l.name = b"convert"
        l.op = abi.OP_CONVERT
        l.dtype = to
        l.n_inputs = 1
        l.n_outer = 1
        l.dims[0] = a.size
        l.inputs[0].dtype = frm
        l.inputs[0].stride[0] = 1
        l.out.dtype = to
        l.out.stride[0] = 1
        self.run(l, [a, out])
        return out

    def widen(self, raw, frm, n):
        """The f32 values of n stored elements of dtype `frm`."""
        out = np.zeros(n, dtype=np.float32)
        l = abi.Launch()
        l.name = b"convert"
        l.op = abi.OP_CONVERT
        l.dtype = abi.F32
        l.n_inputs = 1
        l.n_outer = 1
        l.dims[0] = n
        l.inputs[0].dtype = frm
        l.inputs[0].stride[0] = 1
        l.out.dtype = abi.F32
        l.out.stride[0] = 1
        self.run(l, [np.ascontiguousarray(raw), out])
        return out


def load():
    src = os.path.join(ROOT, "oracle", "psk_oracle.c")
    if not os.path.exists(ORACLE_SO) or not os.path.exists(REF_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-s"], check=True)
    return Oracle(C.CDLL(ORACLE_SO))
