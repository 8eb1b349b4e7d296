"""psk_data_*: .psk.d samples into device buffers, against the reference's own C reader.

The checker is presk_open / presk_read of the reference's C runtime (presk-export-c/c/presk_rt.c), compiled where it
lies into oracle/_ref/libpresk_ref.so: the same files go through both, and every buffer must come out bit for bit,
every refusal with the same code and message. The files: the reference's own four small data files
(tests/golden/data_files.json, made by tests/golden/make_golden.py), and files of versions 2 and 3 written here
byte by byte from the format's statement (presk_rt.c:8-33), with every encoding, every index width and the values
where the roundings differ (ties, the overflow thresholds, subnormals, NaNs with payloads).
"""
import base64
import ctypes as C
import json
import os
import struct

import numpy as np
import pytest

from presk_b200 import DataFile, PreskError, abi

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libpresk_ref.so")
GOLDEN = json.load(open(os.path.join(HERE, "golden", "data_files.json")))

# presk_dtype (presk_rt.h:405) for each of the executor's types
REF_DTYPE = {abi.F32: 1, abi.BF16: 2, abi.I64: 3, abi.F16: 4, abi.E8M15: 5}
NP_OF = {abi.F32: np.uint32, abi.BF16: np.uint16, abi.F16: np.uint16, abi.E8M15: np.uint8, abi.I64: np.int64}
BYTES_OF = {abi.F32: 4, abi.BF16: 2, abi.F16: 2, abi.E8M15: 3, abi.I64: 8}
REAL_DTYPES = (abi.F32, abi.BF16, abi.F16, abi.E8M15)


class RefLeaf(C.Structure):
    _fields_ = [("bound", C.c_uint64), ("n", C.c_uint64)]


class RefReader(C.Structure):
    _fields_ = [("f", C.c_void_p), ("leaves", C.POINTER(RefLeaf)), ("nleaves", C.c_size_t), ("count", C.c_uint64), ("next", C.c_uint64), ("enc", C.c_void_p)]


@pytest.fixture(scope="module")
def ref():
    lib = C.CDLL(REF_SO)
    lib.presk_open.argtypes = [C.POINTER(RefReader), C.c_char_p, C.c_char_p, C.POINTER(RefLeaf), C.c_size_t]
    lib.presk_read.argtypes = [C.POINTER(RefReader), C.POINTER(C.c_void_p), C.POINTER(C.c_int)]
    lib.presk_close.argtypes = [C.POINTER(RefReader)]
    lib.presk_error.restype = C.c_char_p
    return lib


def ref_read_all(lib, path, typ, leaves, dtypes):
    """Every sample through the reference reader: (code, message, [one array a leaf, count x n elements as raw codes])."""
    arr = (RefLeaf * max(len(leaves), 1))()
    for i, (b, n) in enumerate(leaves):
        arr[i].bound, arr[i].n = b, n
    r = RefReader()
    rc = lib.presk_open(C.byref(r), os.fsencode(path), typ.encode(), arr, len(leaves))
    if rc:
        return rc, lib.presk_error().decode(), None
    count = r.count
    outs = [np.zeros(count * n * BYTES_OF[dt], np.uint8) for (b, n), dt in zip(leaves, dtypes)]
    one = [np.zeros(max(n * BYTES_OF[dt], 1), np.uint8) for (b, n), dt in zip(leaves, dtypes)]
    ptrs = (C.c_void_p * max(len(leaves), 1))(*[a.ctypes.data for a in one])
    dts = (C.c_int * max(len(leaves), 1))(*[REF_DTYPE[dt] for dt in dtypes])
    for s in range(count):
        rc = lib.presk_read(C.byref(r), ptrs, dts)
        if rc:
            msg = lib.presk_error().decode()
            lib.presk_close(C.byref(r))
            return rc, msg, None
        for i, ((b, n), dt) in enumerate(zip(leaves, dtypes)):
            w = n * BYTES_OF[dt]
            outs[i][s * w:(s + 1) * w] = one[i][:w]
    lib.presk_close(C.byref(r))
    return 0, "", outs


def write_file(path, typ, version, count, leaves, encodings, data):
    """A .psk.d file from the format's statement. `encodings`: a leaf's byte (0 f64, 1 f32, 2 bf16, "f16", "e8m15", or
    six bytes of another format); `data[s][i]`: leaf i of sample s as the integers to be written, one an element."""
    desc = {"f16": bytes([11, 0xf2, 0xff, 15, 0, 0x01]), "e8m15": bytes([16, 0x82, 0xff, 127, 0, 0x01])}
    t = typ.encode()
    out = bytearray(b"PSKD" + struct.pack("<HI", version, len(t)) + t + struct.pack("<Q", count))
    widths = []
    if version >= 2:
        out += struct.pack("<I", len(leaves))
    for (bound, n), e in zip(leaves, encodings):
        if bound:
            m = bound - 1
            widths.append(1 if m <= 0xff else 2 if m <= 0xffff else 4 if m <= 0xffffffff else 8)
        else:
            widths.append({0: 8, 1: 4, 2: 2, "f16": 2, "e8m15": 3}.get(e, 1) if not isinstance(e, bytes) else 1)
        if version >= 2:
            if e in (0, 1, 2):
                out += bytes([e])
            else:
                out += bytes([3]) + (desc[e] if isinstance(e, str) else e)
    for s in range(count):
        for (bound, n), w, vals in zip(leaves, widths, data[s]):
            for v in vals:
                out += int(v).to_bytes(w, "little")
    with open(path, "wb") as f:
        f.write(out)
    return bytes(out)


def golden_path(tmp_path, name):
    p = tmp_path / name
    p.write_bytes(base64.b64decode(GOLDEN[name]["bytes"]))
    return str(p)


# ---------------------------------------------------------------------------------------------------------------
# the header, on the host (no GPU)
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_the_references_files_open_with_its_counts(tmp_path, ref, name):
    g = GOLDEN[name]
    d = DataFile(golden_path(tmp_path, name), g["type"], g["leaves"])
    assert d.count == g["count"]
    assert d.sample_bytes == sum(n * (8 if not b else 1) for b, n in g["leaves"])  # version 1: f64 reals; idx[64] in one byte
    d.close()
    rc, msg, outs = ref_read_all(ref, golden_path(tmp_path, name), g["type"], g["leaves"], [abi.I64 if b else abi.F32 for b, n in g["leaves"]])
    assert rc == 0 and len(outs[0]) > 0


def refusal(path, typ, leaves):
    with pytest.raises(PreskError) as e:
        DataFile(path, typ, leaves)
    return e.value.code, str(e.value)


def test_header_refusals_are_the_reference_readers(tmp_path, ref):
    """Every way presk_open refuses a file (presk_rt.c:295-460), with its code and its message."""
    g = GOLDEN["windows.psk.d"]
    raw = base64.b64decode(g["bytes"])
    typ, leaves = g["type"], g["leaves"]
    cases = {
        "short": (raw[:3], typ, leaves), "magic": (b"PSKX" + raw[4:], typ, leaves), "version": (raw[:4] + struct.pack("<H", 9) + raw[6:], typ, leaves),
        "cut_header": (raw[:12], typ, leaves), "other_type": (raw, "(idx[64][seq: 9], idx[64][seq: 8])", leaves), "other_length": (raw, typ, [(64, 8), (64, 9)]),
        "truncated": (raw[:-5], typ, leaves), "missing": (None, typ, leaves),
    }
    for name, (data, t, lv) in cases.items():
        p = str(tmp_path / (name + ".psk.d"))
        if data is not None:
            open(p, "wb").write(data)
        code, msg = refusal(p, t, lv)
        rc, rmsg, _ = ref_read_all(ref, p, t, lv, [abi.I64] * len(lv))
        assert code == rc and code in (9002, 9003, 9005), (name, code, rc)
        assert rmsg in msg, (name, msg, rmsg)
    # version 2 and 3 headers: a count of encodings that is not the leaves', an unknown byte, a format not held
    # (named as the reference names it), an index leaf with a real encoding
    lv = [(0, 2), (10, 1)]
    t2 = "(ℝ[2], idx[10])"
    one = [[[0, 0], [3]]]
    p = str(tmp_path / "v.psk.d")
    write_file(p, t2, 2, 1, lv, [1, 0], one)
    DataFile(p, t2, lv).close()
    for name, build in {
        "encodings": lambda: write_file(p, t2, 2, 1, lv + [(0, 1)], [1, 0, 0], [[[0, 0], [3], [0]]]),
        "unknown": lambda: (write_file(p, t2, 2, 1, lv, [1, 0], one), patch(p, -(2 * 4 + 1) - 2, 7)),  # the first leaf's encoding byte
        "e5m2": lambda: write_file(p, t2, 3, 1, lv, [bytes([3, 0xf2, 0xff, 15, 0, 0x01]), 0], [[[0, 0], [3]]]),
        "e4m3fn": lambda: write_file(p, t2, 3, 1, lv, [bytes([4, 0xfa, 0xff, 8, 0, 0x0b]), 0], [[[0, 0], [3]]]),
        "odd_format": lambda: write_file(p, t2, 3, 1, lv, [bytes([5, 0xf0, 0xff, 20, 0, 0x01]), 0], [[[0, 0], [3]]]),
        "real_index": lambda: write_file(p, t2, 2, 1, lv, [1, 1], one),
    }.items():
        build()
        code, msg = refusal(p, t2, lv)
        rc, rmsg, _ = ref_read_all(ref, p, t2, lv, [abi.F32, abi.I64])
        assert code == rc and rc != 0, (name, code, rc, msg, rmsg)
        if name != "odd_format":  # a format outside the reference's table of names is spelled by its parameters there
            assert rmsg in msg, (name, msg, rmsg)


def patch(path, offset_from_end, value):
    b = bytearray(open(path, "rb").read())
    b[offset_from_end] = value
    open(path, "wb").write(b)


# ---------------------------------------------------------------------------------------------------------------
# the samples, on the device
# ---------------------------------------------------------------------------------------------------------------

def device_read(cuda, path, typ, leaves, dtypes, first=0, count=None):
    d = DataFile(path, typ, leaves)
    count = d.count - first if count is None else count
    bufs = [cuda.alloc(max(count * n * BYTES_OF[dt], 16)) for (b, n), dt in zip(leaves, dtypes)]
    try:
        d.read(cuda, first, count, bufs, dtypes)
        outs = [cuda.download(p, count * n * BYTES_OF[dt]) if count * n else np.zeros(0, np.uint8) for p, ((b, n), dt) in zip(bufs, zip(leaves, dtypes))]
    finally:
        for p in bufs:
            cuda.free(p)
        d.close()
    return [np.asarray(o).view(np.uint8).reshape(-1) for o in outs]


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_the_references_files_on_the_device(cuda, ref, tmp_path, name):
    """The reference's own data files, whole, into every type a buffer can have: the reference reader's bytes."""
    g = GOLDEN[name]
    p = golden_path(tmp_path, name)
    for real in REAL_DTYPES:
        dtypes = [abi.I64 if b else real for b, n in g["leaves"]]
        rc, msg, want = ref_read_all(ref, p, g["type"], g["leaves"], dtypes)
        assert rc == 0, msg
        got = device_read(cuda, p, g["type"], g["leaves"], dtypes)
        for i, (a, b) in enumerate(zip(got, want)):
            assert np.array_equal(a, b), (name, real, i)
        if not any(not b for b, n in g["leaves"]):
            break


def special_doubles(rng, n):
    """Bit patterns of doubles where a rounding can go wrong: ties of every target, the overflow thresholds,
    subnormal results, infinities, NaNs with payloads, and random ones of every exponent near the formats' ranges."""
    vals = [0.0, -0.0, 1.0, -1.0, 65504.0, 65519.999, 65520.0, -65520.0, 65536.0, 1e-8, 5.960464477539063e-08, 2.9802322387695312e-08, 2.98023223876953125e-08 * 1.0000001,
            6.103515625e-05, 3.4028234663852886e38, 3.4028235677973366e38, 3.39e38, 1e39, -1e39, 1e-46, 7.006492321624085e-46, 1.401298464324817e-45,
            1.0 + 2.0**-8, 1.0 + 2.0**-9, 1.0 + 3 * 2.0**-9, 1.0 + 2.0**-11, 1.0 + 2.0**-12, 1.0 + 2.0**-16, 1.0 + 2.0**-17, 1.0 + 2.0**-24, 1.0 + 2.0**-25,
            1.0 + 2.0**-24 + 2.0**-40, 1.0 + 2.0**-9 - 2.0**-30, 1.0 + 2.0**-9 + 2.0**-30, float("inf"), float("-inf")]
    bits = [struct.unpack("<Q", struct.pack("<d", v))[0] for v in vals]
    bits += [0x7ff8000000000000, 0xfff8000000000000, 0x7ff0000000000001, 0xfff4000000123456, 0x7ffabcdef0123456, 0x000fffffffffffff, 0x8000000000000001]
    while len(bits) < n:
        e = int(rng.integers(1023 - 160, 1023 + 140))
        bits.append((int(rng.integers(0, 2)) << 63) | (e << 52) | int(rng.integers(0, 1 << 52)))
    return bits[:n]


@pytest.mark.gpu
@pytest.mark.parametrize("version", [1, 2, 3])
def test_every_encoding_and_width_against_the_reference_reader(cuda, ref, tmp_path, version):
    rng = np.random.default_rng(version)
    count = 37
    leaves = [(200, 5), (0, 40), (70000, 3), (1 << 40, 2), (300, 1), (0, 0), (0, 9), (0, 6)]
    typ = "(idx[200][5], ℝ[40], idx[70000][3], idx[1099511627776][2], idx[300], ℝ[0], ℝ[9], ℝ[6])"
    if version == 1:
        enc = [0] * len(leaves)
    elif version == 2:
        enc = [0, 0, 0, 0, 0, 1, 1, 2]
    else:
        enc = [0, 0, 0, 0, 0, 2, "f16", "e8m15"]
    data = []
    for s in range(count):
        row = []
        for (bound, n), e in zip(leaves, enc):
            if bound:
                row.append([int(x) for x in rng.integers(0, bound, size=n)])
            elif e == 0:
                row.append(special_doubles(rng, n))
            elif e == 1:
                row.append([int(x) for x in rng.integers(0, 1 << 32, size=n)])  # every f32 pattern, NaNs included
            elif e in (2, "f16"):
                row.append([int(x) for x in rng.integers(0, 1 << 16, size=n)])
            else:
                row.append([int(x) for x in rng.integers(0, 1 << 24, size=n)])
        data.append(row)
    p = str(tmp_path / f"v{version}.psk.d")
    write_file(p, typ, version, count, leaves, enc, data)
    for real in REAL_DTYPES:
        dtypes = [abi.I64 if b else real for b, n in leaves]
        rc, msg, want = ref_read_all(ref, p, typ, leaves, dtypes)
        assert rc == 0, msg
        got = device_read(cuda, p, typ, leaves, dtypes)
        for i, (a, b) in enumerate(zip(got, want)):
            if not np.array_equal(a, b):
                w = BYTES_OF[dtypes[i]]
                bad = np.nonzero((a.reshape(-1, w) != b.reshape(-1, w)).any(axis=1))[0]
                raise AssertionError((version, real, i, bad[:5], a.reshape(-1, w)[bad[:5]], b.reshape(-1, w)[bad[:5]]))
        # a window of the samples is that window of the whole
        part = device_read(cuda, p, typ, leaves, dtypes, first=5, count=11)
        for i, ((b, n), dt) in enumerate(zip(leaves, dtypes)):
            w = n * BYTES_OF[dt]
            assert np.array_equal(part[i], want[i][5 * w:16 * w]), (version, real, i)
    assert all(len(a) == 0 for a in device_read(cuda, p, typ, leaves, [abi.I64 if b else abi.F32 for b, n in leaves], first=count, count=0))


@pytest.mark.gpu
def test_an_index_not_below_its_bound_is_named_as_the_reference_names_it(cuda, ref, tmp_path):
    leaves = [(0, 3), (200, 4), (300, 2)]
    typ = "(ℝ[3], idx[200][4], idx[300][2])"
    rng = np.random.default_rng(4)
    data = [[[0, 0, 0], [int(x) for x in rng.integers(0, 200, size=4)], [int(x) for x in rng.integers(0, 300, size=2)]] for _ in range(50)]
    data[31][2][1] = 300   # the first offender in file order
    data[31][1][3] = 199   # (allowed)
    data[40][1][0] = 255
    p = str(tmp_path / "bad.psk.d")
    write_file(p, typ, 1, 50, leaves, [0, 0, 0], data)
    dtypes = [abi.F32, abi.I64, abi.I64]
    rc, rmsg, _ = ref_read_all(ref, p, typ, leaves, dtypes)
    assert rc == 9004
    with pytest.raises(PreskError) as e:
        device_read(cuda, p, typ, leaves, dtypes)
    assert e.value.code == 9004 and rmsg in str(e.value), (str(e.value), rmsg)
    # the samples before it read cleanly; a real leaf asked for as indices (and the other way) is 9005, as there
    good = device_read(cuda, p, typ, leaves, dtypes, first=0, count=31)
    assert np.array_equal(good[1].view(np.int64).reshape(31, 4), np.array([r[1] for r in data[:31]], np.int64))
    with pytest.raises(PreskError) as e:
        device_read(cuda, p, typ, leaves, [abi.I64, abi.I64, abi.I64], count=1)
    assert e.value.code == 9005
    with pytest.raises(PreskError) as e:
        device_read(cuda, p, typ, leaves, dtypes, first=49, count=2)
    assert e.value.code == 9003


@pytest.mark.gpu
def test_a_file_of_several_pieces(cuda, ref, tmp_path):
    """80 MB of samples (three pieces through the staging buffer): f32-encoded rows and their labels."""
    n, count = 2047, 10000
    leaves = [(0, n), (1000, 1)]
    typ = "(ℝ[2047], idx[1000])"
    rng = np.random.default_rng(8)
    x = rng.standard_normal((count, n)).astype(np.float32)
    y = rng.integers(0, 1000, size=count).astype(np.uint16)
    t = typ.encode()
    head = b"PSKD" + struct.pack("<HI", 2, len(t)) + t + struct.pack("<Q", count) + struct.pack("<I", 2) + bytes([1, 0])
    rec = np.zeros((count, n * 4 + 2), np.uint8)
    rec[:, :n * 4] = x.view(np.uint8).reshape(count, n * 4)
    rec[:, n * 4:] = y.view(np.uint8).reshape(count, 2)
    p = str(tmp_path / "big.psk.d")
    with open(p, "wb") as f:
        f.write(head)
        f.write(rec.tobytes())
    got = device_read(cuda, p, typ, leaves, [abi.BF16, abi.I64])
    want_x = ((x.view(np.uint32) + 0x7fff + ((x.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(got[0].view(np.uint16).reshape(count, n), want_x)
    assert np.array_equal(got[1].view(np.int64), y.astype(np.int64))
    rc, msg, want = ref_read_all(ref, p, typ, leaves, [abi.BF16, abi.I64])
    assert rc == 0 and np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
