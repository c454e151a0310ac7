"""Saga's tensor file format as written and read by the library (no GPU): the
optimizer-state checkpoint is a set of such files."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from saga_b200 import capi
from saga_b200 import optimizer as opt


def test_tensor_file_layout_is_sagas(tmp_path, built_library):
    """Byte for byte what Tensor::save writes (src/tensor.cpp:1387-1391,1470-1550 of the Saga
    tree): magic, u32 type, u32 rank, u32 dims, row-major elements; no temporary file left."""
    a = (np.arange(24, dtype=np.float32).reshape(2, 3, 4) - 7.5)
    path = tmp_path / "t.saga"
    opt.tensor_save(path, a)
    raw = path.read_bytes()
    assert raw[:8] == b"sagaT001"
    assert struct.unpack("<II", raw[8:16]) == (0, 3)            # float, rank 3
    assert struct.unpack("<III", raw[16:28]) == (2, 3, 4)
    assert raw[28:] == a.tobytes()
    assert not os.path.exists(str(path) + ".tmp")
    h = np.array([1.0, -2.5, 65504.0, 6e-8], dtype=np.float16)
    opt.tensor_save(path, h)                                      # overwrite in place
    raw = path.read_bytes()
    assert struct.unpack("<II", raw[8:16]) == (1, 1) and raw[20:] == h.tobytes()


def test_tensor_file_round_trip_and_hand_written_file(tmp_path, built_library):
    rng = np.random.default_rng(3)
    for arr in (rng.standard_normal((5, 7)).astype(np.float32),
                rng.standard_normal(1000).astype(np.float16),
                np.zeros((0,), np.float32)):
        p = tmp_path / "x.saga"
        opt.tensor_save(p, arr)
        back = opt.tensor_load(p)
        assert back.dtype == arr.dtype and back.shape == arr.shape
        assert back.tobytes() == arr.tobytes()
    # a file laid out by hand the way the reference writes it
    data = np.array([3.0, 4.0, 5.0, 6.0, 7.0, 8.0], np.float32)
    p = tmp_path / "hand.saga"
    p.write_bytes(b"sagaT001" + struct.pack("<II", 0, 2) + struct.pack("<II", 3, 2) + data.tobytes())
    assert np.array_equal(opt.tensor_load(p), data.reshape(3, 2))


def test_tensor_file_errors(tmp_path, built_library):
    L = capi.lib()
    p = tmp_path / "bad.saga"
    p.write_bytes(b"notasaga" + bytes(24))
    with pytest.raises(capi.B200OptError):
        opt.tensor_load(p)
    p.write_bytes(b"sagaT001" + struct.pack("<II", 0, 9))        # rank too high
    with pytest.raises(capi.B200OptError):
        opt.tensor_load(p)
    p.write_bytes(b"sagaT001" + struct.pack("<III", 0, 1, 100) + bytes(8))   # too short
    with pytest.raises(capi.B200OptError):
        opt.tensor_load(p)
    with pytest.raises(capi.B200OptError):
        opt.tensor_load(tmp_path / "missing.saga")
    dims = (C.c_uint32 * 1)(4)
    assert L.b200opt_tensor_save(None, capi.FLOAT, 1, dims, None) == capi.EINVAL
    assert L.b200opt_tensor_save(str(p).encode(), 5, 1, dims, None) == capi.EINVAL
    assert L.b200opt_tensor_save(str(tmp_path / "nodir" / "x").encode(), capi.FLOAT, 1, dims,
                                 (C.c_float * 4)()) == capi.EINVAL
    assert L.b200opt_checkpoint_save(None, b"/tmp", 1.0, 0) == capi.EINVAL
