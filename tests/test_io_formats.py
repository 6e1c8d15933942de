"""File formats of the reference (no GPU): .fvecs reader/writer and index headers."""
import importlib
import struct

import numpy as np
import pytest


def test_fvecs_round_trip(tmp_path):
    io = importlib.import_module("grab-anns_b200.io")
    v = np.random.default_rng(0).standard_normal((17, 12)).astype(np.float32)
    p = tmp_path / "x.fvecs"
    io.write_fvecs(p, v)
    raw = np.fromfile(p, dtype=np.int32)
    assert raw.size == 17 * 13 and raw[0] == 12 and raw[13] == 12     # int32 dim before every vector
    assert np.array_equal(io.read_fvecs(p), v)
    assert io.read_fvecs(p, max_vectors=5).shape == (5, 12)
    (tmp_path / "bad.fvecs").write_bytes(struct.pack("<i3f", 5, 1.0, 2.0, 3.0))
    with pytest.raises(ValueError):
        io.read_fvecs(tmp_path / "bad.fvecs")


def test_index_headers(tmp_path):
    io = importlib.import_module("grab-anns_b200.io")
    p = tmp_path / "a.idx"
    p.write_bytes(struct.pack("<IIQ", 128, 64, 1000) + b"\0" * 16)
    assert io.read_index_header(p) == {"format": "CagraIndex", "dim": 128, "graph_degree": 64, "size": 1000}
    p.write_bytes(b"MCAG" + struct.pack("<IIIQQ", 1, 96, 32, 16, 5000))
    assert io.read_index_header(p) == {"format": "CagraIndexOpt", "version": 1, "dim": 96, "graph_degree": 32,
                                       "local_degree": 16, "size": 5000}
