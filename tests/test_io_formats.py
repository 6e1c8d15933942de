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


def test_benchmark_configs_have_their_shapes():
    import importlib
    ds = importlib.import_module("grab-anns_b200.datasets")
    want = {"C1": (1000, 128, 10, 32), "C2": (10000, 128, 10, 64), "C3": (10000, 768, 10, 64),
            "C4": (10000, 96, 10, 32), "C5": (100000, 96, 100, 64)}
    scale = {"C1": 0.01, "C2": 0.01, "C3": 0.01, "C4": 0.01, "C5": 0.001}
    for name, (n, dim, k, deg) in want.items():
        w = ds.config(name, scale[name])
        assert w["base"].shape == (n, dim) and w["base"].dtype == np.float32
        assert w["queries"].shape[1] == dim and w["k"] == k and w["degree"] == deg
        again = ds.config(name, scale[name])
        assert np.array_equal(w["base"], again["base"])                       # seeded
        if "ts" in w:
            assert (np.diff(w["ts"].astype(np.int64)) >= 0).all()             # non-decreasing timestamps
        if "lo" in w:
            assert (w["hi"] - w["lo"] == max(1, n // 10)).all()
    c3 = ds.config("C3", 0.01)
    assert np.allclose(np.linalg.norm(c3["base"], axis=1), 1.0, atol=1e-5)
    assert c3["labels"].max() < 16 and ((c3["masks"] > 0) & (c3["masks"] < (1 << 16))).all()
    c2 = ds.config("C2", 0.01)
    assert c2["base"].min() >= 0 and c2["base"].max() <= 255 and (c2["base"] == np.rint(c2["base"])).all()
