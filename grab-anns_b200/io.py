"""Dataset / index file formats of the reference.

* ``.fvecs`` (the format every reference test reads, README.md:42 and
  tests/test_cagra_opt_search_range.cu:91-114): per vector an int32 dimension followed by
  that many float32.
* The two index files (written and read by the C++ classes themselves):
  ``CagraIndex``  -- ``dim u32 | degree u32 | size u64 | float[size*dim] | u32[size*degree]``
  (src/cagraIndex.cu:352-395);
  ``CagraIndexOpt`` -- ``"MCAG" | version u32 = 1 | dim u32 | degree u32 | local_degree u64 |
  size u64 | ts_count u64 | u64[ts] | buckets u64 | {key u64, count u64, u32[count]}* |
  data_count u64 | float[] | graph_count u64 | u32[]`` (src/cagraIndexOpt.cu:725-898).
  ``read_index_header`` parses both headers without loading the payload.
"""
from __future__ import annotations

import struct

import numpy as np


def read_fvecs(path, max_vectors=None):
    raw = np.fromfile(path, dtype=np.int32)
    if raw.size == 0:
        return np.empty((0, 0), dtype=np.float32)
    dim = int(raw[0])
    if dim <= 0 or raw.size % (dim + 1) != 0:
        raise ValueError(f"{path}: not an fvecs file (dim {dim}, {raw.size} words)")
    rows = raw.reshape(-1, dim + 1)
    if not np.all(rows[:, 0] == dim):
        raise ValueError(f"{path}: rows with differing dimensions")
    if max_vectors is not None:
        rows = rows[:max_vectors]
    return np.ascontiguousarray(rows[:, 1:]).view(np.float32)


def write_fvecs(path, vectors):
    v = np.ascontiguousarray(vectors, dtype=np.float32)
    out = np.empty((v.shape[0], v.shape[1] + 1), dtype=np.int32)
    out[:, 0] = v.shape[1]
    out[:, 1:] = v.view(np.int32)
    out.tofile(path)


def read_index_header(path):
    with open(path, "rb") as fh:
        head = fh.read(32)
    if head[:4] == b"MCAG":
        version, dim, degree = struct.unpack_from("<III", head, 4)
        local_degree, size = struct.unpack_from("<QQ", head, 16)
        return {"format": "CagraIndexOpt", "version": version, "dim": dim, "graph_degree": degree,
                "local_degree": local_degree, "size": size}
    dim, degree = struct.unpack_from("<II", head, 0)
    (size,) = struct.unpack_from("<Q", head, 8)
    return {"format": "CagraIndex", "dim": dim, "graph_degree": degree, "size": size}
