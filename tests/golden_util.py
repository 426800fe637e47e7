"""Compare a computed tensor with the committed golden vectors (tests/golden/*.npz)."""
import os
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_cache = {}


def _load(family):
    if family not in _cache:
        _cache[family] = np.load(os.path.join(HERE, "golden", family + ".npz"))
    return _cache[family]


def crc(*arrays):
    c = 0
    for a in arrays:
        if a is not None:
            c = zlib.crc32(np.ascontiguousarray(a).tobytes(), c)
    return c


def check(family, name, result, *inputs):
    """Bit-exact check of ``result``; also proves the inputs are the ones the golden run saw."""
    g = _load(family)
    assert int(g[name + "/crc"]) == crc(*inputs), f"{name}: seeded inputs differ from golden run"
    if name in g.files:
        want = g[name]
        assert result.shape == want.shape, (name, result.shape, want.shape)
        bad = int((result != want).sum())
        assert bad == 0, f"{name}: {bad} of {want.size} elements differ from the reference"
    else:
        assert tuple(g[name + "/shape"]) == result.shape
        assert int(g[name + "/out_crc"]) == crc(result), f"{name}: output digest differs"
