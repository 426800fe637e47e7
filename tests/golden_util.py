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


def check_close(family, name, result, rtol, atol, *inputs):
    """fp32 results against the stored reference outputs (sampled positions for large
    tensors): |result - golden| <= atol + rtol * |golden| elementwise."""
    g = _load(family)
    assert int(g[name + "/crc"]) == crc(*inputs), f"{name}: seeded inputs differ from golden run"
    assert tuple(g[name + "/shape"]) == result.shape, (name, result.shape)
    flat = np.asarray(result, np.float64).reshape(-1)
    if name + "/idx" in g.files:
        flat = flat[g[name + "/idx"]]
    want = g[name].astype(np.float64)
    excess = np.abs(flat - want) - (atol + rtol * np.abs(want))
    assert np.isfinite(flat).all() and excess.max() <= 0, \
        f"{name}: worst excess {excess.max():.3e} over the tolerance"
