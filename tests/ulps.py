"""Distance in units in the last place between float arrays (test helper)."""
import numpy as np


def ulp_diff(a, b):
    """0 for equal values; NaN matches NaN; +0 equals -0."""
    a, b = np.asarray(a), np.asarray(b)
    assert a.dtype == b.dtype and a.shape == b.shape, (a.dtype, b.dtype, a.shape, b.shape)
    it = np.int32 if a.dtype == np.float32 else np.int64
    ia, ib = a.reshape(-1).view(it).astype(np.int64), b.reshape(-1).view(it).astype(np.int64)
    lo = np.int64(np.iinfo(it).min)
    ia = np.where(ia < 0, lo - ia, ia)
    ib = np.where(ib < 0, lo - ib, ib)
    d = np.abs(ia - ib)
    both_nan = np.isnan(a.reshape(-1)) & np.isnan(b.reshape(-1))
    return np.where(both_nan, 0, d)
