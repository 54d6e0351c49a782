"""NumPy-backed stand-in for the few `mlx.core` names the reference's op definitions touch on their
generator / float64-truth path (array wrapping, dtype aliases, concatenate, broadcast_to, eval).
Used only by make_golden.py, in a container that has the reference checked out; it contains no
reference code and is not importable from the product."""
import numpy as np

float16, float32, bfloat16, int32, bool_ = np.float16, np.float32, np.float32, np.int32, np.bool_
__version__ = "numpy-standin"


class array(np.ndarray):
    def __new__(cls, a):
        return np.asarray(a).view(cls)

    def astype(self, dtype, *a, **k):
        return np.asarray(self).astype(dtype, *a, **k).view(array)


def concatenate(xs, axis=0):
    return np.concatenate([np.asarray(x) for x in xs], axis=axis).view(array)


def broadcast_to(x, shape):
    return np.broadcast_to(np.asarray(x), shape).view(array)


def eval(*_a, **_k):
    return None


def clear_cache():
    return None
