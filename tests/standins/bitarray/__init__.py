"""A stand-in for the `bitarray` package, which this image does not have: the handful of operations the
reference's tests/features/test_custom_connectivity_update.py uses, over a numpy array of booleans.
Bits are a sequence, index 0 first; `>>` moves every bit towards higher indices and fills with zeros,
as the package documents for its default (big-endian) bit order."""
import numpy as np


class bitarray:
    def __init__(self, length=0):
        self._bits = np.zeros(int(length), dtype=bool)

    @classmethod
    def _of(cls, bits):
        out = cls(0)
        out._bits = np.array(bits, dtype=bool)
        return out

    def __len__(self):
        return len(self._bits)

    def setall(self, value):
        self._bits[:] = bool(value)

    def copy(self):
        return bitarray._of(self._bits)

    def __getitem__(self, index):
        return bool(self._bits[index])

    def __setitem__(self, index, value):
        if isinstance(index, (list, tuple, np.ndarray)):
            index = np.asarray(index, dtype=np.int64)
        self._bits[index] = bool(value)

    def __eq__(self, other):
        return isinstance(other, bitarray) and np.array_equal(self._bits, other._bits)

    def __rshift__(self, count):
        count = int(count)
        out = np.zeros_like(self._bits)
        if count < len(out):
            out[count:] = self._bits[:len(out) - count]
        return bitarray._of(out)

    def __repr__(self):
        return "bitarray('" + "".join("1" if b else "0" for b in self._bits) + "')"
