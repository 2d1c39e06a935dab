"""`bitarray.util.hex2ba` of the stand-in: four bits per hexadecimal digit, most significant first."""
from . import bitarray


def hex2ba(text):
    bits = []
    for digit in text:
        value = int(digit, 16)
        bits += [bool(value & 8), bool(value & 4), bool(value & 2), bool(value & 1)]
    return bitarray._of(bits)
