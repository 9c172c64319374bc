"""Errors shared with the reference's conventions (python/caminus/errors.py): terminal numerical failures a caller must not
retry or reset away. The device kernels never trap: they OR bits into a sticky int32 flag word; the host reads the word
after the stream has drained and raises these."""


class NumericalFailure(RuntimeError):
    """terminal numerical state corruption: refuse further work until the process restarts (python/caminus/errors.py:4-9)"""


class InvalidKVEncoding(NumericalFailure):
    """a Q8_0 KV encoder refused a block (a non-finite value, a scale outside fp16 / fp32 range); other blocks of the same
    append may already be written: the append and its cache state are unusable (python/caminus/errors.py:19-24)"""
