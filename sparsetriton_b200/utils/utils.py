"""Small helpers (reference: sparsetriton/utils/utils.py:15-47)."""


def make_ntuple(value, n):
    """`value` repeated n times, or a sequence cut / padded with its last element to length n."""
    if isinstance(value, (list, tuple)):
        seq = tuple(value)
        return seq[:n] if len(seq) >= n else seq + (seq[-1],) * (n - len(seq))
    if isinstance(value, (int, float)):
        return (value,) * n
    raise TypeError(f"Expected int, float, tuple, or list, got {type(value)}")
