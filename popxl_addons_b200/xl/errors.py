"""`xl.errors` (popxl/errors.py)."""

__all__ = ["UndefinedValue"]


class UndefinedValue(Exception):
    """A property that has no value in the current configuration was read (for instance the device slot of a tensor
    that was never placed)."""
