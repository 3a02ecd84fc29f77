"""Exception types of the package.

Same three-level convention as the reference (packed_encoders/errors.py:11-20):
one base class, one for "no ModernBERT encoder found", one for a failed
validation gate. Nothing here downgrades silently.
"""
from __future__ import annotations


class PackedEncodersError(Exception):
    """Root of every error this package raises itself."""


class UnsupportedTargetError(PackedEncodersError):
    """The object given to pack()/unpack() does not contain a ModernBERT encoder."""


class ValidationError(PackedEncodersError):
    """validate() refused to enable the CUDA path."""
