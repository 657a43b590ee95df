"""Counterpart of the reference's src/gmc/cpp/extensions/pieces/bindings.py (matrix inverse and symmetric
eigen-decomposition of 2x2 / 3x3 matrices)."""
from gmc.cpp.extensions.math import matrix_inverse as _matrix_inverse

matrix_inverse_apply = _matrix_inverse.apply


def symeig_apply(matrices):
    raise NotImplementedError("symeig for 2x2 / 3x3 matrices is not part of this build yet")
