"""CPU checkers for the attention hot path.  TEST INFRASTRUCTURE ONLY.

``oracle.restatement`` loads ``liboracle.so`` (the C restatement in this
directory); ``oracle.reference`` loads ``_ref/libwayruntime_ref*.so`` (the
unmodified reference compiled from its own sources).  Only the test suite, the
smoke check and the bench's CPU-baseline legs may import this package; the
product never does.
"""
from .bindings import Checker, reference, restatement  # noqa: F401
