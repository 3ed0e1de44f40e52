"""Parity checkers for the s2v inference path -- TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
import this package; the product (``graphnn_b200``) never does.

* ``c_oracle``   : ctypes front-end of ``s2v_oracle.c`` (plain-C restatement).
* ``reference``  : ctypes front-end of ``_ref/libs2v_ref.so`` (the reference's own
  C++ compiled against the MKL/TBB stand-ins), when that file exists.
* ``s2v_numpy``  : float64 numpy/scipy restatement used to grade fp32 error.
"""
