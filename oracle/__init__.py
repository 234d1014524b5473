"""CPU oracle of the activation offload codec.  TEST INFRASTRUCTURE ONLY.

Two independent restatements of the reference arithmetic live here:
``codec_oracle.c`` (scalar C, loaded through ctypes by :mod:`oracle.capi`) and
:mod:`oracle.codec_np` (vectorised numpy).  The shipped package never imports
this directory; only the tests, the smoke check and the CPU-baseline leg of the
benchmark do, and only as the checker or the reported baseline.
"""
