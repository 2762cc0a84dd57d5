"""CPU oracles for the GeMKM/GeKMM parity tests.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline legs; never by the product package.

Two checkers live here:

* ``port``      -- ``kron_oracle.c``, a plain-C restatement of the reference's sliced
  multiply (its header lists the reference lines it follows), built by
  ``oracle/Makefile`` into ``libkron_oracle.so``.
* ``reference`` -- the UNMODIFIED reference x86 backend, compiled from the reference's
  own sources by ``oracle/build_ref.sh`` into ``oracle/_ref/libFastKron.so`` and driven
  through its public C API.
"""
from .oracle import (  # noqa: F401
    port_available, ref_available, port_gekmm, ref_gekmm, numpy_gekmm, RefLib,
)
