"""CPU checkers for the B200 backend.  TEST INFRASTRUCTURE ONLY: imported by
tests/, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py``; the product package never imports it."""
