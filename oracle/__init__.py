"""CPU oracle for the quantized matrix-product path.  TEST INFRASTRUCTURE ONLY:
imported by tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs, never
by the product package."""
