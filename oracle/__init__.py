"""CPU restatement of the reference algorithms.  TEST INFRASTRUCTURE ONLY: imported by tests/,
__graft_entry__.smoke() and bench.py's cpu_baseline / reference arm, never by the product package."""
