"""TEST INFRASTRUCTURE: CPU oracles for the row-op path (see oracle_rowops.c, ref_harness.cpp)."""
