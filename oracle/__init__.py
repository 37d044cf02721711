"""CPU oracle for the MXFP4 hot path.  Test infrastructure: imported only by
tests/, the smoke check and the benchmark's CPU-baseline leg."""
