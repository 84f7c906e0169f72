"""CPU checker for the GEMM path. Test infrastructure only: imported by tests/,
the smoke check and the benchmark's CPU-baseline leg, never by llmt_b200."""
