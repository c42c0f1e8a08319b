"""CPU oracle for the tensor-ash GEMM hot path: test infrastructure only."""
