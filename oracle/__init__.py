"""CPU oracle for the LSH + gated-delta forward path: test infrastructure only."""
