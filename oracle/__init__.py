"""CPU oracle for the BCQ LUT-GEMV path — test infrastructure, not product code."""
