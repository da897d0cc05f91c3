"""CPU oracle for dyninfer's direct quantized decoder path (test infrastructure only)."""
