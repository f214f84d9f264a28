"""CPU oracle for the gated-attention path (test infrastructure; never imported by the library)."""
