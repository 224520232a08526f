"""CPU oracle for the gated linear scan (test infrastructure; never on the product path)."""
