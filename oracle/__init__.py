"""CPU oracle package (test infrastructure only; never imported by zinc_b200)."""
