"""CPU oracle for the kten hot path -- test infrastructure, not part of the product."""
