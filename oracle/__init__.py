"""CPU oracle of the int64 fixed-point hot path (test infrastructure only)."""
