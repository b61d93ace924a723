"""CPU oracle (test infrastructure only; see blockscale_ref.py)."""
