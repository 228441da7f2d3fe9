"""CPU oracle package — test infrastructure, never a product path."""
