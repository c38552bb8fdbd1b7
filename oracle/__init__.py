"""CPU checkers for the block ops (test infrastructure; never imported by the product package)."""
