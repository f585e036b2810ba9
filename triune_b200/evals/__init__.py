"""Task-level evaluations of the sequence mixers (no training involved)."""
