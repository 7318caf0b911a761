"""Fusion patterns; each is a function ``pattern(sdfg) -> number of rewrites``."""
PATTERNS = []
