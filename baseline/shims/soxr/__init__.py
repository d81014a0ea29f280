"""Import-time stand-in for `soxr` (not used by the text benchmark path)."""
