"""Import-only stand-in for matplotlib (the reference's trace module imports pyplot)."""
