"""Op library of the decode path."""
