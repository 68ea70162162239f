"""placeholder, filled in below."""
