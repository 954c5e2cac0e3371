"""HTTP serving and production plumbing."""
