"""Placeholder until the MLA model lands in this file."""
