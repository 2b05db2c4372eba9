"""Command-line helpers that ship with the engine (checkpoint export, tensor comparison)."""
