"""Command-line tools that ship with the backend."""
