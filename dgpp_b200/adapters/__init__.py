"""Runtime adapters."""
