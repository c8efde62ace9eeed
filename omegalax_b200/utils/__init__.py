"""Host-side utilities (failure detection)."""
