"""Small host-side utilities shared by every layer of the framework."""
