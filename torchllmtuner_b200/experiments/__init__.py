"""Experimental subsystems that are not reachable from the production CLI."""
