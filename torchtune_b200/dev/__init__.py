"""Experimental components (parity: torchtune/dev)."""
