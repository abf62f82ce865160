"""Experimental components; APIs here may change without notice."""
