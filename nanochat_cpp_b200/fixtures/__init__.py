"""Fixture producers: deterministic record files that pin behaviour which has no upstream oracle."""
