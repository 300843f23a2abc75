"""The process boundary: resource sandbox, GPU job queue, session supervisor (standard library only)."""
