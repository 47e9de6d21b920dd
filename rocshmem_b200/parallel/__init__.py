"""Parallelism helpers above the OpenSHMEM layer: process-grid teams (``layout``), pipeline point-to-point
channels (``pipeline``) and host-side membership / failure detection (``membership``)."""
