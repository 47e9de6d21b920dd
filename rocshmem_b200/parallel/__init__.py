"""Parallelism helpers above the OpenSHMEM layer: process-grid teams (``layout``), data-parallel gradient buckets
(``data_parallel``), pipeline channels and stages (``pipeline``), sequence <-> head re-sharding for attention
(``ulysses``), ring exchange and ring attention (``ring``), host-side membership / failure detection
(``membership``) and shrinking a running job to its survivors (``elastic``). Tensor- and expert-parallel layers live in ``rocshmem_b200.models``."""
