"""Measurement helpers: small command-line drivers that run one operator a few times (targets for
a profiler, quick timings) and a TMA streaming probe in a shared library of its own
(``libgemm_b200_probe.so``).  None of this is on the library's call path and nothing in
``gemm_b200`` outside this folder imports it."""
