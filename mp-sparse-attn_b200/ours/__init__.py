"""Drop-in mirror of the reference project's `ours` package: same module and function names,
argument order, defaults and return tuples, backed by the sm_100a kernels of libmpsa.so
(no Triton, no CPU fallback)."""
