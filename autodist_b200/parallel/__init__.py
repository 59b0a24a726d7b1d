"""Runtime: rank launcher, communication backends, step engine, symmetric-memory kernels."""
