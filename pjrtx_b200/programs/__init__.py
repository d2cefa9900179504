"""Program builders that play the part of `jax.jit` + the StableHLO importer in front of the backend."""
