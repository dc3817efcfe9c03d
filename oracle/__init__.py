"""CPU oracle of the residual LayerNorm path.  Test infrastructure only:
imported by tests, by the smoke entry and by the CPU-baseline leg of the
benchmark, never by the shipped package."""
