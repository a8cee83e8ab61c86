"""CPU oracle of the hot path.  TEST INFRASTRUCTURE: only tests, the smoke check and the
benchmark's CPU-baseline leg may import this package."""
