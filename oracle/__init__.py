"""CPU oracle for the routed MaskedLinear / MaskedFFN path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is the checker used by the tests, by the smoke entry point and by
the CPU-baseline legs of the benchmark.
"""
