"""CPU oracle for the routed-expert MoE FFN path: test infrastructure only.

Nothing in the product package imports this. The tests, the smoke check and
the benchmark's CPU-baseline leg load it to check (never to compute) results.
"""
