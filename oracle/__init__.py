"""CPU checker for the CKKS encrypted-aggregation path (test infrastructure only).

Nothing in the product package may import this: it exists for tests, the smoke entry
and the benchmark's CPU baseline legs.
"""
