"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: CPU restatements of the reference's algorithms.

Only tests, the smoke check and the CPU-baseline legs of the benchmark may import this package.
"""
