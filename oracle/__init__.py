"""CPU oracle of the dense-matmul / policy-MLP path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only tests/, the smoke check
and the CPU-baseline legs of bench.py may import it, and only as the checker.
"""
