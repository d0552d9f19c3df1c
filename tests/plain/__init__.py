"""Plain, slow, whole-sequence implementation used as the oracle by the tests.

Nothing in here is imported by the product package and nothing in here imports
the product package: it rests only on torch (CPU) and on the formulas of the
reference's files, cited beside each function.
"""
