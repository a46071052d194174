"""CPU oracle for sptorch's transformer forward -- test infrastructure only.

Importable only from tests/, the smoke check and the bench's CPU-baseline leg.
"""
