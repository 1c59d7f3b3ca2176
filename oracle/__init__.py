"""CPU oracle for the ternary BitLinear hot path — test infrastructure only.

Importable from tests, the smoke check and the benchmark's CPU-baseline leg;
the shipped package never imports it.
"""
