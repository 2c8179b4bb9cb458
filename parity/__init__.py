"""Parity gates in the reference's manner (parity/<name>_test.py there): standalone scripts with a ``run()``
that count their checks and print ``PARITY-CHECKS: <n>``; pytest only drives them (tests/test_parity_gates.py)."""
