"""B200 (sm_100a) implementation of ZK-DeepSeek's int64 fixed-point hot path.

The directory doubles as a drop-in module path: put it first on ``sys.path`` and the
reference's ``from kernel import ...`` resolves to ``kernel.py`` here.  As a package it
is imported with ``importlib.import_module("zk-deepseek_b200")`` (the hyphen rules out
the plain ``import`` statement).
"""
