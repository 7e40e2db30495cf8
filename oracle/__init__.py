"""CPU oracle for the fused-MoE path. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this; it is the checker used by
``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``.
"""
