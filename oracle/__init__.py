"""CPU oracle for the uneven-collective / sharded-op hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``hap_b200/`` may import this package:
it exists so that ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` can check or time
the CUDA path against a CPU restatement of the reference's algorithm.
"""
