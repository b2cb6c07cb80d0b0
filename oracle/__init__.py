"""CPU oracle for the qs3 mixture-of-experts path (test infrastructure only).

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this package. The product
package never does.
"""
