"""CPU restatement of the reference algorithms.  TEST INFRASTRUCTURE ONLY.

Nothing under `vexact_b200/` imports this package.  It is used by `tests/`, by
`__graft_entry__.smoke()` and by the `cpu_baseline` / `--impl reference` legs of
`bench.py`, always as the checker or the timed CPU baseline, never as the
product path.
"""
