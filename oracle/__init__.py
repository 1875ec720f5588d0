"""CPU oracle for the fused GEMM + epilogue path.  TEST INFRASTRUCTURE ONLY.

Nothing under ``fuseml_b200`` imports this package.  It is used by ``tests/``,
by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py`` as the checker and the timed CPU baseline, never as a
product path.

Two layers:

* :mod:`oracle.chain` — a numpy restatement of what one fused kernel computes
  (fp32-accumulated GEMM, the epilogue operations in order, the reduction
  tails), each function citing the lines of the reference it follows.
* :mod:`oracle.configs` — the five benchmark configurations as seeded input
  generators plus the eager fp32 PyTorch module each one is; that module is
  what the reference itself executes on a CPU (its compiler bypasses fusion
  there and returns ``gm.forward``, fuseml/compiler.py:213-228).

Parity pin: the reference ships no golden vectors for this path, so the
oracle is pinned against outputs of the reference itself — its
``FuseMLCompiler`` run in the authoring container on scaled-down and full
CPU-runnable cases — stored under ``tests/golden/`` together with the script
that generated them (``tests/golden/make_golden.py``).
"""
