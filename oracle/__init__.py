"""CPU oracles: TEST INFRASTRUCTURE, not product code.

Each sub-directory holds a ``model.py`` in the shape the reference workspace gives
its eager model (agent_workdir/model.py:9-26: ``Model``, ``get_inputs``,
``get_init_inputs``) for one operator path. The reference ships no model for
these paths (its only ``model.py`` is ``alpha*a+b``), no golden vector and no
test for them, so these files restate the operator definitions themselves and
their parity is UNPINNED by the reference: the pins are this repository's own
(independent float64 loops, hand-computed cases, committed fixtures under
``tests/golden``).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` import anything from here. Nothing under ``cuda_agent_b200/``
does, and the CUDA path never falls back to it.
"""
