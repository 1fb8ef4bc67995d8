"""CPU oracle for the Daisy attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``daisy_b200/`` imports this package;
only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may.  It is a plain fp32 (or fp64) restatement, in
PyTorch-on-CPU and numpy, of what the reference computes on this path:

* ``oracle.swa``  -- sliding-window causal softmax attention with q/k/v RMS
  normalisation and half-truncated RoPE (reference ``models/daisy/attention.py``,
  ``models/daisy/functional.py``, mask semantics of
  ``models/daisy/daisy_core.py:53-69``) and the ring-buffer KV cache
  (reference ``inference/kv_cache.py``).
* ``oracle.kda``  -- token-by-token Kimi-delta-attention recurrence (semantics
  of the ``chunk_kda`` call at reference ``models/daisy/attention_kimi.py:133-134``;
  the arithmetic itself lives in the third-party ``flash-linear-attention``
  package, which the reference does not pin).

Parity pinning: ``tests/golden/*.npz`` hold outputs of the reference's own code
(``CausalSelfAttention`` / ``KVCache`` imported from the reference tree, and
``fla.ops.kda.naive.naive_recurrent_kda`` 0.5.1) produced by
``tests/golden/make_golden.py``; ``tests/test_oracle_golden.py`` checks this
oracle against them.  KDA parity is pinned only against the third-party naive
recurrence because the reference's own KDA tests cannot run at its current
commit.
"""
