"""CPU oracle for the NAtSL hybrid-attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module;
it exists so that tests, the smoke check and the CPU-baseline leg of the
benchmark can check / time a plain restatement of the reference algorithm.

Every function cites the reference file:line it restates (paths relative to
the reference project root, ``src/nats/...``).  The restatement is plain
PyTorch on CPU (fp32 or fp64), vectorised over batch and heads with Python
loops over tokens or chunks.

Parity pinning
--------------
* Selection tables (``oracle.tables``): pinned against the reference's own
  ``src/nats/ops/nats_util.py`` executed on CPU (loaded by file path) and against
  a known-answer vector produced by that code; the outputs are committed under
  ``tests/golden/`` together with the generating script.
* GDN numerics (``oracle.gdn``): the reference ships no stored vectors and its
  own debug scripts compare against the third-party ``flash-linear-attention``
  kernels.  The oracle is pinned on the all-blocks-selected special case against
  that package's pure-PyTorch ``naive_recurrent_gated_delta_rule`` /
  ``naive_chunk_gated_delta_rule`` (version 0.5.1 on disk; the reference pins
  0.4.0), and its two independent forms (token recurrence with re-roll, chunk
  form following the reference kernels) are checked against each other.
* Mamba2 numerics and the softmax branch have no runnable reference or stored
  vector in the reference project: parity unpinned beyond the internal
  recurrent-vs-chunk cross-check and the mask formula of the reference's own
  debug script (``src/nats/ops/attns/attns.py:2041-2058``).
* Gradients (``oracle.grad``): true gradients by autograd through the forward oracle, and closed forms of what
  the reference's backward returns where it is not the true gradient; parity unpinned (no runnable reference),
  the closed forms are checked against the autograd derivatives they stand for.
"""
from . import tables, gdn, mamba, attn, grad  # noqa: F401
