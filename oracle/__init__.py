"""CPU oracle for the sparse-attention forward path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the checker
and as the timed CPU baseline, never as the product path.

Each function restates, in plain PyTorch/numpy on the CPU, the arithmetic of
one reference function and cites the reference file:line it follows.  The
restatements are pinned against outputs of the reference itself (its Triton
kernels executed on CPU tensors with ``TRITON_INTERPRET=1`` and its pure
PyTorch static attention), stored as fixtures under ``tests/golden/`` together
with the script that generated them.

Parity status per part:
  * DSA indexer / top-k / routing-weighted attention: pinned by golden
    fixtures generated from the reference's own kernels.
  * Static (1-D window) sparse attention, 2-D RoPE: pinned by golden fixtures
    generated from the reference's own modules.
  * 2-D block-sparse attention and NSA: the reference contains no such code;
    those oracles are library-defined ("parity unpinned").
"""
