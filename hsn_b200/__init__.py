"""hsn_b200: the HSN TBPTT window path (router top-K, sparse state gather, gated cell update,
reset masking, reverse state recurrence, carried state) as hand-written sm_100a CUDA behind a
C ABI, with the reference's Python interface on top.

* :mod:`hsn_b200.kernels.window` mirrors the reference's ``hsn.kernels.window`` (custom ops kept).
* :mod:`hsn_b200.window` holds the whole-window entry points (prologue, forward sweep, reverse sweep,
  streaming step, decoder).
* :mod:`hsn_b200.kernels.trainer` mirrors ``hsn.kernels.trainer``; :mod:`hsn_b200.parallel` holds the fused
  gradient exchange + AdamW; :mod:`hsn_b200.state` the carried state's snapshots and checkpoint payload.
* :mod:`hsn_b200.kernels.units`, :mod:`hsn_b200.kernels.scorer`, :mod:`hsn_b200.kernels.tail`,
  :mod:`hsn_b200.kernels.gate` and :mod:`hsn_b200.kernels.messages` are five pieces of the split window's replay:
  ``_scorer_logits``, and ``PDGCell.replay_sparse`` in four (messages and gathered inputs, cell norm and gate,
  ``UnitBank.forward_grouped``, ``W_out`` + candidate norm + ``tanh``), as autograd functions.
* :mod:`hsn_b200.build` compiles ``csrc`` into ``lib/libhsn_window_b200.so``.

Importing the package neither initialises CUDA nor loads the library.
"""

__version__ = "0.1.0"
