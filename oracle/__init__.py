"""Checkers for the CLUSTEN operators.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference legs of
bench.py may import this package; the product (ml-autofocusformer_b200/) never does.

  formula.py        the PyTorch gather formulation the reference's own tests compare against
  clusten_oracle.c  plain-C restatement of the reference's eight kernels (c_oracle.py binds it)
  build_ref.py      compiles the reference's unmodified CUDA extension into oracle/_ref/
  ref_cuda.py       loads that extension on a GPU machine
"""
