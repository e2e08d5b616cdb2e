"""CPU oracle for the paged-KV decode path (reshape_and_cache -> paged_attention).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import, link or
execute anything from this directory: the oracle exists so that the tests, the
smoke check and the CPU-baseline leg of the benchmark have an independent
checker to compare the CUDA path against.

Contents
--------
paged_kv_numpy.py   numpy restatement of the reference's numpy goldens
paged_kv_oracle.c   the same arithmetic in plain C (OpenMP over sequences and
                    heads) for cases too large for the numpy version
c_oracle.py         ctypes loader for the compiled C restatement
ms_stub.py          minimal stand-in for the `mindspore` module so that the
                    reference's own test modules can be imported on a machine
                    that holds a checkout of the reference (fixture generation)
Makefile            builds libpaged_kv_oracle.so

Parity status: paged attention and the plain cache scatter are pinned against
outputs of the reference's own golden functions (see tests/golden).  The
quantising cache scatter has no counterpart in the reference operator and is
"parity unpinned": it is defined here as the exact inverse of the reference's
de-quantisation formula with numpy's round-half-to-even.
"""
