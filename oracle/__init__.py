"""CPU oracle of the forward-Laplacian hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under ``folx_b200/`` may import this package: it exists to check the CUDA kernels
(``tests/``, the smoke test) and to be timed as the CPU baseline of the benchmark.  The
reference (microsoft/folx) is pure Python on JAX, which is not installed on the build or GPU
machines, so this is a restatement of its rules:

* ``rules``  -- closed-form propagation rules in torch-CPU (fp64 for checking, fp32 for timing),
  each citing the reference lines it follows;
* ``brute``  -- brute-force Jacobians / Hessian traces by automatic differentiation, the same
  identity the reference's own tests assert (test/laplacian_testcase.py:22-49);
* ``refmasks`` -- loader that executes the reference's pure-NumPy index-map helpers straight from
  a checkout of the reference (used only to generate the golden fixtures under tests/golden/).

Parity status: the integer index-map paths are pinned by the reference's literal known-answer
arrays (test/test_find_out_idx.py) and by fixtures generated from the reference's own NumPy
code.  The reference stores NO golden floating-point vectors; its float tests assert equality
with brute-force AD on random inputs, and that is what pins ``rules`` here (tests/test_oracle.py).
In the stored-number sense the float paths are therefore "parity unpinned".
"""
