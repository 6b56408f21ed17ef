"""CPU oracle: a restatement of the reference's MoE forward/backward hot path.

TEST INFRASTRUCTURE ONLY.  Only `tests/`, `__graft_entry__.smoke()` and the
`cpu_baseline` / `--impl reference` legs of `bench.py` may import this package,
and only as the checker - the product path (the `sonicmoe` package and its CUDA
library) never does and fails loudly when its CUDA extension is missing.

Parity pin: `oracle.quant` and `oracle.routing` reproduce, bit for bit, the
outputs of the reference's own CPU-loadable goldens stored under
`tests/golden/` (see tests/golden/make_golden.py and tests/test_oracle_golden.py).
The GEMM-level arithmetic of the reference lives in third-party CuTeDSL code and
is pinned at tolerance level only.
"""
