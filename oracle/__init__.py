"""CPU oracle for the two hot paths (test infrastructure, never the product path).

Everything in this package is a plain fp32/fp64 torch-on-CPU restatement of the
reference's algorithm.  Only the tests, the smoke check and the benchmark's
`cpu_baseline` / `--impl reference` legs may import it; the CUDA library never does.

Pinning: `tests/golden/make_golden.py` runs the reference's own Triton kernels under
`TRITON_INTERPRET=1` (CPU) on seeded inputs and stores their outputs; the
`tests/test_oracle_golden.py` cases check this oracle against those stored vectors.
"""
from .attn_oracle import (  # noqa: F401
    varlen_attn_ref,
    varlen_attn_ref_fwd_bwd,
    target_attn_ref,
    target_attn_ref_fwd_bwd,
    lse_combine_ref,
)
from .gen import (  # noqa: F401
    log_uniform_lengths,
    uniform_lengths,
    log_uniform_until,
    lengths_to_cu,
    make_varlen_inputs,
    make_absorb_inputs,
    CONFIGS,
    config_lengths,
)
from .metrics import max_abs, rel_l2, bf16_floor  # noqa: F401
