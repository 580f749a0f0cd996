"""CPU oracle for the calibration-time quantization hot path.

TEST INFRASTRUCTURE ONLY.  This package is a restatement, in plain torch-CPU
arithmetic, of what the reference (ModelTC/LightCompress, `llmc/compression/
quantization/{quant,gptq,awq,auto_clip}.py`) computes on the path this
repository accelerates.  Only the test-suite, the smoke check and the
`cpu_baseline` / `--impl reference` legs of the benchmark may import it; the
product package never does and has no CPU fallback.

Pinning: the reference ships no tests and no golden vectors, so every function
here is pinned differentially against the reference itself, imported and run
on CPU; the resulting input/output pairs are committed under `tests/golden/`
together with the script that produced them (`tests/golden/make_golden.py`).
The one exception is the FP8 rounding step, which the reference delegates to
the un-vendored third-party `qtorch.quant.float_quantize` (no pinned version):
for that single call parity is UNPINNED; it is restated as round-to-nearest-even
onto the float8_e4m3fn grid.
"""
from . import quant_ref, gptq_ref, gptq_block_ref  # noqa: F401
