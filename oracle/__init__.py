"""CPU oracle for the calibrate-and-quantize hot path.

TEST INFRASTRUCTURE ONLY.  This package restates, on CPU tensors, the arithmetic
that llm-compressor and its compressed-tensors dependency perform on the GPTQ /
observer / quantize / pack path.  It exists so that the CUDA kernels can be checked
against an independent statement of the algorithm.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it; the product package
never does and has no CPU fallback.

Where the arithmetic lives in compressed-tensors (pinned by the reference at
``compressed-tensors==0.18.0``, ``setup.py:141-145``; version 0.15.0.1 was the one
available to pin against), each function cites the file and lines of that package
under the prefix ``CT/``; functions following llm-compressor itself cite
``src/llmcompressor/...``.

Pinning: ``tests/golden/`` holds outputs of the real reference functions
(``gptq_quantize.py`` loaded unmodified, the reference observer classes and the
installed compressed-tensors quantize/compress routines) on seeded inputs, and the
known-answer vectors of the reference's own observer/lifecycle tests.  The oracle
is checked against all of them by ``tests/test_oracle_golden.py``.
"""
from .spec import QSpec, preset  # noqa: F401
from .rounding import (  # noqa: F401
    bf16_round,
    cast_e2m1,
    cast_e4m3,
    e8m0_from_amax,
    round_to_power_2,
)
from .qparams import calculate_qparams, generate_gparam, qrange  # noqa: F401
from .quantize import fake_quantize, quantize_codes, dequantize_codes  # noqa: F401
from .pack import (  # noqa: F401
    pack_int32,
    unpack_int32,
    pack_fp4,
    compress_mx_scale,
    compress_weight,
    infer_format,
)
from .observers import flatten_weight, observe_minmax, observe_mse, WeightObserver  # noqa: F401
from .gptq import (make_empty_hessian, accumulate_hessian, accumulate_hessian_running_mean,  # noqa: F401
                   quantize_weight)
from . import awq  # noqa: F401,E402
