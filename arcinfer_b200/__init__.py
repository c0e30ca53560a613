"""B200-native token selection (penalties, top-k / top-p / min-p sampling, constraint masks,
greedy draft acceptance) behind the sampler interface of rizagp/arcinfer.

The compute path is the CUDA library ``lib/libarcsample.so`` (sources in ``csrc/``, C ABI in
``include/arcsample.h``); this package is the thin Python binding used by the tests and the
benchmark. There is no CPU fallback: importing :mod:`arcinfer_b200.capi` fails when the
library has not been built.
"""
from .capi import (  # noqa: F401
    ArcsError,
    PARAMS_DTYPE,
    argmax_batch,
    dfa_mask,
    lib,
    logprobs_batch,
    make_params,
    merge_batch,
    sample_batch,
)
