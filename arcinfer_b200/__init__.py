"""B200-native token selection (penalties, top-k / top-p / min-p sampling, constraint masks,
greedy draft acceptance) behind the sampler interface of rizagp/arcinfer.

The compute path is the CUDA library ``lib/libarcsample.so`` (sources in ``csrc/``, C ABI in
``include/arcsample.h``); this package is the thin Python binding used by the tests and the
benchmark. There is no CPU fallback: the first use of any binding name below imports
:mod:`arcinfer_b200.capi`, which fails when the library has not been built. Importing the
package alone (or :mod:`arcinfer_b200.synth`, :mod:`arcinfer_b200.params`) loads nothing, so a
process that only generates inputs does not map the CUDA library.
"""
from .params import PARAMS_DTYPE, make_params  # noqa: F401

_CAPI_NAMES = ("ArcsError", "accept_batch", "adjusted_batch", "argmax_batch", "dfa_mask", "dflash_select", "lib", "logprobs_batch", "merge_batch", "merge_records", "sample_batch")


def __getattr__(name):
    if name == "capi" or name in _CAPI_NAMES:
        import importlib

        capi = importlib.import_module(".capi", __name__)
        return capi if name == "capi" else getattr(capi, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
