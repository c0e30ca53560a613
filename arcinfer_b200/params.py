"""Row parameters of the sampler as a numpy record (no CUDA library is loaded by this module)."""
import numpy as np

# arcs_row_params: SamplingParams of the reference (tools/sampler.h:15-26) without seed / logit_bias
PARAMS_DTYPE = np.dtype(
    [
        ("temperature", "<f4"),
        ("top_p", "<f4"),
        ("min_p", "<f4"),
        ("presence_penalty", "<f4"),
        ("frequency_penalty", "<f4"),
        ("repeat_penalty", "<f4"),
        ("repeat_last_n", "<i4"),
        ("top_k", "<i4"),
    ]
)


def make_params(n=1, **kw):
    """n rows of SamplingParams defaults (tools/sampler.h:16-22), fields overridden by kw."""
    p = np.zeros(n, PARAMS_DTYPE)
    p["temperature"], p["top_p"], p["repeat_penalty"], p["repeat_last_n"], p["top_k"] = 1.0, 0.95, 1.0, 64, 20
    for k, v in kw.items():
        p[k] = v
    return p
