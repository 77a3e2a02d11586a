"""moba_b200: the MoBA efficient-attention path as sm_100a kernels, behind the reference's Python API.

Same public names as MoonshotAI/MoBA's `moba` package (moba/__init__.py:1-11): `moba_attn_varlen`,
`MoBAConfig`, `register_moba`, `moba_layer`. Importing the package loads libmoba_b200.so (built with
`python moba_b200/build.py`); there is no fallback if it is missing.
"""
from functools import partial

from .config import MoBAConfig
from .host_io import moba_attn_varlen_host
from .moba_efficient import MixedAttention, calc_chunks, check_kernel_status, moba_attn_varlen
from .wrapper import moba_layer

__all__ = ["MixedAttention", "MoBAConfig", "calc_chunks", "check_kernel_status", "moba_attn_varlen",
           "moba_attn_varlen_host", "moba_layer", "register_moba"]


def _moba_naive_impl(*args, **kwargs):
    """The reference's dense-mask implementation (moba/moba_naive.py), used when a model asks for
    attn_implementation="moba_naive": it is the reference's torch oracle, not a kernel path, so it is taken from
    the reference package when that is importable and refused with a clear message otherwise."""
    try:
        from moba.moba_naive import moba_attn_varlen_naive
    except ImportError as e:
        raise RuntimeError('attn_implementation="moba_naive" is the dense torch oracle of the MoonshotAI/MoBA package, '
                           'which is not importable here; moba_b200 ships the kernel path only: use '
                           'attn_implementation="moba"') from e
    return moba_attn_varlen_naive(*args, **kwargs)


def register_moba(cfg: MoBAConfig):
    """Registers "moba" and "moba_naive" in transformers' attention-function registry, the two keys of
    moba/__init__.py:9-11. "moba" is this package's kernel path; "moba_naive" forwards to the reference package's
    dense oracle when it is installed (see _moba_naive_impl)."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    ALL_ATTENTION_FUNCTIONS["moba"] = partial(moba_layer, moba_attn_varlen, cfg)
    ALL_ATTENTION_FUNCTIONS["moba_naive"] = partial(moba_layer, _moba_naive_impl, cfg)
