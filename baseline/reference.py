"""Access to the unmodified reference package installed under baseline/_ref (see install_reference.sh) --
benchmark / test infrastructure, never imported by the product package.

* load_naive()      -> moba.moba_naive.moba_attn_varlen_naive (pure torch; runs on the host cores)
* load_efficient()  -> moba.moba_efficient.moba_attn_varlen with the two private flash-attn entry points it
                       imports rebound for the installed flash-attn 2.8.x: the reference is written against
                       flash-attn 2.6.3 (its requirements.txt:1), whose _flash_attn_varlen_forward returned eight
                       values (2.8 returns four) and whose _flash_attn_varlen_backward took window_size as a pair
                       and returned (dq, dk, dv, softmax_d) (2.8 takes window_size_left / right, writes into
                       caller-provided dq / dk / dv and returns softmax_d). Only the names inside the imported
                       module object are rebound; the installed source files stay as shipped.
"""
import importlib
import os
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available():
    return os.path.isfile(os.path.join(REF_DIR, "moba", "moba_naive.py"))


def _import(name):
    if not available():
        raise ImportError(f"{REF_DIR} holds no reference install (run baseline/install_reference.sh)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module(name)


def load_naive():
    """The reference's moba_attn_varlen_naive (moba/moba_naive.py:7-96), unmodified."""
    return _import("moba.moba_naive").moba_attn_varlen_naive


def load_efficient():
    """The reference's moba_attn_varlen (moba/moba_efficient.py:270-443) on the installed flash-attn."""
    import torch
    from flash_attn import flash_attn_interface as fi

    me = _import("moba.moba_efficient")
    if getattr(me, "_compat_installed", False):
        return me.moba_attn_varlen

    def forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal, dropout_p):
        out, lse, _, rng = fi._flash_attn_varlen_forward(
            q, k, v, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k), dropout_p, softmax_scale,
            causal)
        return None, None, None, None, out, lse, None, rng        # positions 4 and 5 are what the reference reads

    def backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                 max_seqlen_k, softmax_scale, causal, dropout_p, window_size, softcap, alibi_slopes, deterministic):
        dq = torch.empty_like(q) if dq is None else dq
        dk = torch.empty_like(k) if dk is None else dk
        dv = torch.empty_like(v) if dv is None else dv
        d = fi._flash_attn_varlen_backward(
            dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q),
            int(max_seqlen_k), dropout_p, softmax_scale, causal, window_size[0], window_size[1], softcap,
            alibi_slopes, deterministic)
        return dq, dk, dv, d

    me._flash_attn_varlen_forward = forward
    me._flash_attn_varlen_backward = backward
    me._compat_installed = True
    return me.moba_attn_varlen
