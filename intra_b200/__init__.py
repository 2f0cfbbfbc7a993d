"""intra_b200: INTRA forward sparse attention, built for NVIDIA B200 (sm_100a).

Drop-in for the reference's `intra_attn` package: `intra_llm_attn` and `intra_image_attn` keep the
reference's signatures (intra_attn/interface.py:30,48). As in the reference
(intra_attn/__init__.py:1-7) the package imports without the native library and the entry points
raise ImportError when called; there is no non-CUDA fallback.
"""
try:
    from .interface import intra_image_attn, intra_llm_attn
except ImportError as _err:  # native library not built
    def _missing(*args, _err=_err, **kwargs):
        raise ImportError(f"libintra_b200.so is not built ({_err}); run `python -m intra_b200.build`")

    intra_image_attn = intra_llm_attn = _missing

__version__ = "0.1.0"
__all__ = ["intra_llm_attn", "intra_image_attn"]
