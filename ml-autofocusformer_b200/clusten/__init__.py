"""Drop-in `clusten` package: AutoFocusFormer's CLUSTEN operators on B200.

    from clusten import CLUSTENQKFunction, CLUSTENAVFunction, CLUSTENWFFunction
"""
from .clusten import CLUSTENQKFunction, CLUSTENAVFunction, CLUSTENWFFunction
from .ops import clear_inverse_cache

__all__ = ["CLUSTENQKFunction", "CLUSTENAVFunction", "CLUSTENWFFunction", "clear_inverse_cache"]
