from .gemv import bfgemv, hgemv, sgemv

__all__ = ["sgemv", "hgemv", "bfgemv"]
