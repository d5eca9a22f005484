from .gemv import bfgemv, fp8_gemv, hgemv, sgemv

__all__ = ["sgemv", "hgemv", "bfgemv", "fp8_gemv"]
