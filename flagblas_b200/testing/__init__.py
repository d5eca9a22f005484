"""Tolerance helpers with the reference's table and rule
(``src/flag_blas/testing/__init__.py:37-88``): ``atol = atol * reduce_dim``,
``rtol = RESOLUTION[dtype]``; compares of 1 GiB or more are done on the CPU."""
import torch

RESOLUTION = {
    torch.bool: 0,
    torch.uint8: 0,
    torch.int8: 0,
    torch.int16: 0,
    torch.int32: 0,
    torch.int64: 0,
    torch.float16: 1e-3,
    torch.float32: 1.3e-6,
    torch.bfloat16: 0.016,
    torch.float64: 1e-7,
}

_HUGE = 1 << 30


def _maybe_move_to_cpu(res, ref):
    if not (res.is_cuda and ref.is_cuda):
        return res, ref
    need = res.numel() * res.element_size()
    free = None
    try:
        free, _ = torch.cuda.mem_get_info(res.device)
    except RuntimeError:
        pass
    if (free is not None and need >= free) or need >= _HUGE:
        return res.cpu(), ref.cpu()
    return res, ref


def assert_close(res, ref, dtype, equal_nan=False, reduce_dim=1, atol=1e-4):
    if dtype is None:
        dtype = torch.float32
    assert res.dtype == dtype
    ref = ref.to(dtype)
    res, ref = _maybe_move_to_cpu(res, ref)
    torch.testing.assert_close(res, ref, atol=atol * reduce_dim, rtol=RESOLUTION[dtype], equal_nan=equal_nan)


def assert_equal(res, ref, equal_nan=False):
    torch.testing.assert_close(res, ref, atol=0, rtol=0, equal_nan=equal_nan)
