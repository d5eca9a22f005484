"""The sliver of ``flag_blas.runtime`` that callers of the GEMM path touch
(reference: ``src/flag_blas/runtime/backend/device.py:56-159``): a ``device``
object naming the one supported back end and its dtype support flags.  The
reference's vendor / architecture detection and operator-override machinery is
deliberately absent: this package is sm_100a only."""
import torch


class _Device:
    name = "cuda"
    vendor_name = "nvidia"
    support_fp64 = True
    support_bf16 = True
    support_int64 = True

    @property
    def device_count(self):
        return torch.cuda.device_count()


device = _Device()
torch_device_fn = torch.cuda
