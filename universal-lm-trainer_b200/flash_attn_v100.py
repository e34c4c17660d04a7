"""Same public signature as the reference's flash_attn_v100.py:391-396 (its
Triton variant), served by the sm_100a CUDA library: there is no Triton path."""
from flash_attn_v100_cuda import flash_attn_v100, _FlashAttnV100Cuda as _FlashAttnV100  # noqa: F401

__all__ = ['flash_attn_v100']
