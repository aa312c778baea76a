"""b200k — B200 (sm_100a) kernels behind the entry points of the cuTile samples.

Importing this package needs only torch; the first operator call loads
``libb200k.so`` (built by ``cutile-python_b200/build.py``) and raises if it is missing.
"""
from ._lib import B200KError, device_status, raise_on_device_error  # noqa: F401
from .matmul import (bmm, cutile_batch_matmul, cutile_group_matmul, cutile_matmul,  # noqa: F401
                     cutile_persistent_matmul)
from .block_scaled import (block_quantize, cutile_block_scaled_matmul,  # noqa: F401
                           cutile_nvfp4_matmul, cutile_swizzled_scaled_matmul, nvfp4_quantize,
                           swizzle_32_4_4)
from .fmha import cutile_fmha, cutile_fmha_into  # noqa: F401
from .moe import (cutile_moe, cutile_moe_mxfp8, invoke_fused_moe_kernel,  # noqa: F401
                  invoke_silu_and_mul_kernel, moe_align_device, moe_align_tile_size_torch,
                  quantize_expert_weights)
from .allgather import (Nvfp4GatherMatmul, cutile_gather_matmul, cutile_gather_matmul_nvfp4, peer_buffers,  # noqa: F401
                        peer_gather, shard_rows)
from .moe_ep import ExpertParallelMoE, emulate_ranks  # noqa: F401
from . import tune  # noqa: F401
