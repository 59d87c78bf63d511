"""B200-native FP8 (e4m3fn) block-scaled GEMM behind the reference's operator surface.

``custom_kernel((a, b, a_scale, b_scale, c)) -> c`` mirrors
1-amd-fp8-mm/amd-fp8-mm-submission.py:594-604 of the reference; the work is done by
hand-written sm_100a CUDA kernels in ``lib/libb200fp8mm.so`` reached through a C ABI
(``include/b200_fp8_mm.h``). There is no CPU or library fallback: if the shared
library is missing the import of ``_lib`` raises.
"""
from .fp8_mm import Plan, describe, estimate_clocks, fp8_mm, fp8_mm_grouped, fp8_mm_host, workspace_bytes  # noqa: F401
from .inputs import make_inputs  # noqa: F401
from .mla import div_softmax, kv_down_projection_fp8, mla_decode  # noqa: F401
from .sharding import (GridSpec, ShardSpec, choose_grid, gather_c, grid_inputs, grid_spec, shard_inputs,  # noqa: F401
                       shard_spec)
from .submission import custom_kernel  # noqa: F401
