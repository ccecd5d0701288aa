"""b200k: sm_100a kernels for GEMM, attention and (paged) decode attention behind the
iree-turbine operator surface.  Importing the package registers ``torch.ops.b200k.*``.

The directory name contains a hyphen; import it as ``iree_turbine_b200`` (a one-file alias
package beside it forwards to this directory).
"""

from . import op_reg, shapes  # noqa: F401
from .op_reg import CustomOp, KernelSelection, def_library  # noqa: F401
from .shapes import AttentionShape, DecodeShape, GemmShape  # noqa: F401
from . import ops  # noqa: F401  (registers the op library)
from .ops import device_status, reset_device_status  # noqa: F401
from .templates import (  # noqa: F401
    LaunchableKernel,
    get_causal_attention_kernel,
    get_decode_attention_kernel,
    get_fp8_gemm_kernel,
    get_gemm_kernel,
    get_kv_append_kernel,
    get_paged_decode_attention_kernel,
    get_paged_prefill_attention_kernel,
    get_vanilla_attention_kernel,
)

__version__ = "0.1.0"
