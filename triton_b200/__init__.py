"""triton_b200: the MoE hot path of triton_kernels (routing, ragged grouped GEMM bf16 x MXFP4 with
fused bias / SwiGLU / routing-weight epilogue, combine, MXFP4 quantise / dequantise, expert-parallel
dispatch / combine) as hand-written CUDA for sm_100a behind a C ABI (include/moe_b200.h).

Importing the package does not need a GPU; calling an operator does, and needs libmoe_b200.so
(``python -m triton_b200.build``).  There is no fallback path."""
from . import _lib  # noqa: F401
from .matmul import (Epilogue, FlexCtx, FnName, FusedActivation, FusedComm, InapplicableConstraint, PrecisionConfig,  # noqa: F401
                     matmul, matmul_check_status, matmul_ogs, matmul_set_idle_sms, reset_opt_flags_constraints,
                     scoped_opt_flags_constraints, update_opt_flags_constraints)
from .numerics import InFlexData, OutFlexData  # noqa: F401
from .numerics_details.mxfp import DequantScaleRoundingMode, downcast_to_mxfp, upcast_from_mxfp  # noqa: F401
from .reduce import reduce  # noqa: F401
from .router import prepare_router_weight, router_topk  # noqa: F401
from .routing import routing  # noqa: F401
from .specialize import FnSpecs  # noqa: F401
from .swiglu import swiglu, swiglu_fn  # noqa: F401
from .tensor import (FP4, BitmatrixMetadata, RaggedTensorMetadata, SparseMatrix, Storage, Tensor,  # noqa: F401
                     convert_layout, make_bitmatrix_metadata, make_ragged_tensor_metadata,
                     remap_ragged_tensor_metadata, wrap_torch_tensor)
from .topk import topk  # noqa: F401
from .weights_io import from_block_checkpoint, load_layer_weights, save_layer_weights  # noqa: F401
from .distributed import (ExptAssignment, Mesh, SymmetricMemoryPool, convert_dp_to_ep, convert_ep_to_dp,  # noqa: F401
                          make_expt_assignment, make_expt_dict_balanced, make_expt_dict_random,
                          make_expt_dict_uniform)
