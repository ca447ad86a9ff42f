"""`routing()`: the composition the reference's earlier API exposed under this name, written out in
its tests today (python/triton_kernels/tests/test_distributed.py:203-210)."""
import torch

from .tensor import make_ragged_tensor_metadata
from .topk import topk


def routing(logits, n_expts_act, all_gather=False, y_indx=None, symm_mem_pool=None, apply_softmax=True):
    """-> (ragged_metadata, gather_idx, scatter_idx, sparse_logits).

    gather_idx[p] is the token whose activations feed expert-sorted row p, scatter_idx[p] the flat
    (token * k + slot) row its output goes to; sparse_logits.vals holds the routing weights."""
    sparse = topk(logits, n_expts_act, apply_softmax=apply_softmax, all_gather=all_gather, y_indx=y_indx,
                  symm_mem_pool=symm_mem_pool)
    dispatch_indx = sparse.mask_metadata.row_sorted_indx
    combine_indx = sparse.mask_metadata.col_sorted_indx
    ragged = make_ragged_tensor_metadata(sparse.mask_metadata.col_sum, dispatch_indx.shape[0])
    gather_idx = torch.div(combine_indx, n_expts_act, rounding_mode="trunc")
    scatter_idx = combine_indx
    return ragged, gather_idx, scatter_idx, sparse
