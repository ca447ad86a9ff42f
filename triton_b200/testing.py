"""Comparison helpers with the reference's tolerance metric (triton_kernels/testing.py:18-88)."""
import torch


def assert_equal(ref, tri):
    if isinstance(ref, torch.Tensor):
        assert torch.all(ref == tri)
    else:
        assert ref == tri


def assert_close(ref, tri, maxtol=None, rmstol=None, description="--", verbose=True):
    """Both tensors are normalised by max|ref|; the element error is |ref - tri| / max(rms(ref), |ref|);
    its maximum must stay below `maxtol` (default 2e-2) and its RMS below `rmstol` (default 4e-3)."""
    if tri.dtype.itemsize == 1:
        ref_as_type = ref.to(tri.dtype)
        if ref.dtype == tri.dtype:
            assert torch.all(ref_as_type == tri)
            return
        ref = ref_as_type
    if ref.numel() == 0:
        return
    maxtol = 2e-2 if maxtol is None else maxtol
    rmstol = 4e-3 if rmstol is None else rmstol
    ref = ref.to(torch.float32).detach()
    tri = tri.to(torch.float32).detach()
    assert ref.shape == tri.shape, f"Tensors must have same size {ref.shape=} {tri.shape=}"
    inf_ref, inf_tri = torch.isinf(ref), torch.isinf(tri)
    assert torch.equal(inf_ref, inf_tri), "Tensor must have same infinite elements"
    refn = torch.where(inf_ref, 0, ref)
    trin = torch.where(inf_tri, 0, tri)
    eps = 1.0e-30
    mult = 1.0 / (torch.max(torch.abs(refn)) + eps)
    refn, trin = refn * mult, trin * mult
    ref_rms = torch.sqrt(torch.square(refn).mean()) + eps
    rel_err = torch.abs(refn - trin) / torch.maximum(ref_rms, torch.abs(refn))
    max_err = torch.max(rel_err).item()
    rms_err = torch.sqrt(torch.square(rel_err).mean()).item()
    if verbose:
        print(f"{description} maximum relative error = {max_err} (threshold = {maxtol})")
        print(f"{description} RMS relative error = {rms_err} (threshold = {rmstol})")
    assert max_err <= maxtol
    assert rms_err <= rmstol
