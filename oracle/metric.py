"""Tolerance metric of the reference's tests (TEST INFRASTRUCTURE ONLY).

Follows ``triton_kernels/testing.py:27-88`` (``assert_close``): both tensors are normalised by
``max|ref|``; the element error is ``|ref - got| / max(rms(ref), |ref|)``; its maximum and its RMS
are compared with ``maxtol`` (default 2e-2) and ``rmstol`` (default 4e-3).
"""
import torch


def rel_errors(ref: torch.Tensor, got: torch.Tensor):
    ref = ref.detach().float().cpu()
    got = got.detach().float().cpu()
    assert ref.shape == got.shape, (ref.shape, got.shape)
    if ref.numel() == 0:
        return 0.0, 0.0
    inf_r, inf_g = torch.isinf(ref), torch.isinf(got)
    assert torch.equal(inf_r, inf_g), "infinite elements differ"
    r = torch.where(inf_r, torch.zeros(()), ref)
    g = torch.where(inf_g, torch.zeros(()), got)
    eps = 1.0e-30
    mult = 1.0 / (r.abs().max() + eps)
    r, g = r * mult, g * mult
    rms = torch.sqrt((r * r).mean()) + eps
    err = (r - g).abs() / torch.maximum(rms, r.abs())
    return err.max().item(), torch.sqrt((err * err).mean()).item()


def rel_l2(ref: torch.Tensor, got: torch.Tensor) -> float:
    ref = ref.detach().double().cpu()
    got = got.detach().double().cpu()
    den = ref.norm().item()
    return (ref - got).norm().item() / (den if den > 0 else 1.0)


def assert_close_oracle(ref, got, maxtol=2e-2, rmstol=4e-3, what=""):
    mx, rms = rel_errors(ref, got)
    assert mx <= maxtol, f"{what}: max relative error {mx} > {maxtol}"
    if rmstol is not None:
        assert rms <= rmstol, f"{what}: rms relative error {rms} > {rmstol}"
