"""Shared fixtures.  Tests that need a B200 carry ``@pytest.mark.gpu``; everything else runs on CPU."""
import pathlib
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name):
    """Fixture record written by tests/golden/make_golden.py plus its regenerated inputs."""
    from oracle import moe_oracle as orc
    rec = torch.load(GOLDEN / f"{name}.pt", weights_only=True)
    inp = orc.make_inputs(rec["n_tokens"], rec["hidden"], rec["inter"], rec["n_experts"],
                          seed=rec["seed"], bias_mode=rec["bias_mode"], theta_std=rec["theta_std"])
    n_glu = rec["n_glu"]
    for k in ("gate_up_proj", "down_proj", "radial_theta"):
        inp[k] = inp[k][:n_glu].contiguous()
    return rec, inp


def upstream_grad(rec):
    g = torch.Generator().manual_seed(rec["seed"] * 1000 + 77)
    return torch.randn(1, rec["n_tokens"], rec["hidden"], generator=g)[0]


def grad_digest(g, seed):
    probe = torch.randn(g.shape, generator=torch.Generator().manual_seed(seed * 1000 + 99))
    flat, pf = g.reshape(g.shape[0], -1).double().cpu(), probe.reshape(g.shape[0], -1).double()
    return torch.stack([flat.norm(dim=1), (flat * pf).sum(1)], dim=1)


def digest_close(dig, ref, tol):
    """Norm column within ``tol`` relative; probe column within ``tol`` of the norm (the probe is
    N(0,1), so the inner product has the norm's scale and may itself be near zero)."""
    scale = ref[:, 0].clamp_min(1e-30)
    return bool((((dig[:, 0] - ref[:, 0]).abs() / scale) < tol).all()
                and (((dig[:, 1] - ref[:, 1]).abs() / scale) < 4 * tol).all())


def rel_err(a, b):
    """max |a-b| / max |b| -- the reference tests' own relative-error definition."""
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def mean_rel_err(a, b):
    return float((a.double() - b.double()).abs().mean() / b.double().abs().mean().clamp_min(1e-30))


GOLDEN_CASES = ["tiny_glu", "tiny_specials", "tiny_softmax", "tiny_raw", "e64_k6_fp32"]
