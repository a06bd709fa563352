"""Generates the golden fixtures in this directory by running the UNMODIFIED
reference module (models/moe.py: LatentMoELayer, and MoELayer for the tiny_moe* fixtures) on CPU in fp32 through
oracle/ref_shim.py.  Needs the reference source tree; run from the repo root:

    python tests/golden/make_golden.py

Each fixture holds digests of the seeded inputs (to detect RNG drift), the
integer routing results in full, and the float results either in full (small
tensors) or as a strided sample plus norms.
"""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import inputs, ref_shim  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SAMPLE = 4096


def digest(t: torch.Tensor) -> dict:
    """Strided sample + norms of a float tensor (full tensor when small)."""
    flat = t.detach().reshape(-1).to(torch.float32)
    step = max(1, flat.numel() // SAMPLE)
    return dict(shape=tuple(t.shape), step=step, sample=flat[::step].clone(),
                sum=flat.double().sum().item(), l2=flat.double().pow(2).sum().sqrt().item())


def make(name: str, backward: bool):
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w)
    out, grads, layer = ref_shim.run_reference(w, params, buffers, x, dy if backward else None, aux_grad=1.0)
    # canonical routing from the reference's own pieces, for the integer fixtures
    counts, offsets, perm = ref_shim._routing_shim(out["sel"], w.E)
    fx = dict(
        workload=name, seed=0, torch_version=torch.__version__,
        inputs={k: digest(v) for k, v in list(params.items()) + [("x", x)]},
        sel=out["sel"].to(torch.int16), counts=counts.to(torch.int32), offsets=offsets.to(torch.int32),
        perm=perm.to(torch.int32), aux_loss=out["aux_loss"].item(), y=digest(out["y"]),
    )
    if backward:
        fx["grads"] = {k: digest(v) for k, v in grads.items()}
        fx["aux_grad"] = 1.0
    # the bias update that follows backward (models/moe.py:244-275)
    layer.router.update_bias_from_last_forward()
    fx["expert_bias_after_update"] = layer.router.expert_bias.clone()
    fx["load_history_after_update"] = layer.router.load_history.clone()
    path = os.path.join(HERE, f"{name}.pt")
    torch.save(fx, path)
    print(name, os.path.getsize(path), "bytes")


def make_rmsnorm():
    """Reference RMSNorm (models/normalization.py:13-39) forward and backward in fp32 on seeded inputs."""
    models_dir = os.path.join(ref_shim.REFERENCE_ROOT, "models")
    if models_dir not in sys.path:
        sys.path.insert(0, models_dir)
    from normalization import RMSNorm  # the reference class, unmodified
    g = torch.Generator().manual_seed(11)
    T, D = 37, 256
    x = torch.randn(T, D, generator=g).requires_grad_(True)
    w = (1.0 + 0.1 * torch.randn(D, generator=g))
    dy = torch.randn(T, D, generator=g)
    norm = RMSNorm(D, eps=1e-6)
    with torch.no_grad():
        norm.weight.copy_(w)
    y = norm(x)
    (y * dy).sum().backward()
    fx = dict(seed=11, T=T, D=D, eps=1e-6, y=y.detach().clone(), dx=x.grad.clone(), dw=norm.weight.grad.clone(),
              x_l2=x.detach().double().pow(2).sum().sqrt().item())
    path = os.path.join(HERE, "rmsnorm.pt")
    torch.save(fx, path)
    print("rmsnorm", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if not ref_shim.available():
        sys.exit("reference tree not found; fixtures can only be regenerated where it is present")
    make("tiny", True)
    make("tiny_ragged", True)
    make("tiny_shared2", True)       # two shared experts
    make("cfg1", False)
    make("tiny_moe", True)           # the non-latent MoELayer (models/moe.py:294-559)
    make("tiny_moe_ragged", True)
    make_rmsnorm()
