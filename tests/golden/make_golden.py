"""Generate the golden fixtures in this directory from the reference implementation itself.

Run where a checkout of the reference (MOLT 0.12.0) is available:

    python tests/golden/make_golden.py --reference /path/to/MOLT

The script imports ``molt_stream`` from ``<reference>/src`` (CPU only), runs the
reference's own NF4 quantiser / dequantiser, its eager NF4-LoRA autograd
function and its SwiGLU CPU branch on small seeded inputs, and stores inputs and
outputs as ``.npz`` files.  The fixtures travel with the repository; the
reference does not.  bf16 tensors are stored as their int16 bit patterns.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", required=True, help="root of the reference checkout")
    args = parser.parse_args()
    src = Path(args.reference).resolve() / "src"
    sys.path.insert(0, str(src))
    # Some reference modules create a compiler-cache directory in the CWD at import.
    os.chdir(tempfile.mkdtemp(prefix="molt_golden_"))
    torch.set_num_threads(1)  # deterministic reduction order for the fp32 fixtures

    from molt_stream.streaming.nf4 import NF4_CODEBOOK, NF4Tensor
    from molt_stream.streaming.engine import StreamedLoRALinear
    from molt_stream.kernels.gated_activation import fused_silu_multiply
    from molt_stream.kernels.frozen_rmsnorm import _FrozenRMSNormFunction

    sys.path.insert(0, str(HERE.parents[1]))
    from oracle.molt_oracle import NF4_CODEBOOK as ORACLE_CODEBOOK

    assert torch.equal(NF4_CODEBOOK, ORACLE_CODEBOOK), "codebook differs from the reference"
    np.savez(HERE / "nf4_codebook.npz", codebook=NF4_CODEBOOK.numpy())

    # ---- NF4 quantise / dequantise -------------------------------------------------------
    cases = [  # (name, shape, block, seed, std)
        ("q_8x8_b16", (8, 8), 16, 3, 1.0),
        ("q_64x64_b64", (64, 64), 64, 1, 1.0),
        ("q_70x65_b64", (70, 65), 64, 942, 1.0),
        ("q_96x64_b64", (96, 64), 64, 941, 0.02),
        ("q_48x1536_b64", (48, 1536), 64, 1337, 0.02),
        ("q_33x50_b32", (33, 50), 32, 7, 0.5),
    ]
    for name, shape, block, seed, std in cases:
        gen = torch.Generator().manual_seed(seed)
        value = torch.randn(*shape, generator=gen) * std
        q = NF4Tensor.quantize(value, block_size=block)
        np.savez_compressed(
            HERE / f"{name}.npz",
            value=value.numpy(), packed=q.packed.numpy(), scales=q.scales.numpy(),
            shape=np.array(shape), block=np.array(block), elements=np.array(q.elements),
            deq_f32=q.dequantize(dtype=torch.float32).numpy(),
            deq_bf16_bits=_bits(q.dequantize(dtype=torch.bfloat16)),
            storage_bytes=np.array(q.storage_bytes),
        )

    # ---- eager NF4-LoRA forward + backward ----------------------------------------------
    lin_cases = [  # (name, N, K, M, rank, alpha, block, seed)
        ("lin_8x8_r2", 8, 8, 2, 2, 4.0, 16, 3),
        ("lin_96x64_r8", 96, 64, 32, 8, 16.0, 64, 941),
        ("lin_70x65_r7", 70, 65, 5, 7, 0.875, 64, 943),
        ("lin_256x128_r16", 256, 128, 48, 16, 32.0, 64, 1337),
    ]
    for name, n, k, m, rank, alpha, block, seed in lin_cases:
        gen = torch.Generator().manual_seed(seed)
        w = torch.randn(n, k, generator=gen) * 0.02
        a = torch.randn(rank, k, generator=gen) * 0.01
        b = torch.randn(n, rank, generator=gen) * 0.01
        x = torch.randn(m, k, generator=gen).bfloat16().float()
        dy = torch.randn(m, n, generator=gen).bfloat16().float()
        q = NF4Tensor.quantize(w, block_size=block)
        module = StreamedLoRALinear(q, rank=rank, alpha=alpha, device=torch.device("cpu"))
        with torch.no_grad():
            module.lora_a.copy_(a)
            module.lora_b.copy_(b)
        xin = x.clone().requires_grad_(True)
        y = module(xin, q.dequantize())
        y.backward(dy)
        np.savez_compressed(
            HERE / f"{name}.npz",
            w=w.numpy(), a=a.numpy(), b=b.numpy(), x=x.numpy(), dy=dy.numpy(),
            packed=q.packed.numpy(), scales=q.scales.numpy(), block=np.array(block),
            scaling=np.array(module.scaling), y=y.detach().numpy(), dx=xin.grad.numpy(),
            da=module.lora_a.grad.numpy(), db=module.lora_b.grad.numpy(),
        )

    # ---- SwiGLU (CPU branch of the reference's fused op) ---------------------------------
    for name, shape, seed, dtype in [("swiglu_3x5x17_f32", (3, 5, 17), 3401, torch.float32),
                                     ("swiglu_2x31x128_bf16", (2, 31, 128), 3402, torch.bfloat16)]:
        gen = torch.Generator().manual_seed(seed)
        gate = torch.randn(*shape, generator=gen).to(dtype).requires_grad_(True)
        up = torch.randn(*shape, generator=gen).to(dtype).requires_grad_(True)
        grad = torch.randn(*shape, generator=gen).to(dtype)
        out = fused_silu_multiply(gate, up)
        out.backward(grad)
        np.savez_compressed(
            HERE / f"{name}.npz",
            gate=gate.detach().float().numpy(), up=up.detach().float().numpy(), grad=grad.float().numpy(),
            out=out.detach().float().numpy(), dgate=gate.grad.float().numpy(), dup=up.grad.float().numpy(),
        )

    # ---- frozen RMSNorm (norm-replay recipe arithmetic) ----------------------------------
    gen = torch.Generator().manual_seed(77)
    hidden = torch.randn(6, 96, generator=gen).bfloat16().requires_grad_(True)
    weight = (torch.randn(96, generator=gen) * 0.1 + 1.0)
    grad = torch.randn(6, 96, generator=gen).bfloat16()
    out = _FrozenRMSNormFunction.apply(hidden, weight, 1e-6, 0.0)
    out.backward(grad)
    np.savez_compressed(
        HERE / "rmsnorm_6x96.npz",
        hidden=hidden.detach().float().numpy(), weight=weight.numpy(), grad=grad.float().numpy(),
        out_bits=_bits(out.detach()), dhidden_bits=_bits(hidden.grad), eps=np.array(1e-6),
    )
    print("fixtures written to", HERE)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
