"""Generate the golden fixtures in this directory from the reference's own PyTorch code.

Run once, on a CPU, in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/ResidualQuant

It imports scripts/calibration/{quantization,rotation_math,rotation_training}.py from the reference
(nothing is copied), feeds them the seeded inputs of `residualquant_b200.synth`, and stores only the
reference's OUTPUTS; the tests regenerate the inputs from the same seeds.

Fixtures:
  gq_d{D}.npz      affine_qdq (identity rotation; with and without a mean) for INT2 g16, INT2 g32, INT4 g32:
                   bf16 bit patterns of the dequantized rows.  Pins the group quantizer bit-for-bit.
  chain_d{D}_g{g}.npz   FP32Chain([2,2,2,4], "anchor", anchor_index=3).reconstruct for K and V with a
                   signed-Hadamard rotation, and the decode attention (probabilities + p@V) per loop with the
                   last token live.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from residualquant_b200 import synth  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def gq_inputs(dim):
    rng = np.random.default_rng(100 + dim)
    x = synth.loop_rows(rng, 48, 2, dim)[3]
    mean = (0.3 * rng.standard_normal((2, dim))).astype(np.float32)
    return x, mean


def chain_inputs(dim, group, tokens=40, heads=2):
    rng = np.random.default_rng(1000 * dim + group)
    k = synth.loop_rows(rng, tokens, heads, dim)
    v = synth.loop_rows(rng, tokens, heads, dim)
    sg = synth.signs(rng, heads, dim)
    q = synth.to_bf16_f32(rng.standard_normal((1, heads, dim)).astype(np.float32))
    return k, v, sg, q


def main(reference_root):
    sys.path.insert(0, os.path.join(reference_root, "scripts"))
    from calibration.quantization import affine_qdq
    from calibration.rotation_math import hadamard, probabilities
    from calibration.rotation_training import FP32Chain

    torch.set_grad_enabled(False)
    for dim in (128, 96):
        x, mean = gq_inputs(dim)
        xb = torch.from_numpy(x).bfloat16()
        eye = torch.eye(dim).expand(2, dim, dim).contiguous()
        out = {}
        for b, g in ((2, 16), (2, 32), (4, 32)):
            out[f"plain_{b}_{g}"] = bits(affine_qdq(xb, eye, b, g))
            out[f"mean_{b}_{g}"] = bits(affine_qdq(xb, eye, b, g, mean=torch.from_numpy(mean)))
        np.savez_compressed(os.path.join(HERE, f"gq_d{dim}.npz"), **out)

        for group in (32, 16):
            k, v, sg, q = chain_inputs(dim, group)
            tokens = k[0].shape[0]
            rotation = (torch.from_numpy(sg).float()[:, :, None] * hadamard("cpu", dim)[None]).half().float().contiguous()
            chain = FP32Chain([2, 2, 2, 4], "anchor", [group, group, group, 32], anchor_index=3)
            sample = [{"k": torch.from_numpy(a).bfloat16(), "v": torch.from_numpy(b).bfloat16()} for a, b in zip(k, v)]
            k_hat = chain.reconstruct(sample, "k", [rotation], None)
            v_hat = chain.reconstruct(sample, "v", [rotation], None)
            out = {"rscale": np.float32(rotation.abs().max().item())}
            qt = torch.from_numpy(q).bfloat16()
            for loop in range(4):
                out[f"k_hat_{loop}"] = bits(k_hat[loop])
                out[f"v_hat_{loop}"] = bits(v_hat[loop])
                # decode contract: tokens 0..T-2 come from the cache, the last token is live (raw bf16)
                kc = torch.cat([k_hat[loop][: tokens - 1], sample[loop]["k"][tokens - 1:].float()])
                vc = torch.cat([v_hat[loop][: tokens - 1], sample[loop]["v"][tokens - 1:].float()])
                p = probabilities(qt, kc, torch.tensor([tokens - 1]), head_dim=dim)
                out[f"attn_{loop}"] = torch.bmm(p, vc.float().transpose(0, 1)).squeeze(1).numpy().astype(np.float32)
            np.savez_compressed(os.path.join(HERE, f"chain_d{dim}_g{group}.npz"), **out)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference repository>")
    main(sys.argv[1])
