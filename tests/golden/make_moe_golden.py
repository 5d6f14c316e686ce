"""Golden vectors for the MoE routing, produced by EXECUTING THE REFERENCE'S OWN ROUTING LINES.

    python tests/golden/make_moe_golden.py [/path/to/reference]

The reference's ``run()`` (moe/moe_fibench_ref.py) is one function that also dequantises
3.7 GB of FP8 weights, so it cannot be called on small inputs.  This script reads that file,
cuts out the block between its "# 2) No-aux routing" and "# 3) Local expert compute" comments
(lines 106-134) and executes exactly those statements on seeded logits, with the constants the
function defines above them (TOP_K = 8, N_GROUP = 8, TOPK_GROUP = 4).  Output:
tests/golden/moe_routing_vectors.npz with, per case, the logits, the bias, the scaling factor,
the chosen expert ids (sorted per token) and the dense weight matrix.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def routing_block(reference_root):
    path = os.path.join(reference_root, "moe", "moe_fibench_ref.py")
    lines = open(path).read().splitlines()
    start = next(i for i, ln in enumerate(lines) if "# 2) No-aux routing" in ln)
    stop = next(i for i, ln in enumerate(lines) if "# 3) Local expert compute" in ln)
    body = [ln[4:] if ln.startswith("    ") else ln for ln in lines[start:stop]]
    return "\n".join(body)


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(here, "..", "..", "..", "reference")   # beside this repository
    code = compile(routing_block(root), "moe_fibench_ref.py[routing]", "exec")
    out = {}
    cases = [("e256", 57, 256, 0.0, 2.5, 1), ("e256b", 64, 256, 0.1, 1.0, 2), ("e64", 96, 64, 0.05, 2.5, 3)]
    for name, tokens, experts, bias_std, scale, seed in cases:
        gen = torch.Generator().manual_seed(seed)
        logits = torch.randn((tokens, experts), generator=gen)
        bias = torch.randn((experts,), generator=gen) * bias_std
        ns = {"torch": torch, "routing_logits": logits, "routing_bias": bias, "T": tokens, "E_global": experts,
              "TOP_K": 8, "N_GROUP": 8, "TOPK_GROUP": 4, "routed_scaling_factor": scale}
        exec(code, ns)
        out[f"{name}_logits"] = logits.numpy()
        out[f"{name}_bias"] = bias.numpy()
        out[f"{name}_scale"] = np.float32(scale)
        out[f"{name}_topk_sorted"] = np.sort(ns["topk_idx"].numpy(), axis=1)
        out[f"{name}_weights"] = ns["weights"].numpy()
    np.savez_compressed(os.path.join(HERE, "moe_routing_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "moe_routing_vectors.npz"), sorted(out))


if __name__ == "__main__":
    main()
