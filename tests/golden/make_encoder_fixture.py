"""Writes tests/golden/encoder_ref.npz: a seeded dense weight and what the REFERENCE's own encoder
(SplitManifoldLUTLinear.from_dense, split_manifold_lut_experiment/engine/split_manifold_engine.py:90-183,
run on the CPU) makes of it, plus that layer's forward output on a seeded input.

    python tests/golden/make_encoder_fixture.py /path/to/reference
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(reference_root: str) -> None:
    sys.path.insert(0, os.path.join(reference_root, "split_manifold_lut_experiment"))
    from engine.split_manifold_engine import SplitManifoldLUTLinear

    out = {}
    for tag, (M, K, D) in {"d16": (64, 256, 16), "d8": (96, 256, 8)}.items():
        g = torch.Generator().manual_seed(20261104 + D)
        W = torch.randn(M, K, generator=g) * 0.02
        # heavy-tailed cells so that the 3.5-sigma rule finds outliers, as in LLM weights
        hot = torch.rand(M, K, generator=g) < 0.004
        W = torch.where(hot, W * 12.0, W)
        bias = torch.randn(M, generator=g) * 0.01
        layer = SplitManifoldLUTLinear.from_dense(W, bias, block_dim=D, codebook_size=256, outlier_tau=3.5)
        x = torch.randn(3, K, generator=g)
        with torch.no_grad():
            y = layer(x)
        out.update({f"{tag}_W": W.numpy(), f"{tag}_bias": bias.numpy(), f"{tag}_x": x.numpy(), f"{tag}_y": y.float().numpy(),
                    f"{tag}_codebook": layer.codebook.float().numpy(), f"{tag}_codes": layer.codes.numpy(),
                    f"{tag}_scales": layer.scales.float().numpy(),
                    f"{tag}_outlier_indices": layer.outlier_indices.numpy(), f"{tag}_outlier_values": layer.outlier_values.float().numpy()})
        print(tag, "outliers", layer.num_outliers, "max |y - x W^T - b|", float((y - (x @ W.t() + bias)).abs().max()))
    np.savez_compressed(os.path.join(HERE, "encoder_ref.npz"), **out)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
