"""Writes tests/golden/oqpack_toy/ (an OQPack v1 package made by the REFERENCE's own writer) and
tests/golden/oqpack_toy_expected.npz (inputs and the reference modules' CPU outputs).

Run in a checkout that has the reference beside it:
    python tests/golden/make_oqpack_fixture.py /path/to/reference
The package pins this repository's loader (ojasx-vector-24x96_b200/oqpack.py) to the real container:
manifest keys, shard naming, tensor names, dtypes and shapes are whatever ojasx_24x96.oqpack.save_oqpack
(ojasx_24x96/oqpack.py:383-546) wrote.
"""
import os
import shutil
import sys

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from ojasx_24x96 import codec, module, oqpack

    torch.manual_seed(20261104)

    class Toy(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(64, 96, bias=True)     # 8-bit, one stage: the split-manifold layout
            self.b = nn.Linear(96, 32, bias=False)    # 8-bit, one stage, no bias
            self.c = nn.Linear(64, 48, bias=True)     # 4-bit, two stages: the generic residual-VQ layout

    m = Toy()
    cfgs = {
        "a": codec.QuantizationConfig(block_size=8, bits_per_stage=8, max_stages=1, max_relative_error=10.0,
                                      kmeans_iterations=3, min_weight_elements=16, require_compression=False),
        "b": codec.QuantizationConfig(block_size=16, bits_per_stage=8, max_stages=1, max_relative_error=10.0,
                                      kmeans_iterations=3, min_weight_elements=16, require_compression=False),
        "c": codec.QuantizationConfig(block_size=8, bits_per_stage=4, max_stages=2, max_relative_error=10.0,
                                      kmeans_iterations=3, min_weight_elements=16, require_compression=False),
    }
    for name, cfg in cfgs.items():
        lin = getattr(m, name)
        q, report = codec.quantize_weight(lin.weight.detach(), cfg)
        if name == "c":   # the encoder keeps the fewest stages that meet the budget: put the budget between stage 1 and 2
            e = report["stage_relative_errors"]
            import dataclasses
            q, report = codec.quantize_weight(lin.weight.detach(), dataclasses.replace(cfg, max_relative_error=(e[0] + e[1]) / 2))
        assert q is not None, (name, report)
        bias = lin.bias.detach() if lin.bias is not None else None
        setattr(m, name, module.ResidualVQLinear.from_encoded(q, bias=bias, source_dtype=torch.float32,
                                                              device=torch.device("cpu")))
    out_dir = os.path.join(HERE, "oqpack_toy")
    shutil.rmtree(out_dir, ignore_errors=True)
    oqpack.save_oqpack(m, out_dir, model_id="toy")
    oqpack.verify_oqpack_integrity(out_dir)
    expected = {}
    with torch.no_grad():
        for name in cfgs:
            layer = getattr(m, name)
            x = torch.randn(3, layer.in_features)
            expected[f"{name}_x"] = x.numpy()
            expected[f"{name}_y"] = layer(x).numpy()
            expected[f"{name}_stages"] = np.int64(layer.encoded().stages)
    np.savez(os.path.join(HERE, "oqpack_toy_expected.npz"), **expected)
    print("wrote", out_dir, {k: v.shape for k, v in expected.items() if hasattr(v, "shape")})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
