"""OQPack v1 packages read straight into device memory.

The container is the reference's (``ojasx_24x96/oqpack.py``): a directory with ``oqpack_manifest.json``
(``shards`` with file name, SHA-256 and size; ``tensors`` name -> shard, dtype, shape; ``layer_specs``
module path -> geometry, ``:218-276``) and safetensors shards whose tensors carry the state-dict names of
the quantised modules: ``<path>.packed_codes`` u8 ``[stages, ceil(M*G*bits/8)]``, ``<path>.codebooks`` f32
``[stages, 2^bits, D]``, ``<path>.row_scales`` f32 ``[M]`` and ``<path>.bias``.  Optional CSR outliers use
``<path>.csr_row_ptrs`` i32 ``[M+1]``, ``<path>.csr_col_indices`` i32 ``[nnz]`` and ``<path>.csr_values`` f32
``[nnz]`` (an extension of this package: the reference container has no outlier tensors).

``load_quantized_layers`` opens each shard once with safetensors on the target device and wraps the tensors
as they are: 8-bit single-stage layers are already in the layout of the table kernels, so nothing is
unpacked or repacked (the reference loader goes through ``load_state_dict`` on the host,
``ojasx_24x96/oqpack.py:640-720``).  Layers in a codec this package does not execute (the Leech-lattice
codec, rotations, gain bits) are reported, not loaded.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .codec import QuantizedWeight
from .module import ResidualVQLinear

MANIFEST_FILENAME = "oqpack_manifest.json"
_LINEAR_TYPES = {"linear", "residual_vq_linear"}


class OQPackValidationError(ValueError):
    """Same name as the reference's error (``ojasx_24x96/oqpack.py:42``)."""


def read_manifest(package_dir: str) -> Dict[str, object]:
    path = os.path.join(package_dir, MANIFEST_FILENAME)
    if not os.path.isfile(path):
        raise OQPackValidationError(f"OQPack manifest not found: {path}")
    with open(path, "r", encoding="utf-8") as f:
        manifest = json.load(f)
    for key in ("format_version", "shards", "tensors", "layer_specs"):
        if key not in manifest:
            raise OQPackValidationError(f"OQPack manifest lacks '{key}'")
    return manifest


def verify_oqpack_integrity(package_dir: str, *, verify_checksums: bool = True) -> Dict[str, object]:
    """Shard files exist with the recorded size (and SHA-256), and every tensor names a listed shard."""
    manifest = read_manifest(package_dir)
    listed = set()
    for entry in manifest["shards"]:
        path = os.path.join(package_dir, entry["filename"])
        if not os.path.isfile(path):
            raise OQPackValidationError(f"Missing shard: {entry['filename']}")
        if os.path.getsize(path) != int(entry["size_bytes"]):
            raise OQPackValidationError(f"Shard size mismatch: {entry['filename']}")
        if verify_checksums:
            h = hashlib.sha256()
            with open(path, "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    h.update(chunk)
            if h.hexdigest() != entry["sha256"]:
                raise OQPackValidationError(f"Shard checksum mismatch: {entry['filename']}")
        listed.add(entry["filename"])
    for name, rec in manifest["tensors"].items():
        if rec["shard"] not in listed:
            raise OQPackValidationError(f"Tensor {name} names an unlisted shard {rec['shard']}")
    return manifest


def supported_layer(spec: Dict[str, object]) -> Optional[str]:
    """None when this package executes the layer, else the reason it does not."""
    kind = spec.get("module_type") or spec.get("type")
    if kind not in _LINEAR_TYPES:
        return f"module type {kind}"
    if str(spec.get("codec", "adaptive_residual_vq")) != "adaptive_residual_vq":
        return f"codec {spec.get('codec')}"
    if int(spec.get("rotation_reflections", 0)) != 0:
        return "rotated input basis"
    if int(spec.get("gain_bits", 0)) != 0:
        return "gain bits"
    if int(spec.get("bits_per_stage", 0)) not in (1, 2, 4, 8):
        return f"{spec.get('bits_per_stage')}-bit codes"
    return None


def _tensor_names(layer: str, spec: Dict[str, object], tensors: Dict[str, object]) -> List[str]:
    names = [f"{layer}.packed_codes", f"{layer}.codebooks", f"{layer}.row_scales"]
    if spec.get("has_bias", spec.get("bias", False)):
        names.append(f"{layer}.bias")
    names += [n for n in (f"{layer}.csr_row_ptrs", f"{layer}.csr_col_indices", f"{layer}.csr_values") if n in tensors]
    return names


def load_quantized_layers(package_dir: str, device="cuda", names: Optional[Iterable[str]] = None, *,
                          verify_checksums: bool = False) -> Tuple[Dict[str, ResidualVQLinear], Dict[str, str]]:
    """``(layers, skipped)``: module path -> ``ResidualVQLinear`` on ``device``, and path -> reason for the rest."""
    from safetensors import safe_open

    manifest = verify_oqpack_integrity(package_dir, verify_checksums=verify_checksums)
    tensors, specs = manifest["tensors"], manifest["layer_specs"]
    wanted = set(names) if names is not None else None
    device = torch.device(device)
    plan: Dict[str, List[str]] = {}          # shard -> tensor names to read from it
    chosen: Dict[str, Dict[str, object]] = {}
    skipped: Dict[str, str] = {}
    for layer, spec in specs.items():
        if wanted is not None and layer not in wanted:
            continue
        why = supported_layer(spec)
        if why is not None:
            skipped[layer] = why
            continue
        chosen[layer] = spec
        for tname in _tensor_names(layer, spec, tensors):
            if tname not in tensors:
                raise OQPackValidationError(f"Tensor {tname} of layer {layer} is not in the manifest")
            plan.setdefault(tensors[tname]["shard"], []).append(tname)
    loaded: Dict[str, torch.Tensor] = {}
    for shard, tnames in plan.items():
        with safe_open(os.path.join(package_dir, shard), framework="pt", device=str(device)) as f:
            for tname in tnames:
                loaded[tname] = f.get_tensor(tname)
    layers: Dict[str, ResidualVQLinear] = {}
    for layer, spec in chosen.items():
        rows, cols = int(spec["out_features"]), int(spec["in_features"])
        codes, books, scales = (loaded[f"{layer}.{k}"] for k in ("packed_codes", "codebooks", "row_scales"))
        if books.shape[0] != int(spec["stages"]) and int(spec["stages"]) > 0 and not spec.get("adaptive_stages", True):
            raise OQPackValidationError(f"Layer {layer}: {books.shape[0]} codebooks for {spec['stages']} stages")
        outliers = None
        if f"{layer}.csr_values" in loaded:
            outliers = (loaded[f"{layer}.csr_row_ptrs"].to(torch.int32), loaded[f"{layer}.csr_col_indices"].to(torch.int32),
                        loaded[f"{layer}.csr_values"].to(torch.float32))
        enc = QuantizedWeight((rows, cols), int(spec["block_size"]), int(spec["bits_per_stage"]), codes.contiguous(),
                              books.to(torch.float32).contiguous(), scales.to(torch.float32).contiguous(), {},
                              outliers=outliers)
        layers[layer] = ResidualVQLinear(enc, loaded.get(f"{layer}.bias"))
    return layers, skipped


def save_quantized_layers(layers: Dict[str, ResidualVQLinear], package_dir: str, *, model_id: str = "unknown") -> Dict[str, object]:
    """Writes the same container for layers of this package (one shard); used to ship CSR outliers, which the
    reference writer does not know.  Manifest keys follow ``OQPackManifest.to_dict`` (``ojasx_24x96/oqpack.py:96-150``)."""
    from safetensors.torch import save_file

    os.makedirs(package_dir, exist_ok=True)
    state: Dict[str, torch.Tensor] = {}
    specs: Dict[str, Dict[str, object]] = {}
    for name, layer in layers.items():
        enc = layer.encoded()
        state[f"{name}.packed_codes"] = enc.packed_codes.detach().cpu().contiguous()
        state[f"{name}.codebooks"] = enc.codebooks.detach().cpu().contiguous()
        state[f"{name}.row_scales"] = enc.row_scales.detach().cpu().contiguous()
        if layer.bias is not None:
            state[f"{name}.bias"] = layer.bias.detach().cpu().contiguous()
        if enc.outliers is not None:
            for key, t in zip(("csr_row_ptrs", "csr_col_indices", "csr_values"), enc.outliers):
                state[f"{name}.{key}"] = t.detach().cpu().contiguous()
        specs[name] = {"module_type": "linear", "type": "residual_vq_linear", "codec": "adaptive_residual_vq",
                       "in_features": layer.in_features, "out_features": layer.out_features,
                       "block_size": layer.block_size, "bits_per_stage": layer.bits_per_stage, "stages": enc.stages,
                       "gain_bits": 0, "rotation_reflections": 0, "adaptive_stages": True, "source_dtype": "float32",
                       "has_bias": layer.bias is not None, "bias": layer.bias is not None, "active_counts": None}
    shard = "shard-00001-of-00001.safetensors"
    path = os.path.join(package_dir, shard)
    save_file(state, path)
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    manifest = {
        "format_version": 1, "codec_schema_version": 1, "model_id": model_id, "source_checkpoint_sha256": "",
        "architecture_profile": {}, "memory_admission": {}, "quantization_plan": {}, "quality_certificate": None,
        "shards": [{"filename": shard, "sha256": h.hexdigest(), "size_bytes": os.path.getsize(path),
                    "tensor_names": list(state.keys())}],
        "tensors": {n: {"name": n, "shard": shard, "dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape),
                        "nbytes": t.numel() * t.element_size(), "role": "other"} for n, t in state.items()},
        "layer_specs": specs, "tokenizer_files": [], "chat_template": None,
    }
    tmp = os.path.join(package_dir, MANIFEST_FILENAME + ".tmp")
    with open(tmp, "w", encoding="utf-8") as f:
        f.write(json.dumps(manifest, indent=2) + "\n")
    os.replace(tmp, os.path.join(package_dir, MANIFEST_FILENAME))
    return manifest
