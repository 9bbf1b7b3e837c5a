"""Packed expert checkpoints: W8 expert stacks written once and loaded ready-made, so that start-up skips the weight
quantisation (the interface of the reference's src/lemoq/quant/expert_calibration.py: ``validate_packed`` :23,
``file_sha256`` :303, ``save_packed`` :311, ``load_bundle`` :322; consumed by ``replace_moe_blocks(prequantized=...)``,
src/lemoq/kernels/moe_static.py:467-504).

A bundle is a directory: one ``torch.save`` file per decoder layer with the four tensors of a ``QuantFusedExperts``
plus ``bits`` and ``group_size``, and ``manifest.json`` with status, model id and, per layer, file name, SHA-256,
bits and group size.  Only what the decode path needs is here: the reference's calibration passes (GPTQ statistics,
per-layer search) are not part of this project; :func:`export_rtn_bundle` writes the bundle of the canonical
round-to-nearest W8 quantisation, which is what the reference's ``algorithm="rtn"`` arm produces.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any

import torch

from lemoq.kernels.moe_grouped_quant import QuantFusedExperts

_FIELDS = ("packed_gate_up", "scale_gate_up", "packed_down", "scale_down")
MANIFEST = "manifest.json"


def _expected_layout(q: QuantFusedExperts, experts: int, hidden: int, ffn: int) -> dict[str, tuple[tuple[int, ...], Any]]:
    """Field -> (shape, dtype) of a container for ``experts`` experts of the given widths."""
    per_byte = 8 // q.bits  # codes per byte: two for 4-bit payloads
    codes = torch.int8 if q.bits == 8 else torch.uint8
    g = q.group_size
    return {
        "packed_gate_up": ((experts, 2 * ffn, hidden // per_byte), codes),
        "scale_gate_up": ((experts, 2 * ffn, hidden // g), torch.float16),
        "packed_down": ((experts, hidden, ffn // per_byte), codes),
        "scale_down": ((experts, hidden, ffn // g), torch.float16),
    }


def validate_packed(q: Any, *, experts: int, hidden: int, ffn: int) -> None:
    """Raise ``ValueError`` unless ``q`` is a well-formed container for these sizes: 4 or 8 bits, an even group size
    that divides both widths, every tensor of the expected shape, dtype and contiguous, scales finite and not negative
    (zero is allowed: a tiny group's fp32 scale may underflow in fp16, and dequantises to zero), one device."""
    if not isinstance(q, QuantFusedExperts) or q.bits not in (4, 8):
        raise ValueError("invalid pre-quantized expert container")
    g = q.group_size
    if type(g) is not int or g < 2 or g % 2:
        raise ValueError("invalid grouped scale size")
    if hidden % g or ffn % g:
        raise ValueError("group size must divide hidden and ffn")
    devices = set()
    for name, (shape, dtype) in _expected_layout(q, experts, hidden, ffn).items():
        t = getattr(q, name)
        if not (torch.is_tensor(t) and tuple(t.shape) == shape and t.dtype == dtype and t.is_contiguous()):
            raise ValueError("packed shape/dtype/layout mismatch: " + name)
        if dtype == torch.float16 and not bool((torch.isfinite(t) & (t >= 0)).all()):
            raise ValueError("scales must be finite and nonnegative")
        devices.add(t.device)
    if len(devices) != 1:
        raise ValueError("packed buffers must share a device")


def file_sha256(path: Path) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as fh:
        while chunk := fh.read(8 << 20):
            digest.update(chunk)
    return digest.hexdigest()


def save_packed(path: Path, quant: QuantFusedExperts) -> str:
    """Write one layer's container (CPU tensors) to a NEW file; returns the file's SHA-256."""
    path = Path(path)
    payload: dict[str, Any] = {name: getattr(quant, name).detach().cpu().contiguous() for name in _FIELDS}
    payload.update(bits=int(quant.bits), group_size=int(quant.group_size))
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("xb") as fh:  # never overwrites
        torch.save(payload, fh)
    return file_sha256(path)


def _block_sizes(layer: Any) -> tuple[int, int, int]:
    """(experts, hidden, ffn) of a decoder layer's MoE block, before or after its experts were fused."""
    block = layer.mlp
    members = getattr(block, "experts", None)
    if members is not None:
        return len(members), int(members[0].gate_proj.in_features), int(members[0].down_proj.in_features)
    fused = block._static_experts
    return int(fused.num_experts), int(fused.hidden), int(fused.ffn)


def load_bundle(directory: Path, model: Any, *, expected_model_id: str) -> dict[int, QuantFusedExperts]:
    """Read a bundle for ``model``: layer index -> container (CPU), ready for ``replace_moe_blocks(prequantized=...)``.
    Everything is checked before anything is returned: a complete manifest for this model id that lists every layer
    once and in order, plain file names, matching hashes, well-formed payloads that agree with the manifest."""
    directory = Path(directory)
    manifest = json.loads((directory / MANIFEST).read_text())
    if manifest.get("status") != "complete" or manifest.get("model_id") != expected_model_id:
        raise ValueError("incomplete bundle or checkpoint identity mismatch")
    rows = manifest.get("layers", [])
    decoder_layers = list(model.model.layers)
    if [row.get("layer") for row in rows] != list(range(len(decoder_layers))):
        raise ValueError("bundle does not cover every model layer exactly once")
    loaded: dict[int, QuantFusedExperts] = {}
    for row, layer in zip(rows, decoder_layers):
        name = row["file"]
        if Path(name).name != name:
            raise ValueError("bundle paths must be local filenames")
        path = directory / name
        if file_sha256(path) != row["sha256"]:
            raise ValueError("packed checkpoint hash mismatch")
        state = torch.load(path, map_location="cpu", weights_only=True)
        q = QuantFusedExperts(**state)
        experts, hidden, ffn = _block_sizes(layer)
        validate_packed(q, experts=experts, hidden=hidden, ffn=ffn)
        if (q.bits, q.group_size) != (row["bits"], row["group_size"]):
            raise ValueError("precision manifest does not match packed payload")
        loaded[int(row["layer"])] = q
    return loaded


def write_bundle(directory: Path, containers: dict[int, QuantFusedExperts], *, model_id: str, algorithm: str = "rtn") -> dict[str, Any]:
    """Write one file per layer (layers ``0 .. n-1``, all present) and the manifest; returns the manifest."""
    directory = Path(directory)
    if sorted(containers) != list(range(len(containers))):
        raise ValueError("a bundle holds every layer 0 .. n-1 exactly once")
    rows = []
    for index in range(len(containers)):
        quant = containers[index]
        name = "layer_%03d.pt" % index
        rows.append({"layer": index, "file": name, "sha256": save_packed(directory / name, quant), "bits": int(quant.bits),
                     "group_size": int(quant.group_size), "algorithm": algorithm})
    manifest = {"status": "complete", "model_id": model_id, "format": "lemoq packed experts v1", "layers": rows}
    (directory / MANIFEST).write_text(json.dumps(manifest, indent=1))
    return manifest


def export_rtn_bundle(model: Any, directory: Path, *, model_id: str, group_size: int = 128) -> dict[str, Any]:
    """Quantise every layer's experts (symmetric 8-bit round to nearest on the fused stacks, the canonical scheme;
    runs the CUDA quantiser) and write the bundle; returns the manifest.  ``model`` still has its expert modules (call
    before ``replace_moe_blocks``); it is not modified."""
    from lemoq.kernels.moe_grouped_quant import quantize_fused_experts
    from lemoq.kernels.moe_static import fuse_experts

    containers = {}
    for index, layer in enumerate(model.model.layers):
        quant = quantize_fused_experts(fuse_experts(layer.mlp.experts), bits=8, group_size=int(group_size)).to("cpu")
        experts, hidden, ffn = _block_sizes(layer)
        validate_packed(quant, experts=experts, hidden=hidden, ffn=ffn)
        containers[index] = quant
    return write_bundle(directory, containers, model_id=model_id, algorithm="rtn")
