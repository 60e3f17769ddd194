"""``export_for_inference``: a serving checkpoint from a trained model.

The reference's deployment guide calls ``export_utils.export_for_inference`` (``docs/adaptive_training.md:1659-1680``) but ships no
such module.  Here it writes what the chat entry point reads: the weights in the serving dtype plus the model configuration in
one file, and -- for ``quantize="int4"`` -- the packed 4-bit copies of the projections next to it, so that the serving process
neither repeats the calibration nor keeps the bf16 projections in memory.
"""
from __future__ import annotations

import os
from types import SimpleNamespace
from typing import Any, Dict, Iterable, Optional

import torch

EXPORT_FORMAT = "ats-inference-v1"


@torch.no_grad()
def export_for_inference(model, path: str, dtype: torch.dtype = torch.bfloat16, quantize: Optional[str] = None,
                         calibration_batches: Optional[Iterable[torch.Tensor]] = None, symmetric: bool = False) -> Dict[str, Any]:
    """Writes ``path`` (keys ``model_state_dict``, ``model_config``, ``format``; readable by ``Chat.py --checkpoint``).

    ``quantize="int4"`` also writes ``path + ".int4"``: weight-only 4-bit copies of the projections, GPTQ-calibrated block by
    block when ``calibration_batches`` (token id tensors on the model's device) are given, round-to-nearest otherwise; serve
    them with ``Chat.py --quantize int4 --quantized-file <that file>``.  The model itself is left unquantised.
    Returns the paths written and their sizes."""
    if quantize not in (None, "int4"):
        raise ValueError("export_for_inference: only 'int4' copies are stored at rest (fp8 / int8 are quantised when the server loads)")
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    sd = {k: (v.detach().to("cpu", dtype) if v.is_floating_point() else v.detach().cpu()) for k, v in model.state_dict().items()}
    torch.save({"format": EXPORT_FORMAT, "model_state_dict": sd, "model_config": model.config.to_dict(), "dtype": str(dtype)}, path)
    out: Dict[str, Any] = {"checkpoint": path, "checkpoint_bytes": os.path.getsize(path)}
    if quantize == "int4":
        from ..ops import int4
        from ..training.precision import QuantizationManager
        was_training = model.training
        grads = [p.requires_grad for p in model.parameters()]
        qm = QuantizationManager(SimpleNamespace(quantization_method="int4", quantization_bits=4, quantization_symmetric=symmetric))
        try:
            if calibration_batches is not None:
                qm.quantize_sequential(model, list(calibration_batches))
            else:
                qm.quantize_model(model)
            qpath = path + ".int4"
            out.update(quantized=qpath, quantized_tensors=qm.save_quantized(model, qpath), gptq_tensors=qm.gptq_weights)
            out["quantized_bytes"] = os.path.getsize(qpath)
        finally:
            # the exporter's own model keeps running unquantised
            int4.set_enabled(False)
            int4.clear()
            for p, g in zip(model.parameters(), grads):
                p.requires_grad_(g)
            model.train(was_training)
    return out
