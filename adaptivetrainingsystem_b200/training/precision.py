"""Precision and quantisation registries (reference ``training/trainer.py:157-801``).

On this framework parameters live in the compute dtype (bf16 on B200) with fp32 master weights inside the sharded
optimiser, so "mixed_bf16" needs no autocast; autocast contexts are only produced for fp32-parameter CPU / fp16 runs.
fp8 precisions select the block-scaled e4m3 linear path of the model instead of wrapping ``torch.autocast``."""
from __future__ import annotations

from contextlib import nullcontext
from typing import Any, Dict, Optional

import torch

PRECISION_TABLE: Dict[str, Dict[str, Any]] = {
    "fp64": dict(dtype=torch.float64, bits=64, autocast=False), "fp32": dict(dtype=torch.float32, bits=32, autocast=False),
    "tf32": dict(dtype=torch.float32, bits=19, autocast=False, tf32=True),
    "fp16": dict(dtype=torch.float16, bits=16, autocast=False, loss_scale=True),
    "bf16": dict(dtype=torch.bfloat16, bits=16, autocast=False),
    "mixed_fp16": dict(dtype=torch.float16, bits=16, autocast=True, loss_scale=True),
    "mixed_bf16": dict(dtype=torch.bfloat16, bits=16, autocast=True),
    "fp8": dict(dtype=torch.bfloat16, bits=8, fp8="e4m3"), "fp8_e4m3": dict(dtype=torch.bfloat16, bits=8, fp8="e4m3"),
    "fp8_e5m2": dict(dtype=torch.bfloat16, bits=8, fp8="e5m2"), "mixed_fp8": dict(dtype=torch.bfloat16, bits=8, fp8="e4m3"),
    "int8": dict(dtype=torch.bfloat16, bits=8, quant=True), "int4": dict(dtype=torch.bfloat16, bits=4, quant=True),
}


class DynamicLossScaler:
    """x2 after ``growth_interval`` clean steps, x0.5 after ``hysteresis`` overflows (fp16 only)."""

    def __init__(self, init_scale: float = 65536.0, growth_interval: int = 1000, hysteresis: int = 2,
                 min_scale: float = 1.0, max_scale: float = 2.0 ** 32):
        self.scale, self.growth_interval, self.hysteresis = init_scale, growth_interval, hysteresis
        self.min_scale, self.max_scale = min_scale, max_scale
        self._good, self._bad = 0, 0

    def update(self, overflow: bool) -> None:
        if overflow:
            self._bad += 1
            self._good = 0
            if self._bad >= self.hysteresis:
                self.scale = max(self.scale / 2, self.min_scale)
                self._bad = 0
        else:
            self._good += 1
            if self._good >= self.growth_interval:
                self.scale = min(self.scale * 2, self.max_scale)
                self._good = 0


class PrecisionManager:
    def __init__(self, config, device: torch.device):
        self.config, self.device = config, device
        name = config.precision if config.precision != "auto" else "fp32"
        if name not in PRECISION_TABLE:
            raise ValueError(f"unknown precision {name}")
        self.name = name
        self.info = PRECISION_TABLE[name]
        self.loss_scaler: Optional[DynamicLossScaler] = DynamicLossScaler(config.fp16_loss_scale) if self.info.get("loss_scale") else None
        if self.info.get("tf32") or getattr(config, "tf32_enabled", False):
            torch.backends.cuda.matmul.allow_tf32 = True

    @property
    def compute_dtype(self) -> torch.dtype:
        return self.info["dtype"]

    @property
    def uses_fp8(self) -> bool:
        return "fp8" in self.info

    def autocast(self):
        # Parameters already live in the compute dtype; autocast only for fp32-parameter models on request.
        if self.info.get("autocast") and getattr(self.config, "autocast_fp32_params", False):
            return torch.autocast(self.device.type, dtype=self.info["dtype"])
        return nullcontext()

    def supported_precisions(self):
        return list(PRECISION_TABLE)

    def get_precision_info(self) -> Dict[str, Any]:
        return {"name": self.name, "bits": self.info["bits"], "dtype": str(self.info["dtype"]),
                "loss_scaling": self.loss_scaler is not None, "fp8": self.info.get("fp8")}


class QuantizationManager:
    """Post-training quantisation of the projection weights for inference (reference ``training/trainer.py:575-801``).

    The reference swaps ``nn.Linear`` for bitsandbytes / GPTQ / quanto modules, none of which ships here.  The native
    method is ``"fp8"`` (``quantization_method="fp8"`` or ``quantization_bits=8`` without a method): every 2-D projection
    weight is quantised per output channel to e4m3, activations per token at run time, and ``ops.linear`` / the SwiGLU MLP
    run on the ``kind::f8f6f4`` tensor-core GEMM with both scales applied in its epilogue.  ``"int8"`` is the same scheme with
    signed bytes on the ``kind::i8`` GEMM (W8A8), and ``"smoothquant"`` is int8 after :meth:`calibrate` has measured the
    activation range of every projection's input channels and moved it into the weights (``ops/int8.py``).  ``"int4"`` /
    ``"gptq"`` (or ``quantization_bits=4`` without a method) is weight-only 4-bit with groups of 128 input channels
    (``ops/int4.py``): codes by GPTQ for every projection :meth:`calibrate` collected a Hessian for, round-to-nearest for the
    rest; the language-model head, embeddings, routers and stacked expert weights stay in bf16.  The external backends are
    reported and refused when not installed."""

    NATIVE = ("fp8", "fp8_e4m3", "int8", "smoothquant", "int4", "gptq")

    def __init__(self, config):
        self.method = getattr(config, "quantization_method", None)
        self.bits = getattr(config, "quantization_bits", None)
        if self.method is None and self.bits == 8:
            self.method = "fp8"
        if self.method is None and self.bits == 4:
            self.method = "int4"
        self.gptq_weights = 0
        self.symmetric = bool(getattr(config, "quantization_symmetric", False))   # AutoGPTQ's ``sym``: zero point fixed at 8
        self.act_order = bool(getattr(config, "quantization_act_order", False))   # AutoGPTQ's ``desc_act`` with static groups
        self.applied = False
        self.calibrated = False
        self.quantized_tensors = 0
        self.quantized_bytes = 0

    @torch.no_grad()
    def calibrate(self, model, batches, alpha: float = 0.5) -> int:
        """Runs ``batches`` (token id tensors) through the unquantised model while every projection records what its method
        needs: the largest |x| of each input channel (SmoothQuant; returns the number of projections that got smoothing
        factors) or the Hessian sum x^T x of its input rows (``"int4"`` / ``"gptq"``; returns the number of Hessians)."""
        from ..ops import int4, int8
        was = model.training
        model.eval()
        if self.method in ("int4", "gptq"):
            int4.set_enabled(False)
            int4.observe(True, only=[p for _, p in self._int4_targets(model)])
            try:
                for ids in batches:
                    model(ids, return_aux_loss=False)
            finally:
                int4.observe(False)
                model.train(was)
            self.calibrated = int4.hessian_count() > 0
            return int4.hessian_count()
        int8.set_enabled(False)
        int8.observe(True)
        try:
            for ids in batches:
                model(ids, return_aux_loss=False)
        finally:
            int8.observe(False)
            model.train(was)
        n = int8.finish_calibration(alpha)
        self.calibrated = n > 0
        return n

    @staticmethod
    def _int4_targets(model):
        """(name, parameter) of every projection the 4-bit path covers, in model order."""
        from ..ops import int4
        return [(name, p) for name, p in model.named_parameters()
                if p.dim() == 2 and int4.shape_ok(p.shape[0], p.shape[1]) and "embed" not in name and "lm_head" not in name
                and "gate.weight" not in name and "router" not in name and getattr(p, "_ats_z3", None) is None]

    def _register_int4(self, p) -> None:
        from ..ops import int4
        packed, meta, used_gptq = int4.register(p, sym=self.symmetric, act_order=self.act_order)
        self.quantized_tensors += 1
        self.gptq_weights += int(used_gptq)
        self.quantized_bytes += packed.numel() * 4 + meta.numel() * 4

    @torch.no_grad()
    def quantize_sequential(self, model, batches):
        """GPTQ block by block (AutoGPTQ's ``true_sequential``): the Hessians of a block's projections are collected from inputs
        that already went through the quantised blocks before it, so every block compensates for the error made upstream; only
        one block's Hessians exist at a time.  Costs one pass over ``batches`` per block."""
        if self.method not in ("int4", "gptq"):
            raise RuntimeError("block-by-block quantisation is the 4-bit GPTQ path (quantization_method 'int4' or 'gptq')")
        from ..ops import int4
        model.eval()
        for p in model.parameters():
            p.requires_grad_(False)
        blocks: Dict[str, list] = {}
        for name, p in self._int4_targets(model):
            parts = name.split(".")
            key = ".".join(parts[:2]) if parts[0] == "layers" and len(parts) > 2 else parts[0]
            blocks.setdefault(key, []).append(p)
        int4.set_enabled(True)              # registered projections run quantised from the moment they exist
        try:
            for key, params in blocks.items():
                int4.observe(True, only=params)
                for ids in batches:
                    model(ids, return_aux_loss=False)
                int4.observe(False)
                for p in params:
                    self._register_int4(p)
                int4.drop_hessians()
        finally:
            int4.observe(False)
        self.calibrated = self.applied = True
        return model

    # -- 4-bit copies at rest ----------------------------------------------------------------------------------------------------
    def save_quantized(self, model, path: str) -> int:
        """Writes the packed 4-bit copies (codes + scale words per projection, by parameter name) so that a later process can
        serve them without repeating the calibration (AutoGPTQ's ``save_quantized``).  -> number of tensors written."""
        from ..ops import int4
        tensors = {}
        for name, p in self._int4_targets(model):
            hit = int4.lookup(p)
            if hit is not None:
                tensors[name] = {"packed": hit[0].cpu(), "meta": hit[1].cpu(), "group": int(hit[2])}
        if not tensors:
            raise RuntimeError("no projection of this model has a 4-bit copy: run quantize_model / quantize_sequential first")
        torch.save({"format": "ats-int4-v1", "symmetric": self.symmetric, "tensors": tensors}, path)
        return len(tensors)

    @torch.no_grad()
    def load_quantized(self, model, path: str, release_originals: bool = False) -> int:
        """Attaches saved 4-bit copies to the projections of ``model`` (same architecture) and switches the 4-bit path on.  With
        ``release_originals`` the bf16 storage of those projections is freed (see :meth:`release_originals`)."""
        from ..ops import int4
        blob = torch.load(path, map_location="cpu", weights_only=True)
        if not isinstance(blob, dict) or blob.get("format") != "ats-int4-v1":
            raise RuntimeError(f"{path} is not a file written by save_quantized")
        model.eval()
        for p in model.parameters():
            p.requires_grad_(False)
        params = dict(self._int4_targets(model))
        missing = [n for n in blob["tensors"] if n not in params]
        if missing:
            raise RuntimeError(f"saved 4-bit copies for parameters this model does not have: {missing[:4]}")
        for name, t in blob["tensors"].items():
            int4.register_packed(params[name], t["packed"], t["meta"], int(t["group"]))
            self.quantized_tensors += 1
            self.quantized_bytes += t["packed"].numel() * 4 + t["meta"].numel() * 4
        self.method, self.bits, self.symmetric = "int4", 4, bool(blob.get("symmetric", False))
        int4.set_enabled(True)
        self.applied = True
        if release_originals:
            self.release_originals(model)
        return len(blob["tensors"])

    @torch.no_grad()
    def release_originals(self, model) -> int:
        """Frees the bf16 storage of every projection that has a 4-bit copy: the model then holds a quarter of the projection
        bytes (head, embeddings, norms and routers stay).  From here on the model serves only through the 4-bit path: its
        ``state_dict`` no longer holds those weights (use :meth:`save_quantized`), and it cannot be trained.  -> bytes freed."""
        from ..ops import int4
        freed = 0
        for name, p in self._int4_targets(model):
            if int4.lookup(p) is not None and p.stride() != (0, 0):
                freed += int4.release_original(p)
        self.released_bytes = getattr(self, "released_bytes", 0) + freed
        return freed

    def available_backends(self) -> Dict[str, bool]:
        out = {"fp8 (native e4m3 GEMM)": torch.cuda.is_available(), "int8 / smoothquant (native s8 GEMM)": True,
               "int4 / gptq (native weight-only 4-bit)": True}
        for mod in ("bitsandbytes", "auto_gptq", "optimum.quanto"):
            try:
                __import__(mod)
                out[mod] = True
            except Exception:
                out[mod] = False
        return out

    def quantize_model(self, model):
        if not self.method:
            return model
        if self.method not in self.NATIVE:
            raise RuntimeError(f"quantization backend for {self.method!r} is not installed; available: {self.available_backends()}")
        from ..ops import fp8, int4, int8
        if self.method == "gptq" and not self.calibrated:
            raise RuntimeError("gptq needs calibration inputs: call calibrate(model, batches) before quantize_model")
        model.eval()
        for p in model.parameters():
            p.requires_grad_(False)
        if self.method in ("int4", "gptq"):
            for name, p in self._int4_targets(model):
                self._register_int4(p)
            int4.drop_hessians()
            int4.set_enabled(True)
            self.applied = True
            return model
        if self.method in ("int8", "smoothquant"):
            if self.method == "smoothquant" and not self.calibrated:
                raise RuntimeError("smoothquant needs activation ranges: call calibrate(model, batches) before quantize_model")
            int8.set_enabled(True)
            for name, p in model.named_parameters():
                if p.dim() == 2 and p.shape[1] % 16 == 0 and "embed" not in name and "gate.weight" not in name and "router" not in name:
                    q, sc, _ = int8.quantized_weight(p)
                    self.quantized_tensors += 1
                    self.quantized_bytes += q.numel() + sc.numel() * 4
            self.applied = True
            return model
        fp8.set_enabled(True)
        if torch.cuda.is_available():
            # quantise once, up front: the cache is keyed on the storage and stays valid while the weights are frozen
            for name, p in model.named_parameters():
                if p.dim() == 2 and p.is_cuda and p.dtype == torch.bfloat16 and p.shape[1] % 16 == 0 and "embed" not in name \
                        and "gate.weight" not in name and "router" not in name:
                    q, sc = fp8.quantized_weight(p)
                    self.quantized_tensors += 1
                    self.quantized_bytes += q.numel() + sc.numel() * 4
                elif p.dim() == 3 and getattr(p, "_ats_expert", False) and p.is_cuda and p.dtype == torch.bfloat16 and p.shape[2] % 16 == 0 \
                        and not getattr(p, "_ats_packed", False):
                    q, sc = fp8.quantized_expert_weight(p)      # stacked expert weights: per output channel of every expert
                    self.quantized_tensors += 1
                    self.quantized_bytes += q.numel() + sc.numel() * 4
        self.applied = True
        return model

    # -- names of the reference's manager (``training/trainer.py:681-801``) --------------------------------------------------------
    @property
    def is_quantized(self) -> bool:
        return self.applied

    def quantize_model_gptq(self, model, batches=None):
        """GPTQ, 4 bits, groups of 128 (the reference's AutoGPTQ configuration: ``sym=True, true_sequential=True`` are
        ``quantization_symmetric`` and the block-by-block pass taken when ``batches`` are given here)."""
        self.method, self.bits = "gptq", 4
        if batches is not None:
            return self.quantize_sequential(model, batches)
        return self.quantize_model(model)

    def create_quantized_optimizer(self, model):
        """The reference returns an optimiser only for bitsandbytes 8-bit modules; post-training quantisation here freezes the
        model (no parameter requires a gradient), so there is nothing to optimise."""
        return None

    def get_quantization_info(self) -> Dict[str, Any]:
        b = self.available_backends()
        return {"is_quantized": self.applied, "method": self.method, "bits": self.bits,
                "available_methods": {"bnb": b.get("bitsandbytes", False), "gptq": True, "quanto": b.get("optimum.quanto", False),
                                      "fp8": b["fp8 (native e4m3 GEMM)"], "int8": True, "smoothquant": True, "int4": True}}

    def status(self) -> Dict[str, Any]:
        return {"method": self.method, "bits": self.bits, "applied": self.applied, "tensors": self.quantized_tensors,
                "quantized_bytes": self.quantized_bytes, "gptq_weights": self.gptq_weights, "backends": self.available_backends()}
