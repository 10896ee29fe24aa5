"""JSON configuration of a VAR-Q run (same file format and accessors as the reference's
``VAR_Q/config_loader.py:10-128``; files written for the reference load unchanged).

Sections: ``model``, ``quantization``, ``inference``, ``batch_processing`` (optional) and
``checkpoints``.  ``quantization`` understands, beyond the reference's
``enable / q_bits / quant_method / qkv_format``, the optional keys

    "symmetric": bool, "group_size": int, "reduce_batch": bool,
    "k": {...}, "v": {...}      per-tensor overrides of any of the keys above

and the method aliases of the Infinity command line (``G_SCALE_PER_HEAD``, ``PER_DIM``;
Infinity/tools/run_infinity.py:421-422), which the reference class itself rejects.
"""
import copy
import json
import os
from typing import Any, Dict, Optional, Tuple

_SECTIONS = ("model", "quantization", "inference", "checkpoints")
_METHOD_ALIASES = {
    "G_SCALE_PER_HEAD": "G_TOKEN_HEAD", "PER_HEAD": "G_TOKEN_HEAD",
    "PER_DIM": "G_SCALE_HEAD_DIM", "PER_CHANNEL": "G_SCALE_HEAD_DIM",
    "PER_TENSOR": "G_SCALE", "PER_TOKEN": "G_TOKEN",
}
_QUANTIZER_KEYS = ("q_bits", "quant_method", "qkv_format", "symmetric", "group_size", "reduce_batch")


def _merge(base: Dict[str, Any], patch: Dict[str, Any]) -> Dict[str, Any]:
    for key, val in patch.items():
        if isinstance(val, dict):
            base[key] = _merge(base[key] if isinstance(base.get(key), dict) else {}, val)
        else:
            base[key] = val
    return base


class VARQConfig:
    """Holds the parsed JSON in ``self.config`` and hands out copies of its sections."""

    def __init__(self, config_path: Optional[str] = None):
        self._path = config_path or os.path.join(os.path.dirname(__file__), "config.json")
        with open(self._path, "r") as fh:
            self.config = json.load(fh)

    def _section(self, name: str, required: bool = True) -> Dict[str, Any]:
        if required:
            return copy.copy(self.config[name])
        return copy.copy(self.config.get(name, {}))

    def get_model_config(self) -> Dict[str, Any]:
        return self._section("model")

    def get_quantization_config(self) -> Dict[str, Any]:
        return self._section("quantization")

    def get_inference_config(self) -> Dict[str, Any]:
        return self._section("inference")

    def get_checkpoint_config(self) -> Dict[str, Any]:
        return self._section("checkpoints")

    def get_batch_processing_config(self) -> Dict[str, Any]:
        return self._section("batch_processing", required=False)

    def get_checkpoint_paths(self, model_depth: Optional[int] = None) -> Tuple[str, str]:
        """(vae checkpoint, transformer checkpoint); VAR files are named by depth."""
        ck = self.get_checkpoint_config()
        if "model_path" in ck:
            return ck["vae_ckpt"], ck["model_path"]
        if "var_ckpt_template" in ck and model_depth is not None:
            return ck["vae_ckpt"], ck["var_ckpt_template"].format(model_depth)
        raise ValueError("Either 'model_path' or 'var_ckpt_template' with model_depth must be provided")

    def get_device(self) -> str:
        import torch
        want = self.config["inference"]["device"]
        return "cpu" if (want == "cuda" and not torch.cuda.is_available()) else want

    def is_infinity_model(self) -> bool:
        return "infinity" in self.get_model_config().get("model_type", "").lower()

    def is_var_model(self) -> bool:
        return not self.is_infinity_model()

    def update_config(self, updates: Dict[str, Any]):
        self.config = _merge(self.config, updates)

    def save_config(self, save_path: Optional[str] = None):
        target = save_path or os.path.join(os.path.dirname(__file__), "config.json")
        with open(target, "w") as fh:
            json.dump(self.config, fh, indent=2)

    # ---- extension: constructor arguments of the K and V quantizers
    def get_quantizer_kwargs(self, which: str = "k") -> Optional[Dict[str, Any]]:
        """Keyword arguments for ``VAR_Q(...)`` of the K (``which='k'``) or V cache, or None
        when quantization is disabled."""
        if which not in ("k", "v"):
            raise ValueError("which must be 'k' or 'v'")
        q = self.get_quantization_config()
        if not q.get("enable", False):
            return None
        merged = {k: q[k] for k in _QUANTIZER_KEYS if k in q}
        merged.update({k: v for k, v in q.get(which, {}).items() if k in _QUANTIZER_KEYS})
        method = merged.get("quant_method", "G_SCALE_HEAD_DIM")
        kwargs = {
            "quant_bits": int(merged.get("q_bits", 8)),
            "quant_method": _METHOD_ALIASES.get(method, method),
            "qkv_format": merged.get("qkv_format", "BLHc"),
        }
        for opt in ("symmetric", "group_size", "reduce_batch"):
            if opt in merged:
                kwargs[opt] = merged[opt]
        return kwargs


def load_varq_config(config_path: Optional[str] = None) -> VARQConfig:
    return VARQConfig(config_path)
