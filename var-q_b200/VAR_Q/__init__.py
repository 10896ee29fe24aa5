"""Drop-in ``VAR_Q`` package backed by the varq_b200 CUDA library (B200 / sm_100a).

Importable under the module names the VAR and Infinity attention hooks use
(``VAR_Q.quant``, ``VAR_Q.pack_unpack``, ``VAR_Q.config_loader``) once the directory
that contains this package is on ``sys.path`` -- the same convention as the
reference project (VAR/models/basic_var.py:11-21, Infinity/infinity/models/basic.py:24-28).
"""
__all__ = ["quant", "pack_unpack", "config_loader", "attention", "hooks", "sharding"]
