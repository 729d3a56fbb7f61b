"""Model registry for config.json models: architecture name -> model class. ``build_model`` is what every entry point (the generation
command line, the trace replayer, the tests) uses to go from a model folder to a model on the device."""
from __future__ import annotations

from ..config import BF16, F32, read_model_config
from .kodezen import KodezenModel
from .munazen import MunazenModel
from .sopetar import SopetarModel
from .vasosun import VasosunModel

MODEL_CLASSES = {"Munazen": MunazenModel, "Sopetar": SopetarModel, "Vasosun": VasosunModel, "Kodezen": KodezenModel}


def build_model(model_dir: str, dtype: str = "bfloat16", device="cuda", build: bool = False):
    """Read config.json, pick the class of its architecture, load model.safetensors in the storage type of ``dtype``
    ("bfloat16": bf16 matrices, fp32 accumulation and fp32 everywhere the design asks for it; "float32": everything fp32)."""
    import torch

    from .. import weights
    from ..seqops import Ops
    cfg = read_model_config(model_dir)
    w_dtype = {"bfloat16": BF16, "float32": F32}[dtype]
    ops = Ops(w_dtype, build=build)
    dev = torch.device(device)
    return MODEL_CLASSES[cfg.architecture](cfg, weights.load(model_dir, w_dtype, dev), ops, dev)
